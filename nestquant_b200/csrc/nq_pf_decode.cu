// Dense decode of whole experts to fp16 matrices: one warp per 16x128 unit, staged through shared memory so
// that global stores are full 256-byte row segments.  HBM-bound by the fp16 output (2 B per weight written
// against 0.25-0.52 B per weight read).
#include "nq_common.cuh"
#include "nq_unit.cuh"

namespace nq {

constexpr int kTileStride = 68;   // 32-bit words per tile row: 64 + 4 pad keeps rows 16-byte aligned and spreads the 8 rows a fragment
                                  // store touches over all banks

struct TileSink
{
    uint32_t* tile; int g, t4;
    template <int T>
    __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const
    {
#pragma unroll
        for (int q = 0; q < 4; ++q) tile[(g + (q & 1) * 8) * kTileStride + T * 8 + t4 + (q >> 1) * 4] = a[q];
    }
};

// fetch the unit's records into the warp's stage, read them back and decode
template <bool RES, int RC, int BK>
__device__ __forceinline__ void decode_one(const ProjPlanes& P, const StripRef& sr, int ch, int C, int NS, uint32_t sign2, int lane,
                                           uint32_t st, const TileSink& sink)
{
    RecordCursor<BK> cb;
    cb.init(P.base, (size_t)NS * C * 32, sr.unit0 + ch, lane);
    cb.copy(st, 0, lane);
    uint32_t wb[Pattern<BK>::kWords + 2], wr[Pattern<RC>::kWords + 2];
    if constexpr (RES)
    {
        RecordCursor<RC> cr;
        cr.init(P.p4, sr.res_nrec, sr.res0 + refined_before(sr, ch), lane);
        cr.copy(st + kStageBase, 0, lane);
    }
    cp_async_commit();
    cp_async_wait<0>();
    RecordCursor<BK>::read(wb, st, lane);
    if constexpr (RES)
    {
        RecordCursor<RC>::read(wr, st + kStageBase, lane);
        const uint32_t word = __ldg(P.d4 + sr.res0 + refined_before(sr, ch));
        decode_unit<true, RC, BK>(wb, wr, consts_level4(block_multipliers(word), word, sign2), lane, sink);
    }
    else
        decode_unit<false, 0, BK>(wb, wr, consts_level2(sign2), lane, sink);
}

// grid (ceil(max_units / 8), n_experts, 2 = gate|up / down), 256 threads.  The records take the same road as in the
// GEMV and the fused GEMM (cp.async into a per-warp stage, read back by the lane that copied them).
__global__ void __launch_bounds__(256) pf_decode_kernel(const int64_t* __restrict__ table, const int32_t* __restrict__ experts,
                                                        __half* Wgu, __half* Wdn, int H, int I, int nm_gu, int nm_dn,
                                                        int force_level)
{
    __shared__ __align__(16) uint32_t tiles[8][16 * kTileStride];
    __shared__ __align__(16) uint8_t stages[8][kStageBytes];
    const int down = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __half* Wout = down ? Wdn : Wgu;
    if (!Wout) return;
    const int N = down ? H : 2 * I, K = down ? I : H, C = K / 128, NS = N / 16;
    const int unit = blockIdx.x * 8 + warp;
    if (unit >= NS * C) return;   // warp-uniform
    const int strip = unit / C, ch = unit - strip * C;
    const int64_t* row = table + (int64_t)experts[blockIdx.y] * kTableWidth;
    int level = (int)row[0];
    if (force_level > 0 && level > 0) level = force_level;
    uint32_t* tile = tiles[warp];
    uint8_t* st = stages[warp];
    Wout += (size_t)blockIdx.y * N * K + (size_t)strip * 16 * K + (size_t)ch * 128;
    if (level <= 0)
    {
        for (int i = lane; i < 256; i += 32) *(uint4*)(Wout + (size_t)(i >> 4) * K + (i & 15) * 8) = make_uint4(0, 0, 0, 0);
        return;
    }
    const ProjPlanes P = planes_from_row(row, down);
    const int nm = down ? nm_dn : nm_gu, rc = (int)row[10 + down], bk = (int)(row[19] >> (8 * down)) & 0xFF;
    const StripRef sr = locate_strip(P, strip, C, NS, nm, level >= 4);
    const bool refined = chunk_refined(sr, ch);
    const uint32_t sign2 = P.var ? sign_mask(__ldg(P.var + sr.unit0 + ch), lane) : 0u;
    const TileSink sink{tile, lane >> 2, lane & 3};
#define NQ_RUN(RES, RCV, BKV) decode_one<RES, RCV, BKV>(P, sr, ch, C, NS, sign2, lane, smem_addr(st), sink)
    NQ_WITH_CODES(refined, rc, bk, 0x3FF, NQ_RUN);
#undef NQ_RUN
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const int i = lane + 32 * j, r = i >> 4, c8 = i & 15;   // 16 rows x 16 segments of 8 halves
        *(uint4*)(Wout + (size_t)r * K + c8 * 8) = *(const uint4*)(tile + r * kTileStride + c8 * 4);
    }
}

}  // namespace nq

extern "C" int nq_pf_decode(const int64_t* table, const int32_t* experts, int n_experts, void* Wgu, void* Wdn,
                            int H, int I, int nm_gu, int nm_dn, int force_level, void* stream)
{
    NQ_REQUIRE(table && experts, "nq_pf_decode: null table or expert list");
    NQ_REQUIRE(n_experts >= 0, "nq_pf_decode: n_experts = %d", n_experts);
    // gate|up is [2I][H] (K = H), down is [H][I] (K = I): K must be whole 128-wide chunks (at most 64 per strip, the width
    // of a flags word), row counts whole 16-row strips
    NQ_REQUIRE(H > 0 && I > 0 && H % 128 == 0 && H / 128 <= 64 && I % 8 == 0, "nq_pf_decode: H = %d, I = %d", H, I);
    NQ_REQUIRE(!Wdn || (I % 128 == 0 && I / 128 <= 64), "nq_pf_decode: I = %d must be a multiple of 128, at most 64 * 128", I);
    NQ_REQUIRE(nq::aligned16(Wgu) && nq::aligned16(Wdn), "nq_pf_decode: outputs must be 16-byte aligned");
    NQ_REQUIRE(force_level == 0 || force_level == 2 || force_level == 4, "nq_pf_decode: force_level = %d", force_level);
    if (n_experts == 0 || (!Wgu && !Wdn)) return NQ_OK;
    const int ugu = (2 * I / 16) * (H / 128), udn = (H / 16) * (I / 128);
    const int units = ugu > udn ? ugu : udn;
    nq::pf_decode_kernel<<<dim3((units + 7) / 8, n_experts, 2), 256, 0, (cudaStream_t)stream>>>(
        table, experts, (__half*)Wgu, (__half*)Wdn, H, I, nm_gu, nm_dn, force_level);
    return nq::check_launch("nq_pf_decode");
}
