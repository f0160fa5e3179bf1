// Dense decode of whole experts to fp16 matrices: one warp per 16x128 unit, staged through shared memory so
// that global stores are full 256-byte row segments.  HBM-bound by the fp16 output (2 B per weight written
// against 0.25-0.52 B per weight read).
#include "nq_common.cuh"
#include "nq_unit.cuh"

namespace nq {

constexpr int kTileStride = 68;   // 32-bit words per tile row: 64 + 4 pad (16-byte aligned rows, conflict-free fragment stores)

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

// grid (ceil(max_units / 8), n_experts, 2 = gate|up / down), 256 threads
__global__ void __launch_bounds__(256) pf_decode_kernel(const int64_t* __restrict__ table, const int32_t* __restrict__ experts,
                                                        __half* Wgu, __half* Wdn, int H, int I, int nm_gu, int nm_dn,
                                                        int force_level)
{
    __shared__ __align__(16) uint32_t tiles[8][16 * kTileStride];
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
    Wout += (size_t)blockIdx.y * N * K + (size_t)strip * 16 * K + (size_t)ch * 128;
    if (level <= 0)
    {
        for (int i = lane; i < 256; i += 32) *(uint4*)(Wout + (size_t)(i >> 4) * K + (i & 15) * 8) = make_uint4(0, 0, 0, 0);
        return;
    }
    const ProjPlanes P = planes_from_row(row, down);
    const int nm = down ? nm_dn : nm_gu, rc = (int)row[10 + down], bk = (int)(row[19] >> (8 * down)) & 0xFF;
    const UnitRef u = locate_unit(P, strip, ch, C, NS, nm, level);
    decode_unit_dispatch(P, u, rc, bk, lane, TileSink{tile, lane >> 2, lane & 3});
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
