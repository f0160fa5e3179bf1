// One 16x128 unit per warp: locate its records, load them, decode them k-step by k-step.
#pragma once
#include "nq_format.cuh"

namespace nq {

// where a unit's records live and whether it is refined (level 4 and, in mask mode, flagged)
struct UnitRef
{
    size_t base_rec;    // first base record (unit index * 32)
    size_t res_rec;     // first residual record (dense or compact index * 32)
    size_t res_nrec;    // records in the residual plane
    size_t base_nrec;   // records in the base plane
    size_t unit;        // strip * C + chunk
    size_t res_unit;    // index into d4
    bool refined;
};

// Mask mode (sm120/nqmoe.cu:202-206): chunk ch of a strip is refined iff bit ch of flags[strip]; refined chunks are
// stored compactly, nm per strip.
__device__ __forceinline__ UnitRef locate_unit(const ProjPlanes& P, int strip, int ch, int C, int NS, int nm, int level)
{
    UnitRef u;
    u.unit = (size_t)strip * C + ch;
    u.base_rec = u.unit * 32;
    u.refined = level >= 4;
    u.res_unit = u.unit;
    u.res_nrec = u.base_nrec = (size_t)NS * C * 32;
    if (u.refined && P.flags)
    {
        const unsigned long long fl = __ldg((const unsigned long long*)P.flags + strip);
        u.refined = (fl >> ch) & 1ull;
        u.res_unit = (size_t)strip * nm + __popcll(fl & ((1ull << ch) - 1ull));
        u.res_nrec = (size_t)NS * nm * 32;
    }
    u.res_rec = u.res_unit * 32;
    return u;
}

// ring sign of this lane's ring as an fp16x2 xor mask
__device__ __forceinline__ uint32_t ring_sign2(const ProjPlanes& P, const UnitRef& u, int lane)
{
    if (!P.var) return 0u;
    return ((uint32_t)(__ldg(P.var + u.unit) >> (lane >> 2)) & 1u) * 0x80008000u;
}

// Decode the lane's 64 weights of a unit whose words are already in registers.  sink(integral_constant<T>, a[4]) receives,
// for k-step T = 0..7, the m16n8k16 A-fragment registers: a[q] = rows g + 8 (q & 1), k = 16 T + 2 t4 + 8 (q >> 1) + {0, 1}.
template <bool RES, int RC, int BK = 0, class Sink>
__device__ __forceinline__ void decode_words(uint32_t* wb, uint32_t* wr, const UnitConsts& k, int lane, Sink&& sink)
{
    const int nxt = ring_next_lane(lane);
    extend_stream<Pattern<BK>::kBits>(wb, __shfl_sync(0xffffffffu, wb[0], nxt));
    if constexpr (RES) extend_stream<Pattern<RC>::kBits>(wr, __shfl_sync(0xffffffffu, wr[0], nxt));
    static_for<8>([&](auto tc) {
        constexpr int T = decltype(tc)::value;
        uint32_t a[4];
        a[0] = decode_pair<RES, RC, 4 * T + 0, BK>(wb, wr, k);
        a[1] = decode_pair<RES, RC, 4 * T + 1, BK>(wb, wr, k);
        a[2] = decode_pair<RES, RC, 4 * T + 2, BK>(wb, wr, k);
        a[3] = decode_pair<RES, RC, 4 * T + 3, BK>(wb, wr, k);
        sink(tc, a);
    });
}

// base record of the lane: one 128-bit load for base code 0, the sub-array pieces for the others
template <int BK>
__device__ __forceinline__ void load_base(uint32_t* wb, const ProjPlanes& P, const UnitRef& u, int lane)
{
    if constexpr (BK == 0)
    {
        const uint4 b = ldg_stream128(P.base + u.base_rec + lane);
        wb[0] = b.x; wb[1] = b.y; wb[2] = b.z; wb[3] = b.w;
    }
    else load_record<Pattern<BK>::kBits>(wb, (const uint8_t*)P.base, u.base_rec + lane, u.base_nrec);
}
template <int RC, int BK, class Sink>
__device__ __forceinline__ void decode_unit_refined(const ProjPlanes& P, const UnitRef& u, int lane, Sink&& sink)
{
    uint32_t wb[Pattern<BK>::kWords + 2], wr[Pattern<RC>::kWords + 2];
    load_base<BK>(wb, P, u, lane);
    load_record<Pattern<RC>::kBits>(wr, P.p4, u.res_rec + lane, u.res_nrec);
    const uint32_t dl = __ldg(P.d4 + u.res_unit);
    const UnitConsts k = consts_level4(dl, ring_sign2(P, u, lane));
    decode_words<true, RC, BK>(wb, wr, k, lane, sink);
}
template <int BK, class Sink>
__device__ __forceinline__ void decode_unit_base(const ProjPlanes& P, const UnitRef& u, int lane, Sink&& sink)
{
    uint32_t wb[Pattern<BK>::kWords + 2];
    load_base<BK>(wb, P, u, lane);
    const UnitConsts k = consts_level2(ring_sign2(P, u, lane));
    decode_words<false, 0, BK>(wb, nullptr, k, lane, sink);
}

// Base code 1 is built with the residual codes it ships with (3 for gate|up, 9 for down: sm120/NQ_RES_V2.md:9-13).
__host__ __device__ constexpr bool bk1_has_rc(int rc) { return rc == 3 || rc == 9; }

// run-time codes -> compile-time decoder
template <class Sink>
__device__ __forceinline__ void decode_unit_dispatch(const ProjPlanes& P, const UnitRef& u, int rc, int bk, int lane, Sink&& sink)
{
    if (bk == 1)
    {
        if (!u.refined) decode_unit_base<1>(P, u, lane, sink);
        else if (rc == 9) decode_unit_refined<9, 1>(P, u, lane, sink);
        else decode_unit_refined<3, 1>(P, u, lane, sink);
        return;
    }
    if (!u.refined) { decode_unit_base<0>(P, u, lane, sink); return; }
    switch (rc)
    {
        case 1: decode_unit_refined<1, 0>(P, u, lane, sink); break;
        case 2: decode_unit_refined<2, 0>(P, u, lane, sink); break;
        case 3: decode_unit_refined<3, 0>(P, u, lane, sink); break;
        case 4: decode_unit_refined<4, 0>(P, u, lane, sink); break;
        case 5: decode_unit_refined<5, 0>(P, u, lane, sink); break;
        case 6: decode_unit_refined<6, 0>(P, u, lane, sink); break;
        case 7: decode_unit_refined<7, 0>(P, u, lane, sink); break;
        case 8: decode_unit_refined<8, 0>(P, u, lane, sink); break;
        case 9: decode_unit_refined<9, 0>(P, u, lane, sink); break;
        default: decode_unit_refined<0, 0>(P, u, lane, sink); break;
    }
}

}  // namespace nq
