// One 16x128 unit per warp: where its records live, its per-unit constants, and the decode of its 64 weights per lane.
#pragma once
#include "nq_stream.cuh"

namespace nq {

// Mask mode (sm120/nqmoe.cu:202-206): chunk ch of a strip is refined iff bit ch of flags[strip]; refined chunks are
// stored compactly, nm per strip.  Dense mode (no flags): every chunk of a level-4 expert is refined.
struct StripRef
{
    unsigned long long flags;   // bit ch: chunk ch is refined (all ones in dense mode, zero below level 4)
    size_t unit0;               // first unit of the strip in the base / var planes
    size_t res0;                // first refined unit of the strip in the residual / block-word planes
    size_t res_nrec;            // records in the residual plane
    bool compact;
};
__device__ __forceinline__ StripRef locate_strip(const ProjPlanes& P, int strip, int C, int NS, int nm, bool level4)
{
    StripRef s;
    s.unit0 = (size_t)strip * C;
    s.compact = level4 && P.flags != nullptr;
    s.flags = !level4 ? 0ull : s.compact ? (unsigned long long)__ldg((const unsigned long long*)P.flags + strip) : ~0ull;
    s.res0 = s.compact ? (size_t)strip * nm : s.unit0;
    s.res_nrec = (size_t)NS * (s.compact ? nm : C) * 32;
    return s;
}
__device__ __forceinline__ bool chunk_refined(const StripRef& s, int ch) { return (s.flags >> ch) & 1ull; }
// refined units of the strip before chunk ch
__device__ __forceinline__ int refined_before(const StripRef& s, int ch)
{
    return s.compact ? __popcll(s.flags & ((1ull << ch) - 1ull)) : ch;
}

// ring sign of this lane's ring (bit g of the unit's sign byte) as an fp16x2 xor mask
__device__ __forceinline__ uint32_t sign_mask(uint32_t var_byte, int lane) { return ((var_byte >> (lane >> 2)) & 1u) * 0x80008000u; }

// Decode the lane's 64 weights of a unit whose stream words are in registers (wb: the base record, wr: the residual record,
// each already continued with the ring successor's first word: kWords + 2 words).  sink(integral_constant<T>, a[4])
// receives, for k-step T = 0..7, the m16n8k16 A-fragment registers: a[q] = rows g + 8 (q & 1),
// k = 16 T + 2 t4 + 8 (q >> 1) + {0, 1}.
template <bool RES, int RC, int BK, class Sink>
__device__ __forceinline__ void decode_words(const uint32_t* wb, const uint32_t* wr, const UnitConsts& k, Sink&& sink)
{
    static_for<8>([&](auto tc) {
        uint32_t a[4];
        decode_kstep<RES, RC, BK, decltype(tc)::value>(wb, wr, k, a);
        sink(tc, a);
    });
}
// The same for record words as read from the planes: fetches the continuation words from the ring successors first.
// Called by whole warps.
template <bool RES, int RC, int BK, class Sink>
__device__ __forceinline__ void decode_unit(uint32_t* wb, uint32_t* wr, const UnitConsts& k, int lane, Sink&& sink)
{
    const int nxt = ring_successor(lane);
    continue_stream<Pattern<BK>::kBits>(wb, __shfl_sync(0xffffffffu, wb[0], nxt));
    if constexpr (RES) continue_stream<Pattern<RC>::kBits>(wr, __shfl_sync(0xffffffffu, wr[0], nxt));
    decode_words<RES, RC, BK>(wb, wr, k, sink);
}

// Base code 1 is built with the residual codes it ships with (3 for gate|up, 9 for down: sm120/NQ_RES_V2.md:9-13).
__host__ __device__ constexpr bool bk1_has_rc(int rc) { return rc == 3 || rc == 9; }

// run-time (level 4?, residual code, base code) -> compile-time: expands X(RES, RC, BK) for the matching combination.
// CODES: bit c set = residual code c is built (others fall back to code 0, as the reference's kernels do for codes they
// were not compiled with, sm120/nqmoe.cu:547-548).  A macro, not a callback: every decoder instance must be inlined into
// the loop that holds its accumulators.
#define NQ_CODE_CASE(CODES, c, X) case c: if constexpr (((CODES) >> c) & 1) { X(true, c, 0); } break;
#define NQ_WITH_CODES(level4, rc, bk, CODES, X)                                                  \
    do {                                                                                         \
        if ((bk) == 1)                                                                           \
        {                                                                                        \
            if (!(level4)) { X(false, 0, 1); }                                                   \
            else if ((rc) == 9) { X(true, 9, 1); }                                               \
            else { X(true, 3, 1); }                                                              \
        }                                                                                        \
        else if (!(level4)) { X(false, 0, 0); }                                                  \
        else                                                                                     \
            switch ((((CODES) >> (rc)) & 1) ? (rc) : 0)                                          \
            {                                                                                    \
                NQ_CODE_CASE(CODES, 1, X) NQ_CODE_CASE(CODES, 2, X) NQ_CODE_CASE(CODES, 3, X)     \
                NQ_CODE_CASE(CODES, 4, X) NQ_CODE_CASE(CODES, 5, X) NQ_CODE_CASE(CODES, 6, X)     \
                NQ_CODE_CASE(CODES, 7, X) NQ_CODE_CASE(CODES, 8, X) NQ_CODE_CASE(CODES, 9, X)     \
                default: X(true, 0, 0); break;                                                   \
            }                                                                                    \
    } while (0)

}  // namespace nq
