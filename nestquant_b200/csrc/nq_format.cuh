// NestQuant nested-trellis weight format: device-side decode primitives shared by every kernel.
//
// Format (reference: sm120/ref15_spec.py:3-8,43-90; sm120/nqmoe.cu:14-25,146-173; sm120/moe.py:36-63):
//   unit    = 16 rows x 128 k = 32 lane records; record index ((strip * C + chunk) * 32 + lane); lane = 4 g + t4.
//   ring g  = records of lanes 4g..4g+3 concatenated LSB-first (tail-biting); lane weight j is ring position 64 t4 + j.
//   state   = 16-bit window at bit step_off(j) of the lane stream, continued into the next ring lane's first word.
//   S       = sum of the four bytes of state * 0x83DCD12D.
//   level 2 : Q = fp16(A (1024 + Sb) + B), A = 0x1eee, B = 0xc931.
//   level 4 : F = (Mb Sb + N Sr + 128) >> 8, Q = fp16(A' (1024 + F) + C'), A'/C' from the unit's block word.
//   lane weight j = 2 pp + e, pp = 4 t + r  ->  row g + 8 (r & 1), k = 16 t + 2 t4 + 8 (r >> 1) + e, i.e. pair pp is
//   register r of the m16n8k16 A fragment of k-step t.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>
#include <utility>

namespace nq {

constexpr uint32_t kHashMul = 0x83DCD12Du;
constexpr uint32_t kMul1A2 = 0x1eee1eeeu;   // fp16x2 A
constexpr uint32_t kMul1B2 = 0xc931c931u;   // fp16x2 B
constexpr int kTableWidth = 20;              // int64 words per expert row of the device table
constexpr int kNumCodes = 10;

// ---------------------------------------------------------------- window patterns
__host__ __device__ constexpr int pattern_ka(int code)
{
    constexpr int t[kNumCodes] = {2, 1, 2, 2, 3, 1, 1, 2, 1, 2};
    return t[code];
}
__host__ __device__ constexpr int pattern_mask(int code)
{
    constexpr int t[kNumCodes] = {0x0000, 0xEEEE, 0xAAAA, 0x8888, 0x0000, 0xAAAA, 0xFFFE, 0x9248, 0xFEFE, 0xD5AA};
    return t[code];
}
__host__ __device__ constexpr int popcount16(int m)
{
    int c = 0;
    for (int i = 0; i < 16; ++i) c += (m >> i) & 1;
    return c;
}
// bit offset of lane weight j: step i is ka + bit (i mod 16) of mask wide
__host__ __device__ constexpr int step_offset(int j, int code)
{
    const int ka = pattern_ka(code), mask = pattern_mask(code);
    int s = (j >> 4) * (16 * ka + popcount16(mask));
    for (int i = 0; i < (j & 15); ++i) s += ka + ((mask >> i) & 1);
    return s;
}
template <int CODE>
struct Pattern
{
    static constexpr int kBits = 4 * (16 * pattern_ka(CODE) + popcount16(pattern_mask(CODE)));   // bits per lane record
    static constexpr int kWords = (kBits + 31) / 32;
};
__host__ __device__ constexpr int record_bits(int code) { return 4 * (16 * pattern_ka(code) + popcount16(pattern_mask(code))); }

template <int... Is, class F>
__device__ __forceinline__ void static_for_impl(std::integer_sequence<int, Is...>, F&& f)
{
    (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) { static_for_impl(std::make_integer_sequence<int, N>{}, static_cast<F&&>(f)); }

// ---------------------------------------------------------------- 16-bit windows of a lane stream held in registers
// w[] holds the record words followed by two continuation words (see extend_stream).  Windows that start on a
// byte boundary inside one word cost one instruction; the others share a 32-bit funnel anchored every 24 bits
// within their (offset mod 8) class, so one funnel shift serves up to three windows.
template <int O>
__device__ __forceinline__ uint32_t window16(const uint32_t* w)
{
    constexpr int i = O >> 5, s = O & 31;
    if constexpr (s == 0) return w[i] & 0xFFFFu;
    else if constexpr (s == 8) return __byte_perm(w[i], 0u, 0x4421);
    else if constexpr (s == 16) return w[i] >> 16;
    else
    {
        constexpr int r = O & 7, a = r + 24 * ((O - r) / 24), ai = a >> 5, as = a & 31, b = (O - a) >> 3;
        uint32_t f;
        if constexpr (as == 0) f = w[ai];
        else f = __funnelshift_r(w[ai], w[ai + 1], as);
        if constexpr (b == 0) return f & 0xFFFFu;
        else if constexpr (b == 1) return __byte_perm(f, 0u, 0x4421);
        else return f >> 16;
    }
}

// stream bits [BITS, BITS + 32) = first word of the next lane of the ring
template <int BITS>
__device__ __forceinline__ void extend_stream(uint32_t* w, uint32_t next_first)
{
    constexpr int NW = (BITS + 31) / 32, T = BITS % 32;
    if constexpr (T == 0) { w[NW] = next_first; w[NW + 1] = 0u; }
    else
    {
        w[NW - 1] = (w[NW - 1] & ((1u << T) - 1u)) | (next_first << T);
        w[NW] = next_first >> (32 - T);
        w[NW + 1] = 0u;
    }
}
// lane that holds the next quarter of this lane's ring
__device__ __forceinline__ int ring_next_lane(int lane) { return (lane & ~3) | ((lane + 1) & 3); }

__device__ __forceinline__ uint32_t dot4(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t fma_h2(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// per-unit multipliers.  level 2: a2 = A, c2 = B.  level 4: from the block word, computed with individually
// rounded fp32 operations in the order the format defines (sm120/ref15_spec.py:79-83, sm120/moe.py:130-132).
struct UnitConsts
{
    uint32_t a2, c2;       // fp16x2 multiplier / addend (ring sign folded in)
    uint32_t mrep, nrep;   // Mb, N replicated into 4 bytes
};
__device__ __forceinline__ UnitConsts consts_level2(uint32_t sign2)
{
    UnitConsts k;
    k.a2 = kMul1A2 ^ sign2; k.c2 = kMul1B2 ^ sign2; k.mrep = 0x01010101u; k.nrep = 0u;
    return k;
}
__device__ __forceinline__ UnitConsts consts_level4(uint32_t block_word, uint32_t sign2)
{
    const uint32_t mb = block_word & 0xFFu, n = (block_word >> 8) & 0xFFu;
    const float rc = __frcp_rn((float)mb);                                   // IEEE 1.0f / Mb
    const __half ah = __float2half_rn(__fmul_rn(1.732421875f, rc));
    const float t = __fadd_rn(__fmul_rn(__fmul_rn((float)n, rc), -3.453125f), -3.453125f);
    const __half ch = __float2half_rn(__fsub_rn(t, __fmul_rn(1024.0f, __half2float(ah))));
    UnitConsts k;
    k.a2 = ((uint32_t)__half_as_ushort(ah) * 0x00010001u) ^ sign2;
    k.c2 = ((uint32_t)__half_as_ushort(ch) * 0x00010001u) ^ sign2;
    k.mrep = mb * 0x01010101u; k.nrep = n * 0x01010101u;
    return k;
}

// fp16x2 of lane weights 2 PP and 2 PP + 1.  RES: refined (level 4) unit, RC its residual window code, BK the window
// code of the base stream (0 = 2 bits per weight in 128-bit records; 1 = 1.75 bits per weight in 112-bit records,
// sm120/NQ_RES_V2.md:36-50: only the base state walk changes).
template <bool RES, int RC, int PP, int BK = 0>
__device__ __forceinline__ uint32_t decode_pair(const uint32_t* wb, const uint32_t* wr, const UnitConsts& k)
{
    constexpr int b0 = step_offset(2 * PP, BK), b1 = step_offset(2 * PP + 1, BK);
    const uint32_t x0 = window16<b0>(wb) * kHashMul, x1 = window16<b1>(wb) * kHashMul;
    if constexpr (!RES)
    {
        // 0x6400 + S is the fp16 bit pattern of 1024 + S (S <= 1020)
        const uint32_t s0 = dot4(x0, 0x01010101u, 0x6400u), s1 = dot4(x1, 0x01010101u, 0x6400u);
        return fma_h2(__byte_perm(s0, s1, 0x5410), k.a2, k.c2);
    }
    else
    {
        constexpr int o0 = step_offset(2 * PP, RC), o1 = step_offset(2 * PP + 1, RC);
        // Mb Sb + N Sr + 128 + (0x6400 << 8): bits 8..23 are the fp16 pattern of 1024 + F
        uint32_t t0 = dot4(x0, k.mrep, 0x640080u), t1 = dot4(x1, k.mrep, 0x640080u);
        t0 = dot4(window16<o0>(wr) * kHashMul, k.nrep, t0);
        t1 = dot4(window16<o1>(wr) * kHashMul, k.nrep, t1);
        return fma_h2(__byte_perm(t0, t1, 0x6521), k.a2, k.c2);
    }
}

// ---------------------------------------------------------------- plane access
struct ProjPlanes
{
    const uint4* base;        // 128-bit record per lane
    const uint8_t* p4;        // residual plane (sub-array layout)
    const uint32_t* d4;       // block word per refined unit
    const uint64_t* flags;    // per strip, or null (every chunk refined)
    const uint8_t* var;       // per unit ring-sign byte, or null
};
__device__ __forceinline__ ProjPlanes planes_from_row(const int64_t* row, int down)
{
    ProjPlanes p;
    const int o = down ? 5 : 1;
    p.base = (const uint4*)row[o]; p.p4 = (const uint8_t*)row[o + 1]; p.d4 = (const uint32_t*)row[o + 2];
    p.flags = (const uint64_t*)row[o + 3]; p.var = (const uint8_t*)row[down ? 13 : 12];
    return p;
}

__device__ __forceinline__ uint4 ldg_stream128(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream64(const void* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream32(const void* p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream16(const void* p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// words of record `rec` of a residual plane of `nrec` records (sub-arrays: 128-bit pieces record-major, then a
// 64-, 32-, 16-bit piece per record, then a bit-packed tail of BITS % 16 bits per record followed by a 4-byte pad)
template <int BITS>
__device__ __forceinline__ void load_record(uint32_t* w, const uint8_t* __restrict__ p, size_t rec, size_t nrec)
{
    constexpr int n4 = BITS / 128, rem = BITS % 128, T = BITS % 16;
    int k = 0;
#pragma unroll
    for (int i = 0; i < n4; ++i)
    {
        const uint4 v = ldg_stream128(p + (rec * n4 + i) * 16);
        w[k++] = v.x; w[k++] = v.y; w[k++] = v.z; w[k++] = v.w;
    }
    p += nrec * 16 * (size_t)n4;
    if constexpr ((rem & 64) != 0) { const uint2 v = ldg_stream64(p + rec * 8); w[k++] = v.x; w[k++] = v.y; p += nrec * 8; }
    if constexpr ((rem & 32) != 0) { w[k++] = ldg_stream32(p + rec * 4); p += nrec * 4; }
    if constexpr ((rem & 16) != 0) { w[k++] = ldg_stream16(p + rec * 2); p += nrec * 2; }
    if constexpr (T != 0)
    {
        const size_t bit = rec * T;
        const uint8_t* q = p + (bit >> 5) * 4;
        const int sh = (int)(bit & 31);
        uint32_t v;
        if constexpr ((32 % T) != 0) v = __funnelshift_r(ldg_stream32(q), ldg_stream32(q + 4), sh);   // second word: next record word or the pad
        else v = ldg_stream32(q) >> sh;
        v &= (1u << T) - 1u;
        if constexpr (((BITS - T) & 31) == 16) w[k - 1] |= v << 16;
        else w[k++] = v;
    }
}

}  // namespace nq
