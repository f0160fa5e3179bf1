// NestQuant nested-trellis weight format: device-side decode primitives shared by every kernel.
//
// Format (reference: sm120/ref15_spec.py:3-8,43-90; sm120/nqmoe.cu:14-25,146-173; sm120/moe.py:36-63):
//   unit    = 16 rows x 128 k = 32 lane records; record index ((strip * C + chunk) * 32 + lane); lane = 4 g + t4.
//   ring g  = records of lanes 4g..4g+3 concatenated LSB-first (tail-biting); lane weight j is ring position 64 t4 + j.
//   state   = 16-bit window at bit step_offset(j) of the lane stream, continued into the next ring lane's first word.
//   S       = sum of the four bytes of state * 0x83DCD12D.
//   level 2 : Q = fp16(A (1024 + Sb) + B), A = 0x1eee, B = 0xc931.
//   level 4 : F = (Mb Sb + N Sr + 128) >> 8, Q = fp16(A' (1024 + F) + C'), A'/C' from the unit's block word.
//   lane weight j = 2 pp + e, pp = 4 t + r  ->  row g + 8 (r & 1), k = 16 t + 2 t4 + 8 (r >> 1) + e, i.e. pair pp is
//   register r of the m16n8k16 A fragment of k-step t.
//
// How a k-step (8 weights of a lane) is decoded here:
//   windows   the 64 window offsets of a code are known at compile time.  Windows whose offsets agree modulo 8 are
//             packed greedily, in stream order, into 32-bit "views" of the stream (one funnel shift each, none when the
//             view starts on a word); a view serves up to three windows, at its byte offsets 0, 1 and 2, each by one
//             instruction (and / byte-permute / shift).
//   hash      one 32-bit multiply per window.
//   byte sums one dp4a per hashed word (two at level 4, with Mb and N as the byte weights), accumulating onto the bit pattern
//             that turns the sum into fp16(1024 + S).  (The same sums on the tensor pipe - one mma.m16n8k32.u8 per four
//             hashed words, a per-lane selector as the B fragment - were built and measured: legacy mma.sync issues at
//             0.5 per clock per SM on this part, exactly the pipe time of the four dp4a it replaces, and the kernels ran
//             no faster, so that variant is not kept.)
//   affine    one byte-permute packs two sums, one fp16x2 fma applies the unit's multiplier and addend (single rounding).
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

// ---------------------------------------------------------------- window patterns (the format's tables)
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
__host__ __device__ constexpr int record_bits(int code) { return 4 * (16 * pattern_ka(code) + popcount16(pattern_mask(code))); }
template <int CODE>
struct Pattern
{
    static constexpr int kBits = record_bits(CODE);     // bits per lane record
    static constexpr int kWords = (kBits + 31) / 32;
};

template <int... Is, class F>
__device__ __forceinline__ void static_for_impl(std::integer_sequence<int, Is...>, F&& f)
{
    (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, class F>
__device__ __forceinline__ void static_for(F&& f) { static_for_impl(std::make_integer_sequence<int, N>{}, static_cast<F&&>(f)); }

// ---------------------------------------------------------------- 16-bit windows of a lane stream held in registers
// View of window j: the offset of the first window, in stream order, of j's residue class (offset mod 8) that lies
// within 16 bits before j and is not itself covered by an earlier view.
__host__ __device__ constexpr int view_start(int j, int code)
{
    const int oj = step_offset(j, code);
    int v = -1;
    for (int i = 0; i <= j; ++i)
    {
        const int oi = step_offset(i, code);
        if (((oi ^ oj) & 7) != 0) continue;
        if (v < 0 || oi > v + 16) v = oi;
    }
    return v;
}
// w[] = the record's words followed by the continuation word(s) (see continue_stream)
template <int CODE, int J>
__device__ __forceinline__ uint32_t state16(const uint32_t* w)
{
    constexpr int o = step_offset(J, CODE), v = view_start(J, CODE), vi = v >> 5, vs = v & 31, byte = (o - v) >> 3;
    static_assert(byte >= 0 && byte <= 2 && ((o - v) & 7) == 0, "window outside its view");
    uint32_t view;
    if constexpr (vs == 0) view = w[vi];
    else view = __funnelshift_r(w[vi], w[vi + 1], vs);      // identical views of different windows are merged by the compiler
    if constexpr (byte == 0) return view & 0xFFFFu;
    else if constexpr (byte == 1) return __byte_perm(view, 0u, 0x4421);
    else return view >> 16;
}

// A lane's stream continues with the first word of the next lane of its ring (lanes 4g..4g+3, cyclic): append that
// word at bit BITS.  The array must hold kWords + 2 words.
template <int BITS>
__device__ __forceinline__ void continue_stream(uint32_t* w, uint32_t next_word)
{
    constexpr int n = (BITS + 31) / 32, used = BITS & 31;
    if constexpr (used == 0) w[n] = next_word;
    else
    {
        w[n - 1] = __funnelshift_l(w[n - 1] << (32 - used), next_word, used);   // low `used` bits kept, the rest from next_word
        w[n] = next_word >> (32 - used);
    }
    w[n + 1] = 0u;
}
__device__ __forceinline__ int ring_successor(int lane) { return (lane & 28) | ((lane + 1) & 3); }

// ---------------------------------------------------------------- byte sums and the affine map
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
// Per-unit multipliers.  a2 / c2: fp16x2 multiplier and addend with the ring sign folded in (negating both negates the
// result exactly).  m / n: byte weights of the base and the residual sum, replicated into four bytes (1 and 0 at level 2,
// Mb and N at level 4).
struct UnitConsts
{
    uint32_t a2, c2, m, n;
};
// Block word Mb | N << 8 -> fp16 multiplier A' (low half) and addend C' (high half), each fp32 operation rounded on its
// own in the order the format defines (sm120/ref15_spec.py:79-83, sm120/moe.py:130-132):
//   A' = fp16(1.732421875 / Mb),  C' = fp16(((N / Mb) K0 + K0) - 1024 A'),  K0 = -3.453125, 1 / Mb rounded first.
__device__ __forceinline__ uint32_t block_multipliers(uint32_t block_word)
{
    const float inv = __fdiv_rn(1.0f, (float)(block_word & 0xFFu));
    const __half a = __float2half_rn(__fmul_rn(1.732421875f, inv));
    const float ratio = __fmul_rn((float)((block_word >> 8) & 0xFFu), inv);
    const float c = __fsub_rn(__fadd_rn(__fmul_rn(ratio, -3.453125f), -3.453125f), __fmul_rn(1024.0f, __half2float(a)));
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(__float2half_rn(c)) << 16);
}
__device__ __forceinline__ UnitConsts consts_level2(uint32_t sign2)
{
    UnitConsts k;
    k.a2 = kMul1A2 ^ sign2; k.c2 = kMul1B2 ^ sign2; k.m = 0x01010101u; k.n = 0u;
    return k;
}
// ac = block_multipliers(word), mbn = the block word
__device__ __forceinline__ UnitConsts consts_level4(uint32_t ac, uint32_t mbn, uint32_t sign2)
{
    UnitConsts k;
    k.a2 = __byte_perm(ac, 0u, 0x1010) ^ sign2; k.c2 = __byte_perm(ac, 0u, 0x3232) ^ sign2;
    k.m = __byte_perm(mbn, 0u, 0x0000); k.n = __byte_perm(mbn, 0u, 0x1111);
    return k;
}

// The A-fragment registers of k-step T: a[q] = rows g + 8 (q & 1), k = 16 T + 2 t4 + 8 (q >> 1) + {0, 1}, i.e.
// a[q] = fp16x2 of lane weights 2 (4 T + q) and 2 (4 T + q) + 1.
// RES: refined (level 4) unit, RC its residual window code, BK the window code of the base stream (0 = 2 bits per weight
// in 128-bit records; 1 = 1.75 bits per weight in 112-bit records, sm120/NQ_RES_V2.md:36-50: only the base state walk
// changes).
template <bool RES, int RC, int BK, int T>
__device__ __forceinline__ void decode_kstep(const uint32_t* wb, const uint32_t* wr, const UnitConsts& k, uint32_t (&a)[4])
{
    using std::integral_constant;
    // hashed base / residual word of lane weight 8 T + i
    auto hb = [&](auto ic) { return state16<BK, 8 * T + decltype(ic)::value>(wb) * kHashMul; };
    auto hr = [&](auto ic) { return state16<RC, 8 * T + decltype(ic)::value>(wr) * kHashMul; };
    static_for<4>([&](auto qc) {
        constexpr int q = decltype(qc)::value;
        if constexpr (!RES)
        {
            // 0x6400 + S is the fp16 bit pattern of 1024 + S (S <= 1020)
            const uint32_t s0 = dot4(hb(integral_constant<int, 2 * q>{}), k.m, 0x6400u);
            const uint32_t s1 = dot4(hb(integral_constant<int, 2 * q + 1>{}), k.m, 0x6400u);
            a[q] = fma_h2(__byte_perm(s0, s1, 0x5410), k.a2, k.c2);
        }
        else
        {
            // Mb Sb + N Sr + 128 + (0x6400 << 8): bits 8..23 are the fp16 pattern of 1024 + F
            const uint32_t s0 = dot4(hr(integral_constant<int, 2 * q>{}), k.n, dot4(hb(integral_constant<int, 2 * q>{}), k.m, 0x640080u));
            const uint32_t s1 = dot4(hr(integral_constant<int, 2 * q + 1>{}), k.n, dot4(hb(integral_constant<int, 2 * q + 1>{}), k.m, 0x640080u));
            a[q] = fma_h2(__byte_perm(s0, s1, 0x6521), k.a2, k.c2);
        }
    });
}

// ---------------------------------------------------------------- plane pointers of one projection of one expert
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

}  // namespace nq
