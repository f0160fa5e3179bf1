// Asynchronous stream of packed planes into shared memory, shared by the decode-path GEMV and the prefill GEMM.
#pragma once
#include "nq_format.cuh"

namespace nq {

// Each lane copies the words of its own records with cp.async (global -> shared, no registers) a few units ahead and
// later reads back only what it copied itself, so the ring needs no barrier at all.  Per warp and stage:
// 512 B of base records followed by the residual pieces of the unit, one lane-indexed array per piece.
constexpr int kStageBytes = 512 + 768;   // base + the widest residual layout (see ResidualSlots)

__device__ __forceinline__ void cp_async16(void* dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async8(void* dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// byte offsets, inside the residual part of a stage, of each piece of a record of window code RC
template <int RC>
struct ResidualSlots
{
    static constexpr int kBits = Pattern<RC>::kBits;
    static constexpr int n4 = kBits / 128, rem = kBits % 128, T = kBits % 16;
    static constexpr bool has64 = (rem & 64) != 0, has32 = (rem & 32) != 0, has16 = (rem & 16) != 0;
    static constexpr bool tail2 = T != 0 && (32 % T) != 0;          // a tail that can straddle two words
    static constexpr int o128 = 0, o64 = o128 + 512 * n4, o32 = o64 + (has64 ? 256 : 0), o16 = o32 + (has32 ? 128 : 0);
    static constexpr int otail = o16 + (has16 ? 128 : 0), end = otail + (T ? (tail2 ? 256 : 128) : 0);
    static_assert(n4 <= 1 && end <= kStageBytes - 512, "stage too small for this window code");
};

// enqueue the copies of record `rec` (= refined unit * 32 + lane) of a residual plane of `nrec` records
template <int RC>
__device__ __forceinline__ void copy_record(uint8_t* st, const uint8_t* __restrict__ p, size_t rec, size_t nrec, int lane)
{
    using L = ResidualSlots<RC>;
    if constexpr (L::n4) { cp_async16(st + L::o128 + lane * 16, p + rec * 16); p += nrec * 16; }
    if constexpr (L::has64) { cp_async8(st + L::o64 + lane * 8, p + rec * 8); p += nrec * 8; }
    if constexpr (L::has32) { cp_async4(st + L::o32 + lane * 4, p + rec * 4); p += nrec * 4; }
    if constexpr (L::has16) { cp_async4(st + L::o16 + lane * 4, p + ((rec * 2) & ~(size_t)3)); p += nrec * 2; }
    if constexpr (L::T != 0)
    {
        const uint8_t* q = p + ((rec * L::T) >> 5) * 4;
        if constexpr (L::tail2) { cp_async4(st + L::otail + lane * 8, q); cp_async4(st + L::otail + lane * 8 + 4, q + 4); }
        else cp_async4(st + L::otail + lane * 4, q);
    }
}
// read the record back as stream words w[0 .. kWords)
template <int RC>
__device__ __forceinline__ void read_record(uint32_t* w, const uint8_t* st, size_t rec, int lane)
{
    using L = ResidualSlots<RC>;
    int k = 0;
    if constexpr (L::n4) { const uint4 v = *(const uint4*)(st + L::o128 + lane * 16); w[k++] = v.x; w[k++] = v.y; w[k++] = v.z; w[k++] = v.w; }
    if constexpr (L::has64) { const uint2 v = *(const uint2*)(st + L::o64 + lane * 8); w[k++] = v.x; w[k++] = v.y; }
    if constexpr (L::has32) w[k++] = *(const uint32_t*)(st + L::o32 + lane * 4);
    if constexpr (L::has16)
    {
        const uint32_t v = *(const uint32_t*)(st + L::o16 + lane * 4);
        w[k++] = (rec & 1) ? v >> 16 : v & 0xFFFFu;
    }
    if constexpr (L::T != 0)
    {
        const int sh = (int)((rec * L::T) & 31);
        uint32_t v;
        if constexpr (L::tail2)
        {
            const uint2 t = *(const uint2*)(st + L::otail + lane * 8);
            v = __funnelshift_r(t.x, t.y, sh);
        }
        else v = *(const uint32_t*)(st + L::otail + lane * 4) >> sh;
        v &= (1u << L::T) - 1u;
        if constexpr (((L::kBits - L::T) & 31) == 16) w[k - 1] |= v << 16;
        else w[k++] = v;
    }
}

// base records of a unit in the first 512 bytes of a stage: one 16-byte copy per lane for base code 0, the sub-array
// pieces (same slot layout as a residual record) for the others
template <int BK>
__device__ __forceinline__ void copy_base(uint8_t* st, const uint4* __restrict__ base, size_t rec, size_t nrec, int lane)
{
    if constexpr (BK == 0) cp_async16(st + lane * 16, (const uint8_t*)(base + rec));
    else
    {
        static_assert(ResidualSlots<BK>::end <= 512, "base record does not fit the base part of a stage");
        copy_record<BK>(st, (const uint8_t*)base, rec, nrec, lane);
    }
}
template <int BK>
__device__ __forceinline__ void read_base(uint32_t* wb, const uint8_t* st, size_t rec, int lane)
{
    if constexpr (BK == 0)
    {
        const uint4 b = *(const uint4*)(st + lane * 16);
        wb[0] = b.x; wb[1] = b.y; wb[2] = b.z; wb[3] = b.w;
    }
    else read_record<BK>(wb, st, rec, lane);
}

}  // namespace nq
