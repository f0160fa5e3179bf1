// Asynchronous stream of packed planes into shared memory, shared by the decode-path GEMV, the prefill GEMM and the dense
// decode kernel.
//
// Plane layout (sm120/moe.py:36-49): a record of BITS bits is cut into pieces - BITS / 128 pieces of 128 bits, then a
// 64-, a 32- and a 16-bit piece as the binary digits of BITS % 128 say, then a tail of BITS % 16 bits - and every piece
// kind is stored as its own array over all records of the plane (the tail bit-packed, followed by a 4-byte pad).  The
// base plane of window code 0 is the special case of one 128-bit piece.
//
// Each lane copies the pieces of its own record with cp.async (global -> shared, no registers) a few units ahead and
// later reads back only what it copied itself, so the ring needs no barrier at all.  Per warp and stage: 512 B for the
// base records of a unit followed by 768 B for its residual records, one lane-indexed array per piece kind.
// 32 records make a unit, so every piece array advances by a fixed number of bytes per unit and a lane's position
// inside its unit's share of each array never changes: a cursor keeps one pointer per piece kind.
#pragma once
#include "nq_format.cuh"

namespace nq {

constexpr int kStageBase = 512, kStageBytes = kStageBase + 768;

// Shared-memory operands below are 32-bit shared-space addresses (smem_addr of a pointer), so that a stage position plus a
// lane offset is one register and every piece of a record an immediate offset from it.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
// the same with compile-time byte offsets on both addresses
template <int DOFF, int SOFF>
__device__ __forceinline__ void cp_async16_at(uint32_t dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0 + %2], [%1 + %3], 16;" ::"r"(dst), "l"(src), "n"(DOFF), "n"(SOFF));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}

// pieces of a record of window code CODE and where they sit inside a stage part
template <int CODE>
struct RecordLayout
{
    static constexpr int kBits = Pattern<CODE>::kBits;
    static constexpr int n128 = kBits / 128, rem = kBits % 128, T = kBits % 16;
    static constexpr bool has64 = (rem & 64) != 0, has32 = (rem & 32) != 0, has16 = (rem & 16) != 0;
    static constexpr bool tail2 = T != 0 && (32 % (T ? T : 1)) != 0;          // a lane's tail can straddle two words
    static constexpr int o128 = 0, o64 = o128 + 512 * n128, o32 = o64 + (has64 ? 256 : 0), o16 = o32 + (has32 ? 128 : 0);
    static constexpr int otail = o16 + (has16 ? 128 : 0), end = otail + (T ? (tail2 ? 256 : 128) : 0);
    static_assert(n128 <= 1 && end <= kStageBytes - kStageBase, "stage too small for this window code");
    // the tail lands in the upper half of the 16-bit piece's word when the pieces before it end on a half word
    static constexpr bool tail_joins = T != 0 && ((kBits - T) & 31) == 16;
};

// One lane's read position in a plane of `nrec` records, at unit `unit0`; copy(stage, u) fetches unit unit0 + u.
template <int CODE>
struct RecordCursor
{
    using L = RecordLayout<CODE>;
    const uint8_t *p128, *p64, *p32, *p16, *ptail;

    __device__ __forceinline__ void init(const void* plane, size_t nrec, size_t unit0, int lane)
    {
        const uint8_t* p = (const uint8_t*)plane;
        if constexpr (L::n128) { p128 = p + unit0 * 512 + lane * 16; p += nrec * 16; }
        if constexpr (L::has64) { p64 = p + unit0 * 256 + lane * 8; p += nrec * 8; }
        if constexpr (L::has32) { p32 = p + unit0 * 128 + lane * 4; p += nrec * 4; }
        if constexpr (L::has16) { p16 = p + unit0 * 64 + (lane >> 1) * 4; p += nrec * 2; }
        if constexpr (L::T != 0) ptail = p + unit0 * (4 * L::T) + ((lane * L::T) >> 5) * 4;
    }
    // st: shared-space address of the stage part that receives the record pieces
    __device__ __forceinline__ void copy(uint32_t st, int u, int lane) const
    {
        if constexpr (L::n128) cp_async16(st + L::o128 + lane * 16, p128 + (size_t)u * 512);
        if constexpr (L::has64) cp_async8(st + L::o64 + lane * 8, p64 + (size_t)u * 256);
        if constexpr (L::has32) cp_async4(st + L::o32 + lane * 4, p32 + (size_t)u * 128);
        if constexpr (L::has16) cp_async4(st + L::o16 + lane * 4, p16 + (size_t)u * 64);
        if constexpr (L::T != 0)
        {
            const uint8_t* q = ptail + (size_t)u * (4 * L::T);
            if constexpr (L::tail2) { cp_async4(st + L::otail + lane * 8, q); cp_async4(st + L::otail + lane * 8 + 4, q + 4); }
            else cp_async4(st + L::otail + lane * 4, q);
        }
    }
    // the lane's record as stream words w[0 .. kWords), bits past the record zero
    static __device__ __forceinline__ void read(uint32_t* w, uint32_t st, int lane)
    {
        int k = 0;
        if constexpr (L::n128) { const uint4 v = lds128(st + L::o128 + lane * 16); w[k++] = v.x; w[k++] = v.y; w[k++] = v.z; w[k++] = v.w; }
        if constexpr (L::has64) { const uint2 v = lds64(st + L::o64 + lane * 8); w[k++] = v.x; w[k++] = v.y; }
        if constexpr (L::has32) w[k++] = lds32(st + L::o32 + lane * 4);
        if constexpr (L::has16) w[k++] = __byte_perm(lds32(st + L::o16 + lane * 4), 0u, (lane & 1) ? 0x4432 : 0x4410);
        if constexpr (L::T != 0)
        {
            const int sh = (lane * L::T) & 31;
            uint32_t v;
            if constexpr (L::tail2)
            {
                const uint2 t = lds64(st + L::otail + lane * 8);
                v = __funnelshift_r(t.x, t.y, sh);
            }
            else v = lds32(st + L::otail + lane * 4) >> sh;
            v &= (1u << L::T) - 1u;
            if constexpr (L::tail_joins) w[k - 1] |= v << 16;
            else w[k++] = v;
        }
    }
};

}  // namespace nq
