// Warp-level pieces of the layer math around the GEMVs / GEMMs: the 128-point Hadamard rotation and fp16 <-> fp32
// vector access.  A warp holds a 128-vector as 4 consecutive elements per lane (element 4 * lane + i).
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace nq {

// normalised Sylvester-Hadamard transform of order 128 (reference: H128 in sm120/moe.py:168-172; the kernel-side
// butterfly it matches is sm120/nqmoe.cu:337-349)
__device__ __forceinline__ void wht128(float (&v)[4], int lane)
{
    const float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
    v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1)
    {
        const float s = (lane & m) ? -1.f : 1.f;       // o - v or v + o as one fma (exact either way)
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = fmaf(v[i], s, __shfl_xor_sync(0xffffffffu, v[i], m));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= 0.08838834764831845f;   // 1 / sqrt(128)
}
__device__ __forceinline__ void load4h(const __half* p, float (&f)[4])
{
    const uint2 u = *(const uint2*)p;
    const __half2 a = *(const __half2*)&u.x, b = *(const __half2*)&u.y;
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
__device__ __forceinline__ void store4h(__half* p, const float (&v)[4])
{
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint2 u; u.x = *(const uint32_t*)&a; u.y = *(const uint32_t*)&b;
    *(uint2*)p = u;
}

// The same transform for eight 128-vectors per warp: lanes 4 v .. 4 v + 3 hold vector v, 32 elements each (lane bits
// and register bits are index bits of the vector, see the maps below).  Five of the seven butterfly stages stay inside a lane; two cross lanes (8 shuffles per vector
// instead of 20), which is what the HBM-bound prefill passes need to stay off the shuffle pipe.
__device__ __forceinline__ void wht128_x8(float (&v)[32], int lane)
{
#pragma unroll
    for (int h = 1; h < 32; h <<= 1)
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (!(i & h))
            {
                const float a = v[i], b = v[i | h];
                v[i] = a + b; v[i | h] = a - b;
            }
#pragma unroll
    for (int m = 1; m < 4; m <<= 1)
    {
        const float s = (lane & m) ? -1.f : 1.f;       // o - v or v + o as one fma (exact either way)
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(v[i], s, __shfl_xor_sync(0xffffffffu, v[i], m));
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= 0.08838834764831845f;
}
// Which 32 elements of its vector a lane holds is free (any assignment of the 7 index bits to 5 register bits and 2
// lane bits gives the same transform), so it is chosen for coalescing: the 4 lanes of a vector access adjacent pieces.
//   map H (fp16 arrays, 16-byte accesses): register 8 j + e of lane q = element 32 j + 8 q + e   (j < 4, e < 8)
//   map F (fp32 arrays, 16-byte accesses; fp16 vectors alongside them by 8-byte accesses):
//                                          register 4 j + e of lane q = element 16 j + 4 q + e   (j < 8, e < 4)
// p points at the vector's first element, q = lane & 3.
__device__ __forceinline__ void load32h_mapH(const __half* p, int q, float (&f)[32])
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const uint4 u = *(const uint4*)(p + 32 * j + 8 * q);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const __half2 h = *(const __half2*)&w[i];
            f[8 * j + 2 * i] = __low2float(h); f[8 * j + 2 * i + 1] = __high2float(h);
        }
    }
}
__device__ __forceinline__ void store32h_mapH(__half* p, int q, const float (&v)[32])
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const __half2 h = __floats2half2_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
            w[i] = *(const uint32_t*)&h;
        }
        *(uint4*)(p + 32 * j + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
__device__ __forceinline__ void load32f_mapF(const float* p, int q, float (&f)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const float4 u = *(const float4*)(p + 16 * j + 4 * q);
        f[4 * j] = u.x; f[4 * j + 1] = u.y; f[4 * j + 2] = u.z; f[4 * j + 3] = u.w;
    }
}
__device__ __forceinline__ void store32f_mapF(float* p, int q, const float (&v)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j) *(float4*)(p + 16 * j + 4 * q) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}
__device__ __forceinline__ void load32h_mapF(const __half* p, int q, float (&f)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const uint2 u = *(const uint2*)(p + 16 * j + 4 * q);
        const __half2 a = *(const __half2*)&u.x, b = *(const __half2*)&u.y;
        f[4 * j] = __low2float(a); f[4 * j + 1] = __high2float(a); f[4 * j + 2] = __low2float(b); f[4 * j + 3] = __high2float(b);
    }
}
__device__ __forceinline__ void store32h_mapF(__half* p, int q, const float (&v)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const __half2 a = __floats2half2_rn(v[4 * j], v[4 * j + 1]), b = __floats2half2_rn(v[4 * j + 2], v[4 * j + 3]);
        uint2 u; u.x = *(const uint32_t*)&a; u.y = *(const uint32_t*)&b;
        *(uint2*)(p + 16 * j + 4 * q) = u;
    }
}

// k-permuted fp16 stores for the fused prefill GEMM, whose decode warps write weight fragments to tensor memory in
// their register order: inside every group of 16 consecutive k, position 4 i + {0, 1} holds k = 2 i + {0, 1} and
// position 4 i + {2, 3} holds k = 8 + 2 i + {0, 1} (i = 0 .. 3).
// map H: lane q holds 8 consecutive k of a 16-group (first half for even q, second for odd q); the two lanes of a pair
// swap two packed words so that each still writes 16 contiguous bytes.
__device__ __forceinline__ void store32h_mapH_kperm(__half* p, int q, const float (&v)[32], bool live)
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const __half2 h = __floats2half2_rn(v[8 * j + 2 * i], v[8 * j + 2 * i + 1]);
            w[i] = *(const uint32_t*)&h;
        }
        const bool odd = q & 1;
        // even lane (k 0..7 of the group) keeps words 0, 1 and needs the partner's words 0, 1 (k 8..11);
        // odd lane (k 8..15) keeps words 2, 3 and needs the partner's words 2, 3 (k 4..7)
        const uint32_t s0 = __shfl_xor_sync(0xffffffffu, odd ? w[0] : w[2], 1), s1 = __shfl_xor_sync(0xffffffffu, odd ? w[1] : w[3], 1);
        const uint4 o = odd ? make_uint4(s0, w[2], s1, w[3]) : make_uint4(w[0], s0, w[1], s1);
        // group base = 32 j + 16 (q >> 1); even lane writes positions 0..7, odd lane positions 8..15
        if (live) *(uint4*)(p + 32 * j + 16 * (q >> 1) + 8 * (q & 1)) = o;      // every lane takes part in the exchange above
    }
}
// map F: lane q holds k = 4 q .. 4 q + 3 of the 16-group j: two packed words that land at two places
__device__ __forceinline__ void store32h_mapF_kperm(__half* p, int q, const float (&v)[32])
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const __half2 a = __floats2half2_rn(v[4 * j], v[4 * j + 1]), b = __floats2half2_rn(v[4 * j + 2], v[4 * j + 3]);
        // k = 4 q + {0,1} -> pair index i = 2 q (mod 4) in half (q >> 1); k = 4 q + {2,3} -> i = 2 q + 1
        const int half = q >> 1, i0 = (2 * q) & 3;
        uint32_t* g = (uint32_t*)(p + 16 * j);
        g[2 * i0 + half] = *(const uint32_t*)&a;
        g[2 * (i0 + 1) + half] = *(const uint32_t*)&b;
    }
}
// the same permutation for a lane holding 4 consecutive k (element 4 * lane + i of a 128-vector)
__device__ __forceinline__ void store4h_kperm(__half* vec, int lane, const float (&v)[4])
{
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    const int q = lane & 3, half = q >> 1, i0 = (2 * q) & 3;
    uint32_t* g = (uint32_t*)(vec + 16 * (lane >> 2));
    g[2 * i0 + half] = *(const uint32_t*)&a;
    g[2 * (i0 + 1) + half] = *(const uint32_t*)&b;
}

// fused forms (no staging array): v = x * s for packed fp16 x (map H); v *= s, v += z * s, sum v * s for an fp16 vector s (map F)
__device__ __forceinline__ void load16w_mapH(const __half* p, int q, uint32_t (&w)[16])
{
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
        const uint4 u = *(const uint4*)(p + 32 * j + 8 * q);
        w[4 * j] = u.x; w[4 * j + 1] = u.y; w[4 * j + 2] = u.z; w[4 * j + 3] = u.w;
    }
}
// v = x * s for the lane's 32 elements, both given as the packed fp16 words of map H (fp32 products)
__device__ __forceinline__ void mul32w_mapH(const uint32_t (&xw)[16], const uint32_t (&sw)[16], float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 16; ++i)
    {
        const __half2 a = *(const __half2*)&xw[i], b = *(const __half2*)&sw[i];
        v[2 * i] = __low2float(a) * __low2float(b); v[2 * i + 1] = __high2float(a) * __high2float(b);
    }
}
template <class F>
__device__ __forceinline__ void each32h_mapF(const __half* p, int q, F&& f)
{
#pragma unroll
    for (int j = 0; j < 8; ++j)
    {
        const uint2 u = *(const uint2*)(p + 16 * j + 4 * q);
        const __half2 a = *(const __half2*)&u.x, b = *(const __half2*)&u.y;
        f(4 * j, __low2float(a)); f(4 * j + 1, __high2float(a)); f(4 * j + 2, __low2float(b)); f(4 * j + 3, __high2float(b));
    }
}
__device__ __forceinline__ void scale32h_mapF(const __half* p, int q, float (&v)[32]) { each32h_mapF(p, q, [&](int i, float s) { v[i] *= s; }); }
__device__ __forceinline__ void axpy32h_mapF(const __half* p, int q, float z, float (&v)[32]) { each32h_mapF(p, q, [&](int i, float s) { v[i] += z * s; }); }
__device__ __forceinline__ float dot32h_mapF(const __half* p, int q, const float (&v)[32])
{
    float d = 0.f;
    each32h_mapF(p, q, [&](int i, float s) { d += v[i] * s; });
    return d;
}

__device__ __forceinline__ float silu(float g) { return g / (1.f + __expf(-g)); }

}  // namespace nq
