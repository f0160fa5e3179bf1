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
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
            v[i] = (lane & m) ? o - v[i] : v[i] + o;
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

__device__ __forceinline__ float silu(float g) { return g / (1.f + __expf(-g)); }

}  // namespace nq
