// Decode salience export: sal[e] += sum over the picks (t, k) of expert e of (rsf * rw[t][k])^2 * |x[t]|^2.
//
// Replaces sal() of the reference's sm120/nqsal.cu:1-79 (the input of its floating-set predictor): one launch per decode
// call, graph-capturable, running sums in a device fp64 array, every touched entry mirrored to a host-mapped fp64 array
// that the host diffs like the routing-hit counters; picks with weight 0 are skipped, calls on one layer are
// stream-ordered so the sums need no atomics across calls.  Built for this library's decode limits (32 tokens, 256
// picks) instead of the reference's 8 x 8: one warp per token for the squared norms, then one thread per expert adds that
// expert's picks in pick order.
#include <cuda_bf16.h>

#include "nq_common.cuh"

namespace nq {

template <class T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <class T>
__global__ void __launch_bounds__(256) salience_kernel(const T* __restrict__ x, int64_t row_stride, const __half* __restrict__ rw,
                                                       const int64_t* __restrict__ sel, int B, int H, int topk, int E, float rsf,
                                                       double* acc, double* host)
{
    __shared__ float xn[NQ_MAX_TOKENS];
    __shared__ int s_exp[NQ_MAX_PICKS];
    __shared__ double s_val[NQ_MAX_PICKS];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n = B * topk;
    for (int t = warp; t < B; t += 8)
    {
        const T* xr = x + (int64_t)t * row_stride;
        float s = 0.f;
        for (int i = lane; i < H; i += 32) { const float f = to_f32(xr[i]); s += f * f; }
#pragma unroll
        for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) xn[t] = s;
    }
    __syncthreads();
    if (tid < n)
    {
        float w = __half2float(rw[tid]);
        const int64_t e = sel[tid];
        s_exp[tid] = (w != 0.f && e >= 0 && e < E) ? (int)e : -1;
        w *= rsf;
        s_val[tid] = (double)(w * w * xn[tid / topk]);
    }
    __syncthreads();
    // one thread per expert: walk the picks in pick order and add up those of this expert (a fixed order of additions,
    // no election of a writer among the picks)
    for (int e = tid; e < E; e += 256)
    {
        double tot = 0.0;
        bool any = false;
        for (int j = 0; j < n; ++j)
            if (s_exp[j] == e) { tot += s_val[j]; any = true; }
        if (any)
        {
            const double a = acc[e] + tot;
            acc[e] = a;
            if (host) host[e] = a;
        }
    }
}

}  // namespace nq

extern "C" int nq_salience(const void* x, int x_is_bf16, int64_t row_stride, const void* rw, const int64_t* sel, int B, int H, int topk,
                           int E, float rsf, double* acc, double* host, void* stream)
{
    NQ_REQUIRE(B >= 0 && B <= NQ_MAX_TOKENS && topk >= 1 && B * topk <= NQ_MAX_PICKS && H > 0 && E > 0,
               "nq_salience: B = %d, topk = %d, H = %d, E = %d", B, topk, H, E);
    if (B == 0) return NQ_OK;
    NQ_REQUIRE(x && rw && sel && acc && row_stride >= H, "nq_salience: null pointer or row stride %lld < H", (long long)row_stride);
    cudaStream_t st = (cudaStream_t)stream;
    if (x_is_bf16)
        nq::salience_kernel<__nv_bfloat16><<<1, 256, 0, st>>>((const __nv_bfloat16*)x, row_stride, (const __half*)rw, sel, B, H, topk, E, rsf, acc, host);
    else
        nq::salience_kernel<__half><<<1, 256, 0, st>>>((const __half*)x, row_stride, (const __half*)rw, sel, B, H, topk, E, rsf, acc, host);
    return nq::check_launch("nq_salience");
}
