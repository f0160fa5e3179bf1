// Decode-core microbenchmark: the trellis decoder of the library on pseudo-random words held in registers (no memory
// traffic), feeding an mma.m16n8k16 sink as the GEMV does.  Prints weights per clock per SM; argument = CTAs of 8 warps
// per SM (2 = 16 warps, 4 = 32 warps).  Not part of the library build:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr -o decode_rate decode_rate.cu
#include <cuda_runtime.h>
#include <stdio.h>
#include <vector>
#include <algorithm>
#include "../nq_unit.cuh"
using namespace nq;
#define UNITS 256
struct XorSink { uint32_t& acc; template <int T> __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const { acc ^= a[0] + a[1] * 3 + a[2] * 5 + a[3] * 7; } };
struct MmaSink { float (&c)[4]; uint32_t b0, b1; template <int T> __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};" : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1)); } };

template <int VAR, int RC>
__global__ void __launch_bounds__(256) k(long long* dur, uint32_t* out, uint32_t seed)
{
  const int lane = threadIdx.x & 31;
  uint32_t s = seed + threadIdx.x * 2654435761u + blockIdx.x * 40503u;
  float c[4] = {0, 0, 0, 0}; uint32_t acc = 0;
  long long c0 = clock64();
  for (int u = 0; u < UNITS; ++u) {
    uint32_t wb[6], wr[Pattern<RC>::kWords + 2];
    for (int i = 0; i < 4; ++i) { s = s * 1664525u + 1013904223u; wb[i] = s; }
    for (int i = 0; i < Pattern<RC>::kWords; ++i) { s = s * 1664525u + 1013904223u; wr[i] = s; }
    uint32_t dl = 200u | ((s >> 24) << 8 & 0x3F00);
    MmaSink sink{c, s, s ^ 0x5555u};
    if (VAR == 0) decode_words<false, 0>(wb, nullptr, consts_level2(0), lane, sink);
    if (VAR == 1) decode_words<true, RC>(wb, wr, consts_level4(dl, 0), lane, sink);
    if (VAR == 4) { // windows + hash only (base)
      extend_stream<128>(wb, __shfl_sync(~0u, wb[0], ring_next_lane(lane)));
      static_for<64>([&](auto jc) { constexpr int j = decltype(jc)::value; acc ^= window16<2 * j>(wb) * kHashMul; });
    }
    if (VAR == 5) { // windows only
      extend_stream<128>(wb, __shfl_sync(~0u, wb[0], ring_next_lane(lane)));
      static_for<64>([&](auto jc) { constexpr int j = decltype(jc)::value; acc ^= window16<2 * j>(wb); });
    }
  }
  long long c1 = clock64();
  if (threadIdx.x == 0) dur[blockIdx.x] = c1 - c0;
  out[blockIdx.x * 256 + threadIdx.x] = acc ^ __float_as_uint(c[0] + c[1] + c[2] + c[3]);
}
typedef void (*kfn)(long long*, uint32_t*, uint32_t);
int main(int argc, char** argv) {
  int bps = argc > 1 ? atoi(argv[1]) : 2;
  cudaDeviceProp p; cudaGetDeviceProperties(&p, 0); int nsm = p.multiProcessorCount;
  long long* dur; uint32_t* out; cudaMalloc(&dur, 8 * nsm * 8); cudaMalloc(&out, 4 * 256 * nsm * 8);
  struct T { const char* n; kfn f; } tests[] = {
    {"level 2", k<0, 0>}, {"level 4 rc0", k<1, 0>}, {"level 4 rc7", k<1, 7>}, {"level 4 rc9", k<1, 9>},
        {"windows+hash", k<4, 0>}, {"windows", k<5, 0>} };
  for (auto& t : tests) {
    int nb = nsm * bps;
    t.f<<<nb, 256>>>(dur, out, 1); cudaDeviceSynchronize();
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0); t.f<<<nb, 256>>>(dur, out, 2); cudaEventRecord(e1);
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("%s failed\n", t.n); return 1; }
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    std::vector<long long> h(nb); cudaMemcpy(h.data(), dur, 8 * nb, cudaMemcpyDeviceToHost); std::sort(h.begin(), h.end());
    double cyc = (double)h[nb / 2];
    double w = (double)UNITS * 2048 * 8 * bps;   // weights per SM
    printf("%-16s ctas/SM %d: %6.2f weights/clk/SM  (%.0f cycles per unit per warp, %.3f ms)\n", t.n, bps, w / cyc, cyc / UNITS, ms);
  }
  return 0;
}
