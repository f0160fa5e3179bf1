// Instruction issue-rate microbenchmarks for sm_100a (warp-instructions per clock per SM; 8 independent chains per thread).
// Not part of the library build:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o issue_rates issue_rates.cu
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <algorithm>
#include <vector>
#define ITERS 2048
#define PRO long long c0 = clock64();
#define EPI(v) long long c1 = clock64(); if (threadIdx.x == 0) dur[blockIdx.x] = c1 - c0; if ((v) == 0x12345678u) sink[0] = (v);

#define CH8(OP) OP(0) OP(1) OP(2) OP(3) OP(4) OP(5) OP(6) OP(7)

__global__ void k_imad(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x83DCD12Du), "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_shf(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("shf.r.wrap.b32 %0, %0, %1, 7;" : "+r"(x[i]) : "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_prmt(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("prmt.b32 %0, %0, %1, 0x4321;" : "+r"(x[i]) : "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_lop(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("lop3.b32 %0, %0, %1, %2, 0x96;" : "+r"(x[i]) : "r"(s), "r"(s + 5));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_iadd(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("add.u32 %0, %0, %1;" : "+r"(x[i]) : "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_dp4a(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("dp4a.u32.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x01010101u), "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_hfma2(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x3c003c00u), "r"(s));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_ffma(long long* dur, uint32_t* sink, uint32_t s) {
  float x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  float a = __uint_as_float(s | 0x3f800000u), b = (float)s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(x[i]) : "f"(a), "f"(b));
    CH8(OP)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= __float_as_uint(x[i]); EPI(v)
}
// mixes: pairs of different op kinds, 4 chains each
__global__ void k_imad_prmt(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x83DCD12Du), "r"(s));
#define OPB(i) asm volatile("prmt.b32 %0, %0, %1, 0x4321;" : "+r"(x[i]) : "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_imad_dp4a(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x83DCD12Du), "r"(s));
#define OPB(i) asm volatile("dp4a.u32.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x01010101u), "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_prmt_dp4a(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("prmt.b32 %0, %0, %1, 0x4321;" : "+r"(x[i]) : "r"(s));
#define OPB(i) asm volatile("dp4a.u32.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x01010101u), "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_prmt_shf(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("prmt.b32 %0, %0, %1, 0x4321;" : "+r"(x[i]) : "r"(s));
#define OPB(i) asm volatile("shf.r.wrap.b32 %0, %0, %1, 7;" : "+r"(x[i]) : "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_prmt_hfma2(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("prmt.b32 %0, %0, %1, 0x4321;" : "+r"(x[i]) : "r"(s));
#define OPB(i) asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x3c003c00u), "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
__global__ void k_imad_hfma2(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OPA(i) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x83DCD12Du), "r"(s));
#define OPB(i) asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(s | 0x3c003c00u), "r"(s));
    OPA(0) OPB(1) OPA(2) OPB(3) OPA(4) OPB(5) OPA(6) OPB(7)
#undef OPA
#undef OPB
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
// tensor: 4 independent accumulators
__global__ void k_mma_f16(long long* dur, uint32_t* sink, uint32_t s) {
  float c[4][4]; for (int i = 0; i < 16; ++i) c[i / 4][i % 4] = 0.f;
  uint32_t a0 = s + threadIdx.x, a1 = s * 3, a2 = s * 5, a3 = s * 7, b0 = s * 9, b1 = s * 11;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};" \
    : "+f"(c[i][0]), "+f"(c[i][1]), "+f"(c[i][2]), "+f"(c[i][3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    OP(0) OP(1) OP(2) OP(3)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 16; ++i) v ^= __float_as_uint(c[i / 4][i % 4]); EPI(v)
}
__global__ void k_mma_u8(long long* dur, uint32_t* sink, uint32_t s) {
  int c[4][4]; for (int i = 0; i < 16; ++i) c[i / 4][i % 4] = 0;
  uint32_t a0 = s + threadIdx.x, a1 = s * 3, a2 = s * 5, a3 = s * 7, b0 = s * 9, b1 = s * 11;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#define OP(i) asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};" \
    : "+r"(c[i][0]), "+r"(c[i][1]), "+r"(c[i][2]), "+r"(c[i][3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    OP(0) OP(1) OP(2) OP(3)
#undef OP
  }
  uint32_t v = 0; for (int i = 0; i < 16; ++i) v ^= (uint32_t)c[i / 4][i % 4]; EPI(v)
}
// decode-like mix per 4 weights: 5 ALU(prmt/shf), 4 imad, 1 mma_u8, 2 prmt, 2 hfma2  (MMA byte-sum variant)
__global__ void k_mix_mma(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  int c[4] = {0, 0, 0, 0};
  PRO
  for (int it = 0; it < ITERS; ++it) {
    asm volatile("shf.r.wrap.b32 %0, %0, %1, 7;" : "+r"(x[4]) : "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4410;" : "=r"(x[0]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4421;" : "=r"(x[1]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4432;" : "=r"(x[2]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4443;" : "=r"(x[3]) : "r"(x[4]), "r"(s));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[0]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[1]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[2]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[3]) : "r"(s | 0x83DCD12Du));
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(x[0]), "r"(x[1]), "r"(x[2]), "r"(x[3]), "r"(s), "r"(s + 1), "r"(0x6400));
    asm volatile("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(x[5]) : "r"(c[0]), "r"(c[1]));
    asm volatile("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(x[6]) : "r"(c[2]), "r"(c[3]));
    asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[5]) : "r"(s | 0x1eee1eeeu), "r"(s | 0xc931c931u));
    asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[6]) : "r"(s | 0x1eee1eeeu), "r"(s | 0xc931c931u));
    asm volatile("xor.b32 %0, %0, %1;" : "+r"(x[7]) : "r"(x[5]));
    asm volatile("xor.b32 %0, %0, %1;" : "+r"(x[4]) : "r"(x[6]));
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
// same with dp4a byte sums
__global__ void k_mix_dp4a(long long* dur, uint32_t* sink, uint32_t s) {
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = threadIdx.x * 7 + i + s;
  uint32_t c[4];
  PRO
  for (int it = 0; it < ITERS; ++it) {
    asm volatile("shf.r.wrap.b32 %0, %0, %1, 7;" : "+r"(x[4]) : "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4410;" : "=r"(x[0]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4421;" : "=r"(x[1]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4432;" : "=r"(x[2]) : "r"(x[4]), "r"(s));
    asm volatile("prmt.b32 %0, %1, %2, 0x4443;" : "=r"(x[3]) : "r"(x[4]), "r"(s));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[0]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[1]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[2]) : "r"(s | 0x83DCD12Du));
    asm volatile("mul.lo.u32 %0, %0, %1;" : "+r"(x[3]) : "r"(s | 0x83DCD12Du));
    asm volatile("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(c[0]) : "r"(x[0]), "r"(s | 0x01010101u), "r"(0x6400));
    asm volatile("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(c[1]) : "r"(x[1]), "r"(s | 0x01010101u), "r"(0x6400));
    asm volatile("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(c[2]) : "r"(x[2]), "r"(s | 0x01010101u), "r"(0x6400));
    asm volatile("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(c[3]) : "r"(x[3]), "r"(s | 0x01010101u), "r"(0x6400));
    asm volatile("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(x[5]) : "r"(c[0]), "r"(c[1]));
    asm volatile("prmt.b32 %0, %1, %2, 0x5410;" : "=r"(x[6]) : "r"(c[2]), "r"(c[3]));
    asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[5]) : "r"(s | 0x1eee1eeeu), "r"(s | 0xc931c931u));
    asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(x[6]) : "r"(s | 0x1eee1eeeu), "r"(s | 0xc931c931u));
    asm volatile("xor.b32 %0, %0, %1;" : "+r"(x[7]) : "r"(x[5]));
    asm volatile("xor.b32 %0, %0, %1;" : "+r"(x[4]) : "r"(x[6]));
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}
// random 16-bit shared-memory gathers (lookup-table decode): 8 independent loads per iteration
__global__ void k_lds16(long long* dur, uint32_t* sink, uint32_t s) {
  extern __shared__ uint16_t lut[];
  for (int i = threadIdx.x; i < 65536; i += blockDim.x) lut[i] = (uint16_t)(i * 2654435761u >> 13);
  __syncthreads();
  uint32_t x[8]; for (int i = 0; i < 8; ++i) x[i] = (threadIdx.x * 7919u + i * 104729u + s) & 0xFFFF;
  PRO
  for (int it = 0; it < ITERS; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = (lut[x[i]] + x[i] * 5u + 1u) & 0xFFFF;
  }
  uint32_t v = 0; for (int i = 0; i < 8; ++i) v ^= x[i]; EPI(v)
}

typedef void (*kfn)(long long*, uint32_t*, uint32_t);
struct T { const char* name; kfn f; double instr_per_iter; int smem; int bps; };
int main() {
  cudaDeviceProp p; cudaGetDeviceProperties(&p, 0);
  printf("device %s, %d SMs, clock %d kHz\n", p.name, p.multiProcessorCount, p.clockRate);
  int nsm = p.multiProcessorCount;
  long long* dur; uint32_t* sink; cudaMalloc(&dur, sizeof(long long) * nsm * 8); cudaMalloc(&sink, 64);
  T tests[] = {
    {"imad", k_imad, 8, 0, 4}, {"shf", k_shf, 8, 0, 4}, {"prmt", k_prmt, 8, 0, 4}, {"lop3", k_lop, 8, 0, 4}, {"iadd", k_iadd, 8, 0, 4},
    {"dp4a", k_dp4a, 8, 0, 4}, {"hfma2", k_hfma2, 8, 0, 4}, {"ffma", k_ffma, 8, 0, 4},
    {"imad+prmt", k_imad_prmt, 8, 0, 4}, {"imad+dp4a", k_imad_dp4a, 8, 0, 4}, {"prmt+dp4a", k_prmt_dp4a, 8, 0, 4},
    {"prmt+shf", k_prmt_shf, 8, 0, 4}, {"prmt+hfma2", k_prmt_hfma2, 8, 0, 4}, {"imad+hfma2", k_imad_hfma2, 8, 0, 4},
    {"mma_f16_m16n8k16", k_mma_f16, 4, 0, 4}, {"mma_u8_m16n8k32", k_mma_u8, 4, 0, 4},
    {"mix_mma(16 instr / 4 weights)", k_mix_mma, 16, 0, 4}, {"mix_dp4a(19 instr / 4 weights)", k_mix_dp4a, 19, 0, 4},
    {"lds16_gather", k_lds16, 8, 131072, 1},
  };
  for (auto& t : tests) {
    if (t.smem) cudaFuncSetAttribute(t.f, cudaFuncAttributeMaxDynamicSharedMemorySize, t.smem);
    int nb = nsm * t.bps;
    for (int rep = 0; rep < 2; ++rep) t.f<<<nb, 256, t.smem>>>(dur, sink, 0);
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0); t.f<<<nb, 256, t.smem>>>(dur, sink, 0); cudaEventRecord(e1);
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) { printf("%s: %s\n", t.name, cudaGetErrorString(err)); return 1; }
    float ms; cudaEventElapsedTime(&ms, e0, e1);
    std::vector<long long> h(nb); cudaMemcpy(h.data(), dur, sizeof(long long) * nb, cudaMemcpyDeviceToHost);
    std::sort(h.begin(), h.end());
    double cyc = (double)h[nb / 2];
    double wi = (double)ITERS * t.instr_per_iter * 8 /*warps per block*/ * t.bps;   // warp-instructions per SM
    printf("%-34s %8.3f warp-instr/clk/SM  (%6.1f lanes/clk/SM)  cycles %.0f  ms %.3f  eff MHz %.0f\n", t.name, wi / cyc, 32 * wi / cyc, cyc, ms, cyc / ms / 1e3);
  }
  return 0;
}
