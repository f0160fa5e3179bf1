// Prefill path, the work around the grouped GEMMs: per routed pair (token, expert), sorted by expert,
//   pf_pre      x * su_g / su_u -> WHT128 -> fp16 rows xg, xu (the GEMM A operands) and the low-rank input z_gu
//   pf_mid      WHT128(acc) * sv (+ low rank) -> SwiGLU -> * su_d -> WHT128 (or WHT512) -> h fp16, z_dn
//   pf_post     out[token] += rw * (WHT128(y) * sv_o + low rank)           (atomic, as the reference)
//   pf_combine  out[token]  = sum over the token's picks in pick order     (no atomics: bitwise repeatable)
//   pf_hits     routing-hit export
// Replaces nq_pf_pre / nq_pf_mid / nq_pf_post / nq_pf_hits of the reference (sm120/nqmoe.cu:1081-1245,1258-1293).
// All of them are HBM-bound elementwise passes over [pairs][H] or [pairs][I] arrays; a warp owns a 128-wide group
// (one Hadamard block), a CTA owns a pair.
#include "nq_common.cuh"
#include "nq_format.cuh"
#include "nq_rotate.cuh"

namespace nq {

struct LowRank
{
    const __half* lr;     // [V_gu rg x H | U2_g rg x I | U2_u rg x I | V_dn rd x I | U2_d rd x H]
    const __half* lr4;    // level-4 part [U4_g rg x I | U4_u rg x I | U4_d rd x H] or null
    int rg, rd;
};
__device__ __forceinline__ LowRank low_rank_of(const int64_t* row, int level)
{
    LowRank l;
    l.lr = (const __half*)row[14];
    l.rg = l.lr ? (int)row[16] : 0; l.rd = l.lr ? (int)row[17] : 0;
    l.lr4 = level == 4 ? (const __half*)row[15] : nullptr;
    return l;
}
__device__ __forceinline__ float warp_sum(float d)
{
#pragma unroll
    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    return d;
}

// one CTA (256 threads) per pair
__global__ void __launch_bounds__(256) pf_pre_kernel(const __half* __restrict__ x, const int* __restrict__ pt, const int* __restrict__ pe,
                                                     const int64_t* __restrict__ table, __half* xg, __half* xu, float* zg, int H, int I)
{
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t* row = table + (int64_t)pe[p] * kTableWidth;
    const int level = (int)row[0];
    if (level <= 0) return;
    const __half* scales = (const __half*)row[9];
    const __half* xr = x + (size_t)pt[p] * H;
    const int ng = H / 128;
    for (int task = warp; task < 2 * ng; task += 8)
    {
        const int up = task >= ng, k = (task - up * ng) * 128 + lane * 4;
        const __half* su = up ? scales + 2 * H + 3 * I : scales;
        float f[4], s[4];
        load4h(xr + k, f); load4h(su + k, s);
        float v[4] = {f[0] * s[0], f[1] * s[1], f[2] * s[2], f[3] * s[3]};
        wht128(v, lane);
        store4h((up ? xu : xg) + (size_t)p * H + k, v);
    }
    const LowRank L = low_rank_of(row, level);
    if (warp < 4)
    {
        float d = 0.f;
        if (warp < L.rg)
        {
            for (int k = lane * 4; k < H; k += 128)
            {
                float f[4], v[4];
                load4h(xr + k, f); load4h(L.lr + (size_t)warp * H + k, v);
                d += f[0] * v[0] + f[1] * v[1] + f[2] * v[2] + f[3] * v[3];
            }
            d = warp_sum(d);
        }
        if (lane == 0) zg[(size_t)p * 4 + warp] = d;
    }
}

// one CTA (128 threads) per pair; dynamic shared memory: I floats (staging for the 512-wide rotation)
__global__ void __launch_bounds__(128) pf_mid_kernel(const float* __restrict__ acc_g, const float* __restrict__ acc_u, const float* __restrict__ zg,
                                                     const int* __restrict__ pe, const int64_t* __restrict__ table, __half* h, float* zd, int H, int I)
{
    extern __shared__ float stage[];
    __shared__ float zpart[64][4];
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, ng = I / 128;
    const int64_t* row = table + (int64_t)pe[p] * kTableWidth;
    const int level = (int)row[0];
    if (level <= 0) return;
    const __half* scales = (const __half*)row[9];
    const __half *sv_g = scales + H, *sv_u = sv_g + I, *su_d = sv_u + I;
    const LowRank L = low_rank_of(row, level);
    const int hw = (int)row[18];
    float z[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) z[r] = zg[(size_t)p * 4 + r];
    for (int grp = warp; grp < ng; grp += 4)
    {
        const int col = grp * 128 + lane * 4;
        float gu[2][4];
#pragma unroll
        for (int up = 0; up < 2; ++up)
        {
            const float4 f = *(const float4*)((up ? acc_u : acc_g) + (size_t)p * I + col);
            float v[4] = {f.x, f.y, f.z, f.w}, s[4];
            wht128(v, lane);
            load4h((up ? sv_u : sv_g) + col, s);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] *= s[i];
            for (int r = 0; r < L.rg; ++r)
            {
                float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
                const size_t o = (size_t)(up * L.rg + r) * I + col;
                load4h(L.lr + (size_t)L.rg * H + o, u2);
                if (L.lr4) load4h(L.lr4 + o, u4);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] += z[r] * u2[i] + z[r] * u4[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) gu[up][i] = v[i];
        }
        float v[4], s[4];
        load4h(su_d + col, s);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = silu(gu[0][i]) * gu[1][i];
        for (int r = 0; r < L.rd; ++r)
        {
            float vd[4];
            load4h(L.lr + (size_t)L.rg * H + 2 * (size_t)L.rg * I + (size_t)r * I + col, vd);
            const float d = warp_sum(v[0] * vd[0] + v[1] * vd[1] + v[2] * vd[2] + v[3] * vd[3]);
            if (lane == 0) zpart[grp][r] = d;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] *= s[i];
        wht128(v, lane);
        if (hw <= 128) store4h(h + (size_t)p * I + col, v);
        else *(float4*)(stage + col) = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    if (threadIdx.x < 4)      // column groups added in order: the same sum whatever the launch shape
    {
        float s = 0.f;
        if ((int)threadIdx.x < L.rd)
            for (int q = 0; q < ng; ++q) s += zpart[q][threadIdx.x];
        zd[(size_t)p * 4 + threadIdx.x] = s;
    }
    if (hw > 128)             // WHT_hw = H_(hw/128) (x) WHT128: combine the hw/128 rotated blocks of each hw-wide group
    {
        const int nb = hw / 128;
        const float rs = rsqrtf((float)nb);
        for (int blk = warp; blk < ng; blk += 4)
        {
            const int b0 = blk / nb * nb, ob = blk - b0;
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            for (int b = 0; b < nb; ++b)
            {
                const float4 f = *(const float4*)(stage + (b0 + b) * 128 + lane * 4);
                const float sg = (__popc(ob & b) & 1) ? -1.f : 1.f;
                o[0] += sg * f.x; o[1] += sg * f.y; o[2] += sg * f.z; o[3] += sg * f.w;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] *= rs;
            store4h(h + (size_t)p * I + blk * 128 + lane * 4, o);
        }
    }
}

// rw * (WHT128(y) * sv_o + z_dn (U2_d [+ U4_d])) for output columns [col, col + 4) of pair p; false if the pair adds nothing
__device__ __forceinline__ bool pair_output(const float* __restrict__ y, const float* __restrict__ zd, int p, int e, float w,
                                            const int64_t* __restrict__ table, int H, int I, int col, int lane, float (&v)[4])
{
    const int64_t* row = table + (int64_t)e * kTableWidth;
    const int level = (int)row[0];
    if (level <= 0 || w == 0.f) return false;
    const __half* sv_o = (const __half*)row[9] + H + 3 * I;
    const LowRank L = low_rank_of(row, level);
    const float4 f = *(const float4*)(y + (size_t)p * H + col);
    float s[4];
    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    wht128(v, lane);
    load4h(sv_o + col, s);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= s[i];
    const size_t ou = (size_t)L.rg * H + 2 * (size_t)L.rg * I + (size_t)L.rd * I;
    for (int r = 0; r < L.rd; ++r)
    {
        const float z = zd[(size_t)p * 4 + r];
        float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
        load4h(L.lr + ou + (size_t)r * H + col, u2);
        if (L.lr4) load4h(L.lr4 + 2 * (size_t)L.rg * I + (size_t)r * H + col, u4);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] += z * u2[i] + z * u4[i];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= w;
    return true;
}

// one CTA (256 threads) per pair: atomic accumulation into out[token]
__global__ void __launch_bounds__(256) pf_post_kernel(const float* __restrict__ y, const float* __restrict__ zd, const int* __restrict__ pt,
                                                      const int* __restrict__ pe, const __half* __restrict__ prw,
                                                      const int64_t* __restrict__ table, float* out, int H, int I)
{
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float w = __half2float(prw[p]);
    float* op = out + (size_t)pt[p] * H;
    for (int grp = warp; grp < H / 128; grp += 8)
    {
        float v[4];
        const int col = grp * 128 + lane * 4;
        if (!pair_output(y, zd, p, pe[p], w, table, H, I, col, lane, v)) return;   // CTA-uniform
#pragma unroll
        for (int i = 0; i < 4; ++i) atomicAdd(op + col + i, v[i]);
    }
}

// one CTA (256 threads) per token: picks added in pick order, out written once.  pos[t * topk + k] = index of that pick
// in the expert-sorted pair arrays.
__global__ void __launch_bounds__(256) pf_combine_kernel(const float* __restrict__ y, const float* __restrict__ zd, const int* __restrict__ pos,
                                                         const int64_t* __restrict__ sel, const __half* __restrict__ rw,
                                                         const int64_t* __restrict__ table, float* out, int topk, int E, int H, int I)
{
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int grp = warp; grp < H / 128; grp += 8)
    {
        const int col = grp * 128 + lane * 4;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < topk; ++k)
        {
            const int64_t e = sel[(size_t)t * topk + k];
            if (e < 0 || e >= E) continue;
            float v[4];
            if (!pair_output(y, zd, pos[(size_t)t * topk + k], (int)e, __half2float(rw[(size_t)t * topk + k]), table, H, I, col, lane, v))
                continue;
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] += v[i];
        }
        *(float4*)(out + (size_t)t * H + col) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void pf_hits_kernel(const int* __restrict__ counts, int* hits, int E)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < E && counts[e]) atomicAdd(hits + e, counts[e]);
}

}  // namespace nq

extern "C" {

#define NQ_SHAPE_OK(fn) NQ_REQUIRE(H > 0 && I > 0 && H % 128 == 0 && I % 128 == 0 && H / 128 <= 64 && I / 128 <= 64, fn ": H = %d, I = %d must be multiples of 128, at most 64 * 128", H, I)

int nq_pf_pre(const void* x, const int32_t* pt, const int32_t* pe, int R, const int64_t* table, void* xg, void* xu, float* zg,
              int H, int I, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_pre: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(x && pt && pe && table && xg && xu && zg, "nq_pf_pre: null pointer");
    NQ_SHAPE_OK("nq_pf_pre");
    NQ_REQUIRE(nq::aligned16(x) && nq::aligned16(xg) && nq::aligned16(xu), "nq_pf_pre: x, xg, xu must be 16-byte aligned");
    nq::pf_pre_kernel<<<R, 256, 0, (cudaStream_t)stream>>>((const __half*)x, pt, pe, table, (__half*)xg, (__half*)xu, zg, H, I);
    return nq::check_launch("nq_pf_pre");
}

int nq_pf_mid(const float* acc_g, const float* acc_u, const float* zg, const int32_t* pe, int R, const int64_t* table, void* h,
              float* zd, int H, int I, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_mid: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(acc_g && acc_u && zg && pe && table && h && zd, "nq_pf_mid: null pointer");
    NQ_SHAPE_OK("nq_pf_mid");
    NQ_REQUIRE(nq::aligned16(acc_g) && nq::aligned16(acc_u) && nq::aligned16(h), "nq_pf_mid: acc_g, acc_u, h must be 16-byte aligned");
    nq::pf_mid_kernel<<<R, 128, (size_t)I * 4, (cudaStream_t)stream>>>(acc_g, acc_u, zg, pe, table, (__half*)h, zd, H, I);
    return nq::check_launch("nq_pf_mid");
}

int nq_pf_post(const float* y, const float* zd, const int32_t* pt, const int32_t* pe, const void* prw, int R, const int64_t* table,
               float* out, int H, int I, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_post: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(y && zd && pt && pe && prw && table && out, "nq_pf_post: null pointer");
    NQ_SHAPE_OK("nq_pf_post");
    NQ_REQUIRE(nq::aligned16(y) && nq::aligned16(out), "nq_pf_post: y and out must be 16-byte aligned");
    nq::pf_post_kernel<<<R, 256, 0, (cudaStream_t)stream>>>(y, zd, pt, pe, (const __half*)prw, table, out, H, I);
    return nq::check_launch("nq_pf_post");
}

int nq_pf_combine(const float* y, const float* zd, const int32_t* pos, const int64_t* sel, const void* rw, int T, int topk,
                  const int64_t* table, int E, float* out, int H, int I, void* stream)
{
    NQ_REQUIRE(T >= 0 && topk >= 1 && E >= 1, "nq_pf_combine: T = %d, topk = %d, E = %d", T, topk, E);
    if (T == 0) return NQ_OK;
    NQ_REQUIRE(y && zd && pos && sel && rw && table && out, "nq_pf_combine: null pointer");
    NQ_SHAPE_OK("nq_pf_combine");
    NQ_REQUIRE(nq::aligned16(y) && nq::aligned16(out), "nq_pf_combine: y and out must be 16-byte aligned");
    nq::pf_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(y, zd, pos, sel, (const __half*)rw, table, out, topk, E, H, I);
    return nq::check_launch("nq_pf_combine");
}

int nq_pf_hits(const int32_t* counts, int32_t* hits, int E, void* stream)
{
    if (!hits) return NQ_OK;
    NQ_REQUIRE(counts && E > 0, "nq_pf_hits: counts null or E = %d", E);
    nq::pf_hits_kernel<<<(E + 255) / 256, 256, 0, (cudaStream_t)stream>>>(counts, hits, E);
    return nq::check_launch("nq_pf_hits");
}

}  // extern "C"
