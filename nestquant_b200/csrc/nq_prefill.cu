// Prefill path, the work around the grouped GEMMs: per routed pair (token, expert), sorted by expert,
//   pf_pre      x * su_g / su_u -> WHT128 -> fp16 rows xg, xu (the GEMM A operands) and the low-rank input z_gu
//   pf_mid      WHT128(acc) * sv (+ low rank) -> SwiGLU -> * su_d -> WHT128 (or WHT512) -> h fp16, z_dn
//   pf_post     out[token] += rw * (WHT128(y) * sv_o + low rank)           (atomic, as the reference)
//   pf_combine  out[token]  = sum over the token's picks in pick order     (no atomics: bitwise repeatable)
//   pf_hits     routing-hit export
// Replaces nq_pf_pre / nq_pf_mid / nq_pf_post / nq_pf_hits of the reference (sm120/nqmoe.cu:1081-1245,1258-1293).
// All of them are elementwise passes over [pairs][H] or [pairs][I] arrays; a CTA owns a pair, a token or (pf_pre) a run of pairs, a
// warp eight 128-wide groups (Hadamard blocks) at a time, 32 consecutive columns per lane.
#include "nq_common.cuh"
#include "nq_format.cuh"
#include "nq_rotate.cuh"

#ifndef NQ_PF_PRE_BLOCKS
#define NQ_PF_PRE_BLOCKS 2    // pf_pre keeps two scale vectors and a prefetched row in registers
#endif
#ifndef NQ_PF_EW_BLOCKS
#define NQ_PF_EW_BLOCKS 3     // resident 256-thread CTAs the elementwise passes are compiled for (register cap)
#endif

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

// Thread layout of the passes below: a warp task = 8 consecutive 128-wide groups (1024 columns) of one row; lanes
// 4 v .. 4 v + 3 hold group v, 32 columns each (wht128_x8 and its maps).  Groups past the end of the row are idle lanes.
__device__ __forceinline__ float quad_sum(float d)
{
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    return d + __shfl_xor_sync(0xffffffffu, d, 2);
}
// Where the input rows live: token t is row t % tokens_per_rank of buffer t / tokens_per_rank.  One buffer holding every
// token is the single-GPU case; under expert parallelism the buffers are the ranks' symmetric-memory input buffers as seen
// from this GPU, and reading a row IS the dispatch (plain peer loads over NVLink, each pair's row fetched by the rank that
// multiplies it).
constexpr int kPfMaxRanks = 8;
struct TokenRows { const __half* base[kPfMaxRanks]; int tokens_per_rank; };
__device__ __forceinline__ const __half* token_row(const TokenRows& r, int t, int H)
{
    const int owner = t / r.tokens_per_rank;
    return r.base[owner] + (size_t)(t - owner * r.tokens_per_rank) * H;
}

// A CTA takes a contiguous range of the (expert-sorted) pairs, a warp 1,024 columns of every one of them.  The two scale
// vectors of those columns stay in registers while the expert stays the same (the pairs of an expert are consecutive),
// and the input row of the next pair is fetched before the current one is transformed.
struct PairHead { int e; bool live; const __half* xr; const int64_t* row; int level; };
__device__ __forceinline__ PairHead pair_head(const TokenRows& rows, const int* __restrict__ pt, const int* __restrict__ pe,
                                              const int64_t* __restrict__ table, int E, int H, int p, int p1)
{
    PairHead h{-1, false, nullptr, nullptr, 0};
    if (p >= p1) return h;
    h.e = pe[p];
    if (h.e < 0 || h.e >= E) return h;           // a pick with no valid expert id (padding): nothing to prepare
    h.row = table + (int64_t)h.e * kTableWidth;
    h.level = (int)h.row[0];
    if (h.level <= 0) return h;
    h.live = true;
    h.xr = token_row(rows, pt[p], H);
    return h;
}
__global__ void __launch_bounds__(256, NQ_PF_PRE_BLOCKS) pf_pre_kernel(TokenRows rows, const int* __restrict__ pt, const int* __restrict__ pe,
                                                     const int64_t* __restrict__ table, int E, __half* xg, __half* xu, float* zg, int H, int I,
                                                     int kperm, int R)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, ng = H / 128;
    const int per = (R + (int)gridDim.x - 1) / (int)gridDim.x, p0 = (int)blockIdx.x * per, p1 = p0 + per < R ? p0 + per : R;
    const int q = lane & 3;
    for (int g0 = warp * 8; g0 < ng; g0 += nwarp * 8)
    {
        const int grp = g0 + (lane >> 2), k = grp * 128;
        const bool in_row = grp < ng;
        uint32_t sg[16], su[16], xw[16];
        int have = -1;                               // expert whose scales sg / su hold
        PairHead cur = pair_head(rows, pt, pe, table, E, H, p0, p1);
        if (cur.live && in_row) load16w_mapH(cur.xr + k, q, xw);
        for (int p = p0; p < p1; ++p)
        {
            const PairHead nxt = pair_head(rows, pt, pe, table, E, H, p + 1, p1);
            if (cur.live)
            {
                if (cur.e != have)
                {
                    const __half* scales = (const __half*)cur.row[9];
                    if (in_row) { load16w_mapH(scales + k, q, sg); load16w_mapH(scales + 2 * H + 3 * I + k, q, su); }
                    have = cur.e;
                }
                float v[32];
                if (in_row) mul32w_mapH(xw, sg, v);
                else
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.f;
                wht128_x8(v, lane);
                if (kperm) store32h_mapH_kperm(xg + (size_t)p * H + k, q, v, in_row);
                else if (in_row) store32h_mapH(xg + (size_t)p * H + k, q, v);
                if (in_row) mul32w_mapH(xw, su, v);
                // the row is consumed: fetch the next pair's while the second half of this one is transformed
                if (nxt.live && in_row) load16w_mapH(nxt.xr + k, q, xw);
                wht128_x8(v, lane);
                if (kperm) store32h_mapH_kperm(xu + (size_t)p * H + k, q, v, in_row);
                else if (in_row) store32h_mapH(xu + (size_t)p * H + k, q, v);
            }
            else if (nxt.live && in_row) load16w_mapH(nxt.xr + k, q, xw);
            cur = nxt;
        }
    }
    // low-rank inputs z_gu = x V_gu^T: warp r of the CTA takes component r of every pair
    for (int p = p0; p < p1; ++p)
    {
        const PairHead hd = pair_head(rows, pt, pe, table, E, H, p, p1);
        if (!hd.live) continue;
        const LowRank L = low_rank_of(hd.row, hd.level);
        for (int r = warp; r < 4; r += nwarp)
        {
            float d = 0.f;
            if (r < L.rg)
            {
                for (int k = lane * 4; k < H; k += 128)
                {
                    float f[4], v[4];
                    load4h(hd.xr + k, f); load4h(L.lr + (size_t)r * H + k, v);
                    d += f[0] * v[0] + f[1] * v[1] + f[2] * v[2] + f[3] * v[3];
                }
                d = warp_sum(d);
            }
            if (lane == 0) zg[(size_t)p * 4 + r] = d;
        }
    }
}

// one CTA per pair, one warp per 1024 columns; dynamic shared memory: I floats (staging for the 512-wide rotation)
__global__ void __launch_bounds__(256, NQ_PF_EW_BLOCKS) pf_mid_kernel(const float* __restrict__ acc_g, const float* __restrict__ acc_u, const float* __restrict__ zg,
                                                     const int* __restrict__ pe, const int64_t* __restrict__ table, int E, __half* h, float* zd, int H, int I, int kperm)
{
    extern __shared__ float stage[];
    __shared__ float zpart[64][4];
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, ng = I / 128;
    if (pe[p] < 0 || pe[p] >= E) return;
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
    for (int g0 = warp * 8; g0 < ng; g0 += nwarp * 8)
    {
        const int grp = g0 + (lane >> 2), col = grp * 128, q = lane & 3;
        const bool live = grp < ng;
        float g[32], v[32];
#pragma unroll
        for (int up = 0; up < 2; ++up)
        {
            if (live) load32f_mapF((up ? acc_u : acc_g) + (size_t)p * I + col, q, v);
            else
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.f;
            wht128_x8(v, lane);
            if (live)
            {
                scale32h_mapF((up ? sv_u : sv_g) + col, q, v);
                for (int r = 0; r < L.rg; ++r)
                {
                    const size_t o = (size_t)(up * L.rg + r) * I + col;
                    axpy32h_mapF(L.lr + (size_t)L.rg * H + o, q, z[r], v);
                    if (L.lr4) axpy32h_mapF(L.lr4 + o, q, z[r], v);
                }
            }
            if (up == 0)
#pragma unroll
                for (int i = 0; i < 32; ++i) g[i] = v[i];
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = live ? silu(g[i]) * v[i] : 0.f;
        for (int r = 0; r < L.rd; ++r)
        {
            float d = 0.f;
            if (live) d = dot32h_mapF(L.lr + (size_t)L.rg * H + 2 * (size_t)L.rg * I + (size_t)r * I + col, q, v);
            d = quad_sum(d);
            if (live && (lane & 3) == 0) zpart[grp][r] = d;
        }
        if (live) scale32h_mapF(su_d + col, q, v);
        wht128_x8(v, lane);
        if (live)
        {
            if (hw <= 128) { if (kperm) store32h_mapF_kperm(h + (size_t)p * I + col, q, v); else store32h_mapF(h + (size_t)p * I + col, q, v); }
            else store32f_mapF(stage + col, q, v);
        }
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
        for (int blk = warp; blk < ng; blk += nwarp)
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
            if (kperm) store4h_kperm(h + (size_t)p * I + blk * 128, lane, o);
            else store4h(h + (size_t)p * I + blk * 128 + lane * 4, o);
        }
    }
}

// v = rw * (WHT128(y) * sv_o + z_dn (U2_d [+ U4_d])) for the lane's 32 output columns of the group at col of pair p (live lanes
// only load and scale; every lane takes part in the rotation); false if the pair adds nothing (warp-uniform)
__device__ __forceinline__ bool pair_output(const float* __restrict__ y, const float* __restrict__ zd, int p, int e, float w,
                                            const int64_t* __restrict__ table, int H, int I, int col, bool live, int lane, float (&v)[32])
// (col = first column of the lane's group, columns by map F)
{
    const int64_t* row = table + (int64_t)e * kTableWidth;
    const int level = (int)row[0];
    if (level <= 0 || w == 0.f) return false;
    const __half* sv_o = (const __half*)row[9] + H + 3 * I;
    const LowRank L = low_rank_of(row, level);
    const int q = lane & 3;
    if (live) load32f_mapF(y + (size_t)p * H + col, q, v);
    else
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
    wht128_x8(v, lane);
    if (live)
    {
        scale32h_mapF(sv_o + col, q, v);
        const size_t ou = (size_t)L.rg * H + 2 * (size_t)L.rg * I + (size_t)L.rd * I;
        for (int r = 0; r < L.rd; ++r)
        {
            const float z = zd[(size_t)p * 4 + r];
            axpy32h_mapF(L.lr + ou + (size_t)r * H + col, q, z, v);
            if (L.lr4) axpy32h_mapF(L.lr4 + 2 * (size_t)L.rg * I + (size_t)r * H + col, q, z, v);
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= w;
    }
    return true;
}

// one CTA per pair: atomic accumulation into out[token]
__global__ void __launch_bounds__(256, NQ_PF_EW_BLOCKS) pf_post_kernel(const float* __restrict__ y, const float* __restrict__ zd, const int* __restrict__ pt,
                                                      const int* __restrict__ pe, const __half* __restrict__ prw,
                                                      const int64_t* __restrict__ table, int E, float* out, int H, int I)
{
    const int p = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, ng = H / 128;
    if (pe[p] < 0 || pe[p] >= E) return;
    const float w = __half2float(prw[p]);
    float* op = out + (size_t)pt[p] * H;
    for (int g0 = warp * 8; g0 < ng; g0 += nwarp * 8)
    {
        float v[32];
        const int grp = g0 + (lane >> 2), col = grp * 128;
        const bool live = grp < ng;
        if (!pair_output(y, zd, p, pe[p], w, table, H, I, col, live, lane, v)) return;   // CTA-uniform
        if (live)
#pragma unroll
            for (int i = 0; i < 32; ++i) atomicAdd(op + col + 16 * (i >> 2) + 4 * (lane & 3) + (i & 3), v[i]);
    }
}

// one CTA per token: the token's picks whose pairs lie in [pair0, pair0 + npairs) are added in pick order.  pos[t * topk + k] =
// index of that pick in the expert-sorted pair list; y / zd hold the rows of that window only (row = index - pair0).
// accumulate = 0: out[t] is overwritten (zeros if the token has no pick in the window); 1: the sum is added to out[t], and
// tokens without a pick in the window are not touched.  Calling it window after window in a fixed order gives a bitwise
// repeatable result without a pairs-sized buffer.
__global__ void __launch_bounds__(256, NQ_PF_EW_BLOCKS) pf_combine_kernel(const float* __restrict__ y, const float* __restrict__ zd, const int* __restrict__ pos,
                                                         const int64_t* __restrict__ sel, const __half* __restrict__ rw,
                                                         const int64_t* __restrict__ table, float* out, int topk, int E, int H, int I,
                                                         int pair0, int npairs, int accumulate)
{
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, ng = H / 128;
    bool any = false;
    for (int k = 0; k < topk; ++k)
    {
        const int p = pos[(size_t)t * topk + k] - pair0;
        any = any || (p >= 0 && p < npairs);
    }
    if (accumulate && !any) return;      // CTA-uniform
    for (int g0 = warp * 8; g0 < ng; g0 += nwarp * 8)
    {
        const int grp = g0 + (lane >> 2), col = grp * 128;
        const bool live = grp < ng;
        float o[32];
        if (accumulate && live) load32f_mapF(out + (size_t)t * H + col, lane & 3, o);
        else
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
        for (int k = 0; k < topk; ++k)
        {
            const int64_t e = sel[(size_t)t * topk + k];
            const int p = pos[(size_t)t * topk + k] - pair0;
            if (e < 0 || e >= E || p < 0 || p >= npairs) continue;
            float v[32];
            if (!pair_output(y, zd, p, (int)e, __half2float(rw[(size_t)t * topk + k]), table, H, I, col, live, lane, v))
                continue;
            if (live)
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] += v[i];
        }
        if (live) store32f_mapF(out + (size_t)t * H + col, lane & 3, o);
    }
}

__global__ void pf_hits_kernel(const int* __restrict__ counts, int* hits, int E)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e < E && counts[e]) atomicAdd(hits + e, counts[e]);
}

// threads per CTA of the passes above: one warp per 1024 columns of the row, at most 8 warps
// CTAs of pf_pre: enough to fill the device a few times over, each with a run of consecutive pairs
static int pf_pre_grid(int R)
{
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int want = (sms > 0 ? sms : 148) * NQ_PF_PRE_BLOCKS * 4;
    return R < want ? R : want;
}
static int pf_threads(int cols) { const int w = (cols + 1023) / 1024; return 32 * (w > 8 ? 8 : w); }

}  // namespace nq

extern "C" {

#define NQ_SHAPE_OK(fn) NQ_REQUIRE(H > 0 && I > 0 && H % 128 == 0 && I % 128 == 0 && H / 128 <= 64 && I / 128 <= 64, fn ": H = %d, I = %d must be multiples of 128, at most 64 * 128", H, I)

int nq_pf_pre(const void* x, const int32_t* pt, const int32_t* pe, int R, const int64_t* table, int E, void* xg, void* xu, float* zg,
              int H, int I, int kperm, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_pre: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(x && pt && pe && table && xg && xu && zg, "nq_pf_pre: null pointer");
    NQ_SHAPE_OK("nq_pf_pre");
    NQ_REQUIRE(E >= 1, "nq_pf_pre: E = %d", E);
    NQ_REQUIRE(nq::aligned16(x) && nq::aligned16(xg) && nq::aligned16(xu), "nq_pf_pre: x, xg, xu must be 16-byte aligned");
    nq::TokenRows rows{};
    rows.base[0] = (const __half*)x; rows.tokens_per_rank = 0x7fffffff;
    nq::pf_pre_kernel<<<nq::pf_pre_grid(R), nq::pf_threads(H), 0, (cudaStream_t)stream>>>(rows, pt, pe, table, E, (__half*)xg, (__half*)xu, zg, H, I, kperm, R);
    return nq::check_launch("nq_pf_pre");
}

int nq_pf_pre_ep(const void* const* peer_x, int world, int tokens_per_rank, const int32_t* pt, const int32_t* pe, int R, const int64_t* table, int E,
                 void* xg, void* xu, float* zg, int H, int I, int kperm, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_pre_ep: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(peer_x && pt && pe && table && xg && xu && zg, "nq_pf_pre_ep: null pointer");
    NQ_REQUIRE(world >= 1 && world <= nq::kPfMaxRanks && tokens_per_rank >= 1, "nq_pf_pre_ep: world = %d, tokens per rank = %d", world, tokens_per_rank);
    NQ_SHAPE_OK("nq_pf_pre_ep");
    NQ_REQUIRE(E >= 1, "nq_pf_pre_ep: E = %d", E);
    NQ_REQUIRE(nq::aligned16(xg) && nq::aligned16(xu), "nq_pf_pre_ep: xg, xu must be 16-byte aligned");
    nq::TokenRows rows{};
    for (int r = 0; r < world; ++r)
    {
        NQ_REQUIRE(peer_x[r] && nq::aligned16(peer_x[r]), "nq_pf_pre_ep: input buffer of rank %d is null or misaligned", r);
        rows.base[r] = (const __half*)peer_x[r];
    }
    rows.tokens_per_rank = tokens_per_rank;
    nq::pf_pre_kernel<<<nq::pf_pre_grid(R), nq::pf_threads(H), 0, (cudaStream_t)stream>>>(rows, pt, pe, table, E, (__half*)xg, (__half*)xu, zg, H, I, kperm, R);
    return nq::check_launch("nq_pf_pre_ep");
}

int nq_pf_mid(const float* acc_g, const float* acc_u, const float* zg, const int32_t* pe, int R, const int64_t* table, int E, void* h,
              float* zd, int H, int I, int kperm, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_mid: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(acc_g && acc_u && zg && pe && table && h && zd, "nq_pf_mid: null pointer");
    NQ_SHAPE_OK("nq_pf_mid");
    NQ_REQUIRE(E >= 1, "nq_pf_mid: E = %d", E);
    NQ_REQUIRE(nq::aligned16(acc_g) && nq::aligned16(acc_u) && nq::aligned16(h), "nq_pf_mid: acc_g, acc_u, h must be 16-byte aligned");
    nq::pf_mid_kernel<<<R, nq::pf_threads(I), (size_t)I * 4, (cudaStream_t)stream>>>(acc_g, acc_u, zg, pe, table, E, (__half*)h, zd, H, I, kperm);
    return nq::check_launch("nq_pf_mid");
}

int nq_pf_post(const float* y, const float* zd, const int32_t* pt, const int32_t* pe, const void* prw, int R, const int64_t* table, int E,
               float* out, int H, int I, void* stream)
{
    NQ_REQUIRE(R >= 0, "nq_pf_post: R = %d", R);
    if (R == 0) return NQ_OK;
    NQ_REQUIRE(y && zd && pt && pe && prw && table && out, "nq_pf_post: null pointer");
    NQ_SHAPE_OK("nq_pf_post");
    NQ_REQUIRE(E >= 1, "nq_pf_post: E = %d", E);
    NQ_REQUIRE(nq::aligned16(y) && nq::aligned16(out), "nq_pf_post: y and out must be 16-byte aligned");
    nq::pf_post_kernel<<<R, nq::pf_threads(H), 0, (cudaStream_t)stream>>>(y, zd, pt, pe, (const __half*)prw, table, E, out, H, I);
    return nq::check_launch("nq_pf_post");
}

int nq_pf_combine(const float* y, const float* zd, const int32_t* pos, const int64_t* sel, const void* rw, int T, int topk,
                  const int64_t* table, int E, float* out, int H, int I, int pair0, int npairs, int accumulate, void* stream)
{
    NQ_REQUIRE(T >= 0 && topk >= 1 && E >= 1, "nq_pf_combine: T = %d, topk = %d, E = %d", T, topk, E);
    NQ_REQUIRE(pair0 >= 0 && npairs >= 0, "nq_pf_combine: pair window %d + %d", pair0, npairs);
    if (T == 0) return NQ_OK;
    NQ_REQUIRE(y && zd && pos && sel && rw && table && out, "nq_pf_combine: null pointer");
    NQ_SHAPE_OK("nq_pf_combine");
    NQ_REQUIRE(nq::aligned16(y) && nq::aligned16(out), "nq_pf_combine: y and out must be 16-byte aligned");
    nq::pf_combine_kernel<<<T, nq::pf_threads(H), 0, (cudaStream_t)stream>>>(y, zd, pos, sel, (const __half*)rw, table, out, topk, E, H, I, pair0, npairs, accumulate);
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
