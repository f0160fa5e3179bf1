// Decode path of the MoE layer (1..32 tokens): routing, input rotation, gate|up GEMV + SwiGLU, down GEMV + combine.
//
// Replaces moe_forward() of the reference (sm120/nqmoe.cu:858-907 and the kernels it launches, :375-824) with three
// launches on one stream, all reading routing, levels and plane pointers on the device (graph-capturable):
//   route_kernel   one CTA per pick: x * su -> WHT128 -> fp16 for the gate and the up half; one more CTA groups the picks
//                  into runs (one expert + the tokens that picked it), heaviest level first.
//   gemv_kernel<0> gate|up: persistent CTAs pull (run, 128-column group, gate/up, k-slice) items; each warp streams one
//                  16-row strip of packed planes from HBM, decodes it in registers and feeds mma.m16n8k16 with the
//                  run's tokens as N.  The last CTA to finish a (run, group) sums the k-slices in order and applies
//                  WHT128, sv, SwiGLU, su_d, WHT128 -> h (fp16).
//   gemv_kernel<1> down: same stream/decode/MMA; the last CTA of a 128-row output group combines
//                  out[b] = sum_k rw * sv_o * WHT128(y) over every token.
// Split-k partial sums go to separate buffers and are added in a fixed order, so results are bitwise repeatable
// (the reference accumulates with fp32 atomics and is not, sm120/check.py:21).
// HBM-bound by design (0.25 B per level-2 weight, ~0.52 B per level-4 weight); in practice the integer decode
// issue rate bounds it.
#include "nq_common.cuh"
#include "nq_rotate.cuh"
#include "nq_stream.cuh"
#include "nq_unit.cuh"

namespace nq {

// residual window codes built into the decode-path kernels (bit c = code c; code 0 always)
#ifndef NQ_GEMV_CODES
#define NQ_GEMV_CODES 0x3FF
#endif
// stages of the plane ring per warp, and resident CTAs per SM the kernels are compiled for (4 x 8 warps at 64 registers and 4
// stages measured 2 % faster than 3 x 8 warps at 80 registers and 6 stages)
#ifndef NQ_GEMV_DEPTH
#define NQ_GEMV_DEPTH 4
#endif
#ifndef NQ_GEMV_MINBLOCKS
#define NQ_GEMV_MINBLOCKS 4
#endif
constexpr int kDepth = NQ_GEMV_DEPTH;
constexpr int kRunTokens = 8;   // tokens per run = N of one mma.m16n8k16; an expert picked by more tokens gets several runs
struct Run
{
    int expert, level, ntok, pad;
    int slot[kRunTokens];   // pick index b * topk + k of each token of the run, in pick order
};
constexpr int kRunInts = sizeof(Run) / 4;
constexpr int kRouteHdrInts = 4;   // [0] number of runs

struct MoeArgs
{
    const __half* x; const int64_t* sel; const __half* rw;
    int B, topk, E, H, I, nm_gu, nm_dn, force_level, ks_gu, ks_dn;
    const int64_t* table;
    int* route;        // header + Run[B * topk]
    __half* xrot;      // [S][2][H] rotated inputs (gate scale, up scale)
    float* part_gu;    // [ks_gu][S][2I]
    __half* h;         // [S][I]
    float* part_d;     // [ks_dn][S][H]
    int* cnt_gu;       // [2 * S * I/128] arrival counters ((run, group), then (run, 512-block)), zero on entry and exit
    int* cnt_d;        // [H/128]
    int* wq;           // [4] work / exit counters, zero on entry and exit
    float* zd;         // [S][I/128][4] down low-rank partials (gate|up kernel writes, down kernel reads)
    float* out;        // [B][H]
    int* hits;         // optional [E] pick counters (may be host-mapped)
};

__device__ __forceinline__ bool pick_valid(const MoeArgs& a, int s, int* expert, int* level)
{
    const int64_t e = a.sel[s];
    if (e < 0 || e >= a.E || __half2float(a.rw[s]) == 0.f) return false;
    int lv = (int)a.table[e * kTableWidth];
    if (lv <= 0) return false;
    if (a.force_level > 0) lv = a.force_level;
    *expert = (int)e; *level = lv;
    return true;
}

// ---------------------------------------------------------------- routing + input rotation
// grid = B * topk CTAs of 256 threads
// Programmatic dependent launch: a kernel lets its successor in the stream start launching early (launch_dependents)
// and the successor blocks (grid_dependency_wait) until the whole predecessor grid has completed and its writes are
// visible, before it touches anything.  This hides the launch latency between the three kernels of a layer call.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__global__ void __launch_bounds__(256) route_kernel(MoeArgs a)
{
    launch_dependents();
    const int S = a.B * a.topk, s = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int e = 0, lv = 0;
    const bool ok = s < S && pick_valid(a, s, &e, &lv);
    if (a.hits && threadIdx.x == 0 && s < S)
    {
        const int64_t es = a.sel[s];
        if (es >= 0 && es < a.E && __half2float(a.rw[s]) != 0.f) atomicAdd(a.hits + es, 1);   // every pick with a weight, any level
    }
    if (ok)
    {
        const __half* scales = (const __half*)a.table[(int64_t)e * kTableWidth + 9];
        const __half* xr = a.x + (size_t)(s / a.topk) * a.H;
        const int ng = a.H / 128;
        for (int task = warp; task < 2 * ng; task += 8)
        {
            const int up = task / ng, k = (task - up * ng) * 128 + lane * 4;
            const __half* su = up ? scales + 2 * a.H + 3 * a.I : scales;
            float f[4], g[4];
            load4h(xr + k, f); load4h(su + k, g);
            float v[4] = {f[0] * g[0], f[1] * g[1], f[2] * g[2], f[3] * g[3]};
            wht128(v, lane);
            store4h(a.xrot + ((size_t)s * 2 + up) * a.H + k, v);
        }
    }
    if (s != S) return;

    // The extra CTA (it rotates nothing, so it runs beside the others): group the picks into runs.  A run = one expert and up to 8 of its picks in pick order; runs are numbered
    // by first pick, then ordered level 4 before level 2 (heavier items are handed out first).
    __shared__ int s_exp[NQ_MAX_PICKS], s_lvl[NQ_MAX_PICKS], s_pos[NQ_MAX_PICKS], s_cnt[NQ_MAX_PICKS], s_lead[NQ_MAX_PICKS];
    __shared__ int s_ord[NQ_MAX_PICKS], s_rank[NQ_MAX_PICKS], s_warp[8], s_nruns;
    const int t = threadIdx.x;
    int te = -1, tl = 0;
    const bool tv = t < S && pick_valid(a, t, &te, &tl);
    s_exp[t] = tv ? te : -1 - t; s_lvl[t] = tl;
    __syncthreads();
    int pos = 0, cnt = 0;
    if (tv)
        for (int q = 0; q < S; ++q)
            if (s_exp[q] == te) { ++cnt; if (q < t) ++pos; }
    s_pos[t] = pos; s_cnt[t] = cnt;
    const bool lead = tv && (pos % kRunTokens) == 0;
    const unsigned bal = __ballot_sync(0xffffffffu, lead);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = __popc(bal & ((1u << lane) - 1u));
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (t == 0) { int n = 0; for (int w = 0; w < 8; ++w) n += s_warp[w]; s_nruns = n; }
    s_lead[t] = lead ? before : -1;        // run ordinal (by first pick) of leaders
    __syncthreads();
    const int nruns = s_nruns;
    if (lead) { s_ord[before] = t; }
    __syncthreads();
    // rank of run ordinal `t` after the stable sort by level (descending)
    if (t < nruns)
    {
        const int me = s_lvl[s_ord[t]];
        int rk = 0;
        for (int q = 0; q < nruns; ++q)
        {
            const int other = s_lvl[s_ord[q]];
            rk += (other > me) || (other == me && q < t);
        }
        s_rank[t] = rk;
    }
    __syncthreads();
    Run* runs = (Run*)(a.route + kRouteHdrInts);
    if (tv)
    {
        // leader of my run: the pick of my expert at position pos - pos % 8
        int lead_pick = t;
        const int want = pos - pos % kRunTokens;
        if (want != pos)
        {
            int seen = 0;
            for (int q = 0; q < S; ++q)
                if (s_exp[q] == te) { if (seen == want) { lead_pick = q; break; } ++seen; }
        }
        Run* r = runs + s_rank[s_lead[lead_pick]];
        r->slot[pos % kRunTokens] = t;
        if (lead)
        {
            r->expert = te; r->level = tl; r->pad = 0;
            const int left = cnt - pos;
            r->ntok = left < kRunTokens ? left : kRunTokens;
        }
    }
    if (t == 0) { a.route[0] = nruns; a.route[1] = a.route[2] = a.route[3] = 0; }
    if (nruns == 0)   // nothing resident was picked: the layer output is defined as zero
        for (int i = t; i < a.B * a.H; i += 256) a.out[i] = 0.f;
}

// ---------------------------------------------------------------- GEMV
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// tokens of the run as the N operand: lane (g, t4) supplies k = 16 t + 2 t4 (+8) of token 8 nt + g.
// xoff[nt]: element offset of that token's row from `xbase`, or -1 when the tile has no such token.
template <int NT>
struct TokenSink
{
    float (&acc)[NT][4];
    const __half* xbase;
    const int (&xoff)[NT];
    int kbase;   // 128 * chunk + 2 * t4
    template <int T>
    __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const
    {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
        {
            uint32_t b0 = 0, b1 = 0;
            if (xoff[nt] >= 0)
            {
                const __half* p = xbase + (size_t)xoff[nt] + kbase + T * 16;
                b0 = __ldg((const uint32_t*)p); b1 = __ldg((const uint32_t*)(p + 8));
            }
            mma_16816(acc[nt], a, b0, b1);
        }
    }
};

// One warp, one strip, chunks [c0, c1) (at most 64): stream, decode, multiply.  REFINED: the expert is at level 4.
// ring: this warp's kDepth stages.
template <bool REFINED, int RC, int NT, int BK = 0>
__device__ __forceinline__ void strip_gemv(const ProjPlanes& P, int strip, int C, int NS, int nm, int c0, int c1, int lane,
                                           float (&acc)[NT][4], const __half* xbase, const int (&xoff)[NT], uint8_t* ring)
{
    const size_t base_nrec = (size_t)NS * C * 32;
    unsigned long long fl = ~0ull;
    if (REFINED && P.flags) fl = __ldg((const unsigned long long*)P.flags + strip);
    const size_t res_nrec = (size_t)NS * (P.flags ? nm : C) * 32;
    const size_t unit0 = (size_t)strip * C;
    // refined-unit index of chunk ch
    auto res_unit = [&](int ch) -> size_t {
        return P.flags ? (size_t)strip * nm + __popcll(fl & ((1ull << ch) - 1ull)) : unit0 + ch;
    };
    // per-unit scalars of the whole chunk range, one chunk per lane (two rounds cover 64 chunks): ring signs, block words
    uint32_t var_lo = 0, var_hi = 0, dl_lo = 0, dl_hi = 0;
    {
        const int ca = c0 + lane, cb = c0 + 32 + lane;
        if (P.var) { if (ca < c1) var_lo = __ldg(P.var + unit0 + ca); if (cb < c1) var_hi = __ldg(P.var + unit0 + cb); }
        if constexpr (REFINED)
        {
            if (ca < c1 && ((fl >> ca) & 1ull)) dl_lo = __ldg(P.d4 + res_unit(ca));
            if (cb < c1 && ((fl >> cb) & 1ull)) dl_hi = __ldg(P.d4 + res_unit(cb));
        }
    }
    auto issue = [&](int ch, uint8_t* st) {
        copy_base<BK>(st, P.base, (unit0 + ch) * 32 + lane, base_nrec, lane);
        if constexpr (REFINED)
            if ((fl >> ch) & 1ull) copy_record<RC>(st + 512, P.p4, res_unit(ch) * 32 + lane, res_nrec, lane);
    };
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d)
    {
        if (c0 + d < c1) issue(c0 + d, ring + d * kStageBytes);
        cp_async_commit();
    }
    int slot = 0, slot_in = kDepth - 1;
    for (int ch = c0; ch < c1; ++ch)
    {
        if (ch + kDepth - 1 < c1) issue(ch + kDepth - 1, ring + slot_in * kStageBytes);
        cp_async_commit();
        cp_async_wait<kDepth - 1>();
        const uint8_t* st = ring + slot * kStageBytes;
        slot = slot + 1 == kDepth ? 0 : slot + 1;
        slot_in = slot_in + 1 == kDepth ? 0 : slot_in + 1;
        const int rel = ch - c0;
        const uint32_t vb = __shfl_sync(0xffffffffu, rel < 32 ? var_lo : var_hi, rel & 31);
        const uint32_t sign2 = ((vb >> (lane >> 2)) & 1u) * 0x80008000u;
        uint32_t wb[Pattern<BK>::kWords + 2];
        read_base<BK>(wb, st, (unit0 + ch) * 32 + lane, lane);
        const TokenSink<NT> sink{acc, xbase, xoff, ch * 128 + (lane & 3) * 2};
        bool refined = false;
        if constexpr (REFINED) refined = (fl >> ch) & 1ull;
        if (refined)
        {
            const uint32_t dl = __shfl_sync(0xffffffffu, rel < 32 ? dl_lo : dl_hi, rel & 31);
            uint32_t wr[Pattern<RC>::kWords + 2];
            read_record<RC>(wr, st + 512, res_unit(ch) * 32 + lane, lane);
            decode_words<true, RC, BK>(wb, wr, consts_level4(dl, sign2), lane, sink);
        }
        else
            decode_words<false, 0, BK>(wb, nullptr, consts_level2(sign2), lane, sink);
    }
    cp_async_wait<0>();
}

// one warp's share of an item: its strip over chunks [c0, c1) for the run's tokens, then the partial sums
// part[ks][slot][row] of this k-slice
template <int DOWN, int NT>
__device__ __forceinline__ void item_gemv(const MoeArgs& a, const Run& run, const ProjPlanes& P, int level, int rc, int bk, int nm,
                                          int strip, int C, int NS, int c0, int c1, int up, int ks, float* part, int N, int S,
                                          uint8_t* ring)
{
    const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3, ntok = run.ntok;
    const __half* xbase = DOWN ? a.h : a.xrot + (size_t)up * a.H;
    int xoff[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
    {
        const int j = nt * 8 + g;
        xoff[nt] = j < ntok ? run.slot[j] * (DOWN ? a.I : 2 * a.H) : -1;   // at most 256 * 2 * 8192 elements
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
#define NQ_LOOP(REF, RCV) strip_gemv<REF, RCV, NT>(P, strip, C, NS, nm, c0, c1, lane, acc, xbase, xoff, ring)
#define NQ_LOOP1(REF, RCV) strip_gemv<REF, RCV, NT, 1>(P, strip, C, NS, nm, c0, c1, lane, acc, xbase, xoff, ring)
    if (bk == 1)        // 112-bit base records, with the residual codes they ship with
    {
        if (level < 4) NQ_LOOP1(false, 0);
        else if (rc == 9) NQ_LOOP1(true, 9);
        else NQ_LOOP1(true, 3);
    }
    else if (level < 4) NQ_LOOP(false, 0);
    else switch (rc)
    {
#define NQ_CASE(c) case c: if constexpr ((NQ_GEMV_CODES >> c) & 1) { NQ_LOOP(true, c); } break;
        NQ_CASE(1) NQ_CASE(2) NQ_CASE(3) NQ_CASE(4) NQ_CASE(5) NQ_CASE(6) NQ_CASE(7) NQ_CASE(8) NQ_CASE(9)
#undef NQ_CASE
        default: NQ_LOOP(true, 0); break;
    }
#undef NQ_LOOP
#undef NQ_LOOP1
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const int j = nt * 8 + t4 * 2 + (i & 1), rr = strip * 16 + g + (i >> 1) * 8;
            if (j < ntok) __stcg(part + ((size_t)ks * S + run.slot[j]) * N + rr, acc[nt][i]);
        }
}

// DOWN = 0: gate|up (N = 2I, K = H), DOWN = 1: down (N = H, K = I).  Persistent CTAs of 8 warps.
template <int DOWN>
__global__ void __launch_bounds__(256, NQ_GEMV_MINBLOCKS) gemv_kernel(MoeArgs a)
{
    extern __shared__ __align__(16) uint8_t smem_ring[];   // [8 warps][kDepth][kStageBytes]
    __shared__ Run run;
    __shared__ int s_item, s_last;
    launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int S = a.B * a.topk;
    const int N = DOWN ? a.H : 2 * a.I, K = DOWN ? a.I : a.H, C = K / 128, NS = N / 16;
    const int KS = DOWN ? a.ks_dn : a.ks_gu, groups = (DOWN ? a.H : a.I) / 128, parts = DOWN ? KS : 2 * KS;
    const int nruns = a.route[0], per_run = groups * parts, total = nruns * per_run;
    const Run* runs = (const Run*)(a.route + kRouteHdrInts);
    int* wq = a.wq + 2 * DOWN;
    float* part = DOWN ? a.part_d : a.part_gu;

    for (;;)
    {
        __syncthreads();
        if (threadIdx.x == 0) s_item = atomicAdd(wq, 1);
        __syncthreads();
        const int item = s_item;
        if (item >= total) break;
        const int r = item / per_run, rem = item - r * per_run, grp = rem / parts, pt = rem - grp * parts;
        const int up = DOWN ? 0 : pt / KS, ks = pt - up * KS;
        if (threadIdx.x < kRunInts) ((int*)&run)[threadIdx.x] = ((const int*)(runs + r))[threadIdx.x];
        __syncthreads();
        const int ntok = run.ntok, level = run.level;
        const int64_t* row = a.table + (int64_t)run.expert * kTableWidth;
        const ProjPlanes P = planes_from_row(row, DOWN);
        const int rc = (int)row[10 + DOWN], nm = DOWN ? a.nm_dn : a.nm_gu, bk = (int)(row[19] >> (8 * DOWN)) & 0xFF;
        const int row0 = DOWN ? grp * 128 : up * a.I + grp * 128, strip = row0 / 16 + warp;
        const int c0 = ks * (C / KS), c1 = c0 + C / KS;

        item_gemv<DOWN, 1>(a, run, P, level, rc, bk, nm, strip, C, NS, c0, c1, up, ks, part, N, S, smem_ring + warp * (kDepth * kStageBytes));
        int* cnt = DOWN ? a.cnt_d + grp : a.cnt_gu + r * (a.I / 128) + grp;
        const int expect = DOWN ? nruns * KS : 2 * KS;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0)
        {
            int prev;
            asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(cnt) : "memory");
            s_last = prev == expect - 1;
            if (s_last) *cnt = 0;
        }
        __syncthreads();
        if (!s_last) continue;
        __threadfence();

        if constexpr (DOWN == 0)
        {
            // (run, group) complete: WHT128, sv, (+ low rank), SwiGLU, su_d, WHT128 -> h.  One warp per token.
            const __half* scales = (const __half*)row[9];
            const __half *sv_g = scales + a.H, *sv_u = sv_g + a.I, *su_d = sv_u + a.I;
            const __half* lr = (const __half*)row[14];
            const int rg = lr ? (int)row[16] : 0, rd = lr ? (int)row[17] : 0, hw = (int)row[18];
            const __half* lr4 = level == 4 ? (const __half*)row[15] : nullptr;
            const int col = grp * 128 + lane * 4, ng = a.I / 128;
            for (int j = warp; j < ntok; j += 8)
            {
                const int slot = run.slot[j];
                float z[4] = {0.f, 0.f, 0.f, 0.f};
                for (int r = 0; r < rg; ++r)          // z = x V_gu^T on the unrotated input
                {
                    const __half* xr = a.x + (size_t)(slot / a.topk) * a.H;
                    float d = 0.f;
                    for (int k = lane * 4; k < a.H; k += 128)
                    {
                        float f[4], w[4];
                        load4h(xr + k, f); load4h(lr + (size_t)r * a.H + k, w);
                        d += f[0] * w[0] + f[1] * w[1] + f[2] * w[2] + f[3] * w[3];
                    }
#pragma unroll
                    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                    z[r] = d;
                }
                float gu[2][4];
#pragma unroll
                for (int u = 0; u < 2; ++u)
                {
                    float v[4] = {0.f, 0.f, 0.f, 0.f}, sc[4];
                    for (int q = 0; q < KS; ++q)
                    {
                        const float4 f = __ldcg((const float4*)(a.part_gu + ((size_t)q * S + slot) * N + u * a.I + col));
                        v[0] += f.x; v[1] += f.y; v[2] += f.z; v[3] += f.w;
                    }
                    wht128(v, lane);
                    load4h((u ? sv_u : sv_g) + col, sc);
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] *= sc[i];
                    for (int r = 0; r < rg; ++r)
                    {
                        float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
                        const size_t o = (size_t)(u * rg + r) * a.I + col;
                        load4h(lr + (size_t)rg * a.H + o, u2);
                        if (lr4) load4h(lr4 + o, u4);
#pragma unroll
                        for (int i = 0; i < 4; ++i) v[i] += z[r] * u2[i] + z[r] * u4[i];
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) gu[u][i] = v[i];
                }
                float v[4], sc[4];
                load4h(su_d + col, sc);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = silu(gu[0][i]) * gu[1][i];
                for (int r = 0; r < rd; ++r)          // this group's share of z_dn = sw V_dn^T
                {
                    float w[4];
                    load4h(lr + (size_t)rg * a.H + 2 * (size_t)rg * a.I + (size_t)r * a.I + col, w);
                    float d = v[0] * w[0] + v[1] * w[1] + v[2] * w[2] + v[3] * w[3];
#pragma unroll
                    for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                    if (lane == 0) a.zd[((size_t)slot * ng + grp) * 4 + r] = d;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] *= sc[i];
                wht128(v, lane);
                if (hw <= 128) store4h(a.h + (size_t)slot * a.I + col, v);
                else __stcg((float4*)(a.part_gu + (size_t)slot * N + col), make_float4(v[0], v[1], v[2], v[3]));   // fp32 stage: gate columns, k-slice 0
            }
            if (hw > 128)
            {
                // 512-wide rotation = H_4 (x) WHT128 / 2: the last of the hw/128 groups of a block combines their fp32 results
                const int nb = hw / 128, b0 = grp / nb * nb;
                __threadfence();
                __syncthreads();
                if (threadIdx.x == 0)
                {
                    int prev;
                    int* ch = a.cnt_gu + S * ng + r * ng + b0;
                    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(prev) : "l"(ch) : "memory");
                    s_last = prev == nb - 1;
                    if (s_last) *ch = 0;
                }
                __syncthreads();
                if (s_last)
                {
                    __threadfence();
                    const float rs = rsqrtf((float)nb);
                    for (int task = warp; task < ntok * nb; task += 8)
                    {
                        const int j = task / nb, ob = task - j * nb, slot = run.slot[j];
                        const float* p = a.part_gu + (size_t)slot * N + b0 * 128 + lane * 4;
                        float o[4] = {0.f, 0.f, 0.f, 0.f};
                        for (int b = 0; b < nb; ++b)
                        {
                            const float4 f = __ldcg((const float4*)(p + b * 128));
                            const float sg = (__popc(ob & b) & 1) ? -1.f : 1.f;
                            o[0] += sg * f.x; o[1] += sg * f.y; o[2] += sg * f.z; o[3] += sg * f.w;
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) o[i] *= rs;
                        store4h(a.h + (size_t)slot * a.I + (b0 + ob) * 128 + lane * 4, o);
                    }
                }
            }
        }
        else
        {
            // output rows [grp * 128, +128) complete for every run: weighted combine over each token's picks
            const int col = grp * 128 + lane * 4;
            for (int b = warp; b < a.B; b += 8)
            {
                float o[4] = {0.f, 0.f, 0.f, 0.f};
                for (int k = 0; k < a.topk; ++k)
                {
                    const int s = b * a.topk + k;
                    int e, lv;
                    if (!pick_valid(a, s, &e, &lv)) continue;
                    const float w = __half2float(a.rw[s]);
                    const __half* sv_o = (const __half*)a.table[(int64_t)e * kTableWidth + 9] + a.H + 3 * a.I;
                    float v[4] = {0.f, 0.f, 0.f, 0.f}, sc[4];
                    for (int q = 0; q < KS; ++q)
                    {
                        const float4 f = __ldcg((const float4*)(a.part_d + ((size_t)q * S + s) * N + col));
                        v[0] += f.x; v[1] += f.y; v[2] += f.z; v[3] += f.w;
                    }
                    wht128(v, lane);
                    load4h(sv_o + col, sc);
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] *= sc[i];
                    const int64_t* erow = a.table + (int64_t)e * kTableWidth;
                    const __half* lr = (const __half*)erow[14];
                    const int rd = lr ? (int)erow[17] : 0;
                    if (rd)
                    {
                        const int rg = (int)erow[16], ng = a.I / 128;
                        const __half* lr4 = lv == 4 ? (const __half*)erow[15] : nullptr;
                        const size_t ou = (size_t)rg * a.H + 2 * (size_t)rg * a.I + (size_t)rd * a.I;
                        for (int r = 0; r < rd; ++r)
                        {
                            float z = 0.f;
                            for (int gq = 0; gq < ng; ++gq) z += __ldcg(a.zd + ((size_t)s * ng + gq) * 4 + r);
                            float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
                            load4h(lr + ou + (size_t)r * a.H + col, u2);
                            if (lr4) load4h(lr4 + 2 * (size_t)rg * a.I + (size_t)r * a.H + col, u4);
#pragma unroll
                            for (int i = 0; i < 4; ++i) v[i] += z * u2[i] + z * u4[i];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] += w * v[i];
                }
                *(float4*)(a.out + (size_t)b * a.H + col) = make_float4(o[0], o[1], o[2], o[3]);
            }
        }
    }
    // the last CTA to leave resets the work counters (graph replays start from zero)
    if (threadIdx.x == 0)
    {
        __threadfence();
        if (atomicAdd(wq + 1, 1) == (int)gridDim.x - 1) { wq[0] = 0; wq[1] = 0; __threadfence(); }
    }
}

constexpr int kGemvSmem = 8 * kDepth * kStageBytes;

// CTAs that fit on the device at once (the kernels are persistent); also opts the kernel into its shared memory
static int resident_ctas(const void* fn, int threads)
{
    int dev = 0, sms = 0, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmem) != cudaSuccess) return 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, fn, threads, kGemvSmem);
    return sms * (per > 0 ? per : 1);
}

// launch gemv_kernel<DOWN> as a programmatic dependent of the kernel before it in the stream
template <int DOWN>
static int launch_after(int ctas, cudaStream_t st, const MoeArgs& a)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = kGemvSmem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_kernel<DOWN>, a);
    if (e != cudaSuccess) return fail(NQ_ERR_CUDA, "nq_moe_forward(%s): %s", DOWN ? "down" : "gate|up", cudaGetErrorString(e));
    return check_launch(DOWN ? "nq_moe_forward(down)" : "nq_moe_forward(gate|up)");
}

}  // namespace nq

extern "C" {

int nq_moe_workspace(int B, int topk, int H, int I, int ks_gu, int ks_dn, NqMoeWorkspace* w)
{
    NQ_REQUIRE(w, "nq_moe_workspace: null output");
    NQ_REQUIRE(B >= 1 && B <= NQ_MAX_TOKENS && topk >= 1 && B * topk <= NQ_MAX_PICKS, "nq_moe_workspace: B = %d, topk = %d", B, topk);
    NQ_REQUIRE(H > 0 && I > 0 && H % 128 == 0 && I % 128 == 0 && H / 128 <= 64 && I / 128 <= 64, "nq_moe_workspace: H = %d, I = %d", H, I);
    NQ_REQUIRE(ks_gu >= 1 && (H / 128) % ks_gu == 0 && ks_dn >= 1 && (I / 128) % ks_dn == 0, "nq_moe_workspace: k-splits %d / %d must divide %d / %d chunks", ks_gu, ks_dn, H / 128, I / 128);
    const size_t S = (size_t)B * topk;
    w->acc_gu_floats = (size_t)ks_gu * S * 2 * I;
    w->h_halves = S * I + S * 2 * H;                    // h [S][I], then the rotated inputs [S][2][H]
    w->acc_d_floats = (size_t)ks_dn * S * H;
    w->cnt_gu_ints = 2 * S * (I / 128);
    w->cnt_d_ints = H / 128;
    w->wq_ints = 4;
    w->zd_floats = S * (I / 128) * 4;
    w->cnt_h_ints = nq::kRouteHdrInts + S * nq::kRunInts;   // holds the run list
    return NQ_OK;
}

int nq_moe_forward(const NqMoeForward* p, void* stream)
{
    NQ_REQUIRE(p, "nq_moe_forward: null arguments");
    NQ_REQUIRE(p->G == 4, "nq_moe_forward: ring width G = %d (only 4 is built)", p->G);
    NqMoeWorkspace need;
    const int rc = nq_moe_workspace(p->B, p->topk, p->H, p->I, p->ks_gu, p->ks_dn, &need);
    if (rc) return rc;
    NQ_REQUIRE(p->x && p->sel && p->rw && p->table && p->out && p->acc_gu && p->h && p->acc_d && p->cnt_gu && p->cnt_d && p->wq && p->cnt_h && p->zd,
               "nq_moe_forward: null tensor");
    NQ_REQUIRE(p->E > 0, "nq_moe_forward: E = %d", p->E);
    NQ_REQUIRE(p->acc_gu_floats >= need.acc_gu_floats && p->h_halves >= need.h_halves && p->acc_d_floats >= need.acc_d_floats &&
               p->cnt_gu_ints >= need.cnt_gu_ints && p->cnt_d_ints >= need.cnt_d_ints && p->wq_ints >= need.wq_ints && p->cnt_h_ints >= need.cnt_h_ints &&
               p->zd_floats >= need.zd_floats,
               "nq_moe_forward: workspace too small (see nq_moe_workspace)");
    NQ_REQUIRE(p->out_floats >= (size_t)p->B * p->H, "nq_moe_forward: out too small");
    NQ_REQUIRE(nq::aligned16(p->x) && nq::aligned16(p->out) && nq::aligned16(p->acc_gu) && nq::aligned16(p->acc_d) && nq::aligned16(p->h),
               "nq_moe_forward: x, out and workspaces must be 16-byte aligned");
    NQ_REQUIRE(p->force_level == 0 || p->force_level == 2 || p->force_level == 4, "nq_moe_forward: force_level = %d", p->force_level);
    nq::MoeArgs a{};
    a.x = (const __half*)p->x; a.sel = p->sel; a.rw = (const __half*)p->rw;
    a.B = p->B; a.topk = p->topk; a.E = p->E; a.H = p->H; a.I = p->I; a.nm_gu = p->nm_gu; a.nm_dn = p->nm_dn;
    a.force_level = p->force_level; a.ks_gu = p->ks_gu; a.ks_dn = p->ks_dn; a.table = p->table;
    a.route = p->cnt_h; a.h = (__half*)p->h; a.xrot = a.h + (size_t)p->B * p->topk * p->I;
    a.part_gu = p->acc_gu; a.part_d = p->acc_d; a.zd = p->zd; a.cnt_gu = p->cnt_gu; a.cnt_d = p->cnt_d; a.wq = p->wq; a.out = p->out; a.hits = p->hits;
    cudaStream_t st = (cudaStream_t)stream;
    const int S = p->B * p->topk;
    nq::route_kernel<<<S + 1, 256, 0, st>>>(a);
    if (int e = nq::check_launch("nq_moe_forward(route)")) return e;
    if (p->which & 1)
    {
        static int ctas = nq::resident_ctas((const void*)nq::gemv_kernel<0>, 256);
        if (ctas <= 0) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward: cannot reserve %d bytes of shared memory", nq::kGemvSmem);
        if (int e = nq::launch_after<0>(ctas, st, a)) return e;
    }
    if (p->which & 2)
    {
        static int ctas = nq::resident_ctas((const void*)nq::gemv_kernel<1>, 256);
        if (ctas <= 0) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward: cannot reserve %d bytes of shared memory", nq::kGemvSmem);
        if (int e = nq::launch_after<1>(ctas, st, a)) return e;
    }
    return NQ_OK;
}

}  // extern "C"
