// Decode path of the MoE layer (1..32 tokens): routing, input rotation, gate|up GEMV + SwiGLU, down GEMV + combine, in
// ONE persistent launch whose warps pull work pieces from a queue.
//
// Replaces moe_forward() of the reference (sm120/nqmoe.cu:858-907 and the kernels it launches, :375-824).  Every routing,
// level and pointer decision is read on the device (graph-capturable).
//
//   route      every CTA groups the picks into runs (one expert + the tokens that picked it, level 4 first) in its own
//              shared memory: no CTA waits for another one's routing.
//   pieces     the queue holds, in this order,
//                rotation pieces   (pick, 4 blocks of 128): x * su -> WHT128 -> fp16 for the gate and the up scale, stored in
//                                  the k order the GEMV lanes read (see "operand order");
//                gate|up pieces    (run, 16-row strip, k-slice): one warp streams the strip's packed planes from HBM through
//                                  its cp.async ring, decodes them in registers and feeds mma.m16n8k16 with the run's tokens
//                                  as N; the last warp to finish a (run, 128-column group) sums the k-slices in a fixed
//                                  order and applies WHT128, sv, SwiGLU, su_d, WHT128 -> h (fp16);
//                down pieces       the same stream / decode / MMA over h; the last warp to finish a (token, 128-row group)
//                                  combines out[b] = sum_k rw * sv_o * WHT128(y).
//              A warp is the unit of scheduling (no CTA-wide barrier inside the loop), so the tail of the launch is at
//              most one piece per warp.  Pieces are handed out heaviest first.
//   waits      gate|up pieces need the rotated inputs (one global counter), down pieces need h of their run (one counter
//              per run).  A piece is claimed only after every piece it depends on has been claimed by a warp that is
//              already running and waits for nothing that comes later in the queue, so the waits cannot deadlock; they are
//              bounded all the same (2 s, then status[0] = 1 and the launch drains).
//   operand order   inside a 128-wide chunk the fp16 element k = 16 T + 2 t4 + 8 hi + e sits at position 32 t4 + 4 T + 2 hi + e,
//              so lane (g, t4) finds the B fragments of all 8 k-steps of a unit in 64 contiguous bytes.
// Split-k partial sums go to separate buffers and are added in a fixed order, so results are bitwise repeatable
// (the reference accumulates with fp32 atomics and is not, sm120/check.py:21).
// HBM-bound by design (0.25 B per level-2 weight, ~0.52 B per level-4 weight); in practice the integer decode
// issue rate bounds it.
#include "nq_common.cuh"
#include "nq_rotate.cuh"
#include "nq_unit.cuh"

namespace nq {

// residual window codes built into the decode-path kernel (bit c = code c; code 0 always)
#ifndef NQ_GEMV_CODES
#define NQ_GEMV_CODES 0x3FF
#endif
#ifndef NQ_GEMV_DEPTH
#define NQ_GEMV_DEPTH 3          // stages of the plane ring per warp
#endif
#ifndef NQ_GEMV_WARPS
#define NQ_GEMV_WARPS 10         // warps per CTA (independent of one another; the first 8 also build the run list)
#endif
#ifndef NQ_GEMV_MINBLOCKS
#define NQ_GEMV_MINBLOCKS 2      // resident CTAs per SM the kernel is compiled for: 20 warps per SM at <= 96 registers
#endif
constexpr int kDepth = NQ_GEMV_DEPTH;
constexpr int kWarps = NQ_GEMV_WARPS, kThreads = 32 * kWarps;
static_assert(kThreads >= NQ_MAX_PICKS, "the run list is built by one thread per pick");
constexpr int kRunTiles = 4;     // column tiles (8 tokens each) of mma.m16n8k16 per run
constexpr int kRunTokens = 8 * kRunTiles;
constexpr unsigned long long kWaitNs = 2000000000ull;
constexpr int kEpRanks = 8, kEpTokens = NQ_MAX_TOKENS, kEpGroups = 64;   // limits of the in-kernel all-reduce

struct RunRec { int expert, level, first, count; };   // picks of the run: order[first .. first + count)

struct MoeArgs
{
    const __half* x; const int64_t* sel; const __half* rw;
    int B, topk, E, H, I, nm_gu, nm_dn, force_level, ks_gu, ks_dn, which;
    const int64_t* table;
    int* status;       // [0] != 0: a device-side wait ran out
    __half* xrot;      // [S][2][H] rotated inputs (gate scale, up scale), operand order
    float* part_gu;    // [ks_gu][S][2I]
    __half* h;         // [S][I], operand order
    float* part_d;     // [ks_dn][S][H]
    int* cnt_gu;       // [S * I/128] (run, group) arrivals, [S * I/128] (run, 512-block) arrivals, [S] finished groups per run
    int* cnt_d;        // [B][H/128] (token, group) arrivals
    int* wq;           // [0] piece queue, [1] CTAs that left, [2] finished rotation pieces, [3] queue of the all-reduce tasks
    float* zd;         // [S][I/128][4] down low-rank partials
    float* out;        // [B][H]
    int* hits;         // optional [E] pick counters (may be host-mapped)
    // expert parallelism (world > 1): the all-reduce of the partial outputs runs inside this kernel, over peer memory
    int world, rank;
    float* recv[kEpRanks];   // every rank's receive buffer [2][world][32][H] fp32, as seen from this GPU
    int* rcnt[kEpRanks];     // every rank's arrival counters [2][32 * 64], as seen from this GPU
    int* epoch;              // this rank's call counter (device): its parity picks the half of recv / rcnt
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

// Programmatic dependent launch: a kernel lets its successor in the stream start launching early (launch_dependents)
// and the successor blocks (grid_dependency_wait) until the whole predecessor grid has completed and its writes are
// visible, before it touches anything.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ int ld_acquire(const int* p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int add_acq_rel(int* p, int v)
{
    int prev;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(prev) : "l"(p), "r"(v) : "memory");
    return prev;
}
// every lane polls (one broadcast transaction) until *p >= target; false = gave up (status raised by this or another warp)
__device__ __forceinline__ bool wait_counter(const int* p, int target, int* status)
{
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i)
    {
        if (ld_acquire(p) >= target) return true;
        if ((i & 63u) == 63u)
        {
            if (ld_acquire(status) != 0) return false;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > kWaitNs) break;
        }
        __nanosleep(100);
    }
    atomicExch(status, 1);
    return false;
}

// ---------------------------------------------------------------- shared state of a CTA
struct Route
{
    int key[NQ_MAX_PICKS];                // expert of a valid pick, else -1 - pick
    RunRec runs[NQ_MAX_PICKS];
    short lead[NQ_MAX_PICKS];             // run ordinal (by first pick) -> its first pick
    short first_of[NQ_MAX_PICKS];         // first pick of a run -> offset of the run in order[]
    unsigned char lvl[NQ_MAX_PICKS], order[NQ_MAX_PICKS], nvalid[NQ_MAX_TOKENS];
    int warp_sum[NQ_MAX_PICKS / 32], nruns;
};

// Group the picks into runs: a run = one expert and up to 32 of its picks in pick order; runs are numbered by first
// pick, then ordered level 4 before level 2 (heavier pieces are handed out first).  Thread t = pick t (t < 256); every thread
// of the CTA must call it.
__device__ __forceinline__ void build_route(const MoeArgs& a, Route& R)
{
    const int S = a.B * a.topk, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const bool in = t < NQ_MAX_PICKS;
    int e = -1, lv = 0;
    const bool tv = t < S && pick_valid(a, t, &e, &lv);
    if (in) { R.key[t] = tv ? e : -1 - t; R.lvl[t] = (unsigned char)lv; }
    __syncthreads();
    int pos = 0, cnt = 0, first_pick = t;
    if (tv)
        for (int q = 0; q < S; ++q)
            if (R.key[q] == e) { if (cnt == 0) first_pick = q; ++cnt; pos += q < t; }
    const bool lead = tv && (pos % kRunTokens) == 0;
    const unsigned bal = __ballot_sync(0xffffffffu, lead);
    if (lane == 0 && in) R.warp_sum[warp] = __popc(bal);
    __syncthreads();
    int ord = __popc(bal & ((1u << lane) - 1u)), nruns = 0;
    for (int w = 0; w < NQ_MAX_PICKS / 32; ++w) { const int c = R.warp_sum[w]; ord += w < warp ? c : 0; nruns += c; }
    const int my_count = cnt - pos < kRunTokens ? cnt - pos : kRunTokens;
    if (lead) { R.lead[ord] = (short)t; R.first_of[t] = (short)my_count; }      // first_of holds the run's size until the ranks are known
    if (t == 0) R.nruns = nruns;
    __syncthreads();
    int rank = 0, first = 0;
    if (lead)
        for (int q = 0; q < nruns; ++q)
        {
            const int lp = R.lead[q], ol = R.lvl[lp];
            const bool before = ol > lv || (ol == lv && q < ord);
            rank += before; first += before ? (int)R.first_of[lp] : 0;
        }
    __syncthreads();
    if (lead) { R.runs[rank] = RunRec{e, lv, first, my_count}; R.first_of[t] = (short)first; }
    __syncthreads();
    if (tv)
    {
        int lp = first_pick;
        const int want = pos - pos % kRunTokens;
        if (want)                                   // an expert with more than 32 picks: find the first pick of my run
            for (int q = 0, seen = 0; q < S; ++q)
                if (R.key[q] == e) { if (seen == want) { lp = q; break; } ++seen; }
        R.order[R.first_of[lp] + pos % kRunTokens] = (unsigned char)t;
    }
    if (t < a.B)
    {
        int n = 0;
        for (int k = 0; k < a.topk; ++k) n += R.key[t * a.topk + k] >= 0;
        R.nvalid[t] = (unsigned char)n;
    }
    __syncthreads();
}

// ---------------------------------------------------------------- GEMV
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Tokens of the run as the N operand: lane (g, t4) supplies k = 16 T + 2 t4 (+8) of token 8 nt + g, i.e. column g of the
// tile.  A tile column without a token reads the run's first token instead: MMA columns are independent, so whatever is
// multiplied there lands in accumulators that are never stored.
//
// One column tile (runs of up to 8 tokens, the 1..8-token decode case): the 8 k-steps' (b0, b1) pairs of a unit are 64
// contiguous bytes per lane, copied into the plane ring by cp.async together with the unit's records (lanes whose column
// has a token only), so they are in shared memory when the unit is decoded.  A lane's four 16-byte pieces go to four
// lane-indexed arrays (piece i of lane l at 512 i + 16 l): conflict-free, and addressed from the same per-lane register
// as the base records.
constexpr int kStageTokens = kStageBytes;            // offset of the token fragments inside a GEMV stage
constexpr int kGemvStage = kStageBytes + 4 * 512;    // bytes per GEMV stage
struct TokenSink1
{
    float (&acc)[4];
    uint32_t frag;     // shared-space address of this stage's token fragments + 16 lane
    template <int T>
    __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const
    {
        const uint2 b = lds64(frag + 512 * (T >> 1) + 8 * (T & 1));
        mma_16816(acc, a, b.x, b.y);
    }
};
// Up to NT column tiles: B fragments fetched from global memory per k-step.
template <int NT>
struct TokenSinkN
{
    float (&acc)[NT][4];
    const uint8_t* x0;           // token rows (bytes)
    const uint32_t (&xoff)[NT];  // byte offset of the tile's row for this lane (+ 64 t4)
    int ntiles, off;             // off = 256 * chunk
    template <int T>
    __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const
    {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
        {
            if (nt >= ntiles) break;      // warp-uniform
            const uint2 b = *(const uint2*)(x0 + xoff[nt] + off + T * 8);
            mma_16816(acc[nt], a, b.x, b.y);
        }
    }
};

// What one warp does with one strip: filled in by the caller, read once by strip_gemv.
struct StripJob
{
    ProjPlanes P;
    StripRef sr;
    int C, NS, c0, c1;               // chunks per strip, strips of the projection, chunk range [c0, c1)
    const uint8_t* x0;               // token rows (operand order), as bytes
    uint32_t xoff[kRunTiles];        // per column tile: byte offset of this lane's token row + 64 t4
    int ntiles;
    bool has_token;                  // this lane's column of tile 0 holds a token
    uint32_t ring;                   // shared-space address of the warp's kDepth stages
    const int* gate; int gate_target; int* status;   // counter to wait for before the first multiply (or null)
};

// One warp, one strip, chunks [c0, c1): stream, decode, multiply; acc = the 16 x (8 NT) partial sums.  REFINED: the expert
// is at level 4.  false = the wait on the gate counter ran out.
// Not inlined on purpose: each of the decoder variants gets a register allocation of its own, and the bookkeeping of the
// piece loop is saved once per piece around the call instead of being squeezed into the decode loop.
template <bool REFINED, int RC, int BK, int NT>
__device__ __noinline__ bool strip_gemv(const StripJob& J, float (&out)[NT][4])
{
    const int lane = threadIdx.x & 31, c0 = J.c0, c1 = J.c1;
    const unsigned long long flags = J.sr.flags;
    RecordCursor<BK> cb;
    cb.init(J.P.base, (size_t)J.NS * J.C * 32, J.sr.unit0 + c0, lane);
    RecordCursor<RC> cr;
    int issued = 0;                       // refined units whose copies are issued
    if constexpr (REFINED) cr.init(J.P.p4, J.sr.res_nrec, J.sr.res0 + refined_before(J.sr, c0), lane);
    const uint32_t ring = J.ring;
    const uint8_t* xin = J.x0 + J.xoff[0] + (size_t)c0 * 256;       // next token fragment to copy (one column tile)
    const bool has_token = J.has_token;
    auto issue_planes = [&](int ch, uint32_t st) {
        cb.copy(st, ch - c0, lane);
        if constexpr (REFINED)
            if ((flags >> ch) & 1ull) cr.copy(st + kStageBase, issued++, lane);
    };      // (prologue only; the loop below tests its flags from a block-local copy)
    auto issue_tokens = [&](uint32_t st) {
        if constexpr (NT == 1)
        {
            if (has_token)
            {
                const uint32_t dst = st + kStageTokens + lane * 16;
                cp_async16_at<0, 0>(dst, xin); cp_async16_at<512, 16>(dst, xin);
                cp_async16_at<1024, 32>(dst, xin); cp_async16_at<1536, 48>(dst, xin);
            }
            xin += 256;
        }
    };
    // the planes can be fetched before the inputs exist (gate), the token fragments only after
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d)
        if (c0 + d < c1) issue_planes(c0 + d, ring + d * kGemvStage);
    bool ok = true;
    if (J.gate) ok = wait_counter(J.gate, J.gate_target, J.status);
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d)
    {
        if (c0 + d < c1) issue_tokens(ring + d * kGemvStage);
        cp_async_commit();
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
    uint32_t st = ring;                                   // stage to consume; the stage before it (cyclically) is filled
    const int nxt = ring_successor(lane);
    for (int cs = c0; cs < c1; cs += 32)
    {
        // per-unit scalars of chunks cs .. cs + 31, one chunk per lane: ring signs, block word and its multipliers;
        // fl: refinement flags of chunks cs .. cs + 31 (+ kDepth - 1 for the copies that run ahead)
        const unsigned long long fl = flags >> cs;
        uint32_t var_b = 0, ac = 0, mbn = 0;
        {
            const int cl = cs + lane;
            if (cl < c1)
            {
                if (J.P.var) var_b = __ldg(J.P.var + J.sr.unit0 + cl);
                if constexpr (REFINED)
                    if ((fl >> lane) & 1ull)
                    {
                        mbn = __ldg(J.P.d4 + J.sr.res0 + refined_before(J.sr, cl)) & 0xFFFFu;
                        ac = block_multipliers(mbn);
                    }
            }
        }
        const int n = c1 - cs < 32 ? c1 - cs : 32;
        for (int i = 0; i < n; ++i)
        {
            const int ch = cs + i;
            if (ch + kDepth - 1 < c1)
            {
                const uint32_t st_in = st == ring ? ring + (kDepth - 1) * kGemvStage : st - kGemvStage;
                cb.copy(st_in, ch + kDepth - 1 - c0, lane);
                if constexpr (REFINED)
                    if ((fl >> (i + kDepth - 1)) & 1ull) cr.copy(st_in + kStageBase, issued++, lane);
                issue_tokens(st_in);
            }
            cp_async_commit();
            cp_async_wait<kDepth - 1>();
            const uint32_t sign2 = sign_mask(__shfl_sync(0xffffffffu, var_b, i), lane);
            uint32_t wb[Pattern<BK>::kWords + 2], wr[Pattern<RC>::kWords + 2];
            RecordCursor<BK>::read(wb, st, lane);
            continue_stream<Pattern<BK>::kBits>(wb, __shfl_sync(0xffffffffu, wb[0], nxt));
            bool refined = false;
            if constexpr (REFINED) refined = (fl >> i) & 1ull;
            UnitConsts k;
            if (refined)
            {
                const uint32_t acw = __shfl_sync(0xffffffffu, ac, i), mb = __shfl_sync(0xffffffffu, mbn, i);
                RecordCursor<RC>::read(wr, st + kStageBase, lane);
                continue_stream<Pattern<RC>::kBits>(wr, __shfl_sync(0xffffffffu, wr[0], nxt));
                k = consts_level4(acw, mb, sign2);
            }
            else k = consts_level2(sign2);
            if constexpr (NT == 1)
            {
                const TokenSink1 sink{acc[0], st + kStageTokens + lane * 16};
                if (refined) decode_words<true, RC, BK>(wb, wr, k, sink);
                else decode_words<false, 0, BK>(wb, wr, k, sink);
            }
            else
            {
                const TokenSinkN<NT> sink{acc, J.x0, J.xoff, J.ntiles, ch * 256};
                if (refined) decode_words<true, RC, BK>(wb, wr, k, sink);
                else decode_words<false, 0, BK>(wb, wr, k, sink);
            }
            st = st + kGemvStage == ring + kDepth * kGemvStage ? ring : st + kGemvStage;
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) out[nt][i] = acc[nt][i];
    return ok;
}

// 4 consecutive elements k = 4 lane + i of a 128-chunk -> operand order (two 4-byte stores)
__device__ __forceinline__ void store4h_operand(__half* chunk, int lane, const float (&v)[4])
{
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint32_t* w = (uint32_t*)chunk + (lane & 1) * 32 + (lane >> 2) * 2 + ((lane & 3) >> 1);
    w[0] = *(const uint32_t*)&a;
    w[16] = *(const uint32_t*)&b;
}

struct Shape
{
    int S, ng, ngH, KSg, KSd, nparts, rot_blocks, nruns;
    int n_rot, n_gu, n_dn, per_run_gu, per_run_dn;
};

// ---------------------------------------------------------------- rotation piece: (pick, blocks [rb part, rb part + rb))
// rb = 1 whenever there are at least as many warps as (pick, block) pairs: every gate|up piece waits for the rotations, so
// they are spread as thin as possible, and the inputs of the next block are fetched before the current one is transformed.
struct RotIn { uint2 x, g, u; };
__device__ __forceinline__ RotIn rot_fetch(const __half* xr, const __half* scales, const __half* su_u, int k)
{
    return RotIn{*(const uint2*)(xr + k), *(const uint2*)(scales + k), *(const uint2*)(su_u + k)};
}
__device__ __forceinline__ void unpack4h(const uint2& w, float (&f)[4])
{
    const __half2 a = *(const __half2*)&w.x, b = *(const __half2*)&w.y;
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
__device__ __forceinline__ void rotate_piece(const MoeArgs& a, const Shape& sh, const Route& R, int piece, int lane)
{
    const int s = piece / sh.nparts, part = piece - s * sh.nparts;
    const int e = R.key[s];
    if (e >= 0)
    {
        const __half* scales = (const __half*)a.table[(int64_t)e * kTableWidth + 9];
        const __half* su_u = scales + 2 * a.H + 3 * a.I;
        const __half* xr = a.x + (size_t)(s / a.topk) * a.H;
        __half* dst = a.xrot + (size_t)s * 2 * a.H;
        const int b0 = part * sh.rot_blocks, b1 = b0 + sh.rot_blocks < sh.ngH ? b0 + sh.rot_blocks : sh.ngH;
        RotIn in = rot_fetch(xr, scales, su_u, b0 * 128 + lane * 4);
        for (int blk = b0; blk < b1; ++blk)
        {
            const RotIn cur = in;
            if (blk + 1 < b1) in = rot_fetch(xr, scales, su_u, (blk + 1) * 128 + lane * 4);
            float f[4], g[4], u[4];
            unpack4h(cur.x, f); unpack4h(cur.g, g); unpack4h(cur.u, u);
            float vg[4] = {f[0] * g[0], f[1] * g[1], f[2] * g[2], f[3] * g[3]};
            float vu[4] = {f[0] * u[0], f[1] * u[1], f[2] * u[2], f[3] * u[3]};
            wht128(vg, lane); wht128(vu, lane);
            store4h_operand(dst + blk * 128, lane, vg);
            store4h_operand(dst + a.H + blk * 128, lane, vu);
        }
    }
    __syncwarp();                      // the lanes' stores happen before lane 0's release below
    if (lane == 0) add_acq_rel(a.wq + 2, 1);
}

// ---------------------------------------------------------------- finishers
// (run, group) complete: WHT128, sv, (+ low rank), SwiGLU, su_d, WHT128 -> h, one token after the other.
__device__ __forceinline__ void finish_gate_up(const MoeArgs& a, const Shape& sh, const Route& R, int r, int grp, int lane)
{
    __syncwarp();        // lane 0's acquiring arrival is ordered before every lane's loads below
    const RunRec run = R.runs[r];
    const int64_t* row = a.table + (int64_t)run.expert * kTableWidth;
    const int S = sh.S, N = 2 * a.I, KS = sh.KSg, ng = sh.ng;
    const __half* scales = (const __half*)row[9];
    const __half *sv_g = scales + a.H, *sv_u = sv_g + a.I, *su_d = sv_u + a.I;
    const __half* lr = (const __half*)row[14];
    const int rg = lr ? (int)row[16] : 0, rd = lr ? (int)row[17] : 0, hw = (int)row[18];
    const __half* lr4 = run.level == 4 ? (const __half*)row[15] : nullptr;
    const int col = grp * 128 + lane * 4;
    for (int j = 0; j < run.count; ++j)
    {
        const int slot = R.order[run.first + j];
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        for (int q = 0; q < rg; ++q)          // z = x V_gu^T on the unrotated input
        {
            const __half* xr = a.x + (size_t)(slot / a.topk) * a.H;
            float d = 0.f;
            for (int k = lane * 4; k < a.H; k += 128)
            {
                float f[4], w[4];
                load4h(xr + k, f); load4h(lr + (size_t)q * a.H + k, w);
                d += f[0] * w[0] + f[1] * w[1] + f[2] * w[2] + f[3] * w[3];
            }
#pragma unroll
            for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            z[q] = d;
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
            for (int q = 0; q < rg; ++q)
            {
                float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
                const size_t o = (size_t)(u * rg + q) * a.I + col;
                load4h(lr + (size_t)rg * a.H + o, u2);
                if (lr4) load4h(lr4 + o, u4);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] += z[q] * u2[i] + z[q] * u4[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) gu[u][i] = v[i];
        }
        float v[4], sc[4];
        load4h(su_d + col, sc);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = silu(gu[0][i]) * gu[1][i];
        for (int q = 0; q < rd; ++q)          // this group's share of z_dn = sw V_dn^T
        {
            float w[4];
            load4h(lr + (size_t)rg * a.H + 2 * (size_t)rg * a.I + (size_t)q * a.I + col, w);
            float d = v[0] * w[0] + v[1] * w[1] + v[2] * w[2] + v[3] * w[3];
#pragma unroll
            for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (lane == 0) a.zd[((size_t)slot * ng + grp) * 4 + q] = d;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] *= sc[i];
        wht128(v, lane);
        if (hw <= 128) store4h_operand(a.h + (size_t)slot * a.I + grp * 128, lane, v);
        else __stcg((float4*)(a.part_gu + (size_t)slot * N + col), make_float4(v[0], v[1], v[2], v[3]));   // fp32 stage: gate columns, k-slice 0
    }
    int done = 1;       // groups of this run whose h is now complete
    if (hw > 128)
    {
        // 512-wide rotation = H_4 (x) WHT128 / 2: the last of the hw/128 groups of a block combines their fp32 results
        const int nb = hw / 128, b0 = grp / nb * nb;
        __syncwarp();
        int last = 0;
        if (lane == 0)
        {
            int* ch = a.cnt_gu + S * ng + r * ng + b0;
            last = add_acq_rel(ch, 1) == nb - 1;
            if (last) *ch = 0;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        done = 0;
        if (last)
        {
            __syncwarp();
            const float rs = rsqrtf((float)nb);
            for (int task = 0; task < run.count * nb; ++task)
            {
                const int j = task / nb, ob = task - j * nb, slot = R.order[run.first + j];
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
                store4h_operand(a.h + (size_t)slot * a.I + (b0 + ob) * 128, lane, o);
            }
            done = nb;
        }
    }
    if (done)
    {
        __syncwarp();
        if (lane == 0) add_acq_rel(a.cnt_gu + 2 * S * ng + r, done);
    }
}

// ---- all-reduce of the partial outputs inside the kernel (expert parallelism) --------------------------------------------
// Every rank computes, for each (token, 128-column group), the weighted sum over ITS experts.  It stores that slice into
// slot [parity][its rank][token] of every rank's receive buffer (plain peer stores over NVLink, its own buffer included),
// then adds 1 to the (token, group) arrival counter of every rank (release, system scope).  After its own pieces are done, a
// rank's warps take (token, group) tasks: wait until the counter shows all `world` slices (acquire; bounded), add the slices
// in rank order - every rank gets bitwise the same sums - and write out.  The parity of a per-rank call counter alternates
// two halves of the buffers: a rank can run at most one call ahead of a peer (it needs the peer's slices of call n to finish
// call n), so the slices of call n + 1 never land on slices of call n that are still being read.
__device__ __forceinline__ void ep_send(const MoeArgs& a, const Shape& sh, int par, int b, int grp, int lane, const float (&o)[4])
{
    const size_t at = (((size_t)par * a.world + a.rank) * kEpTokens + b) * a.H + grp * 128 + lane * 4;
    for (int p = 0; p < a.world; ++p) *(float4*)(a.recv[p] + at) = make_float4(o[0], o[1], o[2], o[3]);
    __syncwarp();       // the lanes' stores happen before the releasing adds below, which publish them (cumulativity)
    if (lane < a.world)
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(a.rcnt[lane] + (par * kEpTokens + b) * kEpGroups + grp) : "memory");
}
// false = the wait ran out
__device__ __forceinline__ bool ep_sum(const MoeArgs& a, const Shape& sh, int par, int b, int grp, int lane)
{
    int* cnt = a.rcnt[a.rank] + (par * kEpTokens + b) * kEpGroups + grp;
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i)
    {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
        if (v >= a.world) break;
        if ((i & 31u) == 31u)
        {
            if (ld_acquire(a.status) != 0) return false;
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > kWaitNs) { atomicExch(a.status, 1); return false; }
        }
        if (i > 8) __nanosleep(50);
    }
    __syncwarp();
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < a.world; ++p)
    {
        const float4 v = __ldcg((const float4*)(a.recv[a.rank] + (((size_t)par * a.world + p) * kEpTokens + b) * a.H + grp * 128 + lane * 4));
        o[0] += v.x; o[1] += v.y; o[2] += v.z; o[3] += v.w;
    }
    *(float4*)(a.out + (size_t)b * a.H + grp * 128 + lane * 4) = make_float4(o[0], o[1], o[2], o[3]);
    __syncwarp();
    if (lane == 0) *cnt = 0;          // this half is next used two calls from now
    return true;
}

// output rows [grp * 128, +128) of token b are complete in every k-slice of every pick: weighted combine
__device__ __forceinline__ void finish_down(const MoeArgs& a, const Shape& sh, const Route& R, int b, int grp, int lane, int par)
{
    __syncwarp();        // the acquiring arrival (some lane's) is ordered before every lane's loads below
    const int S = sh.S, N = a.H, KS = sh.KSd, col = grp * 128 + lane * 4;
    float o[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < a.topk; ++k)
    {
        const int s = b * a.topk + k, e = R.key[s];
        if (e < 0) continue;
        const int lv = R.lvl[s];
        const float w = __half2float(a.rw[s]);
        const int64_t* erow = a.table + (int64_t)e * kTableWidth;
        const __half* sv_o = (const __half*)erow[9] + a.H + 3 * a.I;
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
        const __half* lr = (const __half*)erow[14];
        const int rd = lr ? (int)erow[17] : 0;
        if (rd)
        {
            const int rg = (int)erow[16], ng = sh.ng;
            const __half* lr4 = lv == 4 ? (const __half*)erow[15] : nullptr;
            const size_t ou = (size_t)rg * a.H + 2 * (size_t)rg * a.I + (size_t)rd * a.I;
            for (int q = 0; q < rd; ++q)
            {
                float z = 0.f;
                for (int gq = 0; gq < ng; ++gq) z += __ldcg(a.zd + ((size_t)s * ng + gq) * 4 + q);
                float u2[4], u4[4] = {0.f, 0.f, 0.f, 0.f};
                load4h(lr + ou + (size_t)q * a.H + col, u2);
                if (lr4) load4h(lr4 + 2 * (size_t)rg * a.I + (size_t)q * a.H + col, u4);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] += z * u2[i] + z * u4[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] += w * v[i];
    }
    if (a.world > 1) ep_send(a, sh, par, b, grp, lane, o);
    else *(float4*)(a.out + (size_t)b * a.H + col) = make_float4(o[0], o[1], o[2], o[3]);
}

// ---------------------------------------------------------------- GEMV pieces
// One warp's piece: strip `strip` of the projection over chunks [c0, c1) for the run's tokens; the partial sums go to
// part[ks][slot][row].  false = a wait ran out.
template <int NT>
__device__ __forceinline__ bool gemv_piece(const MoeArgs& a, const Shape& sh, const Route& R, const RunRec& run, int DOWN, int strip, int c0, int c1,
                                           int up, int ks, const int* gate_counter, int gate_target, uint32_t ring, int lane)
{
    const int g = lane >> 2, t4 = lane & 3;
    const int N = DOWN ? a.H : 2 * a.I, K = DOWN ? a.I : a.H;
    const int64_t* row = a.table + (int64_t)run.expert * kTableWidth;
    const int rc = (int)row[10 + DOWN], nm = DOWN ? a.nm_dn : a.nm_gu, bk = (int)(row[19] >> (8 * DOWN)) & 0xFF;
    const bool level4 = run.level >= 4;
    StripJob J;
    J.P = planes_from_row(row, DOWN);
    J.C = K / 128; J.NS = N / 16; J.c0 = c0; J.c1 = c1;
    J.sr = locate_strip(J.P, strip, J.C, J.NS, nm, level4);
    J.ntiles = (run.count + 7) >> 3;
    J.has_token = g < run.count;
    J.x0 = (const uint8_t*)(DOWN ? a.h : a.xrot);
#pragma unroll
    for (int nt = 0; nt < kRunTiles; ++nt)
    {
        const int j = nt * 8 + g;
        const int slot = R.order[run.first + (j < run.count ? j : 0)];
        J.xoff[nt] = (uint32_t)((DOWN ? (size_t)slot * a.I : ((size_t)slot * 2 + up) * a.H) * 2 + t4 * 64);
    }
    J.ring = ring; J.gate = gate_counter; J.gate_target = gate_target; J.status = a.status;
    float acc[NT][4];
    bool ok = true;
#define NQ_RUN(RES, RCV, BKV) ok = strip_gemv<RES, RCV, BKV, NT>(J, acc)
    NQ_WITH_CODES(level4, rc, bk, NQ_GEMV_CODES, NQ_RUN);
#undef NQ_RUN
    if (!ok) return false;
    float* part = DOWN ? a.part_d : a.part_gu;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const int j = nt * 8 + t4 * 2 + (i & 1), rr = strip * 16 + g + (i >> 1) * 8;
            if (j < run.count) __stcg(part + ((size_t)ks * sh.S + R.order[run.first + j]) * N + rr, acc[nt][i]);
        }
    return true;
}

__device__ __forceinline__ Shape make_shape(const MoeArgs& a, int nruns, int nwarps)
{
    Shape sh;
    sh.S = a.B * a.topk; sh.ng = a.I / 128; sh.ngH = a.H / 128; sh.KSg = a.ks_gu; sh.KSd = a.ks_dn;
    sh.rot_blocks = (sh.S * sh.ngH + nwarps - 1) / nwarps;
    sh.nparts = (sh.ngH + sh.rot_blocks - 1) / sh.rot_blocks; sh.nruns = nruns;
    sh.per_run_gu = sh.ng * 2 * sh.KSg * 8; sh.per_run_dn = sh.ngH * sh.KSd * 8;
    sh.n_rot = (a.which & 1) ? sh.S * sh.nparts : 0;
    sh.n_gu = (a.which & 1) ? nruns * sh.per_run_gu : 0;
    sh.n_dn = (a.which & 2) ? nruns * sh.per_run_dn : 0;
    return sh;
}

// persistent CTAs of independent warps
__global__ void __launch_bounds__(kThreads, NQ_GEMV_MINBLOCKS) moe_decode_kernel(MoeArgs a)
{
    extern __shared__ __align__(16) uint8_t smem_ring[];   // [kWarps][kDepth][kGemvStage]
    __shared__ Route R;
    launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    build_route(a, R);
    const int nwarps = (int)gridDim.x * kWarps;
    const Shape sh = make_shape(a, R.nruns, nwarps);
    if (blockIdx.x == 0 && a.hits && (int)threadIdx.x < sh.S)
    {
        const int64_t es = a.sel[threadIdx.x];
        if (es >= 0 && es < a.E && __half2float(a.rw[threadIdx.x]) != 0.f) atomicAdd(a.hits + es, 1);   // every pick with a weight, any level
    }
    const bool ep = a.world > 1 && a.which == 3;
    const int par = ep ? (*(volatile int*)a.epoch & 1) : 0;
    // rows of tokens none of whose picks is resident here are defined as zero (nothing else writes them); under expert
    // parallelism this rank's slice of such a token is a zero slice, sent like any other
    if (a.which & 2)
    {
        if (!ep)
        {
            for (int b = blockIdx.x; b < a.B; b += gridDim.x)
                if (R.nvalid[b] == 0)
                    for (int i = threadIdx.x; i < a.H; i += kThreads) a.out[(size_t)b * a.H + i] = 0.f;
        }
        else
        {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
            for (int task = (int)blockIdx.x * kWarps + warp; task < a.B * sh.ngH; task += (int)gridDim.x * kWarps)
                if (R.nvalid[task / sh.ngH] == 0) ep_send(a, sh, par, task / sh.ngH, task % sh.ngH, lane, zero);
        }
    }

    const uint32_t ring = smem_addr(smem_ring) + warp * (kDepth * kGemvStage);
    const int total = sh.n_rot + sh.n_gu + sh.n_dn;
    bool rotated = false;      // this warp has seen every rotation piece finished
    int ready_run = -1;        // the run whose h this warp has seen complete
    // a warp's first piece is its own index (thousands of warps start at once: no burst of atomics on one address); later
    // ones come from the queue counter, which therefore counts from the number of warps
    for (int round = 0;; ++round)
    {
        int piece = (int)blockIdx.x * kWarps + warp;
        if (round)
        {
            if (lane == 0) piece = nwarps + atomicAdd(a.wq, 1);
            else if (lane == 1) piece = ld_acquire(a.status);
            const int raised = __shfl_sync(0xffffffffu, piece, 1);
            piece = __shfl_sync(0xffffffffu, piece, 0);
            if (raised) break;
        }
        if (piece >= total) break;
        if (piece < sh.n_rot) { rotate_piece(a, sh, R, piece, lane); continue; }
        piece -= sh.n_rot;
        // gate|up: (run, group, gate / up, k-slice, strip of the group); down: (run, group, k-slice, strip of the group)
        const int down = piece >= sh.n_gu;
        if (down) piece -= sh.n_gu;
        const int per_run = down ? sh.per_run_dn : sh.per_run_gu, KS = down ? sh.KSd : sh.KSg;
        const int r = piece / per_run, rem = piece - r * per_run;
        const int per_grp = (down ? 1 : 2) * KS * 8, grp = rem / per_grp, rem2 = rem - grp * per_grp;
        const int up = rem2 / (KS * 8), rem3 = rem2 - up * (KS * 8), ks = rem3 >> 3, s8 = rem3 & 7;
        const RunRec run = R.runs[r];
        const int C = (down ? a.I : a.H) / 128, c0 = ks * (C / KS), c1 = c0 + C / KS;
        const int strip = down ? grp * 8 + s8 : (up * a.I + grp * 128) / 16 + s8;
        const int* gate = nullptr;
        int target = 0;
        if (!down) { if (!rotated) { gate = a.wq + 2; target = sh.n_rot; } }
        else if ((a.which & 1) && ready_run != r) { gate = a.cnt_gu + 2 * sh.S * sh.ng + r; target = sh.ng; }
        bool ok;
        if (run.count <= 8) ok = gemv_piece<1>(a, sh, R, run, down, strip, c0, c1, up, ks, gate, target, ring, lane);
        else ok = gemv_piece<kRunTiles>(a, sh, R, run, down, strip, c0, c1, up, ks, gate, target, ring, lane);
        if (!ok) break;
        // Every arrival below is an acq_rel atomic issued after this warp barrier: the barrier orders all lanes' partial-sum
        // stores before it, the release half publishes them, the acquire half of the last arrival sees everybody's.
        __syncwarp();
        if (!down)
        {
            rotated = true;
            int last = 0;
            if (lane == 0)
            {
                int* cnt = a.cnt_gu + r * sh.ng + grp;
                last = add_acq_rel(cnt, 1) == 2 * KS * 8 - 1;
                if (last) *cnt = 0;
            }
            if (__shfl_sync(0xffffffffu, last, 0)) finish_gate_up(a, sh, R, r, grp, lane);
        }
        else
        {
            ready_run = r;
            // one arrival per token of the run on its (token, group) counter
            int last = 0, b = 0;
            if (lane < run.count)
            {
                b = R.order[run.first + lane] / a.topk;
                int* cnt = a.cnt_d + b * sh.ngH + grp;
                last = add_acq_rel(cnt, 1) == (int)R.nvalid[b] * KS * 8 - 1;
                if (last) *cnt = 0;
            }
            unsigned todo = __ballot_sync(0xffffffffu, last);
            while (todo)
            {
                const int src = __ffs(todo) - 1;
                todo &= todo - 1;
                finish_down(a, sh, R, __shfl_sync(0xffffffffu, b, src), grp, lane, par);
            }
        }
    }
    // this rank's pieces are done (or handed out): add up the slices of all ranks, one (token, group) at a time
    // (tasks are dealt out by warp index: there are more warps than tasks for every supported shape, and no counter to fight over)
    if (ep)
        for (int task = (int)blockIdx.x * kWarps + warp; task < a.B * sh.ngH; task += nwarps)
            if (!ep_sum(a, sh, par, task / sh.ngH, task % sh.ngH, lane)) break;
    // the last CTA to leave resets the queue and the per-run counters (graph replays start from zero)
    __syncthreads();
    if (threadIdx.x == 0)
    {
        __threadfence();
        if (atomicAdd(a.wq + 1, 1) == (int)gridDim.x - 1)
        {
            a.wq[0] = 0; a.wq[1] = 0; a.wq[2] = 0; a.wq[3] = 0;
            if (ep) *a.epoch = *(volatile int*)a.epoch + 1;
            for (int r = 0; r < sh.nruns; ++r) a.cnt_gu[2 * sh.S * sh.ng + r] = 0;
            if (ld_acquire(a.status) != 0)      // a wait ran out: leave every counter clean all the same
            {
                for (int i = 0; i < 2 * sh.S * sh.ng; ++i) a.cnt_gu[i] = 0;
                for (int i = 0; i < a.B * sh.ngH; ++i) a.cnt_d[i] = 0;
            }
            __threadfence();
        }
    }
}

constexpr int kGemvSmem = kWarps * kDepth * kGemvStage;
constexpr int kMaxDevices = 64;

// CTAs that fit on the current device at once (the kernel is persistent); the first call on a device also opts the kernel
// into its shared memory there.  0 = failure.
static int resident_ctas()
{
    static int cached[kMaxDevices] = {0};
    int dev = 0, sms = 0, per = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    if (cached[dev]) return cached[dev];
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaFuncSetAttribute((const void*)moe_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvSmem) != cudaSuccess) return 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, (const void*)moe_decode_kernel, kThreads, kGemvSmem);
    cached[dev] = sms * (per > 0 ? per : 1);
    return cached[dev];
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
    w->cnt_gu_ints = 2 * S * (I / 128) + S;
    w->cnt_d_ints = (size_t)B * (H / 128);
    w->wq_ints = 4;
    w->zd_floats = S * (I / 128) * 4;
    w->cnt_h_ints = 4;                                  // [0] status
    return NQ_OK;
}

static int moe_forward(const NqMoeForward* p, const NqMoeEp* ep, void* stream)
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
    NQ_REQUIRE(((size_t)p->B * p->topk * p->I) % 8 == 0, "nq_moe_forward: h and the rotated inputs must both be 16-byte aligned");
    nq::MoeArgs a{};
    a.x = (const __half*)p->x; a.sel = p->sel; a.rw = (const __half*)p->rw;
    a.B = p->B; a.topk = p->topk; a.E = p->E; a.H = p->H; a.I = p->I; a.nm_gu = p->nm_gu; a.nm_dn = p->nm_dn;
    a.force_level = p->force_level; a.ks_gu = p->ks_gu; a.ks_dn = p->ks_dn; a.which = p->which & 3; a.table = p->table;
    a.status = p->cnt_h; a.h = (__half*)p->h; a.xrot = a.h + (size_t)p->B * p->topk * p->I;
    a.part_gu = p->acc_gu; a.part_d = p->acc_d; a.zd = p->zd; a.cnt_gu = p->cnt_gu; a.cnt_d = p->cnt_d; a.wq = p->wq; a.out = p->out; a.hits = p->hits;
    a.world = 1; a.rank = 0;
    if (ep && ep->world > 1)
    {
        NQ_REQUIRE(ep->world <= nq::kEpRanks && ep->rank >= 0 && ep->rank < ep->world, "nq_moe_forward_ep: rank %d of %d", ep->rank, ep->world);
        NQ_REQUIRE(ep->peer_recv && ep->peer_counters && ep->epoch, "nq_moe_forward_ep: null exchange buffers");
        NQ_REQUIRE((p->which & 3) == 3, "nq_moe_forward_ep: the in-kernel all-reduce needs the whole layer call (which = 3)");
        NQ_REQUIRE(p->H / 128 <= nq::kEpGroups && p->B <= nq::kEpTokens, "nq_moe_forward_ep: shape beyond the exchange buffers");
        a.world = ep->world; a.rank = ep->rank; a.epoch = ep->epoch;
        for (int r = 0; r < ep->world; ++r)
        {
            NQ_REQUIRE(ep->peer_recv[r] && ep->peer_counters[r] && nq::aligned16(ep->peer_recv[r]), "nq_moe_forward_ep: buffers of rank %d are null or misaligned", r);
            a.recv[r] = (float*)ep->peer_recv[r]; a.rcnt[r] = (int*)ep->peer_counters[r];
        }
    }
    const int ctas = nq::resident_ctas();
    if (ctas <= 0) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward: cannot reserve %d bytes of shared memory", nq::kGemvSmem);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas); cfg.blockDim = dim3(nq::kThreads); cfg.dynamicSmemBytes = nq::kGemvSmem; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, nq::moe_decode_kernel, a);
    if (e != cudaSuccess) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward: %s", cudaGetErrorString(e));
    return nq::check_launch("nq_moe_forward");
}

int nq_moe_forward(const NqMoeForward* p, void* stream) { return moe_forward(p, nullptr, stream); }

int nq_moe_forward_ep(const NqMoeForward* p, const NqMoeEp* ep, void* stream)
{
    NQ_REQUIRE(ep, "nq_moe_forward_ep: null exchange description");
    return moe_forward(p, ep, stream);
}

size_t nq_moe_ep_recv_floats(int world, int H) { return world >= 1 && H > 0 ? (size_t)2 * world * nq::kEpTokens * H : 0; }
size_t nq_moe_ep_counter_ints(void) { return (size_t)2 * nq::kEpTokens * nq::kEpGroups; }

}  // extern "C"
