/*
 * nestquant_b200 C ABI: the NestQuant quantized routed-expert MoE layer on NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device/host pointers and sizes, enqueues its work on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), never synchronises and
 * returns 0 or a negative NQ_ERR_* code.  nq_last_error() gives the message of the calling thread's last failure.
 * Unless a function says otherwise it allocates nothing: all memory is caller-owned.
 *
 * Each declaration names the interface of the reference implementation (jarrelscy/nestquant) that it
 * replaces, as file:line of that project.  The reference binds these through a torch C++ extension
 * (sm120/nqmoe.cu:1294-1295); a ctypes binding with the same Python-visible names ships in nestquant_b200/ext.py.
 *
 * Device table: int64 [E][20] per layer, one row per expert (sm120/nqmoe.cu:26-45, sm120/moe.py:216-229):
 *   [0] level (0 = not resident here, 2, 4)   [1..4] gate|up: base, p4, d4, flags (0 = dense)   [5..8] down: same
 *   [9] fp16 scales [H su_g | I sv_g | I sv_u | I su_d | H sv_o | H su_u]   [10],[11] residual window codes
 *   [12],[13] ring-sign planes (0 = none)   [14] low-rank plane, [15] its level-4 part, [16] r_gu, [17] r_dn
 *   [18] width of the down-input rotation (0 or 128, or 512)   [19] base window codes bk_gu | bk_dn << 8 (0, or 1: see nq_bk_codes)
 */
#ifndef NESTQUANT_B200_H
#define NESTQUANT_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NQ_TABLE_WIDTH 20
#define NQ_MAX_TOKENS 32          /* tokens per decode-path call */
#define NQ_MAX_PICKS 256          /* tokens * topk per decode-path call */

enum {
    NQ_OK = 0,
    NQ_ERR_ARG = -1,              /* bad shape, size, alignment or configuration */
    NQ_ERR_CUDA = -2,             /* a CUDA runtime call or launch failed */
    NQ_ERR_UNSUPPORTED = -3       /* valid in the format but not built into this library */
};

const char* nq_last_error(void);
/* library build info: compute capability it was compiled for (100), as a sanity check for loaders */
int nq_build_arch(void);

/* Residual window codes compiled in, bit c = code c: out[0] gate|up, out[1] down.
 * Replaces rk_codes() (sm120/nqmoe.cu:938-940). */
int nq_rk_codes(int64_t out[2]);
/* Base window codes compiled in, bit c = code c: 0 = the 128-bit ring base (2 bits per weight), 1 = the pattern-rate base
 * of sm120/NQ_RES_V2.md:36-50 (1.75 bits per weight, 112-bit records in the sub-array layout; table field [19] =
 * bk_gu | bk_dn << 8).  Code 1 is built at level 2 and, at level 4, with the residual codes that build ships with (3 and
 * 9); the reference kernel has no base code other than 0.  Replaces the optional bk_codes() that sm120/moe.py:247-249
 * probes for. */
int nq_bk_codes(int64_t out[2]);

/* Bytes of a residual plane of `nrec` lane records of window code `code` (sm120/moe.py:27-30), or 0 for a bad code. */
size_t nq_plane_bytes(size_t nrec, int code);

/* Dense decode of `n_experts` experts to fp16 matrices, level and pointers read from the live table rows:
 * Wgu [n][2I][H], Wdn [n][H][I] (either may be NULL to skip that projection); experts = int32 expert ids (device).
 * Level-0 experts decode to zeros.  Replaces pf_decode() (sm120/nqmoe.cu:1013-1080,1247-1257) and, with one expert,
 * the NQ_WDUMP debug hook set_wdump() (sm120/nqmoe.cu:246-248,852-853) used for the bit-exactness checks. */
int nq_pf_decode(const int64_t* table, const int32_t* experts, int n_experts, void* Wgu, void* Wdn,
                 int H, int I, int nm_gu, int nm_dn, int force_level, void* stream);

/* Graph-safe table switch: table[e] = stage[e] wherever seq[e] != applied[e], then applied[e] = seq[e]
 * (also mirrored to applied_host when it is not NULL; host-mapped memory).  Replaces mailbox()
 * (sm120/nqmoe.cu:908-929). */
int nq_mailbox(int64_t* table, const int64_t* stage, const int32_t* seq, int32_t* applied, int32_t* applied_host,
               int E, void* stream);

/* Promotion (level 2 -> 4) or demotion of one expert, enqueued on a side stream: copy the pinned host record (the
 * expert's residual planes, see nestquant_b200/p4rec.py) into its slot, then the new table row into stage[e], then the
 * new sequence number into seq[e] - three copies in stream order, so the row is never visible before its bytes.  A
 * demotion passes slot = host_record = NULL.  The compute stream's next nq_mailbox applies the row.  All host buffers
 * must be pinned and must stay valid until the stream has executed the copies; one outstanding operation per expert.
 * Replaces Engine::issue_copies (streaming/nqstream.cu:183-191). */
int nq_promote(void* slot, const void* host_record, size_t record_bytes, int64_t* stage_row, const int64_t* host_row,
               int32_t* seq_entry, const int32_t* host_seq, void* stream);

/* ---- prefill path: stream-ordered helpers around the grouped GEMMs ---------------------------------------------
 * Pairs = (token, expert) picks sorted by expert: pt[p] = token, pe[p] = expert, prw[p] = routing weight (fp16).
 * R = number of pairs in this call.  z arrays are fp32 [R][4] (low-rank inputs, rank <= 4). */

/* The permutation of a prefill window: the T * topk picks sorted by expert with a stable counting sort on the device (three
 * small kernels, no host sync).  Bin E collects the picks that contribute nothing - expert id outside [0, E), expert not
 * resident (level <= 0), routing weight 0 - behind every real pair.
 *   pe [P] expert (or E) and pt [P] token of sorted pair p;  pos [P]: sorted index of pick t * topk + k;
 *   start [E + 2]: first pair of each bin (start[E] = number of live pairs, start[E + 1] = P);
 *   hit_counts [E] or NULL: += picks with a valid id and a non-zero weight, whatever the level (caller zeroes it; feed it to
 *   nq_pf_hits);  scratch: int32 [nq_pf_sort_scratch_ints(P, E)].
 * Replaces the host side of the reference's prefill (sm120/moe.py:293-298: argsort, scatter_add, .cpu() of the counts). */
int nq_pf_sort_scratch_ints(int pairs, int E);
int nq_pf_sort(const int64_t* sel, const void* rw, const int64_t* table, int T, int topk, int E, int32_t* pe, int32_t* pt,
               int32_t* pos, int32_t* start, int32_t* hit_counts, int32_t* scratch, int scratch_ints, void* stream);

/* xg[p] = fp16(WHT128(x[pt[p]] * su_g)), xu[p] likewise with su_u, both [R][H]; zg[p][r] = x . V_gu[r].
 * Pairs of level-0 experts and pairs whose expert id is outside [0, E) (padding) are skipped (their rows are left untouched).
 * kperm != 0 writes xg / xu in the k order nq_pf_gemm reads: inside every 16 consecutive k, position 4 i + {0, 1}
 * holds k = 2 i + {0, 1} and position 4 i + {2, 3} holds k = 8 + 2 i + {0, 1} (i < 4); 0 = plain order (the reference's).
 * Replaces pf_pre() (sm120/nqmoe.cu:1081-1117,1258-1267). */
int nq_pf_pre(const void* x, const int32_t* pt, const int32_t* pe, int R, const int64_t* table, int E, void* xg, void* xu, float* zg,
              int H, int I, int kperm, void* stream);

/* The same pass when the tokens' input rows are spread over the ranks of an expert-parallel group: token t is row
 * t % tokens_per_rank of peer_x[t / tokens_per_rank] (host array of `world` device addresses as seen from this GPU:
 * symmetric memory / peer mappings; fp16 [tokens_per_rank][H] each).  Reading a pair's row from its owner is the dispatch
 * step of the expert-parallel prefill, done by plain peer loads inside this kernel (the caller's nq_ep_barrier makes the
 * peers' rows complete first).  No counterpart in the reference (its serving path is tensor-parallel). */
int nq_pf_pre_ep(const void* const* peer_x, int world, int tokens_per_rank, const int32_t* pt, const int32_t* pe, int R,
                 const int64_t* table, int E, void* xg, void* xu, float* zg, int H, int I, int kperm, void* stream);

/* acc_g, acc_u fp32 [R][I] (GEMM outputs) -> h fp16 [R][I] = WHT_w(silu(g) u su_d), g = WHT128(acc_g) sv_g + low rank,
 * w = 128 or the expert's 512-wide rotation; zd[p][r] = (silu(g) u) . V_dn[r].  kperm: k order of h as for nq_pf_pre.
 * Replaces pf_mid() (sm120/nqmoe.cu:1118-1203,1268-1277). */
int nq_pf_mid(const float* acc_g, const float* acc_u, const float* zg, const int32_t* pe, int R, const int64_t* table, int E, void* h,
              float* zd, int H, int I, int kperm, void* stream);

/* out[pt[p]] += prw[p] * (WHT128(y[p]) * sv_o + low rank), y fp32 [R][H]; atomic adds into a caller-zeroed out.
 * Replaces pf_post() (sm120/nqmoe.cu:1204-1240,1278-1287). */
int nq_pf_post(const float* y, const float* zd, const int32_t* pt, const int32_t* pe, const void* prw, int R, const int64_t* table, int E,
               float* out, int H, int I, void* stream);

/* Same sum without atomics, one window of the expert-sorted pair list at a time: y / zd hold the rows of the pairs
 * [pair0, pair0 + npairs) (row = pair index - pair0); pos[t * topk + k] = pair index of that pick.  Each token's picks
 * inside the window are added in pick order.  accumulate = 0: out[t] is overwritten (zeros for a token without a pick in
 * the window); accumulate = 1: the sum is added to out[t].  Window after window in a fixed order this is bitwise
 * repeatable with scratch for one window only.  No counterpart in the reference (its pf_post order depends on atomics). */
int nq_pf_combine(const float* y, const float* zd, const int32_t* pos, const int64_t* sel, const void* rw, int T, int topk,
                  const int64_t* table, int E, float* out, int H, int I, int pair0, int npairs, int accumulate, void* stream);

/* Fused prefill GEMM (decode in registers -> weight tiles in tensor memory -> tcgen05.mma): the replacement of the reference's
 * pf_decode + grouped GEMM pair (sm120/moe.py:303-324, sm120/pf_gemm.py:7-34, sm120/nqmoe.cu:1013-1080); the dense fp16
 * weights are never materialised.
 *   nq_pf_plan   from per-expert pair counts (int32 [E], pairs sorted by expert) build the pass list on the device:
 *                a pass = one resident expert x up to 384 of its pairs.  plan: int32 [nq_pf_plan_ints(E, pairs)].
 *   nq_pf_gemm   down = 0: acc_g[p] = xg[p] Wg^T, acc_u[p] = xu[p] Wu^T (act0 = xg, act1 = xu fp16 [pairs][H];
 *                out0 = acc_g, out1 = acc_u fp32 [pairs][I]); down = 1: y[p] = h[p] Wd^T (act0 = h fp16 [pairs][I],
 *                out0 = y fp32 [pairs][H], act1 / out1 unused).  The activation matrices must be in the k order
 *                nq_pf_pre / nq_pf_mid write with kperm = 1.  Rows of pairs whose expert is not resident are not
 *                written.  status: int32 [1] on the device, set to 1 if a device-side wait timed out (bounded waits;
 *                the outputs are then invalid) - read it after synchronising.
 *   nq_pf_plan_window   the same from nq_pf_sort's start array for the pairs [pair0, pair0 + npairs) of the sorted list
 *                (rows counted from pair0): the pass list of one scratch chunk. */
int nq_pf_plan_ints(int E, int pairs);
int nq_pf_plan_window(const int32_t* start, const int64_t* table, int E, int pair0, int npairs, int32_t* plan, int plan_ints,
                      void* stream);
int nq_pf_plan(const int32_t* counts, const int64_t* table, int E, int pairs, int32_t* plan, int plan_ints, void* stream);
int nq_pf_gemm(const int64_t* table, const int32_t* plan, const void* act0, const void* act1, int pairs, float* out0, float* out1,
               int H, int I, int nm_gu, int nm_dn, int down, int32_t* status, void* stream);

/* hits[e] += counts[e] (hits may be host-mapped; NULL = no-op).  Replaces pf_hits() (sm120/nqmoe.cu:1241-1245,1288-1293). */
int nq_pf_hits(const int32_t* counts, int32_t* hits, int E, void* stream);

/* ---- decode path: one MoE layer call for 1..NQ_MAX_TOKENS tokens -------------------------------------------
 * Replaces moe_forward() (sm120/nqmoe.cu:858-907).  The argument block carries the same tensors, in the same roles,
 * as the reference's positional arguments; element counts travel with the pointers because nothing here can ask a
 * tensor for its size.  Differences a caller can see:
 *   - up to 32 tokens per call (the reference: 8), B * topk <= 256;
 *   - split-k partial sums are written to acc_gu / acc_d and summed in a fixed order: results are bitwise repeatable,
 *     and those two buffers need no zeroing.  cnt_gu, cnt_d and wq must be zero on entry and are zero again on exit;
 *   - workspace sizes depend on the k-splits: ask nq_moe_workspace() (the reference sized them from B * topk alone);
 *     h also holds the rotated inputs;
 *   - cnt_h[0] is a status word: the call leaves it alone unless a device-side wait ran out (2 s), then it is 1 and the
 *     outputs are invalid.  Clear it before the first call and read it after synchronising if you want to know;
 *   - if no resident expert with a non-zero weight is picked at all, out is written with zeros
 *     (the reference leaves it untouched, sm120/nqmoe.cu:789); so is the row of any token none of whose picks is resident;
 *   - tiling is two integers (ks_gu, ks_dn = k-slices per strip) instead of cfg_gu / cfg_dn = (cpw, sb, nst[, pers]).
 * One persistent launch on `stream` does the routing, the input rotations, both GEMVs and the combine (the reference: two
 * launches); every routing, level and pointer decision is read on the device, so the call can be captured in a CUDA graph
 * and replayed while a mailbox flips table rows.
 * which = 1 stops after h (gate|up, SwiGLU); which = 2 starts from the h that is in the workspace.  Both h [S][I] and the
 * rotated inputs [S][2][H] behind it are fp16 in "operand order": inside every 128 consecutive k, element
 * k = 16 T + 2 t4 + 8 hi + e (T < 8, t4 < 4, hi, e < 2) sits at position 32 t4 + 4 T + 2 hi + e.  With which = 1 the
 * split-k partial sums of the gate|up projection stay readable in acc_gu [ks_gu][S][2I], with which = 2 those of the down
 * projection in acc_d [ks_dn][S][H] (S = B * topk pick slots): fed one-hot inputs they hold columns of the decoded weight
 * matrices, which is how the tests check the decoder inside this kernel bit for bit (the role of the reference's
 * NQ_WDUMP hook, sm120/nqmoe.cu:246-248,852-853). */
typedef struct NqMoeWorkspace {
    size_t acc_gu_floats, h_halves, acc_d_floats, cnt_gu_ints, cnt_d_ints, wq_ints, zd_floats, cnt_h_ints;
} NqMoeWorkspace;

/* Required element counts of the workspace tensors for a call shape. */
int nq_moe_workspace(int B, int topk, int H, int I, int ks_gu, int ks_dn, NqMoeWorkspace* out);

typedef struct NqMoeForward {
    const void* x;            /* fp16 [B][H] */
    const int64_t* sel;       /* int64 [B][topk] expert ids */
    const void* rw;           /* fp16 [B][topk] routing weights */
    const int64_t* table;     /* int64 [E][20] */
    float* out;               /* fp32 [>= B][H], overwritten */
    float* acc_gu;            /* workspaces, see nq_moe_workspace */
    void* h;
    float* acc_d;
    int32_t* cnt_gu;
    int32_t* cnt_d;
    int32_t* wq;
    float* zd;
    int32_t* cnt_h;
    int32_t* hits;            /* optional int32 [E] pick counters (device or host-mapped), or NULL */
    size_t out_floats, acc_gu_floats, h_halves, acc_d_floats, cnt_gu_ints, cnt_d_ints, wq_ints, zd_floats, cnt_h_ints;
    int B, topk, E, H, I;
    int nm_gu, nm_dn;         /* flagged chunks per strip of masked experts (per layer) */
    int ks_gu, ks_dn;         /* k-slices per strip: must divide H/128 and I/128 */
    int G;                    /* ring width, must be 4 */
    int force_level;          /* 0, or 2 / 4 to override the level of every resident expert */
    int which;                /* bit 0: gate|up, bit 1: down + combine */
} NqMoeForward;

int nq_moe_forward(const NqMoeForward* args, void* stream);

/* The same layer call on one rank of an expert-parallel group, with the all-reduce of the partial outputs done inside the
 * kernel over peer memory: every rank calls it with the same tokens and picks and a table that marks the other ranks'
 * experts level 0; out receives the sum over all ranks, bitwise equal on every rank (slices are added in rank order).
 * peer_recv[r] / peer_counters[r]: device addresses, as seen from this GPU, of rank r's receive buffer (fp32
 * [nq_moe_ep_recv_floats(world, H)]) and arrival counters (int32 [nq_moe_ep_counter_ints()], zero before the first call);
 * symmetric memory or peer mappings over NVLink.  epoch: device int32, zero before the first call, private to this rank.
 * Plain peer stores, one remote atomic add per (token, 128-column group) and peer, bounded waits (2 s, then cnt_h[0] = 1).
 * All ranks must make the same sequence of calls with these buffers; which must be 3.  No counterpart in the reference (its
 * evaluation harness all-reduces with the collective library, sm120/eval/eval_reg.py:137-142,181). */
typedef struct NqMoeEp {
    int world, rank;
    void* const* peer_recv;
    int32_t* const* peer_counters;
    int32_t* epoch;
} NqMoeEp;
size_t nq_moe_ep_recv_floats(int world, int H);
size_t nq_moe_ep_counter_ints(void);
int nq_moe_forward_ep(const NqMoeForward* args, const NqMoeEp* ep, void* stream);

/* The same layer call for hosts that must not allocate - a plugin inside a serving engine that has already handed all
 * device memory to its caches, or a process that bans allocator calls on its hot thread.  No counterpart in the reference
 * (its workspaces are always torch tensors owned by the caller).  The workspaces of nq_moe_forward live in an array that
 * is part of the library image: nq_moe_static_scratch_bytes() = 4 MiB, held by every GPU that loads the library until
 * the process exits.  A call shape whose workspaces (nq_moe_workspace) do not fit is refused with NQ_ERR_ARG; 4 MiB
 * covers the GLM-5 shape (H 6144, I 2048, top-8) for 1 token at any k-split up to (8, 4) and for up to 4 tokens at k-split
 * (2, 1); 4 tokens at (4, 2) need 4.6 MB and are refused.  The call issues no cudaMalloc / cudaFree and no allocating library
 * routine.  The first call on a device looks up the array's device address (cudaGetSymbolAddress): make that call at
 * start-up, before any stream capture on the device.  All calls share the array, which keeps the previous call's
 * contents; the counters are cleared at the start of each call, and calls that overlap on the GPU race - keep them in
 * one stream order.  x fp16 [B][H], sel int64 [B][topk], rw fp16 [B][topk], table int64 [E][20], out fp32 [B][H];
 * hits may be NULL. */
size_t nq_moe_static_scratch_bytes(void);
int nq_moe_forward_static(const void* x, const int64_t* sel, const void* rw, const int64_t* table, float* out,
                          int B, int topk, int E, int H, int I, int nm_gu, int nm_dn, int ks_gu, int ks_dn,
                          int32_t* hits, void* stream);

/* Decode salience export: acc[e] += sum over the picks (t, k) with sel[t][k] == e and rw[t][k] != 0 of
 * (rsf * rw[t][k])^2 * sum_i x[t][i]^2; every touched entry is also stored to host[e] (host-mapped fp64 [E], may be NULL).
 * x fp16 or bf16 [B][row_stride >= H] (the layer input), rw fp16 [B][topk], sel int64 [B][topk], acc fp64 [E] on the
 * device.  One launch, no host sync; calls on one layer must be stream-ordered.
 * Replaces sal() (sm120/nqsal.cu:18-77), with this library's decode limits (32 tokens, 256 picks). */
int nq_salience(const void* x, int x_is_bf16, int64_t row_stride, const void* rw, const int64_t* sel, int B, int H, int topk,
                int E, float rsf, double* acc, double* host, void* stream);

/* Expert-parallel dispatch over peer memory: for every global token t (rank t / tokens_per_rank owns it) that has a pick
 * with a non-zero weight among this rank's experts (expert / experts_per_rank == rank), copy its fp16 input row from the
 * owner's buffer peer_x[owner] ([tokens_per_rank][H], device addresses as seen from this GPU) into xstage[t]
 * ([world * tokens_per_rank][H]); other rows of xstage are left untouched.  sel int64 / rw fp16: the picks of ALL tokens
 * ([world * tokens_per_rank][topk], e.g. from an all-gather).  Plain peer loads; the caller's barrier makes the peers'
 * rows complete first.  No counterpart in the reference; it takes the place of the dispatch all-to-all. */
int nq_ep_gather(void* xstage, const void* const* peer_x, const int64_t* sel, const void* rw, int tokens_per_rank, int topk, int H,
                 int world, int rank, int experts_per_rank, void* stream);

/* The picks of every rank's tokens, fetched from the ranks' buffers (plain peer loads; the caller's nq_ep_barrier makes
 * them complete first): peer_sel[w] / peer_rw[w] = int64 / fp16 [tokens_per_rank][topk] of rank w, as seen from this GPU
 * (host arrays of `world` device addresses).  sel_all (int64 [world * tokens_per_rank][topk]) gets every pick's expert id;
 * rw_mine (fp16, same shape) its weight where the expert belongs to this rank (id / experts_per_rank == rank), else 0.
 * Takes the place of an all-gather of the picks and the masking that follows it.  No counterpart in the reference. */
int nq_ep_picks(const int64_t* const* peer_sel, const void* const* peer_rw, int tokens_per_rank, int topk, int world, int rank,
                int experts_per_rank, int64_t* sel_all, void* rw_mine, void* stream);

/* Barrier over the ranks of an expert-parallel group, as one small kernel per rank on `stream`: rank `rank` stores its call
 * number (*epoch + 1) into flag [rank] of every peer_flags[r] (int32 [world] per rank, zero-initialised symmetric memory;
 * host array of `world` device addresses as seen from this GPU), waits until its own flags have all reached that number,
 * then advances *epoch (device int32, zero-initialised, private to this rank and this group of buffers).  Everything the
 * stream wrote before the barrier is visible to the peers' kernels after theirs.  The wait is bounded by timeout_ns: when
 * it runs out *status (device int32) is set to 1 and the kernel returns - read it after synchronising.  Graph-capturable
 * (the call number is read on the device).  No counterpart in the reference. */
int nq_ep_barrier(int32_t* const* peer_flags, int rank, int world, int32_t* epoch, int32_t* status, long long timeout_ns,
                  void* stream);

/* Expert-parallel combine over peer memory: out[t] (fp32 [T][H]) = sum over the ranks r = 0 .. world - 1, in that order,
 * of row rows[r * T + t] (int32, -1 = none) of peer_parts[r] (fp32 [.][H], device addresses of every rank's partial-row
 * buffer as seen from this GPU: symmetric memory / peer mappings; host array of `world` pointers).  Plain peer loads.
 * The caller makes the peers' rows complete before the call and keeps them unchanged until it has run (barriers).
 * No counterpart in the reference (its serving path is tensor-parallel); it takes the place of the combine all-to-all
 * plus the indexed add of an expert-parallel prefill. */
int nq_ep_combine(float* out, const void* const* peer_parts, const int32_t* rows, int T, int H, int world, void* stream);

/* ---- promotion engine (host side) -------------------------------------------------------------------------------
 * One engine per GPU process, reading that process's record file (fixed-size records, see nestquant_b200/p4rec.py).
 * Replaces the torch-extension class Engine of streaming/nqstream.cu:46-283 (upgrade / post / poll / cancel /
 * tier_load / tier_drop / stats / close, same meaning):
 *   upgrade  record `rec` -> pinned host entry (drive read, or a hit in the host cache / RAM tier) -> device `slot`
 *            -> `row` into stage_row -> `seq` into seq_entry, in that order on the engine's own side stream
 *   post     row and sequence number only (demotion)
 *   poll     operations whose device writes have completed: hit = the bytes were already in host memory;
 *            t_read_s / t_done_s = seconds from the call to bytes-in-host-memory / device-writes-done.
 *            A failed read reports hit 0, t_read_s < 0 (-errno, or -1 for a short read), t_done_s -1 and never posts
 *            the row; a cancelled operation reports t_read_s = t_done_s = -1e9
 *   cancel   best effort: drops an operation that has touched neither a drive nor the device yet
 *   tier_load / tier_drop   pinned RAM copy of chosen records (read once, blocking); upgrades of those skip the drive
 * Operations start in arrival order; the caller keeps at most one operation per expert outstanding.  Calls return
 * at once (tier_load and close excepted).  device < 0 runs the engine against host memory (slot, stage_row and
 * seq_entry are then host pointers): the mode the CPU tests use.  alt_path = an identical copy of the file on a second
 * drive ("" or NULL for none); each read goes to the drive with fewer reads in flight (caps qd, qd_alt).
 * Environment (host-side fault injection, as the reference): NQ_FAULT_READ_MS = minimum spacing of drive reads,
 * NQ_FAULT_FAIL_PPM = share of completed reads reported as failed. */
typedef struct NqEngine NqEngine;
typedef struct { int64_t tag; int32_t hit; double t_read_s, t_done_s; } NqEngineDone;
typedef struct
{
    int64_t upgrades, posts, host_hits, bytes_read, fault_injected, cancelled, device_errors;
    int64_t queued, waiting, reading, copying;                 /* operations not yet seen / waiting / reading / copying */
    int64_t drive_reads[2], drive_bytes[2], drive_inflight[2], drive_qd[2];
    double drive_read_s[2];
    int64_t drives, n_host, tier_state, tier_recs, tier_hits, tier_bytes;   /* tier_state: 0 none, 1 active, 2 dropping, 3 dropped */
    double now_s;
} NqEngineStats;

int nq_engine_open(const char* path, const char* alt_path, size_t rec_bytes, int n_host, int qd, int qd_alt, int device,
                   NqEngine** out);
int nq_engine_upgrade(NqEngine* e, int64_t tag, int64_t rec, void* slot, void* stage_row, const int64_t* row /* [20] */,
                      void* seq_entry, int32_t seq);
int nq_engine_post(NqEngine* e, int64_t tag, void* stage_row, const int64_t* row /* [20] */, void* seq_entry, int32_t seq);
int nq_engine_cancel(NqEngine* e, int64_t tag);
int nq_engine_poll(NqEngine* e, NqEngineDone* out, int max);        /* returns the number of entries written */
int nq_engine_tier_load(NqEngine* e, const int64_t* recs, int n);   /* returns n */
int nq_engine_tier_drop(NqEngine* e);
int nq_engine_stats(NqEngine* e, NqEngineStats* out);
int nq_engine_close(NqEngine* e);

#ifdef __cplusplus
}
#endif
#endif
