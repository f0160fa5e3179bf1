// Prefill grouped GEMM with the trellis decode fused in: acc[pair][n] = sum_k act[pair][k] * W_expert(pair)[n][k].
//
// Replaces the reference's prefill sequence pf_decode -> dense fp16 weights in VRAM -> cuBLAS / Triton grouped GEMM
// (sm120/moe.py:303-324, sm120/pf_gemm.py, sm120/nqmoe.cu:1013-1080): the dense weights are never written to HBM.
//
// One work item = (pass, 128-row weight group): a pass is one expert and up to 384 of its tokens.  Per item a CTA
// walks K in blocks of 64:
//   warp 0        TMA: the tokens' activation tile [ntok x 64] fp16 (SWIZZLE_128B boxes of 64 rows) -> shared memory
//   warps 2..17   decode: a warp streams every other chunk of one strip with cp.async, decodes each unit in registers
//                 (bit-exact fp16) and stores it with tcgen05.st as two weight tiles [128 x 64] in TENSOR MEMORY
//                 (k-blocks 2 c and 2 c + 1): the m16n8k16-style fragment a lane holds is exactly what the 16x256b
//                 store shape takes, so a tile costs 4 stores per warp and no shared memory at all
//   warp 1        one elected lane issues tcgen05.mma with the A operand in tensor memory (M 128 = weight rows, N =
//                 tokens, K 16) into a [128 x 384] fp32 accumulator, also in tensor memory; tcgen05.commit frees the
//                 stages.  Token tiles run 3..8 k-blocks ahead (160 KB), weight tiles 4 stages (32 columns each)
//   warps 2..17   epilogue: tcgen05.ld the accumulator and store fp32 rows acc[pair][128 columns] (coalesced); it runs
//                 after the first unit of the CTA's next item has been decoded
// A lane's fragment registers of a k-step hold k = 2 t4 + {0, 1} and 8 + 2 t4 + {0, 1}; stored side by side they make
// the tile's k order inside every 16: position 4 i + {0, 1} = k 2 i + {0, 1}, position 4 i + {2, 3} = k 8 + 2 i + {0, 1}.
// The activation matrices must be in the same order (nq_pf_pre / nq_pf_mid with kperm = 1).
// Each decoded weight is used for every token of the pass, so decode cost is paid once per expert (for up to 384
// tokens).  Tensor-pipe bound by intent; the decode instruction rate is the practical limit.
// Every mbarrier wait is bounded: on time-out the CTA raises status[0], drains and returns.
#include <cuda.h>

#include "nq_common.cuh"
#include "nq_unit.cuh"

namespace nq {

#ifndef NQ_PF_SPLIT
#define NQ_PF_SPLIT 256      // token tiles wider than this are multiplied as two column halves
#endif
#ifndef NQ_PF_GROUPS
#define NQ_PF_GROUPS 2      // groups of 8 decode warps; group g takes the chunks c = g (mod groups) of its strips.  3 groups
                            // (24 decode warps at 72 registers) measured the same time as 2: the kernel runs at the power cap
#endif
constexpr int kPfGroups = NQ_PF_GROUPS;
constexpr int kPfDecodeWarps = 8 * kPfGroups;
constexpr int kPfAStages = 2 * kPfGroups;            // weight tiles in tensor memory: each unit fills two consecutive stages
constexpr int kPfACols = 32;                         // [128 lanes x 64 k] fp16 = 32 columns
constexpr int kPfTmemCols = 512;                     // [0, kPfAccCols) accumulator, the rest weight tiles
constexpr int kPfAccCols = kPfTmemCols - kPfAStages * kPfACols;
constexpr int kPfTokens = kPfAccCols;                // tokens per pass = accumulator columns (384 with 2 groups, 320 with 3)
constexpr int kPfBoxRows = 64;                       // token rows per TMA box
constexpr int kPfBoxBytes = kPfBoxRows * 128;        // [64 rows][64 k] fp16
constexpr int kPfBBoxes = 20;                        // token-tile region: 8 x 2, 5 x 4, 4 x 5 or 3 x 6 boxes per stage
constexpr int kPfBStages = 8;                        // most token-tile stages
constexpr int kPfRingDepth = 2;
constexpr int kPfThreads = 32 * (2 + kPfDecodeWarps);
constexpr int kPfSmem = kPfBBoxes * kPfBoxBytes + kPfDecodeWarps * kPfRingDepth * kStageBytes + 1024 + 256;
static_assert(kPfSmem <= 232448, "shared memory of the prefill GEMM");
constexpr unsigned long long kPfWaitNs = 2000000000ull;   // a wait that lasts 2 s is treated as a hang

struct PfPass { int expert, row0, ntok, pad; };

struct PfGemmArgs
{
    const int64_t* table;
    const int* plan;          // [0] number of passes, then PfPass records from int 4 on
    float* out0; float* out1; // gate|up: acc_g, acc_u [pairs][I]; down: y [pairs][H]
    int* status;              // [0] != 0: a wait timed out (device side), the results are invalid
    int H, I, nm_gu, nm_dn, down;
};

// ---------------------------------------------------------------- mbarrier / tcgen05 / TMA primitives
__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
// bounded wait for the phase with the given parity; false = aborted (by this or another thread of the CTA)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    const uint32_t a = saddr(bar);
    unsigned long long t0 = 0;
    for (uint32_t i = 0;; ++i)
    {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if ((i & 255u) == 255u)
        {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (t0 == 0) t0 = t;
            else if (t - t0 > kPfWaitNs) break;
        }
    }
    *abort_flag = 1;
    return false;
}
// The producer and MMA warps run their loops with all 32 lanes converged (so that addresses, descriptors and
// coordinates are warp-uniform values) and one elected lane issues the asynchronous instruction.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag)) != 0;
}
__device__ __forceinline__ void mbar_expect_tx_elect(uint64_t* bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_elect(uint64_t* bar)
{
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t@e mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d_elect(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n\t}"
                 ::"r"(saddr(dst)), "l"(map), "r"(saddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(saddr(dst)), "l"(map), "r"(saddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit_elect(uint64_t* bar)
{
    asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; fp16 operands, fp32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The four K = 16 steps of one 64-wide k-block, issued by one elected lane of a converged warp.  The weight operand is
// in tensor memory (8 columns per step), the token operand in shared memory (descriptor advances by 32 B, in 16-byte
// units on the low word: shared-memory addresses fit its 14-bit field).  first == 0: the first MMA overwrites the
// accumulator.
__device__ __forceinline__ void tc_mma_kblock(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t first)
{
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 db;\n\t.reg .b32 ta, tb;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
        "setp.eq.b32 p, %4, %4;\n\t"
        "add.u32 ta, %1, 8;\n\tadd.u32 tb, %2, 2;\n\tmov.b64 db, {tb, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
        "add.u32 ta, %1, 16;\n\tadd.u32 tb, %2, 4;\n\tmov.b64 db, {tb, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
        "add.u32 ta, %1, 24;\n\tadd.u32 tb, %2, 6;\n\tmov.b64 db, {tb, %3};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, p;\n\t"
        "}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(first) : "memory");
}
// The same for a token tile cut into two column halves with their own accumulator columns (alternating chains).
__device__ __forceinline__ void tc_mma_kblock2(uint32_t tmem_d0, uint32_t tmem_d1, uint32_t tmem_a, uint32_t b_lo0, uint32_t b_lo1,
                                               uint32_t b_hi, uint32_t idesc0, uint32_t idesc1, uint32_t first)
{
    asm volatile(
        "{\n\t.reg .pred p, e;\n\t.reg .b64 db;\n\t.reg .b32 ta, tb;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %8, 0;\n\t"
        "mov.b64 db, {%3, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%2], db, %6, p;\n\t"
        "mov.b64 db, {%4, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], db, %7, p;\n\t"
        "setp.eq.b32 p, %6, %6;\n\t"
        "add.u32 ta, %2, 8;\n\tadd.u32 tb, %3, 2;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %6, p;\n\t"
        "add.u32 tb, %4, 2;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], [ta], db, %7, p;\n\t"
        "add.u32 ta, %2, 16;\n\tadd.u32 tb, %3, 4;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %6, p;\n\t"
        "add.u32 tb, %4, 4;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], [ta], db, %7, p;\n\t"
        "add.u32 ta, %2, 24;\n\tadd.u32 tb, %3, 6;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %6, p;\n\t"
        "add.u32 tb, %4, 6;\n\tmov.b64 db, {tb, %5};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], [ta], db, %7, p;\n\t"
        "}"
        ::"r"(tmem_d0), "r"(tmem_d1), "r"(tmem_a), "r"(b_lo0), "r"(b_lo1), "r"(b_hi), "r"(idesc0), "r"(idesc1), "r"(first) : "memory");
}
// 16 lanes x 256 bits of tensor memory from a warp: lane (g, t4) supplies lane g columns 2 t4, 2 t4 + 1 (r0, r1) and
// lane g + 8, same columns (r2, r3) - the layout of an m16n8 fragment
__device__ __forceinline__ void tmem_st_16x256b(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3)
{
    asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// shared-memory operand descriptor: start address, leading / stride byte offsets (all >> 4), descriptor version 1,
// layout 0 = no swizzle, 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout)
{
    const uint32_t lo = ((addr >> 4) & 0x3FFFu) | (((lbo >> 4) & 0x3FFFu) << 16);
    const uint32_t hi = ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (layout << 29);
    return ((uint64_t)hi << 32) | lo;
}
// kind::f16 instruction descriptor: D fp32, A/B fp16 K-major, M 128, N tokens
__device__ __forceinline__ uint32_t instr_desc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | (8u << 24); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, "
                 "%26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                   "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                   "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- decode warps
struct PfShared
{
    uint64_t full_b[kPfBStages], empty_b[kPfBStages], full_a[kPfAStages], empty_a[kPfAStages], acc_full, acc_empty;
    uint32_t tmem_base;
    volatile int abort_flag;
};
// The token-tile region (20 boxes) is cut into stages of 2, 4, 5 or 6 boxes (8, 5, 4 or 3 stages) for a pass of nbox
// boxes per k-block.  Passes with the same stage size share the stage barriers freely; when the stage size changes
// between two items of a CTA the new stages overlap old ones at other indices, so the producer first waits until every
// stage of the old layout has been released.
__device__ __forceinline__ int b_stage_boxes(int nbox) { return nbox <= 2 ? 2 : nbox <= 4 ? 4 : nbox <= 5 ? 5 : 6; }
__device__ __forceinline__ int b_stages(int nbox) { return nbox <= 2 ? 8 : nbox <= 4 ? 5 : nbox <= 5 ? 4 : 3; }

// A unit is decoded whole (8 k-steps) by one warp: k-steps 0..3 fill the weight tile of k-block 2 c, k-steps 4..7 the
// tile of k-block 2 c + 1.  The sink does the stage hand-over in between: wait until the MMAs that last read the
// stage are done, store the fragments, wait for the stores, signal "full".
struct UnitSink
{
    uint32_t tmem_a;      // tensor-memory address of the warp's 16 lanes in weight-tile stage 0
    PfShared* sh; uint32_t it0; int lane; bool* ok;
    template <int T>
    __device__ __forceinline__ void operator()(std::integral_constant<int, T>, const uint32_t (&a)[4]) const
    {
        const uint32_t it = it0 + (T >> 2), sa = it % kPfAStages;
        if constexpr ((T & 3) == 0)
        {
            if (*ok && !mbar_wait(&sh->empty_a[sa], ((it / kPfAStages) & 1u) ^ 1u, &sh->abort_flag)) *ok = false;
            *ok = __shfl_sync(0xffffffffu, (int)*ok, 0) != 0;
            tc_fence_after();
        }
        if (*ok)      // warp-uniform
        {
            // a[0], a[2]: row g, k = 2 t4 + {0,1} and 8 + 2 t4 + {0,1}; a[1], a[3]: row g + 8
            tmem_st_16x256b(tmem_a + sa * kPfACols + (T & 3) * 8, a[0], a[2], a[1], a[3]);
            if constexpr ((T & 3) == 3)
            {
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&sh->full_a[sa]);
            }
        }
    }
};

// One decode warp, one item: its strip over the chunks c = GROUP, GROUP + 2, ... (the other group of 8 warps takes the
// other parity), i.e. k-blocks 4 i + 2 GROUP and + 1.  it_base = k-blocks of earlier items.  false = aborted.
template <bool REFINED, int RC, int BK, class Mid>
__device__ __forceinline__ bool decode_strip(const ProjPlanes& P, const StripRef& sr, int C, int NS, int lane, int group,
                                             uint32_t tmem_a, uint32_t ring, PfShared* sh, uint32_t it_base, Mid& mid)
{
    // per-unit scalars of this warp's chunks, one chunk (group + kPfGroups * lane) per lane: ring signs and, for refined units,
    // the block word with its fp16 multiplier / addend (computed once here instead of by every lane of every unit)
    uint32_t var_b = 0, ac = 0, mbn = 0;
    {
        const int ch = group + kPfGroups * lane;
        if (ch < C)
        {
            if (P.var) var_b = __ldg(P.var + sr.unit0 + ch);
            if constexpr (REFINED)
                if (chunk_refined(sr, ch))
                {
                    mbn = __ldg(P.d4 + sr.res0 + refined_before(sr, ch)) & 0xFFFFu;
                    ac = block_multipliers(mbn);
                }
        }
    }
    RecordCursor<BK> cb;
    cb.init(P.base, (size_t)NS * C * 32, sr.unit0, lane);
    RecordCursor<RC> cr;
    if constexpr (REFINED) cr.init(P.p4, sr.res_nrec, sr.res0, lane);
    auto issue = [&](int ch, uint32_t st) {
        cb.copy(st, ch, lane);
        if constexpr (REFINED)
            if (chunk_refined(sr, ch)) cr.copy(st + kStageBase, refined_before(sr, ch), lane);
    };
#pragma unroll
    for (int d = 0; d < kPfRingDepth - 1; ++d)
    {
        if (group + kPfGroups * d < C) issue(group + kPfGroups * d, ring + d * kStageBytes);
        cp_async_commit();
    }
    int slot = 0, slot_in = kPfRingDepth - 1, i = 0;
    bool ok = true;
    for (int ch = group; ch < C; ch += kPfGroups, ++i)
    {
        if (ch + kPfGroups * (kPfRingDepth - 1) < C) issue(ch + kPfGroups * (kPfRingDepth - 1), ring + slot_in * kStageBytes);
        cp_async_commit();
        cp_async_wait<kPfRingDepth - 1>();
        const uint32_t st = ring + slot * kStageBytes;
        slot = slot + 1 == kPfRingDepth ? 0 : slot + 1;
        slot_in = slot_in + 1 == kPfRingDepth ? 0 : slot_in + 1;
        const uint32_t sign2 = sign_mask(__shfl_sync(0xffffffffu, var_b, i), lane);
        uint32_t wb[Pattern<BK>::kWords + 2], wr[Pattern<RC>::kWords + 2];
        RecordCursor<BK>::read(wb, st, lane);
        const UnitSink sink{tmem_a, sh, it_base + 2 * (uint32_t)ch, lane, &ok};
        bool refined = false;
        if constexpr (REFINED) refined = chunk_refined(sr, ch);
        if (refined)
        {
            const uint32_t acw = __shfl_sync(0xffffffffu, ac, i), mb = __shfl_sync(0xffffffffu, mbn, i);
            RecordCursor<RC>::read(wr, st + kStageBase, lane);
            decode_unit<true, RC, BK>(wb, wr, consts_level4(acw, mb, sign2), lane, sink);
        }
        else
            decode_unit<false, 0, BK>(wb, wr, consts_level2(sign2), lane, sink);
        if (i == 0) mid();      // the previous item's epilogue, once this item's first tiles are on their way
    }
    cp_async_wait<0>();
    return ok;
}

template <class Mid>
__device__ __forceinline__ bool decode_item(const ProjPlanes& P, int level, int rc, int bk, int strip, int C, int NS, int nm, int lane, int group,
                                            uint32_t tmem_a, uint8_t* ring, PfShared* sh, uint32_t it_base, Mid& mid)
{
    const StripRef sr = locate_strip(P, strip, C, NS, nm, level >= 4);
    bool ok = true;
#define NQ_RUN(REF, RCV, BKV) ok = decode_strip<REF, RCV, BKV>(P, sr, C, NS, lane, group, tmem_a, smem_addr(ring), sh, it_base, mid)
    NQ_WITH_CODES(level >= 4, rc, bk, 0x3FF, NQ_RUN);
#undef NQ_RUN
    return ok;
}

// grid = resident CTAs (one per SM), 576 threads
__global__ void __launch_bounds__(kPfThreads, 1) pf_gemm_kernel(const __grid_constant__ CUtensorMap tmap0,
                                                                const __grid_constant__ CUtensorMap tmap1, PfGemmArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* b_tiles = smem;                                  // token tiles [rows][64 k] fp16, 128-byte swizzle (TMA boxes)
    uint8_t* rings = smem + kPfBBoxes * kPfBoxBytes;          // per decode warp: kPfRingDepth plane stages
    PfShared* sh = (PfShared*)(rings + kPfDecodeWarps * kPfRingDepth * kStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0)
    {
        for (int s = 0; s < kPfBStages; ++s) { mbar_init(&sh->full_b[s], 1); mbar_init(&sh->empty_b[s], 1); }
        for (int s = 0; s < kPfAStages; ++s) { mbar_init(&sh->full_a[s], 8); mbar_init(&sh->empty_a[s], 1); }
        mbar_init(&sh->acc_full, 1); mbar_init(&sh->acc_empty, kPfDecodeWarps);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1)
    {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&sh->tmem_base)), "r"(kPfTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    const int N = a.down ? a.H : 2 * a.I, K = a.down ? a.I : a.H, C = K / 128, NS = N / 16, groups = N / 128, nkb = K / 64;
    const int npass = a.plan[0], nitems = npass * groups;
    const PfPass* passes = (const PfPass*)(a.plan + 4);
    uint32_t it = 0, nitem = 0;     // k-blocks / items handled so far by this role (phases of the A-stage and accumulator barriers)
    uint32_t par_b = 0;                  // bit s: parity of the times token-tile stage s was used (its stage count changes from pass to pass)
    int last_sbox = 0;                   // producer: stage size of the previous item

    // decode warps: accumulator [128 weight rows x ntok] of item number n of this CTA -> out.  TMEM lanes 32 q .. 32 q + 31
    // (the quarter this warp may read) are weight rows; the four warps of a quarter take 32-column chunks in turn.
    PfPass prev{};
    int prev_wg = 0, prev_up = 0;
    bool have_prev = false;
    auto epilogue = [&](const PfPass& ps, int wg, int up, uint32_t n) {
        bool ok = true;
        if (lane == 0 && !mbar_wait(&sh->acc_full, n & 1u, &sh->abort_flag)) ok = false;
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) return;
        tc_fence_after();
        const int q = warp & 3, cpart = (warp - 2) >> 2;
        const int ncol = (up ? wg - a.I / 128 : wg) * 128 + q * 32 + lane;
        float* out = up ? a.out1 : a.out0;
        const int ld = a.down ? a.H : a.I;
        for (int c0 = cpart * 32; c0 < ps.ntok; c0 += 32 * (kPfDecodeWarps / 4))
        {
            uint32_t v[32];
            tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + c0, v);
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (c0 + j < ps.ntok) out[(size_t)(ps.row0 + c0 + j) * ld + ncol] = __uint_as_float(v[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh->acc_empty);
    };

    for (int item = blockIdx.x; item < nitems; item += gridDim.x, ++nitem)
    {
        const int pi = item / groups, wg = item - pi * groups;
        const PfPass ps = passes[pi];
        const int ntok16 = (ps.ntok + 15) & ~15, nbox = (ps.ntok + kPfBoxRows - 1) / kPfBoxRows, nb = b_stages(nbox);
        const int sbox = b_stage_boxes(nbox);
        const int up = !a.down && wg >= a.I / 128;
        if (warp == 0)
        {
            // ---- token tiles by TMA, up to nb k-blocks ahead of the MMAs
            const CUtensorMap* map = up ? &tmap1 : &tmap0;
            bool ok = true;
            if (sbox != last_sbox)
                for (int s = 0; ok && s < kPfBStages; ++s) ok = mbar_wait_warp(&sh->empty_b[s], ((par_b >> s) & 1u) ^ 1u, &sh->abort_flag);
            last_sbox = sbox;
            for (int kb = 0, s = 0; ok && kb < nkb; ++kb, s = s + 1 == nb ? 0 : s + 1)
            {
                if (!mbar_wait_warp(&sh->empty_b[s], ((par_b >> s) & 1u) ^ 1u, &sh->abort_flag)) break;
                par_b ^= 1u << s;
                mbar_expect_tx_elect(&sh->full_b[s], (uint32_t)nbox * kPfBoxBytes);
                for (int j = 0; j < nbox; ++j)
                    tma_load_2d_elect(b_tiles + (s * sbox + j) * kPfBoxBytes, map, kb * 64, ps.row0 + j * kPfBoxRows, &sh->full_b[s]);
            }
        }
        else if (warp == 1)
        {
            // ---- MMA issue
            bool ok = mbar_wait_warp(&sh->acc_empty, (nitem & 1u) ^ 1u, &sh->abort_flag);   // epilogue of the previous item has drained TMEM
            tc_fence_after();
            // N <= 256 per instruction: one MMA per k-step, or two of (nearly) equal width
            const int n0 = ntok16 <= NQ_PF_SPLIT ? ntok16 : ((ntok16 / 2 + 15) & ~15), n1 = ntok16 - n0;
            const uint32_t idesc0 = instr_desc(n0), idesc1 = instr_desc(n1 > 0 ? n1 : 16);
            const uint64_t bdesc0 = smem_desc(saddr(b_tiles), 16, 1024, 2);
            const uint32_t b_lo0 = (uint32_t)bdesc0, b_hi = (uint32_t)(bdesc0 >> 32);
            const uint32_t b_step = (uint32_t)(sbox * (kPfBoxBytes >> 4));
            uint32_t s = 0, b_lo = b_lo0;                 // token-tile stage of this k-block and its descriptor
            for (int kb = 0; ok && kb < nkb; ++kb, ++it)
            {
                const uint32_t sa = it % kPfAStages;
                if (!mbar_wait_warp(&sh->full_b[s], (par_b >> s) & 1u, &sh->abort_flag) ||
                    !mbar_wait_warp(&sh->full_a[sa], (it / kPfAStages) & 1u, &sh->abort_flag)) { ok = false; break; }
                par_b ^= 1u << s;
                tc_fence_after();
                const uint32_t ta = tmem + kPfAccCols + sa * kPfACols;
                if (n1 > 0) tc_mma_kblock2(tmem, tmem + n0, ta, b_lo, b_lo + (uint32_t)(n0 * 8), b_hi, idesc0, idesc1, (uint32_t)kb);
                else tc_mma_kblock(tmem, ta, b_lo, b_hi, idesc0, (uint32_t)kb);
                tc_commit_elect(&sh->empty_a[sa]);       // both arrive when the MMAs above have read their operands
                tc_commit_elect(&sh->empty_b[s]);
                if (++s == (uint32_t)nb) { s = 0; b_lo = b_lo0; } else b_lo += b_step;
            }
            if (ok) tc_commit_elect(&sh->acc_full);
        }
        else
        {
            // ---- decode, then epilogue
            // A warp may touch only the 32 tensor-memory lanes of its quarter (warp % 4): the four decode warps of a
            // quarter take its two strips x the chunk groups.
            const int dw = warp - 2, qd = warp & 3, sub = (dw >> 2) & 1, half = dw >> 3, sidx = 2 * qd + sub;      // half = chunk group
            const uint32_t tmem_a = tmem + ((uint32_t)(32 * qd + 16 * sub) << 16) + kPfAccCols;
            const int64_t* row = a.table + (int64_t)ps.expert * kTableWidth;
            const int level = (int)row[0];
            const ProjPlanes P = planes_from_row(row, a.down);
            const int rc = (int)row[10 + a.down], nm = a.down ? a.nm_dn : a.nm_gu, bk = (int)(row[19] >> (8 * a.down)) & 0xFF;
            uint8_t* ring = rings + dw * kPfRingDepth * kStageBytes;
            // group `half` of 8 warps decodes the chunks c = half (mod kPfGroups): k-blocks 2 c and 2 c + 1.  The epilogue
            // of the previous item runs after this item's first unit is decoded: the MMAs of the previous item's last
            // k-blocks finish meanwhile, and the tensor pipe finds tiles waiting when the accumulator is free again.
            auto mid = [&]() { if (have_prev) { epilogue(prev, prev_wg, prev_up, nitem - 1); have_prev = false; } };
            const bool ok = decode_item(P, level, rc, bk, wg * 8 + sidx, C, NS, nm, lane, half, tmem_a, ring, sh, it, mid);
            it += nkb;
            mid();                                   // (an item of fewer than two chunks: its second warp group decodes nothing)
            if (ok) { prev = ps; prev_wg = wg; prev_up = up; have_prev = true; }
        }
        if (sh->abort_flag) break;
    }
    if (warp >= 2 && have_prev && !sh->abort_flag) epilogue(prev, prev_wg, prev_up, nitem - 1);
    if (sh->abort_flag && threadIdx.x == 0) atomicExch(a.status, 1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPfTmemCols) : "memory");
}

// ---------------------------------------------------------------- pass plan (device side, no host sync)
// counts[e] = routed pairs of expert e (pairs are sorted by expert).  A pass = one expert x up to 384 of its pairs;
// experts at level 0 get none.  plan: [0] passes, [1] pairs covered, then PfPass records from int 4 on.
__global__ void pf_plan_kernel(const int* __restrict__ counts, const int64_t* __restrict__ table, int E, int* plan, int max_passes)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    PfPass* out = (PfPass*)(plan + 4);
    int n = 0, row = 0, covered = 0;
    for (int e = 0; e < E; ++e)
    {
        const int c = counts[e];
        if (c > 0 && table[(int64_t)e * kTableWidth] > 0)
            for (int t0 = 0; t0 < c && n < max_passes; t0 += kPfTokens)
            {
                out[n].expert = e; out[n].row0 = row + t0; out[n].ntok = c - t0 < kPfTokens ? c - t0 : kPfTokens; out[n].pad = 0;
                covered += out[n].ntok; ++n;
            }
        row += c;
    }
    plan[0] = n; plan[1] = covered; plan[2] = plan[3] = 0;
}

// The same from the sorted pair list of a whole window: start[e] = first pair of expert e (start[E] = end of the last
// expert's pairs); the plan covers the pairs [pair0, pair0 + npairs) with rows counted from pair0.
__global__ void pf_plan_window_kernel(const int* __restrict__ start, const int64_t* __restrict__ table, int E, int pair0, int npairs,
                                      int* plan, int max_passes)
{
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    PfPass* out = (PfPass*)(plan + 4);
    int n = 0, covered = 0;
    for (int e = 0; e < E; ++e)
    {
        const int a = max(start[e], pair0), b = min(start[e + 1], pair0 + npairs), c = b - a;
        if (c > 0 && table[(int64_t)e * kTableWidth] > 0)
            for (int t0 = 0; t0 < c && n < max_passes; t0 += kPfTokens)
            {
                out[n].expert = e; out[n].row0 = a - pair0 + t0; out[n].ntok = c - t0 < kPfTokens ? c - t0 : kPfTokens; out[n].pad = 0;
                covered += out[n].ntok; ++n;
            }
    }
    plan[0] = n; plan[1] = covered; plan[2] = plan[3] = 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// tensor map of a row-major fp16 matrix [rows][cols]: boxes of 64 columns x 64 rows, 128-byte swizzle, zero fill
static int make_tile_map(CUtensorMap* map, const void* base, size_t rows, size_t cols)
{
    static EncodeTiledFn fn = nullptr;
    if (!fn)
    {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p)
            return fail(NQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = (EncodeTiledFn)p;
    }
    const cuuint64_t dims[2] = {cols, rows}, strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kPfBoxRows}, estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return NQ_OK;
}

}  // namespace nq

extern "C" {

int nq_pf_plan_ints(int E, int pairs) { return 4 + 4 * (E + pairs / nq::kPfTokens + 1); }

int nq_pf_plan(const int32_t* counts, const int64_t* table, int E, int pairs, int32_t* plan, int plan_ints, void* stream)
{
    NQ_REQUIRE(counts && table && plan && E > 0 && pairs >= 0, "nq_pf_plan: bad arguments");
    NQ_REQUIRE(plan_ints >= nq_pf_plan_ints(E, pairs), "nq_pf_plan: plan needs %d ints", nq_pf_plan_ints(E, pairs));
    nq::pf_plan_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counts, table, E, plan, (plan_ints - 4) / 4);
    return nq::check_launch("nq_pf_plan");
}

int nq_pf_plan_window(const int32_t* start, const int64_t* table, int E, int pair0, int npairs, int32_t* plan, int plan_ints, void* stream)
{
    NQ_REQUIRE(start && table && plan && E > 0 && pair0 >= 0 && npairs >= 0, "nq_pf_plan_window: bad arguments");
    NQ_REQUIRE(plan_ints >= nq_pf_plan_ints(E, npairs), "nq_pf_plan_window: plan needs %d ints", nq_pf_plan_ints(E, npairs));
    nq::pf_plan_window_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(start, table, E, pair0, npairs, plan, (plan_ints - 4) / 4);
    return nq::check_launch("nq_pf_plan_window");
}

int nq_pf_gemm(const int64_t* table, const int32_t* plan, const void* act0, const void* act1, int pairs, float* out0, float* out1,
               int H, int I, int nm_gu, int nm_dn, int down, int32_t* status, void* stream)
{
    NQ_REQUIRE(table && plan && act0 && out0 && status, "nq_pf_gemm: null pointer");
    NQ_REQUIRE(down || (act1 && out1), "nq_pf_gemm: the gate|up projection needs both activation matrices and both outputs");
    NQ_REQUIRE(H > 0 && I > 0 && H % 128 == 0 && I % 128 == 0 && H / 128 <= 64 && I / 128 <= 64, "nq_pf_gemm: H = %d, I = %d", H, I);
    NQ_REQUIRE(pairs >= 0, "nq_pf_gemm: pairs = %d", pairs);
    if (pairs == 0) return NQ_OK;
    NQ_REQUIRE(nq::aligned16(act0) && nq::aligned16(act1) && nq::aligned16(out0), "nq_pf_gemm: matrices must be 16-byte aligned");
    // SM count and the shared-memory opt-in are per device: cached per device ordinal
    static int ctas_of[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nq::fail(NQ_ERR_CUDA, "nq_pf_gemm: no usable current device");
    if (!ctas_of[dev])
    {
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (cudaFuncSetAttribute((const void*)nq::pf_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, nq::kPfSmem) != cudaSuccess)
            return nq::fail(NQ_ERR_CUDA, "nq_pf_gemm: cannot reserve %d bytes of shared memory", nq::kPfSmem);
        ctas_of[dev] = sms;
    }
    const int ctas = ctas_of[dev];
    CUtensorMap m0, m1;
    const size_t K = down ? I : H;
    if (int e = nq::make_tile_map(&m0, act0, (size_t)pairs, K)) return e;
    if (int e = nq::make_tile_map(&m1, down ? act0 : act1, (size_t)pairs, K)) return e;
    nq::PfGemmArgs a{};
    a.table = table; a.plan = plan; a.out0 = out0; a.out1 = out1; a.status = status;
    a.H = H; a.I = I; a.nm_gu = nm_gu; a.nm_dn = nm_dn; a.down = down ? 1 : 0;
    nq::pf_gemm_kernel<<<ctas, nq::kPfThreads, nq::kPfSmem, (cudaStream_t)stream>>>(m0, m1, a);
    return nq::check_launch("nq_pf_gemm");
}

}  // extern "C"
