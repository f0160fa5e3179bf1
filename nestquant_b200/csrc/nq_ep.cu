// Expert-parallel exchange over peer memory (plain peer loads over NVLink, no collective on the data path).
//
// Dispatch: every rank keeps its tokens' input rows in a symmetric buffer.  The prefill's first pass (nq_pf_pre with
// peer row pointers, nq_prefill.cu) reads the row of each of its pairs straight from the owner's buffer while it scales and
// rotates it: the dispatch is part of that kernel.  nq_ep_gather is the stand-alone form (a staging matrix indexed by
// global token gets the rows of exactly those tokens that picked one of this rank's experts).
// Combine: out[t] = sum over the ranks r, in rank order, of the partial row rank r computed for token t, read straight
// from rank r's buffer.
//
// This is the return leg of the expert-parallel prefill (the reference names the exchange, sm120/eval/eval_reg.py:137-142;
// its serving path is tensor-parallel and has no counterpart kernel): instead of an all-to-all of the partial rows into a
// receive buffer followed by an indexed add, the owner of a token gathers and sums its partial rows in one pass.  The
// buffers are symmetric-memory allocations whose peer addresses the host passes in; the host brackets the call with
// nq_ep_barrier, which makes the peers' rows complete before and keeps them untouched during the reads.
//
// Barrier: one small kernel per rank.  Rank r stores its call number into flag [r] of every peer (release, system scope)
// and waits until all of its own flags have reached that number (acquire, system scope).  The wait is bounded: when it
// runs out the kernel raises a status word and returns, so a peer that died or never arrives cannot hang this GPU.  The
// call number lives in device memory and is advanced by the kernel itself, so the call can be replayed from a CUDA graph.
// The kernels of different ranks run on different GPUs; never launch two ranks' barriers on one GPU and expect them to
// meet.
#include <cuda_fp16.h>

#include "nq_common.cuh"

namespace nq {

constexpr int kEpMaxRanks = 8;
struct EpPeers { const float* part[kEpMaxRanks]; };

// one CTA per token; rows[r * T + t] = row of token t in rank r's buffer, or -1 if rank r holds none of its picks
__global__ void __launch_bounds__(256) ep_combine_kernel(float* __restrict__ out, EpPeers peers, const int32_t* __restrict__ rows, int T, int H,
                                                         int world)
{
    const int t = blockIdx.x;
    int row[kEpMaxRanks];
#pragma unroll
    for (int r = 0; r < kEpMaxRanks; ++r) row[r] = r < world ? rows[(size_t)r * T + t] : -1;
    for (int c = threadIdx.x * 4; c < H; c += blockDim.x * 4)
    {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kEpMaxRanks; ++r)
            if (row[r] >= 0)
            {
                const float4 v = *(const float4*)(peers.part[r] + (size_t)row[r] * H + c);
                o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
            }
        *(float4*)(out + (size_t)t * H + c) = o;
    }
}

// one CTA per global token: copy its row from the owner's buffer if any of its picks with a weight belongs to `rank`
__global__ void __launch_bounds__(128) ep_gather_kernel(__half* __restrict__ xstage, EpPeers peers, const int64_t* __restrict__ sel,
                                                        const __half* __restrict__ rw, int tokens_per_rank, int topk, int H, int rank, int per)
{
    const int t = blockIdx.x;
    bool need = false;
    for (int k = 0; k < topk; ++k)
    {
        const int64_t e = sel[(size_t)t * topk + k];
        need |= e >= 0 && e / per == rank && __half2float(rw[(size_t)t * topk + k]) != 0.f;
    }
    if (!need) return;
    const int owner = t / tokens_per_rank;
    const uint4* src = (const uint4*)((const __half*)peers.part[owner] + (size_t)(t - owner * tokens_per_rank) * H);
    uint4* dst = (uint4*)(xstage + (size_t)t * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

struct EpFlags { int32_t* flags[kEpMaxRanks]; };

__global__ void __launch_bounds__(32) ep_barrier_kernel(EpFlags peers, int rank, int world, int32_t* epoch, int32_t* status,
                                                        unsigned long long timeout_ns)
{
    const int r = threadIdx.x;
    const int32_t e = *(volatile int32_t*)epoch + 1;
    __syncwarp();
    bool ok = true;
    if (r < world)
    {
        __threadfence_system();       // everything this GPU wrote before the barrier is visible to the peers first
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.flags[r] + rank), "r"(e) : "memory");
        const int32_t* mine = peers.flags[rank] + r;
        unsigned long long t0 = 0;
        for (unsigned i = 0;; ++i)
        {
            int32_t v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v - e >= 0) break;
            if ((i & 15u) == 15u)
            {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                if (t0 == 0) t0 = t;
                else if (t - t0 > timeout_ns) { ok = false; break; }
            }
            __nanosleep(200);
        }
    }
    if (!ok) atomicExch(status, 1);
    __syncwarp();
    if (r == 0) *epoch = e;
}

// The picks of every rank's tokens, read from the ranks' buffers: sel_all[w * T + t][k] = sel of rank w's token t;
// rw_mine = its weight where the pick belongs to one of this rank's experts, else 0 (other ranks' picks then sort away
// in this rank's prefill).
struct EpPicks { const int64_t* sel[kEpMaxRanks]; const __half* rw[kEpMaxRanks]; };
__global__ void __launch_bounds__(256) ep_picks_kernel(EpPicks peers, int n_per_rank, int world, int rank, int per, int64_t* __restrict__ sel_all,
                                                       __half* __restrict__ rw_mine)
{
    const int n = n_per_rank * world;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    {
        const int w = i / n_per_rank, j = i - w * n_per_rank;
        const int64_t e = peers.sel[w][j];
        const __half r = peers.rw[w][j];
        sel_all[i] = e;
        const bool mine = e >= 0 && e / per == rank;
        rw_mine[i] = mine ? r : __ushort_as_half((unsigned short)0);
    }
}

}  // namespace nq

extern "C" int nq_ep_barrier(int32_t* const* peer_flags, int rank, int world, int32_t* epoch, int32_t* status, long long timeout_ns,
                             void* stream)
{
    NQ_REQUIRE(world >= 1 && world <= nq::kEpMaxRanks && rank >= 0 && rank < world, "nq_ep_barrier: rank %d of %d", rank, world);
    NQ_REQUIRE(peer_flags && epoch && status && timeout_ns > 0, "nq_ep_barrier: null pointer or timeout %lld", timeout_ns);
    nq::EpFlags f{};
    for (int r = 0; r < world; ++r)
    {
        NQ_REQUIRE(peer_flags[r], "nq_ep_barrier: flags of rank %d are null", r);
        f.flags[r] = peer_flags[r];
    }
    nq::ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, rank, world, epoch, status, (unsigned long long)timeout_ns);
    return nq::check_launch("nq_ep_barrier");
}

extern "C" int nq_ep_picks(const int64_t* const* peer_sel, const void* const* peer_rw, int tokens_per_rank, int topk, int world, int rank,
                           int experts_per_rank, int64_t* sel_all, void* rw_mine, void* stream)
{
    NQ_REQUIRE(tokens_per_rank >= 0 && topk >= 1 && world >= 1 && world <= nq::kEpMaxRanks && rank >= 0 && rank < world && experts_per_rank >= 1,
               "nq_ep_picks: bad shape (tokens %d, topk %d, world %d, rank %d)", tokens_per_rank, topk, world, rank);
    if (tokens_per_rank == 0) return NQ_OK;
    NQ_REQUIRE(peer_sel && peer_rw && sel_all && rw_mine, "nq_ep_picks: null pointer");
    NQ_REQUIRE((long long)tokens_per_rank * topk * world < (1ll << 31), "nq_ep_picks: too many picks");
    nq::EpPicks p{};
    for (int r = 0; r < world; ++r)
    {
        NQ_REQUIRE(peer_sel[r] && peer_rw[r], "nq_ep_picks: buffer of rank %d is null", r);
        p.sel[r] = peer_sel[r]; p.rw[r] = (const __half*)peer_rw[r];
    }
    const int n = tokens_per_rank * topk * world, blocks = (n + 255) / 256;
    nq::ep_picks_kernel<<<blocks < 1184 ? blocks : 1184, 256, 0, (cudaStream_t)stream>>>(p, tokens_per_rank * topk, world, rank, experts_per_rank,
                                                                                        sel_all, (__half*)rw_mine);
    return nq::check_launch("nq_ep_picks");
}

extern "C" int nq_ep_gather(void* xstage, const void* const* peer_x, const int64_t* sel, const void* rw, int tokens_per_rank, int topk, int H,
                            int world, int rank, int experts_per_rank, void* stream)
{
    NQ_REQUIRE(tokens_per_rank >= 0 && topk >= 1 && H > 0 && H % 8 == 0 && world >= 1 && world <= nq::kEpMaxRanks && rank >= 0 && rank < world &&
               experts_per_rank >= 1, "nq_ep_gather: bad shape (tokens %d, topk %d, H %d, world %d, rank %d)", tokens_per_rank, topk, H, world, rank);
    if (tokens_per_rank == 0) return NQ_OK;
    NQ_REQUIRE(xstage && peer_x && sel && rw && nq::aligned16(xstage), "nq_ep_gather: null or misaligned pointer");
    nq::EpPeers p{};
    for (int r = 0; r < world; ++r)
    {
        NQ_REQUIRE(peer_x[r] && nq::aligned16(peer_x[r]), "nq_ep_gather: buffer of rank %d is null or misaligned", r);
        p.part[r] = (const float*)peer_x[r];
    }
    nq::ep_gather_kernel<<<world * tokens_per_rank, 128, 0, (cudaStream_t)stream>>>((__half*)xstage, p, sel, (const __half*)rw, tokens_per_rank, topk, H,
                                                                                    rank, experts_per_rank);
    return nq::check_launch("nq_ep_gather");
}

extern "C" int nq_ep_combine(float* out, const void* const* peer_parts, const int32_t* rows, int T, int H, int world, void* stream)
{
    NQ_REQUIRE(T >= 0 && H > 0 && H % 4 == 0 && world >= 1 && world <= nq::kEpMaxRanks, "nq_ep_combine: T = %d, H = %d, world = %d", T, H, world);
    if (T == 0) return NQ_OK;
    NQ_REQUIRE(out && peer_parts && rows && nq::aligned16(out), "nq_ep_combine: null or misaligned pointer");
    nq::EpPeers p{};
    for (int r = 0; r < world; ++r)
    {
        NQ_REQUIRE(peer_parts[r] && nq::aligned16(peer_parts[r]), "nq_ep_combine: buffer of rank %d is null or misaligned", r);
        p.part[r] = (const float*)peer_parts[r];
    }
    nq::ep_combine_kernel<<<T, 256, 0, (cudaStream_t)stream>>>(out, p, rows, T, H, world);
    return nq::check_launch("nq_ep_combine");
}
