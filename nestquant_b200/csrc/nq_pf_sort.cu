// Prefill path, the permutation: the (token, pick) pairs of a window sorted by expert, as a stable counting sort in three
// small kernels and without a host sync.
//
// Replaces the host side of the reference's prefill (sm120/moe.py:293-298: torch.argsort of the flattened expert ids,
// scatter_add for the counts, a .cpu() of the counts) and this library's earlier use of the same torch operators.
//   bins     expert id 0 .. E - 1, plus bin E for the picks that contribute nothing (id outside [0, E), expert not resident
//            on this GPU, routing weight 0): they sort behind every real pair and no kernel touches their rows.
//   slices   a warp owns 256 consecutive picks.  Pass 1 counts its picks per bin; pass 2 (one CTA) turns the counts into the
//            offset of every (slice, bin) and the start of every bin; pass 3 walks the slice again, 32 picks at a time in pick
//            order, and places each pick at start[bin] + offset[slice][bin] + its rank among the slice's earlier picks of that
//            bin (match.any gives the lanes of a step that share a bin).  Equal experts keep pick order: the result does
//            not depend on timing.
// Outputs: pe[p] = expert (or E) and pt[p] = token of sorted pair p, pos[t * topk + k] = sorted index of a pick,
// start[0 .. E + 1] = first pair of each bin (start[E] = number of live pairs, start[E + 1] = all pairs), and, optionally,
// the routing-hit counts of this call (every pick with a valid id and a non-zero weight, whatever the expert's level) added
// to a device array that the caller zeroed.
#include <cuda_fp16.h>

#include "nq_common.cuh"
#include "nq_format.cuh"

namespace nq {

constexpr int kSortSlice = 256;      // picks per warp
constexpr int kSortWarps = 8;        // warps per CTA
constexpr int kSortMaxBins = 1025;   // experts + 1

__device__ __forceinline__ int pick_bin(const int64_t* __restrict__ sel, const __half* __restrict__ rw, const int64_t* __restrict__ table,
                                        int E, int i, bool* hit)
{
    const int64_t e = sel[i];
    const bool valid = e >= 0 && e < E && __half2float(rw[i]) != 0.f;
    *hit = valid;
    return valid && table[e * kTableWidth] > 0 ? (int)e : E;
}

// pass 1: hist[slice][bin] (and hits[e] += picks with a weight)
__global__ void __launch_bounds__(32 * kSortWarps) sort_count_kernel(const int64_t* __restrict__ sel, const __half* __restrict__ rw,
                                                                    const int64_t* __restrict__ table, int P, int E, int* hist, int* hits)
{
    extern __shared__ int s_hist[];      // [kSortWarps][E + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, slice = blockIdx.x * kSortWarps + warp, nb = E + 1;
    int* h = s_hist + warp * nb;
    for (int b = lane; b < nb; b += 32) h[b] = 0;
    __syncwarp();
    const int i0 = slice * kSortSlice;
    for (int i = i0 + lane; i < i0 + kSortSlice && i < P; i += 32)
    {
        bool hit;
        const int b = pick_bin(sel, rw, table, E, i, &hit);
        atomicAdd(h + b, 1);
        if (hits && hit) atomicAdd(hits + (int)sel[i], 1);
    }
    __syncwarp();
    if (i0 < P)
        for (int b = lane; b < nb; b += 32) hist[(size_t)slice * nb + b] = h[b];
}

// pass 2 (one CTA): hist[slice][bin] -> offset of the slice inside the bin; start[bin] = first pair of the bin
__global__ void __launch_bounds__(1024) sort_scan_kernel(int* hist, int nslices, int E, int* start)
{
    __shared__ int s_total[kSortMaxBins + 1];
    const int nb = E + 1;
    for (int b = threadIdx.x; b < nb; b += blockDim.x)
    {
        int run = 0;
        for (int s = 0; s < nslices; ++s)
        {
            const int c = hist[(size_t)s * nb + b];
            hist[(size_t)s * nb + b] = run;
            run += c;
        }
        s_total[b] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0)
    {
        int run = 0;
        for (int b = 0; b < nb; ++b) { start[b] = run; run += s_total[b]; }
        start[nb] = run;
    }
}

// pass 3: place every pick
__global__ void __launch_bounds__(32 * kSortWarps) sort_place_kernel(const int64_t* __restrict__ sel, const __half* __restrict__ rw,
                                                                    const int64_t* __restrict__ table, int P, int E, int topk,
                                                                    const int* __restrict__ hist, const int* __restrict__ start,
                                                                    int* pe, int* pt, int* pos)
{
    extern __shared__ int s_next[];      // [kSortWarps][E + 1]: next free place of each bin for this slice
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, slice = blockIdx.x * kSortWarps + warp, nb = E + 1;
    int* nx = s_next + warp * nb;
    const int i0 = slice * kSortSlice;
    if (i0 >= P) return;                 // warp-uniform
    for (int b = lane; b < nb; b += 32) nx[b] = start[b] + hist[(size_t)slice * nb + b];
    __syncwarp();
    for (int base = i0; base < i0 + kSortSlice && base < P; base += 32)
    {
        const int i = base + lane;
        const bool in = i < P;
        bool hit;
        const int b = in ? pick_bin(sel, rw, table, E, i, &hit) : -1 - lane;      // idle lanes get bins of their own
        const unsigned same = __match_any_sync(0xffffffffu, b);
        const int rank = __popc(same & ((1u << lane) - 1u));
        int p = 0;
        if (in) p = nx[b] + rank;
        __syncwarp();
        if (in && rank == __popc(same) - 1) nx[b] = p + 1;                         // the last lane of each bin moves the bin on
        __syncwarp();
        if (in) { pe[p] = b; pt[p] = i / topk; pos[i] = p; }
    }
}

}  // namespace nq

extern "C" {

int nq_pf_sort_scratch_ints(int pairs, int E)
{
    if (pairs < 0 || E < 1) return 0;
    const long long slices = ((long long)pairs + nq::kSortSlice - 1) / nq::kSortSlice;
    const long long n = slices * (E + 1);
    return n > 0x7fffffffLL ? 0 : (int)n;
}

int nq_pf_sort(const int64_t* sel, const void* rw, const int64_t* table, int T, int topk, int E, int32_t* pe, int32_t* pt, int32_t* pos,
               int32_t* start, int32_t* hits, int32_t* scratch, int scratch_ints, void* stream)
{
    NQ_REQUIRE(T >= 0 && topk >= 1 && E >= 1 && E + 1 <= nq::kSortMaxBins, "nq_pf_sort: T = %d, topk = %d, E = %d", T, topk, E);
    NQ_REQUIRE((long long)T * topk <= 0x7fffffffLL, "nq_pf_sort: too many pairs");
    const int P = T * topk;
    NQ_REQUIRE(start, "nq_pf_sort: null start array");
    cudaStream_t st = (cudaStream_t)stream;
    if (P == 0) return cudaMemsetAsync(start, 0, sizeof(int32_t) * (E + 2), st) == cudaSuccess ? NQ_OK : nq::fail(NQ_ERR_CUDA, "nq_pf_sort: memset failed");
    NQ_REQUIRE(sel && rw && table && pe && pt && pos && scratch, "nq_pf_sort: null pointer");
    NQ_REQUIRE(scratch_ints >= nq_pf_sort_scratch_ints(P, E), "nq_pf_sort: scratch needs %d ints", nq_pf_sort_scratch_ints(P, E));
    const int slices = (P + nq::kSortSlice - 1) / nq::kSortSlice, ctas = (slices + nq::kSortWarps - 1) / nq::kSortWarps;
    const size_t smem = sizeof(int) * nq::kSortWarps * (E + 1);
    nq::sort_count_kernel<<<ctas, 32 * nq::kSortWarps, smem, st>>>(sel, (const __half*)rw, table, P, E, scratch, hits);
    if (int e = nq::check_launch("nq_pf_sort(count)")) return e;
    nq::sort_scan_kernel<<<1, 1024, 0, st>>>(scratch, slices, E, start);
    if (int e = nq::check_launch("nq_pf_sort(scan)")) return e;
    nq::sort_place_kernel<<<ctas, 32 * nq::kSortWarps, smem, st>>>(sel, (const __half*)rw, table, P, E, topk, scratch, start, pe, pt, pos);
    return nq::check_launch("nq_pf_sort(place)");
}

}  // extern "C"
