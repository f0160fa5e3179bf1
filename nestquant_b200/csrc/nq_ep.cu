// Expert-parallel combine over peer memory: out[t] = sum over the ranks r, in rank order, of the partial row rank r
// computed for token t, read straight from rank r's buffer over NVLink (plain peer loads).
//
// This is the return leg of the expert-parallel prefill (the reference names the exchange, sm120/eval/eval_reg.py:137-142;
// its serving path is tensor-parallel and has no counterpart kernel): instead of an all-to-all of the partial rows into a
// receive buffer followed by an indexed add, the owner of a token gathers and sums its partial rows in one pass.  The
// buffers are symmetric-memory allocations whose peer addresses the host passes in; the host brackets the call with the
// barriers that make the peers' rows complete before and keep them untouched during the reads.
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

}  // namespace nq

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
