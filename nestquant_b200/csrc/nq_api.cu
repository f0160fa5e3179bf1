// C ABI: error reporting, format queries and the table mailbox.
#include "nq_common.cuh"
#include "nq_format.cuh"

namespace nq {

char* error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}
int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

// One thread per expert.  The staged row is copied before the sequence number is published, so a host that sees
// applied_host[e] == seq knows every later launch on this stream reads the new row.
__global__ void mailbox_kernel(int64_t* table, const int64_t* stage, const int32_t* seq, int32_t* applied,
                               int32_t* applied_host, int E)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const int32_t s = *(const volatile int32_t*)(seq + e);
    if (s == applied[e]) return;
    const volatile int64_t* src = stage + (size_t)e * kTableWidth;
    int64_t* dst = table + (size_t)e * kTableWidth;
#pragma unroll
    for (int i = 0; i < kTableWidth; ++i) dst[i] = src[i];
    __threadfence_system();
    applied[e] = s;
    if (applied_host) *(volatile int32_t*)(applied_host + e) = s;
}

}  // namespace nq

extern "C" {

const char* nq_last_error(void) { return nq::error_buffer(); }
int nq_build_arch(void) { return 100; }

int nq_rk_codes(int64_t out[2])
{
    if (!out) return nq::fail(NQ_ERR_ARG, "nq_rk_codes: null output");
    out[0] = out[1] = (1 << nq::kNumCodes) - 1;   // every window code 0..9 is compiled into both projections
    return NQ_OK;
}
int nq_bk_codes(int64_t out[2])
{
    if (!out) return nq::fail(NQ_ERR_ARG, "nq_bk_codes: null output");
    out[0] = out[1] = 3;      // base codes 0 and 1 (code 1 with residual codes 3 and 9 at level 4)
    return NQ_OK;
}
size_t nq_plane_bytes(size_t nrec, int code)
{
    if (code < 0 || code >= nq::kNumCodes) return 0;
    const int bits = nq::record_bits(code);
    return nrec * (size_t)bits / 8 + ((bits % 16) ? 4 : 0);
}

int nq_mailbox(int64_t* table, const int64_t* stage, const int32_t* seq, int32_t* applied, int32_t* applied_host,
               int E, void* stream)
{
    NQ_REQUIRE(table && stage && seq && applied, "nq_mailbox: null pointer");
    NQ_REQUIRE(E > 0, "nq_mailbox: E = %d", E);
    nq::mailbox_kernel<<<(E + 127) / 128, 128, 0, (cudaStream_t)stream>>>(table, stage, seq, applied, applied_host, E);
    return nq::check_launch("nq_mailbox");
}

}  // extern "C"

// Promotion / demotion of one expert: bytes, then the staged table row, then the sequence number, in that order on one
// (side) stream, so the row can never become visible before the bytes it points at.  The next nq_mailbox on the compute
// stream picks the row up.  Host buffers must be pinned and stay untouched until the stream has passed the copies.
extern "C" int nq_promote(void* slot, const void* host_record, size_t record_bytes, int64_t* stage_row, const int64_t* host_row,
                          int32_t* seq_entry, const int32_t* host_seq, void* stream)
{
    NQ_REQUIRE(stage_row && host_row && seq_entry && host_seq, "nq_promote: null row or sequence pointer");
    NQ_REQUIRE(!(slot || host_record || record_bytes) || (slot && host_record && record_bytes),
               "nq_promote: slot, record and its size must be given together (or none of them for a demotion)");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaSuccess;
    if (slot && host_record && record_bytes)
        e = cudaMemcpyAsync(slot, host_record, record_bytes, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(stage_row, host_row, sizeof(int64_t) * nq::kTableWidth, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(seq_entry, host_seq, sizeof(int32_t), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return nq::fail(NQ_ERR_CUDA, "nq_promote: %s", cudaGetErrorString(e));
    return NQ_OK;
}
