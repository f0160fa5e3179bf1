// Decode-path MoE layer call for hosts that must not allocate.
//
// Some callers of this library cannot create device buffers at the moment they need a layer call: a plugin that runs
// inside a serving engine whose device memory was carved up at start-up (every remaining byte already belongs to the
// KV cache, so a late cudaMalloc fails or evicts something), or a process whose rules forbid allocator calls on its
// latency-critical thread.  For them nq_moe_forward_static() runs the same three kernels as nq_moe_forward() with the
// workspaces taken from a fixed array that is part of the library image.
//
// The array is a file-scope __device__ array of NQ_STATIC_SCRATCH_BYTES (4 MiB): every GPU that loads the library
// holds it until the process exits.  Its name is only a host-side handle; the device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and handed to the kernels.  That lookup happens inside
// the FIRST call on each device, so make the first call on a device during start-up, before any stream capture begins
// on it.  The call itself uses no cudaMalloc / cudaFree and no allocating library routine.
//
// All calls on a device share the one array and it keeps whatever the previous call left in it.  The counters the
// kernels expect to be zero are cleared at the start of every call (a stream-ordered memset); everything else is
// fully rewritten before it is read.  Two calls that overlap on the GPU (different streams, or replays that can run
// concurrently) would race on the array: issue them in one stream order.
#include <mutex>

#include "nq_common.cuh"

#define NQ_STATIC_SCRATCH_BYTES (4u << 20)

static __device__ __align__(256) unsigned char nq_static_scratch[NQ_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {nullptr};

// device address of the scratch array on the current device (looked up once per device)
int scratch_base(unsigned char** out)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return nq::fail(NQ_ERR_ARG, "nq_moe_forward_static: device index %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_ptr[dev])
    {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, nq_static_scratch);
        if (e != cudaSuccess || !p)
            return nq::fail(NQ_ERR_CUDA, "nq_moe_forward_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = (unsigned char*)p;
    }
    *out = g_scratch_ptr[dev];
    return NQ_OK;
}

size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

}  // namespace

extern "C" {

size_t nq_moe_static_scratch_bytes(void) { return NQ_STATIC_SCRATCH_BYTES; }

int nq_moe_forward_static(const void* x, const int64_t* sel, const void* rw, const int64_t* table, float* out,
                          int B, int topk, int E, int H, int I, int nm_gu, int nm_dn, int ks_gu, int ks_dn,
                          int32_t* hits, void* stream)
{
    NqMoeWorkspace w;
    if (int rc = nq_moe_workspace(B, topk, H, I, ks_gu, ks_dn, &w)) return rc;
    // carve the workspaces: counters first (one contiguous region to clear), then the buffers that are fully rewritten
    size_t off = 0;
    const size_t o_cnt_gu = off; off = align256(off + w.cnt_gu_ints * 4);
    const size_t o_cnt_d = off; off = align256(off + w.cnt_d_ints * 4);
    const size_t o_wq = off; off = align256(off + w.wq_ints * 4);
    const size_t counters_end = off;
    const size_t o_cnt_h = off; off = align256(off + w.cnt_h_ints * 4);
    const size_t o_zd = off; off = align256(off + w.zd_floats * 4);
    const size_t o_acc_gu = off; off = align256(off + w.acc_gu_floats * 4);
    const size_t o_h = off; off = align256(off + w.h_halves * 2);
    const size_t o_acc_d = off; off = align256(off + w.acc_d_floats * 4);
    if (off > NQ_STATIC_SCRATCH_BYTES)
        return nq::fail(NQ_ERR_ARG,
                        "nq_moe_forward_static: this call shape (B %d, topk %d, H %d, I %d, k-slices %d/%d) needs %zu bytes of workspace, "
                        "the built-in array holds %u; use nq_moe_forward with caller-owned workspaces",
                        B, topk, H, I, ks_gu, ks_dn, off, NQ_STATIC_SCRATCH_BYTES);
    unsigned char* base = nullptr;
    if (int rc = scratch_base(&base)) return rc;
    const cudaError_t e = cudaMemsetAsync(base, 0, counters_end, (cudaStream_t)stream);
    if (e != cudaSuccess) return nq::fail(NQ_ERR_CUDA, "nq_moe_forward_static: clearing the counters: %s", cudaGetErrorString(e));
    NqMoeForward a{};
    a.x = x; a.sel = sel; a.rw = rw; a.table = table; a.out = out; a.hits = hits;
    a.cnt_gu = (int32_t*)(base + o_cnt_gu); a.cnt_d = (int32_t*)(base + o_cnt_d); a.wq = (int32_t*)(base + o_wq);
    a.cnt_h = (int32_t*)(base + o_cnt_h); a.zd = (float*)(base + o_zd); a.acc_gu = (float*)(base + o_acc_gu);
    a.h = base + o_h; a.acc_d = (float*)(base + o_acc_d);
    a.out_floats = (size_t)B * H; a.acc_gu_floats = w.acc_gu_floats; a.h_halves = w.h_halves; a.acc_d_floats = w.acc_d_floats;
    a.cnt_gu_ints = w.cnt_gu_ints; a.cnt_d_ints = w.cnt_d_ints; a.wq_ints = w.wq_ints; a.zd_floats = w.zd_floats; a.cnt_h_ints = w.cnt_h_ints;
    a.B = B; a.topk = topk; a.E = E; a.H = H; a.I = I; a.nm_gu = nm_gu; a.nm_dn = nm_dn; a.ks_gu = ks_gu; a.ks_dn = ks_dn;
    a.G = 4; a.force_level = 0; a.which = 3;
    return nq_moe_forward(&a, stream);
}

}  // extern "C"
