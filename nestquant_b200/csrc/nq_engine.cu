// Promotion engine, host side: record file -> pinned host entry -> device slot -> staged table row -> sequence number.
//
// Takes the place of the reference's streaming/nqstream.cu (Engine: upgrade / post / poll / cancel / tier_load /
// tier_drop / stats / close, lines 46-283) behind a C ABI.  Same contract: an upgrade reads one fixed-size record of
// the rank's record file (or finds it in the host cache / RAM tier), copies it into the device slot, then writes the
// staged row, then the sequence number, in that order on ONE side stream, so an expert can only go live (next mailbox
// pass of the compute stream) after its bytes have landed; a post writes only row and sequence number (demotion).
// Operations start in arrival order.  poll() reports (tag, hit, seconds until the bytes were in host memory, seconds
// until the device writes completed); a failed read reports hit = 0, t_read < 0 and t_done = -1 and never posts the
// row; a cancelled operation that had not started reports t_read = t_done = -1e9.
//
// Built differently from the reference: no io_uring (liburing is not a dependency) - a pool of reader threads issues
// O_DIRECT preads, a dispatcher thread owns ordering, the host cache (LRU over pinned entries) and every device call;
// device work goes through a small backend so that `device < 0` runs the whole engine against plain host memory
// (memcpy instead of cudaMemcpyAsync).  That mode is what the CPU tests drive: cache hits, eviction, cancellation,
// failing and slow drives, the RAM tier and the two-drive split need no GPU.
#include <fcntl.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <list>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../include/nestquant_b200.h"
#include "nq_common.cuh"

namespace nq {
namespace {

double now_s()
{
    timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

// ---------------------------------------------------------------- where copies go
struct Backend
{
    virtual ~Backend() {}
    virtual void* host_alloc(size_t n) = 0;                 // page-aligned, pinned when there is a device
    virtual void host_free(void* p) = 0;
    virtual bool copy(void* dst, const void* src, size_t n) = 0;   // stream-ordered
    virtual void* mark() = 0;                               // completion token for everything enqueued so far
    virtual bool done(void* token) = 0;
    virtual void release(void* token) = 0;
    virtual void sync() = 0;
    virtual void bind() {}                                  // called once by every thread that uses the backend
};

struct HostBackend : Backend
{
    void* host_alloc(size_t n) override { void* p = nullptr; return posix_memalign(&p, 4096, n ? n : 4096) == 0 ? p : nullptr; }
    void host_free(void* p) override { free(p); }
    bool copy(void* dst, const void* src, size_t n) override { memcpy(dst, src, n); return true; }
    void* mark() override { return this; }
    bool done(void*) override { return true; }
    void release(void*) override {}
    void sync() override {}
};

struct CudaBackend : Backend
{
    int dev;
    cudaStream_t st = nullptr;
    std::vector<cudaEvent_t> pool;
    bool ok = true;
    explicit CudaBackend(int d) : dev(d)
    {
        ok = cudaSetDevice(dev) == cudaSuccess && cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess;
    }
    ~CudaBackend() override
    {
        cudaSetDevice(dev);
        for (auto e : pool) cudaEventDestroy(e);
        if (st) cudaStreamDestroy(st);
    }
    void bind() override { cudaSetDevice(dev); }
    void* host_alloc(size_t n) override { void* p = nullptr; return cudaHostAlloc(&p, n ? n : 4096, cudaHostAllocPortable) == cudaSuccess ? p : nullptr; }
    void host_free(void* p) override { cudaFreeHost(p); }
    bool copy(void* dst, const void* src, size_t n) override { return cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, st) == cudaSuccess; }
    void* mark() override
    {
        cudaEvent_t e = nullptr;
        if (pool.empty()) { if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr; }
        else { e = pool.back(); pool.pop_back(); }
        cudaEventRecord(e, st);
        return e;
    }
    bool done(void* t) override { return cudaEventQuery((cudaEvent_t)t) != cudaErrorNotReady; }
    void release(void* t) override { pool.push_back((cudaEvent_t)t); }
    void sync() override { cudaStreamSynchronize(st); }
};

// ---------------------------------------------------------------- one operation
struct Op
{
    int64_t tag = 0, rec = -1;
    bool read = false;                 // upgrade (bytes + row + seq) or post (row + seq)
    void *slot = nullptr, *stage = nullptr, *seqp = nullptr;
    int32_t seq = 0;
    int64_t row[20];
    double t0 = 0, t_read = 0, t_sub = 0;
    int entry = -1, ring = -1, drive = -1;
    bool hit = false;
    const uint8_t* tier_src = nullptr;
    void* token = nullptr;
    long read_result = 0;              // bytes read, or -errno
};

}  // namespace
}  // namespace nq

struct NqEngine
{
    using Op = nq::Op;
    // configuration
    size_t rb = 0;
    int nh = 0, nd = 1, qd[2] = {0, 0}, fds[2] = {-1, -1};
    nq::Backend* be = nullptr;
    // host cache: nh entries of rb bytes; an entry is reusable when no operation in flight uses it
    uint8_t* host = nullptr;
    std::vector<int64_t> ent_rec;
    std::vector<int> ent_pin;
    std::list<int> lru;                                     // front = least recently used
    std::vector<std::list<int>::iterator> lru_it;
    std::unordered_map<int64_t, int> where;
    // staging ring for rows and sequence numbers (must outlive the copies)
    int64_t* rows = nullptr;
    int32_t* seqs = nullptr;
    std::vector<int> ring_free;
    // RAM tier: 0 none, 1 active, 2 drop requested, 3 dropped
    std::atomic<int> tier_state{0};
    uint8_t* tier_mem = nullptr;
    std::unordered_map<int64_t, const uint8_t*> tier_at;
    int tier_inflight = 0;
    // queues.  mu guards: inbox, cancel_req, done, jobs, finished, counters read by stats()
    std::mutex mu;
    std::condition_variable cv_dispatch, cv_reader;
    std::deque<Op*> inbox;
    std::vector<int64_t> cancel_req;
    std::vector<NqEngineDone> done;
    std::deque<Op*> jobs, finished;                         // reader pool in / out
    std::atomic<bool> stop{false};
    std::thread dispatcher;
    std::vector<std::thread> readers;
    // dispatcher-private
    std::deque<Op*> waiting, ready;
    std::vector<Op*> copying;
    int inflight[2] = {0, 0}, n_reading = 0;
    // fault injection from the environment (host side only): a slow drive and a failing drive
    double fault_gap = 0, next_ok = 0;
    int64_t fault_ppm = 0;
    uint64_t frng = 88172645463325252ull;
    NqEngineStats st{};

    int pick_drive() const
    {
        int b = -1;
        for (int i = 0; i < nd; ++i)
            if (inflight[i] < qd[i] && (b < 0 || inflight[i] < inflight[b])) b = i;
        return b;
    }
    int take_entry(int64_t rec, bool& hit)
    {
        auto it = where.find(rec);
        if (it != where.end())
        {
            hit = true;
            const int e = it->second;
            ++ent_pin[e];
            lru.splice(lru.end(), lru, lru_it[e]);
            return e;
        }
        hit = false;
        for (auto li = lru.begin(); li != lru.end(); ++li)
            if (ent_pin[*li] == 0)
            {
                const int e = *li;
                if (ent_rec[e] >= 0) where.erase(ent_rec[e]);
                ent_rec[e] = -1; ent_pin[e] = 1;
                lru.splice(lru.end(), lru, li);
                return e;
            }
        return -1;
    }
    void report(const Op* o, bool hit, double t_read, double t_done)
    {
        std::lock_guard<std::mutex> g(mu);
        done.push_back(NqEngineDone{o->tag, hit ? 1 : 0, t_read, t_done});
    }
    // bytes (upgrade) -> staged row -> sequence number, in order
    void issue_copies(Op* o)
    {
        o->ring = ring_free.back(); ring_free.pop_back();
        int64_t* r = rows + (size_t)o->ring * 20;
        memcpy(r, o->row, sizeof o->row);
        seqs[o->ring] = o->seq;
        bool ok = true;
        if (o->read) ok = be->copy(o->slot, o->tier_src ? (const void*)o->tier_src : (const void*)(host + (size_t)o->entry * rb), rb);
        ok = ok && be->copy(o->stage, r, sizeof o->row) && be->copy(o->seqp, seqs + o->ring, sizeof(int32_t));
        o->token = be->mark();
        if (!ok || !o->token) { std::lock_guard<std::mutex> g(mu); ++st.device_errors; }
        copying.push_back(o);
    }
    void retire()
    {
        for (size_t i = 0; i < copying.size();)
        {
            Op* o = copying[i];
            if (o->token && !be->done(o->token)) { ++i; continue; }
            if (o->token) be->release(o->token);
            ring_free.push_back(o->ring);
            if (o->tier_src) --tier_inflight;
            else if (o->read) --ent_pin[o->entry];
            report(o, o->hit, o->t_read - o->t0, nq::now_s() - o->t0);
            delete o;
            copying[i] = copying.back(); copying.pop_back();
        }
    }
    void reader_loop()
    {
        for (;;)
        {
            Op* o = nullptr;
            {
                std::unique_lock<std::mutex> g(mu);
                cv_reader.wait(g, [&] { return stop.load() || !jobs.empty(); });
                if (jobs.empty()) return;
                o = jobs.front(); jobs.pop_front();
            }
            uint8_t* dst = host + (size_t)o->entry * rb;
            size_t got = 0;
            long res = 0;
            while (got < rb)
            {
                const ssize_t r = pread(fds[o->drive], dst + got, rb - got, (off_t)((size_t)o->rec * rb + got));
                if (r < 0) { res = -(long)errno; break; }
                if (r == 0) break;
                got += (size_t)r;
            }
            o->read_result = res < 0 ? res : (long)got;
            {
                std::lock_guard<std::mutex> g(mu);
                finished.push_back(o);
            }
            cv_dispatch.notify_one();
        }
    }
    void dispatch_loop()
    {
        be->bind();
        while (!stop.load())
        {
            std::deque<Op*> fin;
            {
                std::unique_lock<std::mutex> g(mu);
                if (inbox.empty() && finished.empty() && cancel_req.empty() && copying.empty() && ready.empty() &&
                    (waiting.empty() || n_reading > 0) && tier_state.load() != 2)
                    cv_dispatch.wait_for(g, std::chrono::milliseconds(2));
                while (!inbox.empty()) { waiting.push_back(inbox.front()); inbox.pop_front(); }
                fin.swap(finished);
                if (!cancel_req.empty())
                {
                    // operations still waiting here have touched neither a drive nor the device
                    std::unordered_set<int64_t> cs(cancel_req.begin(), cancel_req.end());
                    cancel_req.clear();
                    std::deque<Op*> keep;
                    for (Op* o : waiting)
                        if (cs.count(o->tag)) { done.push_back(NqEngineDone{o->tag, 0, -1e9, -1e9}); ++st.cancelled; delete o; }
                        else keep.push_back(o);
                    waiting.swap(keep);
                }
            }
            retire();
            if (tier_state.load(std::memory_order_acquire) == 2 && tier_inflight == 0)
            {
                tier_at.clear();
                be->host_free(tier_mem); tier_mem = nullptr;
                std::lock_guard<std::mutex> g(mu);
                st.tier_recs = 0;
                tier_state.store(3);
            }
            const bool tier_on = tier_state.load(std::memory_order_acquire) == 1;
            // reads that came back
            for (Op* o : fin)
            {
                --n_reading; --inflight[o->drive];
                bool fail = o->read_result != (long)rb;
                if (!fail && fault_ppm)
                {
                    frng ^= frng << 13; frng ^= frng >> 7; frng ^= frng << 17;
                    if ((int64_t)(frng % 1000000) < fault_ppm) { fail = true; std::lock_guard<std::mutex> g(mu); ++st.fault_injected; }
                }
                {
                    std::lock_guard<std::mutex> g(mu);
                    ++st.drive_reads[o->drive]; st.drive_read_s[o->drive] += nq::now_s() - o->t_sub;
                    if (!fail) { st.bytes_read += (int64_t)rb; st.drive_bytes[o->drive] += (int64_t)rb; }
                }
                if (fail)
                {
                    // the expert stays where it is: the row is never posted
                    --ent_pin[o->entry];
                    report(o, false, o->read_result < 0 ? (double)o->read_result : -1.0, -1.0);
                    delete o;
                    continue;
                }
                o->t_read = nq::now_s();
                ent_rec[o->entry] = o->rec; where[o->rec] = o->entry;
                ready.push_back(o);
            }
            while (!ready.empty() && !ring_free.empty()) { issue_copies(ready.front()); ready.pop_front(); }
            // start operations in arrival order (the caller keeps one outstanding operation per expert)
            bool handed = false, throttled = false;
            while (ready.empty() && !waiting.empty() && !ring_free.empty())
            {
                Op* o = waiting.front();
                if (!o->read)
                {
                    waiting.pop_front(); o->t_read = o->t0;
                    issue_copies(o);
                    std::lock_guard<std::mutex> g(mu); ++st.posts;
                    continue;
                }
                if (tier_on)
                {
                    auto ti = tier_at.find(o->rec);
                    if (ti != tier_at.end())
                    {
                        waiting.pop_front();
                        o->tier_src = ti->second; o->hit = true; o->t_read = nq::now_s(); ++tier_inflight;
                        { std::lock_guard<std::mutex> g(mu); ++st.upgrades; ++st.tier_hits; st.tier_bytes += (int64_t)rb; }
                        issue_copies(o);
                        continue;
                    }
                }
                const int dv = pick_drive();
                if (dv < 0) break;
                if (fault_gap > 0 && !where.count(o->rec) && nq::now_s() < next_ok) { throttled = true; break; }
                bool hit;
                const int e = take_entry(o->rec, hit);
                if (e < 0) break;
                waiting.pop_front();
                o->entry = e; o->hit = hit;
                { std::lock_guard<std::mutex> g(mu); ++st.upgrades; if (hit) ++st.host_hits; }
                if (hit) { o->t_read = nq::now_s(); issue_copies(o); continue; }
                o->drive = dv; ++inflight[dv]; ++n_reading; o->t_sub = nq::now_s();
                if (fault_gap > 0) next_ok = nq::now_s() + fault_gap;
                { std::lock_guard<std::mutex> g(mu); jobs.push_back(o); }
                handed = true;
            }
            if (handed) cv_reader.notify_all();
            {
                std::lock_guard<std::mutex> g(mu);
                st.waiting = (int64_t)(waiting.size() + ready.size());
                st.reading = (int64_t)n_reading; st.copying = (int64_t)copying.size();
                for (int i = 0; i < 2; ++i) st.drive_inflight[i] = inflight[i];
            }
            if (!copying.empty() && fin.empty() && !handed) usleep(20);     // copies in flight only: do not spin a core
            if (throttled && fin.empty()) usleep(200);
        }
        // drain: reads in flight finish (their buffers must not be freed under them), device work completes
        {
            std::unique_lock<std::mutex> g(mu);
            for (Op* o : jobs) { delete o; --n_reading; }
            jobs.clear();
        }
        cv_reader.notify_all();
        for (auto& t : readers) t.join();
        for (Op* o : finished) delete o;
        finished.clear();
        be->sync();
        for (Op* o : copying) { if (o->token) be->release(o->token); delete o; }
        for (Op* o : waiting) delete o;
        for (Op* o : ready) delete o;
        for (Op* o : inbox) delete o;
    }
};

extern "C" {

int nq_engine_open(const char* path, const char* alt_path, size_t rec_bytes, int n_host, int qd, int qd_alt, int device, NqEngine** out)
{
    NQ_REQUIRE(path && out, "nq_engine_open: null argument");
    const bool two = alt_path && alt_path[0];
    const int q1 = two ? (qd_alt > 0 ? qd_alt : qd) : 0;
    NQ_REQUIRE(rec_bytes > 0 && rec_bytes % 4096 == 0 && qd >= 1 && n_host >= qd + q1,
               "nq_engine_open: rec_bytes %% 4096 == 0 and n_host >= qd (+ qd_alt) >= 1 required");
    NqEngine* e = new NqEngine();
    e->rb = rec_bytes; e->nh = n_host; e->nd = two ? 2 : 1; e->qd[0] = qd; e->qd[1] = q1;
    auto open_ro = [](const char* p) { int f = open(p, O_RDONLY | O_DIRECT); return f >= 0 ? f : open(p, O_RDONLY); };   // O_DIRECT where the file system has it
    e->fds[0] = open_ro(path);
    if (e->fds[0] < 0) { delete e; return nq::fail(NQ_ERR_ARG, "nq_engine_open: cannot open %s", path); }
    if (two)
    {
        e->fds[1] = open_ro(alt_path);
        struct stat a, b;
        if (e->fds[1] < 0 || fstat(e->fds[0], &a) || fstat(e->fds[1], &b) || a.st_size != b.st_size)
        {
            close(e->fds[0]); if (e->fds[1] >= 0) close(e->fds[1]);
            delete e;
            return nq::fail(NQ_ERR_ARG, "nq_engine_open: %s cannot be opened or differs in size from %s", alt_path, path);
        }
    }
    if (device >= 0)
    {
        auto* cb = new nq::CudaBackend(device);
        if (!cb->ok) { delete cb; close(e->fds[0]); if (two) close(e->fds[1]); delete e; return nq::fail(NQ_ERR_CUDA, "nq_engine_open: cannot create a stream on device %d", device); }
        e->be = cb;
    }
    else e->be = new nq::HostBackend();
    const int nring = 4 * (qd + q1);
    e->host = (uint8_t*)e->be->host_alloc((size_t)n_host * rec_bytes);
    e->rows = (int64_t*)e->be->host_alloc((size_t)nring * 20 * sizeof(int64_t));
    e->seqs = (int32_t*)e->be->host_alloc((size_t)nring * sizeof(int32_t));
    if (!e->host || !e->rows || !e->seqs)
    {
        if (e->host) e->be->host_free(e->host);
        if (e->rows) e->be->host_free(e->rows);
        if (e->seqs) e->be->host_free(e->seqs);
        close(e->fds[0]); if (two) close(e->fds[1]);
        delete e->be; delete e;
        return nq::fail(NQ_ERR_CUDA, "nq_engine_open: cannot allocate %zu bytes of host memory", (size_t)n_host * rec_bytes);
    }
    for (int i = 0; i < nring; ++i) e->ring_free.push_back(i);
    e->ent_rec.assign(n_host, -1); e->ent_pin.assign(n_host, 0); e->lru_it.resize(n_host);
    for (int i = 0; i < n_host; ++i) { e->lru.push_back(i); e->lru_it[i] = std::prev(e->lru.end()); }
    if (const char* v = getenv("NQ_FAULT_READ_MS")) e->fault_gap = atof(v) * 1e-3;
    if (const char* v = getenv("NQ_FAULT_FAIL_PPM")) e->fault_ppm = atoll(v);
    e->st.drives = e->nd; e->st.n_host = n_host; e->st.drive_qd[0] = qd; e->st.drive_qd[1] = q1;
    for (int i = 0; i < qd + q1; ++i) e->readers.emplace_back([e] { e->reader_loop(); });
    e->dispatcher = std::thread([e] { e->dispatch_loop(); });
    *out = e;
    return NQ_OK;
}

static int engine_enqueue(NqEngine* e, nq::Op* o, const int64_t* row)
{
    memcpy(o->row, row, sizeof o->row);
    o->t0 = nq::now_s();
    { std::lock_guard<std::mutex> g(e->mu); e->inbox.push_back(o); }
    e->cv_dispatch.notify_one();
    return NQ_OK;
}

int nq_engine_upgrade(NqEngine* e, int64_t tag, int64_t rec, void* slot, void* stage_row, const int64_t* row, void* seq_entry, int32_t seq)
{
    NQ_REQUIRE(e && slot && stage_row && row && seq_entry && rec >= 0, "nq_engine_upgrade: bad argument");
    NQ_REQUIRE(!e->stop.load(), "nq_engine_upgrade: engine is closed");
    auto* o = new nq::Op();
    o->tag = tag; o->rec = rec; o->read = true; o->slot = slot; o->stage = stage_row; o->seqp = seq_entry; o->seq = seq;
    return engine_enqueue(e, o, row);
}

int nq_engine_post(NqEngine* e, int64_t tag, void* stage_row, const int64_t* row, void* seq_entry, int32_t seq)
{
    NQ_REQUIRE(e && stage_row && row && seq_entry, "nq_engine_post: bad argument");
    NQ_REQUIRE(!e->stop.load(), "nq_engine_post: engine is closed");
    auto* o = new nq::Op();
    o->tag = tag; o->stage = stage_row; o->seqp = seq_entry; o->seq = seq;
    return engine_enqueue(e, o, row);
}

int nq_engine_cancel(NqEngine* e, int64_t tag)
{
    NQ_REQUIRE(e, "nq_engine_cancel: null engine");
    { std::lock_guard<std::mutex> g(e->mu); e->cancel_req.push_back(tag); }
    e->cv_dispatch.notify_one();
    return NQ_OK;
}

int nq_engine_poll(NqEngine* e, NqEngineDone* out, int max)
{
    NQ_REQUIRE(e && (out || max == 0) && max >= 0, "nq_engine_poll: bad argument");
    std::lock_guard<std::mutex> g(e->mu);
    const int n = (int)e->done.size() < max ? (int)e->done.size() : max;
    for (int i = 0; i < n; ++i) out[i] = e->done[i];
    e->done.erase(e->done.begin(), e->done.begin() + n);
    return n;
}

int nq_engine_tier_load(NqEngine* e, const int64_t* recs, int n)
{
    NQ_REQUIRE(e && (recs || n == 0) && n >= 0, "nq_engine_tier_load: bad argument");
    NQ_REQUIRE(e->tier_state.load() == 0, "nq_engine_tier_load: the tier was already loaded or dropped");
    if (n == 0) return 0;
    e->be->bind();
    uint8_t* m = (uint8_t*)e->be->host_alloc((size_t)n * e->rb);
    if (!m) return nq::fail(NQ_ERR_CUDA, "nq_engine_tier_load: cannot allocate %zu bytes", (size_t)n * e->rb);
    std::atomic<int> next{0}, bad{0};
    std::vector<std::thread> ths;
    for (int t = 0; t < 8; ++t)
        ths.emplace_back([&, t] {
            const int f = e->fds[t % e->nd];
            for (int i; (i = next.fetch_add(1)) < n;)
            {
                size_t got = 0;
                while (got < e->rb)
                {
                    const ssize_t r = pread(f, m + (size_t)i * e->rb + got, e->rb - got, (off_t)((size_t)recs[i] * e->rb + got));
                    if (r <= 0) break;
                    got += (size_t)r;
                }
                if (got != e->rb) ++bad;
            }
        });
    for (auto& t : ths) t.join();
    if (bad.load()) { e->be->host_free(m); return nq::fail(NQ_ERR_ARG, "nq_engine_tier_load: %d short reads", bad.load()); }
    e->tier_mem = m;
    for (int i = 0; i < n; ++i) e->tier_at[recs[i]] = m + (size_t)i * e->rb;
    { std::lock_guard<std::mutex> g(e->mu); e->st.tier_recs = n; }
    e->tier_state.store(1, std::memory_order_release);
    e->cv_dispatch.notify_one();
    return n;
}

int nq_engine_tier_drop(NqEngine* e)
{
    NQ_REQUIRE(e, "nq_engine_tier_drop: null engine");
    int one = 1;
    e->tier_state.compare_exchange_strong(one, 2);
    e->cv_dispatch.notify_one();
    return NQ_OK;
}

int nq_engine_stats(NqEngine* e, NqEngineStats* out)
{
    NQ_REQUIRE(e && out, "nq_engine_stats: null argument");
    std::lock_guard<std::mutex> g(e->mu);
    *out = e->st;
    out->queued = (int64_t)e->inbox.size();
    out->tier_state = e->tier_state.load();
    out->now_s = nq::now_s();
    return NQ_OK;
}

int nq_engine_close(NqEngine* e)
{
    if (!e) return NQ_OK;
    if (!e->stop.exchange(true))
    {
        e->cv_dispatch.notify_all(); e->cv_reader.notify_all();
        if (e->dispatcher.joinable()) e->dispatcher.join();
        e->be->bind();
        if (e->tier_mem) e->be->host_free(e->tier_mem);
        e->be->host_free(e->host); e->be->host_free(e->rows); e->be->host_free(e->seqs);
        close(e->fds[0]); if (e->fds[1] >= 0) close(e->fds[1]);
        delete e->be;
    }
    delete e;
    return NQ_OK;
}

}  // extern "C"
