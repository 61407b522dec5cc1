// Host side of the batch readers: a multi-threaded row gather (memory-mapped cache
// shard -> page-locked staging) and the native double-buffered pipeline behind
// ZeroCopyTensorStreamer / FeatureCacheDataset.iter_batches.
//
// Pipeline per batch b (slot = b mod n_slots):
//   producer thread : wait until the H2D copy that last read pinned[slot] is done
//                     -> gather rows into pinned[slot] on the worker pool
//                     -> copy stream waits for the decode that last read
//                        dev[slot] -> three async H2D copies -> record h2d[slot]
//   tcb_streamer_next (caller's thread): consumer stream waits for h2d[slot]
//                     -> decode kernel into out[slot] -> record decoded[slot]
// The producer runs ahead of the consumer by up to n_slots batches, so the host
// gather, the PCIe copy and the decode of three different batches overlap.  The
// reference (src/tensorcache/streamer.py:459-495) has the same ring but runs the
// gather on the consumer's Python thread and has no event from the decode back
// to the copy stream nor from the copy back to the host.
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "tcb_common.h"

#if defined(__x86_64__)
#include <immintrin.h>
#endif
#if defined(__linux__)
#include <sys/mman.h>
#endif

namespace tcb {
int launch_decompress(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out, int64_t numel,
                      int group_size, cudaStream_t st);
}

namespace {

// Runs fn(task) for task in [0, n) on the calling thread plus up to (n_workers)
// helper threads; returns when every task has finished.
class WorkerPool {
public:
    explicit WorkerPool(int n_helpers) {
        for (int i = 0; i < n_helpers; ++i) helpers_.emplace_back([this] { loop(); });
    }
    ~WorkerPool() {
        {
            std::lock_guard<std::mutex> lk(mu_);
            stop_ = true;
        }
        cv_.notify_all();
        for (auto& t : helpers_) t.join();
    }
    void run(int n_tasks, const std::function<void(int)>& fn) {
        if (n_tasks <= 0) return;
        {
            std::lock_guard<std::mutex> lk(mu_);
            fn_ = &fn;
            n_tasks_ = n_tasks;
            next_ = 0;
            pending_ = n_tasks;
            ++generation_;
        }
        cv_.notify_all();
        work();
        std::unique_lock<std::mutex> lk(mu_);
        done_cv_.wait(lk, [this] { return pending_ == 0; });
        fn_ = nullptr;
    }
    int size() const { return int(helpers_.size()) + 1; }

private:
    void work() {
        for (;;) {
            int t;
            const std::function<void(int)>* fn;
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (!fn_ || next_ >= n_tasks_) return;
                t = next_++;
                fn = fn_;
            }
            (*fn)(t);
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (--pending_ == 0) done_cv_.notify_all();
            }
        }
    }
    void loop() {
        uint64_t seen = 0;
        for (;;) {
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return stop_ || generation_ != seen; });
                if (stop_) return;
                seen = generation_;
            }
            work();
        }
    }
    std::vector<std::thread> helpers_;
    std::mutex mu_;
    std::condition_variable cv_, done_cv_;
    const std::function<void(int)>* fn_ = nullptr;
    int n_tasks_ = 0, next_ = 0, pending_ = 0;
    uint64_t generation_ = 0;
    bool stop_ = false;
};

// Row copy into page-locked staging.  The destination is written once and next read by the
// DMA engine, never by this core, so the stores bypass the cache (non-temporal): no
// read-for-ownership of the destination lines and no eviction of the source's page-cache
// lines.  Falls back to memcpy for short or unaligned-tail pieces and on CPUs without AVX2.
#if defined(__x86_64__)
__attribute__((target("avx2"))) static void copy_stream_avx2(uint8_t* dst, const uint8_t* src, size_t n) {
    // head: bring dst to 32-byte alignment
    size_t head = (32 - (reinterpret_cast<uintptr_t>(dst) & 31)) & 31;
    if (head > n) head = n;
    if (head) {
        std::memcpy(dst, src, head);
        dst += head; src += head; n -= head;
    }
    size_t blocks = n / 128;
    for (size_t i = 0; i < blocks; ++i) {
        const __m256i a = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src));
        const __m256i b = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + 32));
        const __m256i c = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + 64));
        const __m256i d = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(src + 96));
        _mm256_stream_si256(reinterpret_cast<__m256i*>(dst), a);
        _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + 32), b);
        _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + 64), c);
        _mm256_stream_si256(reinterpret_cast<__m256i*>(dst + 96), d);
        src += 128; dst += 128;
    }
    _mm_sfence();
    const size_t tail = n - blocks * 128;
    if (tail) std::memcpy(dst, src, tail);
}
#endif

static void copy_row(uint8_t* dst, const uint8_t* src, size_t n) {
#if defined(__x86_64__)
    static const bool have_avx2 = __builtin_cpu_supports("avx2");
    if (have_avx2 && n >= 4096) {
        copy_stream_avx2(dst, src, n);
        return;
    }
#endif
    std::memcpy(dst, src, n);
}

// dst row i <- src_of(i), rows split over the pool.  Rows of a cache are hundreds
// of KB, so one memcpy per row already streams at full speed.
template <typename SrcOf>
void gather_rows(WorkerPool& pool, uint8_t* dst, int64_t row_bytes, int64_t n, const SrcOf& src_of) {
    if (n <= 0 || row_bytes <= 0) return;
    int parts = pool.size();
    if (parts > n) parts = int(n);
    pool.run(parts, [&](int t) {
        const int64_t lo = n * t / parts, hi = n * (t + 1) / parts;
        for (int64_t i = lo; i < hi; ++i) copy_row(dst + i * row_bytes, src_of(i), size_t(row_bytes));
    });
}

std::mutex g_shared_pool_call_mu;  // the shared pool runs one job at a time, whichever entry point asks

WorkerPool& shared_pool(int want) {
    static std::mutex mu;
    static WorkerPool* pool = nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!pool || pool->size() < want) {
        // grown pools replace smaller ones; the old one is drained and joined
        WorkerPool* old = pool;
        pool = new WorkerPool(want - 1);
        delete old;
    }
    return *pool;
}

}  // namespace

extern "C" int tcb_gather_rows(void* dst, const void* src_base, int64_t row_bytes, const int64_t* idx, int64_t first_row,
                               int64_t n, int nthreads) {
    if (n < 0 || row_bytes < 0 || first_row < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_gather_rows: negative size");
    if (n == 0 || row_bytes == 0) return TCB_OK;
    if (!dst || !src_base) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_gather_rows: null pointer");
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 64) nthreads = 64;
    std::lock_guard<std::mutex> lk(g_shared_pool_call_mu);
    const uint8_t* src = static_cast<const uint8_t*>(src_base);
    gather_rows(shared_pool(nthreads), static_cast<uint8_t*>(dst), row_bytes, n,
                [&](int64_t i) { return src + (idx ? idx[i] : first_row + i) * row_bytes; });
    return TCB_OK;
}

// Block copy into a freshly created, still sparse file mapping (the cache writer's output).  Every
// 4 KB page of such a mapping is allocated and zero-filled by a page fault on first touch; taken one
// by one inside the copy loop those faults, not the copy, set the writer's speed.  Each worker
// therefore first asks the kernel to populate its slice in one call (MADV_POPULATE_WRITE, Linux 5.14+;
// older kernels refuse it and the copy faults the pages as before), then streams its slice.
extern "C" int tcb_write_block(void* dst, const void* src, int64_t bytes, int nthreads) {
    if (bytes < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_write_block: negative size");
    if (bytes == 0) return TCB_OK;
    if (!dst || !src) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_write_block: null pointer");
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 64) nthreads = 64;
    constexpr int64_t kSlice = 2 << 20;   // slices start on 2 MB boundaries of the destination
    uint8_t* d = static_cast<uint8_t*>(dst);
    const uint8_t* s = static_cast<const uint8_t*>(src);
    const uintptr_t d0 = reinterpret_cast<uintptr_t>(d);
    const int64_t first = int64_t(d0 / kSlice), last = int64_t((d0 + uintptr_t(bytes) - 1) / kSlice);
    const int64_t n_slices = last - first + 1;
    std::lock_guard<std::mutex> lk(g_shared_pool_call_mu);
    WorkerPool& pool = shared_pool(nthreads);
    int parts = nthreads < n_slices ? nthreads : int(n_slices);
    pool.run(parts, [&](int t) {
        const int64_t s_lo = first + n_slices * t / parts, s_hi = first + n_slices * (t + 1) / parts;
        uintptr_t lo = uintptr_t(s_lo) * kSlice, hi = uintptr_t(s_hi) * kSlice;
        if (lo < d0) lo = d0;
        if (hi > d0 + uintptr_t(bytes)) hi = d0 + uintptr_t(bytes);
        if (hi <= lo) return;
#if defined(__linux__)
        const uintptr_t page = 4096, p_lo = (lo + page - 1) & ~(page - 1), p_hi = hi & ~(page - 1);
        if (p_hi > p_lo) (void)madvise(reinterpret_cast<void*>(p_lo), p_hi - p_lo, 23 /* MADV_POPULATE_WRITE */);
#endif
        copy_row(reinterpret_cast<uint8_t*>(lo), s + (lo - d0), size_t(hi - lo));
    });
    return TCB_OK;
}

// ------------------------------------------------------------------ streamer

// Resident-shard mode, scattered order: ONE kernel pulls the batch's rows (codes, scales, zero points) straight out of
// the page-locked host mapping over PCIe and writes them, packed, into device staging.  The SMs issue the reads; a few
// dozen blocks keep enough 16-byte loads in flight to fill the link (a stand-alone run of the code rows alone: 50.5 GB/s
// against 55 GB/s for one large copy-engine transfer, 24 to 296 blocks alike; one cudaMemcpyAsync per row: 32 GB/s,
// bound by the 8 us each call costs the host).  The three arrays share the launch, each with a share of the blocks in
// proportion to its bytes, so that the small ones neither wait for the codes nor run with too few loads in flight.
// `rows` tables hold host pointers and live in mapped page-locked memory themselves.
struct GatherSegment {
    uint4* dst;
    const uint4* const* rows;
    int64_t units_per_row;   // 16-byte units
    int first_block, blocks; // this segment's share of the grid
};
struct GatherBatch {
    GatherSegment seg[3];
    int n_segments;
    int64_t n_rows;
};

__global__ void __launch_bounds__(256)
gather_host_rows_kernel(const GatherBatch g) {
    int k = 0;
    while (k + 1 < g.n_segments && int(blockIdx.x) >= g.seg[k + 1].first_block) ++k;
    const GatherSegment sg = g.seg[k];
    const int64_t total = sg.units_per_row * g.n_rows;
    const int64_t stride = int64_t(sg.blocks) * blockDim.x;
    constexpr int kInFlight = 8;   // 16-byte loads per thread before the first store (4: 2-5 % less on the same link)
    for (int64_t u0 = int64_t(int(blockIdx.x) - sg.first_block) * blockDim.x + threadIdx.x; u0 < total; u0 += kInFlight * stride) {
        uint4 v[kInFlight];
#pragma unroll
        for (int i = 0; i < kInFlight; ++i) {
            const int64_t u = u0 + i * stride;
            if (u < total) {
                const int64_t r = u / sg.units_per_row;
                v[i] = sg.rows[r][u - r * sg.units_per_row];
            }
        }
#pragma unroll
        for (int i = 0; i < kInFlight; ++i) {
            const int64_t u = u0 + i * stride;
            if (u < total) sg.dst[u] = v[i];
        }
    }
}

struct tcb_streamer {
    tcb_streamer_desc d{};
    std::vector<const uint8_t*> q_bases, s_bases, zp_bases;
    std::vector<int64_t> shard_start;  // first global sample of each shard, plus the total at the end
    std::vector<void*> pinned_q, pinned_s, pinned_zp, dev_q, dev_s, dev_zp, dev_out;
    int device = 0;
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> h2d_done, released;
    WorkerPool* pool = nullptr;
    // resident mode: per slot three tables of row pointers (codes, scales, zero points) in mapped pinned memory
    const uint4** row_tables = nullptr;       // host view
    const uint4** row_tables_dev = nullptr;   // the same memory as the device addresses it
    std::vector<const uint8_t*> q_dev, s_dev, zp_dev;  // device views of the page-locked mappings
    bool rows_vectorisable = false;
    bool has_zp = true;  // false: symmetric cache (signed codes, no zero-point file)

    std::thread producer;
    std::mutex mu;
    std::condition_variable cv;
    // pass state (guarded by mu)
    std::vector<int64_t> order;
    bool have_order = false;
    int64_t n_indices = 0, n_batches = 0;
    int64_t produced = 0;   // batches whose H2D has been enqueued
    int64_t acquired = 0;   // batches handed to the consumer
    int64_t consumed = 0;   // batches whose device staging the consumer has released
    bool pass_active = false;
    bool producer_idle = true;
    bool abort_pass = false;
    bool quit = false;
    int producer_error = TCB_OK;
    char producer_msg[256] = "";
};

namespace {

int64_t batch_rows_of(const tcb_streamer* s, int64_t b) {
    const int64_t start = b * s->d.batch_size;
    const int64_t left = s->n_indices - start;
    return left < s->d.batch_size ? left : s->d.batch_size;
}

void producer_fail(tcb_streamer* s, cudaError_t e, const char* what) {
    std::lock_guard<std::mutex> lk(s->mu);
    s->producer_error = TCB_ERR_CUDA;
    snprintf(s->producer_msg, sizeof(s->producer_msg), "streamer producer: %s: %s", what, cudaGetErrorString(e));
    s->cv.notify_all();
}

// global sample id -> shard and local row
inline void locate(const tcb_streamer* s, int64_t gid, int& shard, int64_t& local) {
    int sh = 0;
    const int n = int(s->shard_start.size()) - 1;
    while (sh + 1 < n && gid >= s->shard_start[sh + 1]) ++sh;
    shard = sh;
    local = gid - s->shard_start[sh];
}

void producer_main(tcb_streamer* s) {
    cudaSetDevice(s->device);
    const int64_t qrow = s->d.values_per_sample;
    const int64_t srow = s->d.groups_per_sample * 2;
    const int64_t zrow = s->d.groups_per_sample;
    for (;;) {
        {
            std::unique_lock<std::mutex> lk(s->mu);
            s->producer_idle = true;
            s->cv.notify_all();
            s->cv.wait(lk, [&] { return s->quit || (s->pass_active && !s->abort_pass); });
            if (s->quit) return;
            s->producer_idle = false;
        }
        for (int64_t b = 0;; ++b) {
            const int64_t* idx;
            int64_t first, rows;
            const int slot = int(b % s->d.n_slots);
            {
                std::unique_lock<std::mutex> lk(s->mu);
                if (b >= s->n_batches) break;
                // device staging of this slot is free once batch b - n_slots has been released
                s->cv.wait(lk, [&] { return s->quit || s->abort_pass || s->consumed >= b - s->d.n_slots + 1; });
                if (s->quit || s->abort_pass) break;
                rows = batch_rows_of(s, b);
                first = b * s->d.batch_size;
                idx = s->have_order ? s->order.data() + first : nullptr;
            }
            // The copy that last read this pinned slot must have finished (a no-op for
            // an event that was never recorded; also covers the previous pass).
            cudaError_t e = cudaEventSynchronize(s->h2d_done[slot]);
            if (e != cudaSuccess) { producer_fail(s, e, "cudaEventSynchronize(h2d)"); break; }
            auto src = [&](const std::vector<const uint8_t*>& bases, int64_t row_bytes) {
                return [&, row_bytes](int64_t i) {
                    int sh;
                    int64_t local;
                    locate(s, idx ? idx[i] : first + i, sh, local);
                    return bases[sh] + local * row_bytes;
                };
            };
            if (!s->d.direct_dma) {
                // one pass over the batch's rows: each worker copies the codes, scales and zero points of its rows
                int parts = s->pool->size();
                if (parts > rows) parts = int(rows);
                uint8_t* pq = static_cast<uint8_t*>(s->pinned_q[slot]);
                uint8_t* ps = static_cast<uint8_t*>(s->pinned_s[slot]);
                uint8_t* pz = s->has_zp ? static_cast<uint8_t*>(s->pinned_zp[slot]) : nullptr;
                s->pool->run(parts, [&](int t) {
                    const int64_t lo = rows * t / parts, hi = rows * (t + 1) / parts;
                    for (int64_t i = lo; i < hi; ++i) {
                        int sh;
                        int64_t local;
                        locate(s, idx ? idx[i] : first + i, sh, local);
                        copy_row(pq + i * qrow, s->q_bases[sh] + local * qrow, size_t(qrow));
                        copy_row(ps + i * srow, s->s_bases[sh] + local * srow, size_t(srow));
                        if (pz) copy_row(pz + i * zrow, s->zp_bases[sh] + local * zrow, size_t(zrow));
                    }
                });
            }
            // the consumer's last read of this device slot (this pass or the one before)
            e = cudaStreamWaitEvent(s->copy_stream, s->released[slot], 0);
            if (e != cudaSuccess) { producer_fail(s, e, "cudaStreamWaitEvent(released)"); break; }
            if (!s->d.direct_dma) {
                // a full batch in a slot whose three arrays lie back to back (host and device alike) is one copy
                const uint8_t *hq = static_cast<const uint8_t*>(s->pinned_q[slot]), *hs = static_cast<const uint8_t*>(s->pinned_s[slot]);
                const uint8_t *dq = static_cast<const uint8_t*>(s->dev_q[slot]), *ds = static_cast<const uint8_t*>(s->dev_s[slot]);
                bool one = hs == hq + rows * qrow && ds == dq + rows * qrow;
                if (one && s->has_zp)
                    one = static_cast<const uint8_t*>(s->pinned_zp[slot]) == hs + rows * srow &&
                          static_cast<const uint8_t*>(s->dev_zp[slot]) == ds + rows * srow;
                if (one) {
                    e = cudaMemcpyAsync(s->dev_q[slot], s->pinned_q[slot], size_t(rows * (qrow + srow + (s->has_zp ? zrow : 0))),
                                        cudaMemcpyHostToDevice, s->copy_stream);
                } else {
                    e = cudaMemcpyAsync(s->dev_q[slot], s->pinned_q[slot], size_t(rows * qrow), cudaMemcpyHostToDevice, s->copy_stream);
                    if (e == cudaSuccess)
                        e = cudaMemcpyAsync(s->dev_s[slot], s->pinned_s[slot], size_t(rows * srow), cudaMemcpyHostToDevice, s->copy_stream);
                    if (e == cudaSuccess && s->has_zp)
                        e = cudaMemcpyAsync(s->dev_zp[slot], s->pinned_zp[slot], size_t(rows * zrow), cudaMemcpyHostToDevice, s->copy_stream);
                }
            } else {
                // The mapped shards are page-locked: the copy engine reads them directly.  Runs of
                // consecutive rows of one shard become one copy.  Codes always go straight from the
                // mapping (rows are hundreds of KB); when the order is scattered the small side
                // arrays are gathered by the CPU first so that they cost one copy each, not one per row.
                std::vector<int64_t> run_first, run_len;   // in units of batch rows
                std::vector<int> run_shard;
                std::vector<int64_t> run_local;
                for (int64_t i = 0; i < rows; ++i) {
                    int sh;
                    int64_t local;
                    locate(s, idx ? idx[i] : first + i, sh, local);
                    if (!run_first.empty() && run_shard.back() == sh && run_local.back() + run_len.back() == local) {
                        ++run_len.back();
                    } else {
                        run_first.push_back(i);
                        run_len.push_back(1);
                        run_shard.push_back(sh);
                        run_local.push_back(local);
                    }
                }
                const bool scattered = run_first.size() > 8;
                if (scattered && s->rows_vectorisable) {
                    const int64_t B = s->d.batch_size;
                    const int64_t o = int64_t(slot) * 3 * B;
                    const uint4** tq = s->row_tables + o;
                    const uint4** ts = tq + B;
                    const uint4** tz = ts + B;
                    for (int64_t i = 0; i < rows; ++i) {
                        int sh;
                        int64_t local;
                        locate(s, idx ? idx[i] : first + i, sh, local);
                        tq[i] = reinterpret_cast<const uint4*>(s->q_dev[sh] + local * qrow);
                        ts[i] = reinterpret_cast<const uint4*>(s->s_dev[sh] + local * srow);
                        if (s->has_zp) tz[i] = reinterpret_cast<const uint4*>(s->zp_dev[sh] + local * zrow);
                    }
                    const uint4** dq = s->row_tables_dev + o;
                    GatherBatch g;
                    g.n_rows = rows;
                    g.n_segments = s->has_zp ? 3 : 2;
                    // blocks in proportion to the bytes (all blocks draw on the link at about the same rate, so equal bytes per
                    // block means they finish together): 48 for the codes, the others rounded up
                    const int bs = int((48 * srow + qrow - 1) / qrow), bz = s->has_zp ? int((48 * zrow + qrow - 1) / qrow) : 0;
                    g.seg[0] = {static_cast<uint4*>(s->dev_q[slot]), dq, qrow / 16, 0, 48};
                    g.seg[1] = {static_cast<uint4*>(s->dev_s[slot]), dq + B, srow / 16, 48, bs > 0 ? bs : 1};
                    g.seg[2] = {static_cast<uint4*>(s->dev_zp[slot]), dq + 2 * B, zrow / 16, 48 + g.seg[1].blocks, bz > 0 ? bz : 1};
                    gather_host_rows_kernel<<<48 + g.seg[1].blocks + (s->has_zp ? g.seg[2].blocks : 0), 256, 0, s->copy_stream>>>(g);
                    e = cudaGetLastError();
                } else {
                    if (scattered) {
                        gather_rows(*s->pool, static_cast<uint8_t*>(s->pinned_s[slot]), srow, rows, src(s->s_bases, srow));
                        if (s->has_zp) gather_rows(*s->pool, static_cast<uint8_t*>(s->pinned_zp[slot]), zrow, rows, src(s->zp_bases, zrow));
                    }
                    for (size_t r = 0; e == cudaSuccess && r < run_first.size(); ++r) {
                        const int sh = run_shard[r];
                        const int64_t at = run_first[r], n = run_len[r], loc = run_local[r];
                        e = cudaMemcpyAsync(static_cast<uint8_t*>(s->dev_q[slot]) + at * qrow, s->q_bases[sh] + loc * qrow, size_t(n * qrow),
                                            cudaMemcpyHostToDevice, s->copy_stream);
                        if (!scattered && e == cudaSuccess)
                            e = cudaMemcpyAsync(static_cast<uint8_t*>(s->dev_s[slot]) + at * srow, s->s_bases[sh] + loc * srow, size_t(n * srow),
                                                cudaMemcpyHostToDevice, s->copy_stream);
                        if (!scattered && e == cudaSuccess && s->has_zp)
                            e = cudaMemcpyAsync(static_cast<uint8_t*>(s->dev_zp[slot]) + at * zrow, s->zp_bases[sh] + loc * zrow, size_t(n * zrow),
                                                cudaMemcpyHostToDevice, s->copy_stream);
                    }
                    if (scattered && e == cudaSuccess)
                        e = cudaMemcpyAsync(s->dev_s[slot], s->pinned_s[slot], size_t(rows * srow), cudaMemcpyHostToDevice, s->copy_stream);
                    if (scattered && e == cudaSuccess && s->has_zp)
                        e = cudaMemcpyAsync(s->dev_zp[slot], s->pinned_zp[slot], size_t(rows * zrow), cudaMemcpyHostToDevice, s->copy_stream);
                }
            }
            if (e == cudaSuccess) e = cudaEventRecord(s->h2d_done[slot], s->copy_stream);
            if (e != cudaSuccess) { producer_fail(s, e, "H2D enqueue"); break; }
            {
                std::lock_guard<std::mutex> lk(s->mu);
                s->produced = b + 1;
            }
            s->cv.notify_all();
        }
        {
            std::lock_guard<std::mutex> lk(s->mu);
            s->pass_active = false;  // finished, aborted or failed: park until the next begin
        }
    }
}

// Stops the current pass (if any) and waits until the producer is parked and the
// copy stream is empty.
int quiesce(tcb_streamer* s) {
    {
        std::unique_lock<std::mutex> lk(s->mu);
        s->abort_pass = true;
        s->cv.notify_all();
        s->cv.wait(lk, [&] { return s->producer_idle; });
        s->pass_active = false;
        s->abort_pass = false;
    }
    TCB_CUDA_TRY(cudaStreamSynchronize(s->copy_stream));
    return TCB_OK;
}

}  // namespace

extern "C" int tcb_pin_host_range(void* p, int64_t bytes) {
    if (!p || bytes <= 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_pin_host_range: null pointer or empty range");
    cudaError_t e = cudaHostRegister(p, size_t(bytes), cudaHostRegisterPortable | cudaHostRegisterMapped);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tcb::fail(TCB_ERR_CUDA, "tcb_pin_host_range: cudaHostRegister(%lld bytes): %s (read-only and shared file mappings "
                         "cannot be page-locked; map the file privately and writable)", (long long)bytes, cudaGetErrorString(e));
    }
    return TCB_OK;
}

extern "C" int tcb_unpin_host_range(void* p) {
    if (!p) return TCB_OK;
    cudaError_t e = cudaHostUnregister(p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return tcb::cuda_fail(e, "tcb_unpin_host_range: cudaHostUnregister");
    }
    return TCB_OK;
}

extern "C" int tcb_streamer_create(const tcb_streamer_desc* desc, tcb_streamer** out) {
    if (!desc || !out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: null argument");
    *out = nullptr;
    if (!tcb::group_size_ok(desc->group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "tcb_streamer_create: group_size %d not in {8, 16, 24, 32, 48, 64, 128}", desc->group_size);
    if (desc->n_slots < 1 || desc->n_slots > 8) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: n_slots %d outside 1..8", desc->n_slots);
    if (desc->n_shards < 1 || desc->n_shards > 4096) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: n_shards %d outside 1..4096", desc->n_shards);
    if (desc->batch_size < 1 || desc->values_per_sample < 1) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: bad sizes");
    if (desc->groups_per_sample != (desc->values_per_sample + desc->group_size - 1) / desc->group_size)
        return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: groups_per_sample does not match values_per_sample / group_size");
    if (desc->values_per_sample % desc->group_size != 0)
        return tcb::fail(TCB_ERR_BAD_ARG,
                         "tcb_streamer_create: values per sample (%lld) must be a multiple of the group size so that "
                         "a batch decodes as one flat tensor", (long long)desc->values_per_sample);
    if (!desc->q_bases || !desc->s_bases || !desc->shard_sizes)
        return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: null shard table");
    const bool has_zp = desc->zp_bases != nullptr;  // a symmetric cache has no zero points
    for (int i = 0; i < desc->n_shards; ++i) {
        if (desc->shard_sizes[i] < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: shard %d has negative size", i);
        if (desc->shard_sizes[i] > 0 && (!desc->q_bases[i] || !desc->s_bases[i] || (has_zp && !desc->zp_bases[i])))
            return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: shard %d has a null mapping", i);
    }
    if (!desc->pinned_q || !desc->pinned_s || !desc->dev_q || !desc->dev_s || !desc->dev_out ||
        (has_zp && (!desc->pinned_zp || !desc->dev_zp)))
        return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: null buffer table");
    for (int i = 0; i < desc->n_slots; ++i)
        if ((!desc->pinned_q[i] && !desc->direct_dma) || !desc->pinned_s[i] || !desc->dev_q[i] || !desc->dev_s[i] || !desc->dev_out[i] ||
            (has_zp && (!desc->pinned_zp[i] || !desc->dev_zp[i])))
            return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_create: null buffer in slot %d", i);

    tcb_streamer* s = new tcb_streamer();
    s->d = *desc;
    s->has_zp = has_zp;
    int64_t total = 0;
    for (int i = 0; i < desc->n_shards; ++i) {
        s->q_bases.push_back(static_cast<const uint8_t*>(desc->q_bases[i]));
        s->s_bases.push_back(static_cast<const uint8_t*>(desc->s_bases[i]));
        s->zp_bases.push_back(has_zp ? static_cast<const uint8_t*>(desc->zp_bases[i]) : nullptr);
        s->shard_start.push_back(total);
        total += desc->shard_sizes[i];
    }
    s->shard_start.push_back(total);
    for (int i = 0; i < desc->n_slots; ++i) {
        s->pinned_q.push_back(desc->pinned_q[i]);
        s->pinned_s.push_back(desc->pinned_s[i]);
        s->pinned_zp.push_back(has_zp ? desc->pinned_zp[i] : nullptr);
        s->dev_q.push_back(desc->dev_q[i]);
        s->dev_s.push_back(desc->dev_s[i]);
        s->dev_zp.push_back(has_zp ? desc->dev_zp[i] : nullptr);
        s->dev_out.push_back(desc->dev_out[i]);
    }
    // the caller's tables need not outlive this call
    s->d.q_bases = s->d.s_bases = s->d.zp_bases = nullptr;
    s->d.shard_sizes = nullptr;
    s->d.pinned_q = s->d.pinned_s = s->d.pinned_zp = s->d.dev_q = s->d.dev_s = s->d.dev_zp = s->d.dev_out = nullptr;
    cudaError_t e = cudaGetDevice(&s->device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&s->copy_stream, cudaStreamNonBlocking);
    for (int i = 0; e == cudaSuccess && i < desc->n_slots; ++i) {
        cudaEvent_t a = nullptr, b = nullptr;
        e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
        if (a) s->h2d_done.push_back(a);
        if (b) s->released.push_back(b);
    }
    if (e != cudaSuccess) {
        int rc = tcb::cuda_fail(e, "tcb_streamer_create");
        for (auto ev : s->h2d_done) cudaEventDestroy(ev);
        for (auto ev : s->released) cudaEventDestroy(ev);
        if (s->copy_stream) cudaStreamDestroy(s->copy_stream);
        delete s;
        return rc;
    }
    if (desc->direct_dma) {
        // the gather kernel moves 16-byte units: rows and mapping bases must be multiples of 16 bytes
        bool ok16 = desc->values_per_sample % 16 == 0 && (desc->groups_per_sample * 2) % 16 == 0 &&
                    (!has_zp || desc->groups_per_sample % 16 == 0);
        for (int i = 0; i < desc->n_shards; ++i)
            ok16 = ok16 && ((reinterpret_cast<uintptr_t>(s->q_bases[i]) | reinterpret_cast<uintptr_t>(s->s_bases[i]) |
                             reinterpret_cast<uintptr_t>(s->zp_bases[i])) & 15) == 0;
        for (int i = 0; i < desc->n_slots; ++i)
            ok16 = ok16 && ((reinterpret_cast<uintptr_t>(s->dev_q[i]) | reinterpret_cast<uintptr_t>(s->dev_s[i]) |
                             reinterpret_cast<uintptr_t>(s->dev_zp[i])) & 15) == 0;
        // device-side addresses of the mappings (they were registered as mapped memory)
        for (int i = 0; ok16 && i < desc->n_shards; ++i) {
            void *dq = nullptr, *ds = nullptr, *dz = nullptr;
            if (desc->shard_sizes[i] > 0 &&
                (cudaHostGetDevicePointer(&dq, const_cast<uint8_t*>(s->q_bases[i]), 0) != cudaSuccess ||
                 cudaHostGetDevicePointer(&ds, const_cast<uint8_t*>(s->s_bases[i]), 0) != cudaSuccess ||
                 (has_zp && cudaHostGetDevicePointer(&dz, const_cast<uint8_t*>(s->zp_bases[i]), 0) != cudaSuccess))) {
                cudaGetLastError();
                ok16 = false;
            }
            s->q_dev.push_back(static_cast<const uint8_t*>(dq));
            s->s_dev.push_back(static_cast<const uint8_t*>(ds));
            s->zp_dev.push_back(static_cast<const uint8_t*>(dz));
        }
        if (ok16) {
            void *t = nullptr, *td = nullptr;
            const size_t bytes = size_t(desc->n_slots) * 3 * size_t(desc->batch_size) * sizeof(void*);
            if (cudaHostAlloc(&t, bytes, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
                cudaHostGetDevicePointer(&td, t, 0) == cudaSuccess) {
                s->row_tables = static_cast<const uint4**>(t);
                s->row_tables_dev = static_cast<const uint4**>(td);
                s->rows_vectorisable = true;
            } else {
                cudaGetLastError();  // fall back to one copy per row
                if (t) cudaFreeHost(t);
            }
        }
    }
    int nt = desc->n_threads < 1 ? 1 : desc->n_threads > 64 ? 64 : desc->n_threads;
    s->pool = new WorkerPool(nt - 1);
    s->producer = std::thread(producer_main, s);
    *out = s;
    return TCB_OK;
}

extern "C" int tcb_streamer_num_samples(const tcb_streamer* s, int64_t* out) {
    if (!s || !out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_num_samples: null argument");
    *out = s->shard_start.back();
    return TCB_OK;
}

extern "C" int tcb_streamer_begin(tcb_streamer* s, const int64_t* order, int64_t n_indices) {
    if (!s) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_begin: null streamer");
    if (n_indices < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_begin: negative count");
    const int64_t total = s->shard_start.back();
    if (!order && n_indices > total)
        return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_begin: %lld samples asked, cache has %lld", (long long)n_indices, (long long)total);
    if (order)
        for (int64_t i = 0; i < n_indices; ++i)
            if (order[i] < 0 || order[i] >= total)
                return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_begin: index %lld out of range at position %lld", (long long)order[i], (long long)i);
    int rc = quiesce(s);
    if (rc != TCB_OK) return rc;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        if (s->producer_error != TCB_OK) return tcb::fail(s->producer_error, "%s", s->producer_msg);
        s->have_order = order != nullptr;
        if (order) s->order.assign(order, order + n_indices); else s->order.clear();
        s->n_indices = n_indices;
        s->n_batches = (n_indices + s->d.batch_size - 1) / s->d.batch_size;
        s->produced = s->acquired = s->consumed = 0;
        s->pass_active = s->n_batches > 0;
    }
    s->cv.notify_all();
    return TCB_OK;
}

extern "C" int tcb_streamer_acquire(tcb_streamer* s, void* consumer_stream, int* slot_out, int* rows_out) {
    if (!s || !slot_out || !rows_out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_acquire: null argument");
    int64_t b, rows;
    {
        std::unique_lock<std::mutex> lk(s->mu);
        if (s->acquired != s->consumed)
            return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_acquire: the previous batch has not been released");
        b = s->acquired;
        if (b >= s->n_batches) {
            *slot_out = 0;
            *rows_out = 0;
            return TCB_OK;
        }
        s->cv.wait(lk, [&] { return s->produced > b || s->producer_error != TCB_OK; });
        if (s->producer_error != TCB_OK) return tcb::fail(s->producer_error, "%s", s->producer_msg);
        rows = batch_rows_of(s, b);
    }
    const int slot = int(b % s->d.n_slots);
    TCB_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(consumer_stream), s->h2d_done[slot], 0));
    {
        std::lock_guard<std::mutex> lk(s->mu);
        s->acquired = b + 1;
    }
    *slot_out = slot;
    *rows_out = int(rows);
    return TCB_OK;
}

extern "C" int tcb_streamer_release(tcb_streamer* s, void* consumer_stream) {
    if (!s) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_release: null streamer");
    int64_t b;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        if (s->acquired != s->consumed + 1) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_streamer_release: no batch is acquired");
        b = s->consumed;
    }
    const int slot = int(b % s->d.n_slots);
    TCB_CUDA_TRY(cudaEventRecord(s->released[slot], static_cast<cudaStream_t>(consumer_stream)));
    {
        std::lock_guard<std::mutex> lk(s->mu);
        s->consumed = b + 1;
    }
    s->cv.notify_all();
    return TCB_OK;
}

extern "C" int tcb_streamer_next(tcb_streamer* s, void* consumer_stream, int* slot_out, int* rows_out) {
    int rc = tcb_streamer_acquire(s, consumer_stream, slot_out, rows_out);
    if (rc != TCB_OK || *rows_out == 0) return rc;
    const int slot = *slot_out;
    rc = tcb::launch_decompress(static_cast<const uint8_t*>(s->dev_q[slot]), static_cast<const uint16_t*>(s->dev_s[slot]),
                                s->has_zp ? static_cast<const uint8_t*>(s->dev_zp[slot]) : nullptr,
                                static_cast<uint16_t*>(s->dev_out[slot]),
                                int64_t(*rows_out) * s->d.values_per_sample, s->d.group_size,
                                static_cast<cudaStream_t>(consumer_stream));
    int rc2 = tcb_streamer_release(s, consumer_stream);
    return rc != TCB_OK ? rc : rc2;
}

extern "C" int tcb_streamer_destroy(tcb_streamer* s) {
    if (!s) return TCB_OK;
    {
        std::lock_guard<std::mutex> lk(s->mu);
        s->quit = true;
        s->abort_pass = true;
    }
    s->cv.notify_all();
    if (s->producer.joinable()) s->producer.join();
    cudaStreamSynchronize(s->copy_stream);
    for (auto ev : s->h2d_done) cudaEventDestroy(ev);
    for (auto ev : s->released) cudaEventDestroy(ev);
    cudaStreamDestroy(s->copy_stream);
    if (s->row_tables) cudaFreeHost(const_cast<uint4**>(s->row_tables));
    delete s->pool;
    delete s;
    return TCB_OK;
}
