// Status / error plumbing of the C ABI.
#include <atomic>
#include <cstring>

#include "tcb_common.h"

namespace tcb {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

void clear_error() { g_err[0] = 0; }

int sm_count() {
    static std::atomic<int> cached[64];   // zero-initialised; the look-up is idempotent
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace tcb

extern "C" int tcb_version(void) { return TCB_VERSION; }

extern "C" const char* tcb_last_error(void) { return tcb::g_err; }

// ---------------------------------------------------------------- sum-order self-test
//
// The encoders pick, per group, the candidate with the smallest squared-error SUM, and the sums are
// compared bit for bit with the host's torch.sum(dim=-1) over the group's G fp32 terms
// (src/tensorcache/codec.py:877).  Floating-point addition is not associative, so the kernels add the
// terms in the order torch's CPU reduction uses: vectors of 8 lanes, runs of four vectors feeding four
// accumulators per lane, left-over vectors into accumulator 0, accumulators combined in order, lane
// totals left to right, a scalar tail last.  That order is a property of the torch build and the CPU's
// vector ISA, not of the algorithm, so it is re-checked on the host the library runs on.
namespace {

float sum_in_kernel_order(const float* e, int g) {
    const int vectors = g / 8, in_runs = vectors & ~3;
    float total = 0.0f;
    for (int lane = 0; lane < 8 && vectors > 0; ++lane) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int v = 0; v < in_runs; ++v) acc[v & 3] = acc[v & 3] + e[v * 8 + lane];
        for (int v = in_runs; v < vectors; ++v) acc[0] = acc[0] + e[v * 8 + lane];
        total = total + (((acc[0] + acc[1]) + acc[2]) + acc[3]);
    }
    for (int i = vectors * 8; i < g; ++i) total = total + e[i];
    return total;
}

}  // namespace

extern "C" int tcb_selftest_sum_order(const float* rows, int64_t n_rows, int group_size, const float* host_sums) {
    if (!tcb::group_size_ok(group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "tcb_selftest_sum_order: group_size %d not in {8, 16, 24, 32, 48, 64, 128}", group_size);
    if (n_rows < 0 || (n_rows > 0 && (!rows || !host_sums))) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_selftest_sum_order: bad arguments");
    for (int64_t r = 0; r < n_rows; ++r) {
        const float mine = sum_in_kernel_order(rows + r * group_size, group_size);
        if (std::memcmp(&mine, host_sums + r, sizeof(float)) != 0)
            return tcb::fail(TCB_ERR_SUM_ORDER,
                             "tcb_selftest_sum_order: row %lld of %d terms sums to %.9g in the encoders' order but the host "
                             "computed %.9g: this host's reduction order differs, encoded scales may differ from the host's own",
                             (long long)r, group_size, double(mine), double(host_sums[r]));
    }
    return TCB_OK;
}
