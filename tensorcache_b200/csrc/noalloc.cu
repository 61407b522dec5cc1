// Decode of host-resident AMO-BQ codes without any device allocation.
//
// Some callers may not allocate device memory at the moment they need a decode: a
// serving or training process that handed the whole GPU to its own allocator at
// start-up (a raw cudaMalloc from a plug-in then fails or fragments that plan), or a
// loader hook that runs while another thread of the process is capturing a CUDA
// graph (cudaMalloc is not permitted then).  For them the staging area that the
// batch readers normally get from the caller lives here, inside the library image:
// a fixed array in device memory that exists on every GPU that loads the library,
// from load until exit.
//
// The array's name is only meaningful to device code.  Host code must ask the
// runtime where the array lives on the current device (cudaGetSymbolAddress) and
// hand that address to copies and kernels; this file does so once per device.
#include "tcb_common.h"

#include <atomic>

namespace tcb {
int launch_decompress(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out, int64_t numel,
                      int group_size, cudaStream_t st);
cudaError_t prime_amo_decompress();
}

namespace {

constexpr int64_t kMaxValues = TCB_NOALLOC_MAX_VALUES;            // codes per call
constexpr int64_t kMaxGroups = kMaxValues / 16;                    // smallest group size
constexpr int64_t kOffScales = kMaxValues;                         // 256-byte aligned by construction
constexpr int64_t kOffZp = kOffScales + kMaxGroups * 2;
constexpr int64_t kScratchBytes = kOffZp + kMaxGroups;

static __device__ __align__(256) uint8_t g_decode_staging[kScratchBytes];

// Address of g_decode_staging on the current device.  The first call on a device looks it up (which is also what
// makes the runtime place the array and load this file's module there) and, in the same set-up step, makes every
// decode kernel this entry point can choose resident, so that later calls neither load code nor query occupancy.
// Two host threads making their first call at once both do the idempotent look-up; the cache word is atomic.
cudaError_t staging_address(uint8_t** out) {
    static std::atomic<uint8_t*> cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    uint8_t* base = cached[dev].load(std::memory_order_acquire);
    if (!base) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_staging);
        if (e != cudaSuccess) return e;
        e = tcb::prime_amo_decompress();
        if (e != cudaSuccess) return e;
        base = static_cast<uint8_t*>(p);
        cached[dev].store(base, std::memory_order_release);
    }
    *out = base;
    return cudaSuccess;
}

}  // namespace

extern "C" int tcb_decompress_amo_host_noalloc(const uint8_t* q_host, const uint16_t* scales_host, const uint8_t* zp_host,
                                               uint16_t* out_dev, int64_t numel, int group_size, void* stream) {
    const char* who = "tcb_decompress_amo_host_noalloc";
    if (numel < 0) return tcb::fail(TCB_ERR_BAD_ARG, "%s: numel %lld < 0", who, (long long)numel);
    if (!tcb::core_group_size_ok(group_size)) return tcb::fail(TCB_ERR_GROUP_SIZE, "%s: group_size %d not in {16, 32, 64}", who, group_size);
    if (numel > kMaxValues)
        return tcb::fail(TCB_ERR_TOO_LARGE, "%s: %lld values asked, the built-in staging area holds at most %lld per call "
                         "(split the tensor at a multiple of the group size)", who, (long long)numel, (long long)kMaxValues);
    if (numel == 0) return TCB_OK;
    if (!q_host || !scales_host || !zp_host || !out_dev) return tcb::fail(TCB_ERR_BAD_ARG, "%s: null pointer", who);
    if (reinterpret_cast<uintptr_t>(out_dev) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "%s: out not 2-byte aligned", who);
    uint8_t* base = nullptr;
    cudaError_t e = staging_address(&base);
    if (e != cudaSuccess) return tcb::cuda_fail(e, "cudaGetSymbolAddress(decode staging)");
    const int64_t groups = (numel + group_size - 1) / group_size;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // every byte the kernel reads is written by these copies first, so nothing has to be cleared
    TCB_CUDA_TRY(cudaMemcpyAsync(base, q_host, size_t(numel), cudaMemcpyHostToDevice, st));
    TCB_CUDA_TRY(cudaMemcpyAsync(base + kOffScales, scales_host, size_t(groups) * 2, cudaMemcpyHostToDevice, st));
    TCB_CUDA_TRY(cudaMemcpyAsync(base + kOffZp, zp_host, size_t(groups), cudaMemcpyHostToDevice, st));
    return tcb::launch_decompress(base, reinterpret_cast<const uint16_t*>(base + kOffScales), base + kOffZp, out_dev, numel,
                                  group_size, st);
}
