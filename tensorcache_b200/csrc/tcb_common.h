// Shared host-side helpers of the tcb200 library: status codes, the per-thread
// error message, and CUDA error mapping.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../include/tcb200.h"

namespace tcb {

// Stores a printf-style message for tcb_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);
void clear_error();

inline int cuda_fail(cudaError_t e, const char* what) {
    return fail(TCB_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define TCB_CUDA_TRY(expr)                                       \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) return ::tcb::cuda_fail(_e, #expr); \
    } while (0)

// Group sizes of the codec kernels (encode and decode); the fused GEMM and the no-allocation decode accept 16 / 32 / 64 only.
inline bool group_size_ok(int g) { return g == 8 || g == 16 || g == 24 || g == 32 || g == 48 || g == 64 || g == 128; }
inline bool core_group_size_ok(int g) { return g == 16 || g == 32 || g == 64; }

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace tcb
