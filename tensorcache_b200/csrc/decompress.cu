// AMO-BQ decode kernel for sm_100a:  out = bf16((q - zp) * scale) per group of G codes.
//
// The kernel is HBM-bound (1 + 3/G bytes read and 2 bytes written per value), so
// the design is about bytes in flight and full-width transactions:
//   - each thread owns 16 consecutive codes: one 128-bit load of codes, one bf16
//     scale and one zero point (read once per chunk, never per element), and one
//     256-bit store of 16 bf16 values (two 128-bit stores when `out` is only
//     16-byte aligned);
//   - UNROLL independent chunks per thread are loaded before any is converted,
//     so every SM keeps tens of KB of loads outstanding;
//   - the grid is a multiple of the SM count and strides over tiles.
// Arithmetic: a code byte is spliced into the mantissa of 2^23 (one PRMT), the
// subtraction of (2^23 + zp) yields the exact integer q - zp, and its product with
// a bf16 scale has at most 16 significant bits, so the fp32 product is exact and
// the only rounding is the final round-to-nearest-even to bf16 -- the same value
// the reference computes (src/tensorcache/codec.py:959-965).
#include <cuda_bf16.h>

#include "tcb_common.h"

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 ldg_stream_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void stg_v8(uint16_t* p, const uint32_t (&o)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(o[0]), "r"(o[1]),
                 "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
}

__device__ __forceinline__ void stg_v4x2(uint16_t* p, const uint32_t (&o)[8]) {
    uint4* d = reinterpret_cast<uint4*>(p);
    d[0] = make_uint4(o[0], o[1], o[2], o[3]);
    d[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), one cvt.rn.bf16x2.f32
    return *reinterpret_cast<uint32_t*>(&v);
}

// 4 code bytes of `w` -> 2 packed bf16 pairs
__device__ __forceinline__ void convert_word(uint32_t w, float zmagic, float scale, uint32_t& o0, uint32_t& o1) {
    const uint32_t magic = 0x4B000000u;  // 2^23
    float f0 = __uint_as_float(__byte_perm(w, magic, 0x7650));
    float f1 = __uint_as_float(__byte_perm(w, magic, 0x7651));
    float f2 = __uint_as_float(__byte_perm(w, magic, 0x7652));
    float f3 = __uint_as_float(__byte_perm(w, magic, 0x7653));
    o0 = pack_bf16x2(__fmul_rn(__fsub_rn(f0, zmagic), scale), __fmul_rn(__fsub_rn(f1, zmagic), scale));
    o1 = pack_bf16x2(__fmul_rn(__fsub_rn(f2, zmagic), scale), __fmul_rn(__fsub_rn(f3, zmagic), scale));
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

__device__ __forceinline__ uint16_t decode_one(uint8_t code, uint8_t z, uint16_t sbits) {
    float v = __fmul_rn(__fsub_rn(float(code), float(z)), bf16_bits_to_float(sbits));
    __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&b);
}

// LOG2_CPG: log2(chunks of 16 codes per group) = log2(G / 16)
template <int LOG2_CPG, bool STORE256>
__global__ void __launch_bounds__(kThreads)
decompress_vec_kernel(const uint4* __restrict__ q, const uint16_t* __restrict__ scales,
                      const uint8_t* __restrict__ zp, uint16_t* __restrict__ out, int64_t numel) {
    const int64_t full_chunks = numel >> 4;
    const int64_t tile_chunks = int64_t(kThreads) * kUnroll;
    const int64_t n_tiles = (full_chunks + tile_chunks - 1) / tile_chunks;

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t c0 = tile * tile_chunks + threadIdx.x;
        uint4 w[kUnroll];
        uint16_t sb[kUnroll];
        uint8_t zb[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < full_chunks) {
                w[u] = ldg_stream_v4(q + c);
                const int64_t g = c >> LOG2_CPG;
                sb[u] = __ldg(scales + g);
                zb[u] = __ldg(zp + g);
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < full_chunks) {
                const float scale = bf16_bits_to_float(sb[u]);
                const float zmagic = 8388608.0f + float(zb[u]);
                uint32_t o[8];
                convert_word(w[u].x, zmagic, scale, o[0], o[1]);
                convert_word(w[u].y, zmagic, scale, o[2], o[3]);
                convert_word(w[u].z, zmagic, scale, o[4], o[5]);
                convert_word(w[u].w, zmagic, scale, o[6], o[7]);
                uint16_t* dst = out + (c << 4);
                if (STORE256)
                    stg_v8(dst, o);
                else
                    stg_v4x2(dst, o);
            }
        }
    }

    // ragged tail: numel % 16 codes, handled by the first threads of block 0
    const int tail = int(numel & 15);
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const int64_t i = (full_chunks << 4) + threadIdx.x;
        const int64_t g = i >> (LOG2_CPG + 4);
        out[i] = decode_one(reinterpret_cast<const uint8_t*>(q)[i], zp[g], scales[g]);
    }
}

// Any alignment, one value per thread-iteration.  Same arithmetic as above.
__global__ void __launch_bounds__(kThreads)
decompress_scalar_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scales,
                         const uint8_t* __restrict__ zp, uint16_t* __restrict__ out, int64_t numel, int log2_g) {
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < numel; i += int64_t(gridDim.x) * kThreads) {
        const int64_t g = i >> log2_g;
        out[i] = decode_one(q[i], zp[g], scales[g]);
    }
}

template <int LOG2_CPG>
cudaError_t launch_vec(const uint8_t* q, const uint16_t* s, const uint8_t* zp, uint16_t* out, int64_t numel,
                       bool store256, int grid, cudaStream_t st) {
    if (store256)
        decompress_vec_kernel<LOG2_CPG, true><<<grid, kThreads, 0, st>>>(reinterpret_cast<const uint4*>(q), s, zp, out, numel);
    else
        decompress_vec_kernel<LOG2_CPG, false><<<grid, kThreads, 0, st>>>(reinterpret_cast<const uint4*>(q), s, zp, out, numel);
    return cudaGetLastError();
}

}  // namespace

namespace tcb {

// Shared by the public entry point and the streamer.
int launch_decompress(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out, int64_t numel,
                      int group_size, cudaStream_t st) {
    if (numel == 0) return TCB_OK;
    const int sms = sm_count();
    const bool aligned16 = (reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (!aligned16) {
        const int log2g = group_size == 16 ? 4 : group_size == 32 ? 5 : 6;
        int64_t blocks = (numel + kThreads - 1) / kThreads;
        int grid = int(blocks < int64_t(sms) * 16 ? blocks : int64_t(sms) * 16);
        decompress_scalar_kernel<<<grid, kThreads, 0, st>>>(q, scales, zp, out, numel, log2g);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? TCB_OK : cuda_fail(e, "decompress_scalar_kernel launch");
    }
    const bool store256 = (reinterpret_cast<uintptr_t>(out) & 31) == 0;
    const int64_t tile_chunks = int64_t(kThreads) * kUnroll;
    int64_t n_tiles = ((numel >> 4) + tile_chunks - 1) / tile_chunks;
    if (n_tiles < 1) n_tiles = 1;
    const int64_t max_grid = int64_t(sms) * 8;
    const int grid = int(n_tiles < max_grid ? n_tiles : max_grid);
    cudaError_t e;
    switch (group_size) {
    case 16: e = launch_vec<0>(q, scales, zp, out, numel, store256, grid, st); break;
    case 32: e = launch_vec<1>(q, scales, zp, out, numel, store256, grid, st); break;
    default: e = launch_vec<2>(q, scales, zp, out, numel, store256, grid, st); break;
    }
    return e == cudaSuccess ? TCB_OK : cuda_fail(e, "decompress_vec_kernel launch");
}

}  // namespace tcb

extern "C" int tcb_decompress_amo(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out,
                                  int64_t numel, int group_size, void* stream) {
    if (numel < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_amo: numel %lld < 0", (long long)numel);
    if (!tcb::group_size_ok(group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "tcb_decompress_amo: group_size %d not in {16, 32, 64}", group_size);
    if (numel == 0) return TCB_OK;
    if (!q || !scales || !zp || !out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_amo: null pointer");
    if (reinterpret_cast<uintptr_t>(scales) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_amo: scales not 2-byte aligned");
    if (reinterpret_cast<uintptr_t>(out) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_amo: out not 2-byte aligned");
    return tcb::launch_decompress(q, scales, zp, out, numel, group_size, static_cast<cudaStream_t>(stream));
}
