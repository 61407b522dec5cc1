// AMO-BQ decode kernel for sm_100a:  out = bf16((q - zp) * scale) per group of G codes.
//
// The kernel is HBM-bound (1 + 3/G bytes read and 2 bytes written per value), so
// the design is about bytes in flight, full-width transactions and L2 policy:
//   - each thread owns 32 consecutive codes: one 256-bit load of codes, the bf16
//     scale(s) and zero point(s) of those codes (read once, never per element), and
//     two 256-bit stores of 16 bf16 values each; a warp instruction therefore moves
//     1 KB of contiguous memory and every store fills whole 32-byte sectors;
//   - codes and output are streamed once, so loads and stores carry the
//     L2::evict_first policy -- without it the 88 MB of output written per call
//     pushes dirty lines through L2 in LRU order and costs ~8 % of the bandwidth;
//   - UNROLL independent loads per thread are issued before any is converted;
//   - the grid is exactly one wave (occupancy x SM count) and every block owns an
//     equal contiguous share of the input;
//   - launches opt into programmatic dependent launch, so back-to-back decodes on
//     one stream overlap the next launch's scheduling with this one's tail.
// Pointers that are only 16-byte aligned take a 128-bit variant of the same
// kernel, anything else an element-wise kernel; all three compute the same bits.
// Arithmetic: a code byte is spliced into the mantissa of 2^23 (one PRMT), the
// subtraction of (2^23 + zp) yields the exact integer q - zp, and its product with
// a bf16 scale has at most 16 significant bits, so the fp32 product is exact and
// the only rounding is the final round-to-nearest-even to bf16 -- the same value
// the reference computes (src/tensorcache/codec.py:959-965).
// The symmetric codec (signed codes, no zero point; src/tensorcache/codec.py:685-695)
// runs through the same kernels with SYM = true: the sign bit of every code byte is
// flipped, which turns the int8 value v into the unsigned byte v + 128, and the
// zero point becomes the constant 128.
// Group sizes: the 32- and 16-code kernels cover the powers of two 16..128; 8, 24
// and 48 take a kernel that owns 8 codes per thread (no group straddles an octet).
#include <cuda_bf16.h>

#include <atomic>

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

constexpr uint32_t kSignFlip = 0x80808080u;

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(uint32_t(b) << 16); }

template <bool SYM>
__device__ __forceinline__ uint16_t decode_one(uint8_t code, const uint8_t* __restrict__ zp, int64_t g, uint16_t sbits) {
    const float centred = SYM ? float(int8_t(code)) : __fsub_rn(float(code), float(zp[g]));
    float v = __fmul_rn(centred, bf16_bits_to_float(sbits));
    __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&b);
}

__device__ __forceinline__ void ldg_stream_v8(const uint8_t* p, uint32_t (&w)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}

__device__ __forceinline__ void stg_stream_v8(uint16_t* p, const uint32_t (&o)[8]) {
    asm volatile("st.global.L2::evict_first.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(o[0]), "r"(o[1]),
                 "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
}

constexpr int kUnroll32 = 2;

// Main kernel: 32 codes per thread.  LOG2_G = log2(group size) in {4, 5, 6, 7}.
// Needs q and out 32-byte aligned.  Every block owns one contiguous, equally
// sized range of 32-code units; the grid is exactly the number of blocks the
// device holds at once, so there is a single wave and no block does more work
// than another.
template <int LOG2_G, bool SYM>
__global__ void __launch_bounds__(kThreads)
decompress_v8_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scales,
                     const uint8_t* __restrict__ zp, uint16_t* __restrict__ out, int64_t numel) {
    // Programmatic dependent launch: let the next kernel of the stream get
    // scheduled while this one drains, and do not touch memory before the
    // previous kernel of the stream has completed and flushed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int64_t units = numel >> 5;
    const int64_t begin = units * blockIdx.x / gridDim.x;
    const int64_t end = units * (blockIdx.x + 1) / gridDim.x;

    for (int64_t t0 = begin + threadIdx.x; t0 < end; t0 += int64_t(kThreads) * kUnroll32) {
        uint32_t w[kUnroll32][8];
        uint16_t sb[kUnroll32][2];
        uint8_t zb[kUnroll32][2];
#pragma unroll
        for (int u = 0; u < kUnroll32; ++u) {
            const int64_t t = t0 + int64_t(u) * kThreads;
            if (t < end) {
                ldg_stream_v8(q + (t << 5), w[u]);
                if (LOG2_G == 4) {  // two groups of 16 per unit
                    sb[u][0] = __ldg(scales + 2 * t);
                    sb[u][1] = __ldg(scales + 2 * t + 1);
                    if (!SYM) {
                        zb[u][0] = __ldg(zp + 2 * t);
                        zb[u][1] = __ldg(zp + 2 * t + 1);
                    }
                } else {  // one group (G32) or part of a group (G64, G128)
                    const int64_t g = t >> (LOG2_G >= 5 ? LOG2_G - 5 : 0);
                    sb[u][0] = sb[u][1] = __ldg(scales + g);
                    if (!SYM) zb[u][0] = zb[u][1] = __ldg(zp + g);
                }
                if (SYM) {
                    zb[u][0] = zb[u][1] = 128;
#pragma unroll
                    for (int k = 0; k < 8; ++k) w[u][k] ^= kSignFlip;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll32; ++u) {
            const int64_t t = t0 + int64_t(u) * kThreads;
            if (t < end) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float scale = bf16_bits_to_float(sb[u][h]);
                    const float zmagic = 8388608.0f + float(zb[u][h]);
                    uint32_t o[8];
                    convert_word(w[u][4 * h + 0], zmagic, scale, o[0], o[1]);
                    convert_word(w[u][4 * h + 1], zmagic, scale, o[2], o[3]);
                    convert_word(w[u][4 * h + 2], zmagic, scale, o[4], o[5]);
                    convert_word(w[u][4 * h + 3], zmagic, scale, o[6], o[7]);
                    stg_stream_v8(out + (t << 5) + 16 * h, o);
                }
            }
        }
    }

    // ragged tail: numel % 32 codes, handled by the first threads of block 0
    const int tail = int(numel & 31);
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const int64_t i = (units << 5) + threadIdx.x;
        const int64_t g = i >> LOG2_G;
        out[i] = decode_one<SYM>(q[i], zp, g, scales[g]);
    }
}

// Variant for pointers that are 16- but not 32-byte aligned: 16 codes per thread,
// 128-bit load, two 128-bit stores.  LOG2_CPG = log2(G / 16).
template <int LOG2_CPG, bool SYM>
__global__ void __launch_bounds__(kThreads)
decompress_vec_kernel(const uint4* __restrict__ q, const uint16_t* __restrict__ scales,
                      const uint8_t* __restrict__ zp, uint16_t* __restrict__ out, int64_t numel) {
    // Programmatic dependent launch: let the next kernel of the stream get
    // scheduled while this one drains, and do not touch memory before the
    // previous kernel of the stream has completed and flushed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int64_t full_chunks = numel >> 4;
    const int64_t begin = full_chunks * blockIdx.x / gridDim.x;
    const int64_t end = full_chunks * (blockIdx.x + 1) / gridDim.x;

    for (int64_t c0 = begin + threadIdx.x; c0 < end; c0 += int64_t(kThreads) * kUnroll) {
        uint4 w[kUnroll];
        uint16_t sb[kUnroll];
        uint8_t zb[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < end) {
                w[u] = ldg_stream_v4(q + c);
                const int64_t g = c >> LOG2_CPG;
                sb[u] = __ldg(scales + g);
                if (SYM) {
                    zb[u] = 128;
                    w[u].x ^= kSignFlip, w[u].y ^= kSignFlip, w[u].z ^= kSignFlip, w[u].w ^= kSignFlip;
                } else {
                    zb[u] = __ldg(zp + g);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < end) {
                const float scale = bf16_bits_to_float(sb[u]);
                const float zmagic = 8388608.0f + float(zb[u]);
                uint32_t o[8];
                convert_word(w[u].x, zmagic, scale, o[0], o[1]);
                convert_word(w[u].y, zmagic, scale, o[2], o[3]);
                convert_word(w[u].z, zmagic, scale, o[4], o[5]);
                convert_word(w[u].w, zmagic, scale, o[6], o[7]);
                stg_v4x2(out + (c << 4), o);
            }
        }
    }

    // ragged tail: numel % 16 codes, handled by the first threads of block 0
    const int tail = int(numel & 15);
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const int64_t i = (full_chunks << 4) + threadIdx.x;
        const int64_t g = i >> (LOG2_CPG + 4);
        out[i] = decode_one<SYM>(reinterpret_cast<const uint8_t*>(q)[i], zp, g, scales[g]);
    }
}

// Group sizes that are a multiple of 8 but not a power of two >= 16 (8, 24, 48), 32-byte aligned
// pointers: the main kernel's data movement (32 codes per thread, one 256-bit load, two 256-bit
// stores) with one scale / zero point per octet of codes.  OPG = octets per group.  A thread's four
// octets belong to four groups at G = 8 and to at most two neighbouring groups at G = 24 / 48, so the
// scales and zero points come in one 64-bit + one 32-bit load (G = 8, VEC_META: scales 8-byte and zero
// points 4-byte aligned) or in two loads of each (G = 24 / 48) instead of four scalar loads of each.
template <int OPG, bool SYM, bool VEC_META>
__global__ void __launch_bounds__(kThreads)
decompress_v8_oct_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scales, const uint8_t* __restrict__ zp,
                         uint16_t* __restrict__ out, int64_t numel) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int64_t units = numel >> 5;
    const int64_t begin = units * blockIdx.x / gridDim.x;
    const int64_t end = units * (blockIdx.x + 1) / gridDim.x;

    for (int64_t t0 = begin + threadIdx.x; t0 < end; t0 += int64_t(kThreads) * kUnroll32) {
        uint32_t w[kUnroll32][8];
        uint32_t ms[kUnroll32][2];   // the four octets' scales, two bf16 per word
        uint32_t mz[kUnroll32];      // their zero points, one per byte
#pragma unroll
        for (int u = 0; u < kUnroll32; ++u) {
            const int64_t t = t0 + int64_t(u) * kThreads;
            if (t < end) {
                ldg_stream_v8(q + (t << 5), w[u]);
                if (OPG == 1 && VEC_META) {
                    const uint2 s4 = __ldg(reinterpret_cast<const uint2*>(scales + 4 * t));
                    ms[u][0] = s4.x, ms[u][1] = s4.y;
                    mz[u] = SYM ? kSignFlip : __ldg(reinterpret_cast<const uint32_t*>(zp + 4 * t));
                } else if (OPG == 1) {
                    ms[u][0] = uint32_t(__ldg(scales + 4 * t)) | uint32_t(__ldg(scales + 4 * t + 1)) << 16;
                    ms[u][1] = uint32_t(__ldg(scales + 4 * t + 2)) | uint32_t(__ldg(scales + 4 * t + 3)) << 16;
                    mz[u] = SYM ? kSignFlip
                                : uint32_t(__ldg(zp + 4 * t)) | uint32_t(__ldg(zp + 4 * t + 1)) << 8 |
                                      uint32_t(__ldg(zp + 4 * t + 2)) << 16 | uint32_t(__ldg(zp + 4 * t + 3)) << 24;
                } else {
                    const int64_t g0 = (4 * t) / OPG;
                    const int first = int((g0 + 1) * OPG - 4 * t);  // this thread's octets [0, first) are of group g0, the rest of g0 + 1
                    const bool two = first < 4;
                    const uint32_t s0 = __ldg(scales + g0), s1 = two ? uint32_t(__ldg(scales + g0 + 1)) : s0;
                    const uint32_t z0 = SYM ? 128u : uint32_t(__ldg(zp + g0)), z1 = (SYM || !two) ? z0 : uint32_t(__ldg(zp + g0 + 1));
                    // first is 1, 2, 3 or >= 4: octet j takes group g0 when j < first
                    ms[u][0] = s0 | (first > 1 ? s0 : s1) << 16;
                    ms[u][1] = (first > 2 ? s0 : s1) | (first > 3 ? s0 : s1) << 16;
                    mz[u] = z0 | (first > 1 ? z0 : z1) << 8 | (first > 2 ? z0 : z1) << 16 | (first > 3 ? z0 : z1) << 24;
                }
                if (SYM) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) w[u][k] ^= kSignFlip;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll32; ++u) {
            const int64_t t = t0 + int64_t(u) * kThreads;
            if (t < end) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t o[8];
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int oct = 2 * h + j;
                        // bf16 bits -> fp32 bits: the even octet's scale sits in the low half of its word
                        const float scale = __uint_as_float((oct & 1) ? (ms[u][oct >> 1] & 0xFFFF0000u) : (ms[u][oct >> 1] << 16));
                        // 2^23 + zp is exactly the fp32 whose low mantissa byte is zp
                        const float zmagic = __uint_as_float(__byte_perm(mz[u], 0x4B000000u, 0x7650 + oct));
                        convert_word(w[u][4 * h + 2 * j], zmagic, scale, o[4 * j], o[4 * j + 1]);
                        convert_word(w[u][4 * h + 2 * j + 1], zmagic, scale, o[4 * j + 2], o[4 * j + 3]);
                    }
                    stg_stream_v8(out + (t << 5) + 16 * h, o);
                }
            }
        }
    }

    const int tail = int(numel & 31);
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const int64_t i = (units << 5) + threadIdx.x;
        const int64_t g = i / (8 * OPG);
        out[i] = decode_one<SYM>(q[i], zp, g, scales[g]);
    }
}

// The same group sizes with pointers that are not 32-byte aligned: 8 codes per
// thread, one 64-bit load and one 128-bit store; OPG = octets per group.  Needs q 8-byte and out
// 16-byte aligned.
template <int OPG, bool SYM>
__global__ void __launch_bounds__(kThreads)
decompress_oct_kernel(const uint2* __restrict__ q, const uint16_t* __restrict__ scales, const uint8_t* __restrict__ zp,
                      uint16_t* __restrict__ out, int64_t numel) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int64_t octs = numel >> 3;
    const int64_t begin = octs * blockIdx.x / gridDim.x;
    const int64_t end = octs * (blockIdx.x + 1) / gridDim.x;

    for (int64_t c0 = begin + threadIdx.x; c0 < end; c0 += int64_t(kThreads) * kUnroll) {
        uint2 w[kUnroll];
        uint16_t sb[kUnroll];
        uint8_t zb[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < end) {
                w[u] = __ldg(q + c);
                const int64_t g = c / OPG;
                sb[u] = __ldg(scales + g);
                if (SYM) {
                    zb[u] = 128;
                    w[u].x ^= kSignFlip, w[u].y ^= kSignFlip;
                } else {
                    zb[u] = __ldg(zp + g);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t c = c0 + int64_t(u) * kThreads;
            if (c < end) {
                const float scale = bf16_bits_to_float(sb[u]);
                const float zmagic = 8388608.0f + float(zb[u]);
                uint32_t o0, o1, o2, o3;
                convert_word(w[u].x, zmagic, scale, o0, o1);
                convert_word(w[u].y, zmagic, scale, o2, o3);
                *reinterpret_cast<uint4*>(out + (c << 3)) = make_uint4(o0, o1, o2, o3);
            }
        }
    }

    const int tail = int(numel & 7);
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const int64_t i = (octs << 3) + threadIdx.x;
        const int64_t g = i / (8 * OPG);
        out[i] = decode_one<SYM>(reinterpret_cast<const uint8_t*>(q)[i], zp, g, scales[g]);
    }
}

// Any alignment, one value per thread-iteration.  Same arithmetic as above.
template <bool SYM>
__global__ void __launch_bounds__(kThreads)
decompress_scalar_kernel(const uint8_t* __restrict__ q, const uint16_t* __restrict__ scales,
                         const uint8_t* __restrict__ zp, uint16_t* __restrict__ out, int64_t numel, int group_size) {
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < numel; i += int64_t(gridDim.x) * kThreads) {
        const int64_t g = i / group_size;
        out[i] = decode_one<SYM>(q[i], zp, g, scales[g]);
    }
}

// Blocks of `kernel` one device holds at once (occupancy x SM count), cached per device.  The look-up is
// idempotent, so concurrent first calls may both do it; the cache word itself is atomic.
typedef std::atomic<int> WaveCache[64];

template <typename K>
int resident_blocks(K kernel, WaveCache& cache) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return tcb::sm_count() * 4;
    int have = cache[dev].load(std::memory_order_relaxed);
    if (have == 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
        have = per_sm * tcb::sm_count();
        cache[dev].store(have, std::memory_order_relaxed);
    }
    return have;
}

// The per-device wave sizes of the power-of-two kernels, outside the launch functions so that they can be filled ahead of time.
template <int LOG2_G, bool SYM>
struct AlignedWaves {
    static WaveCache v8, vec;
};
template <int LOG2_G, bool SYM>
WaveCache AlignedWaves<LOG2_G, SYM>::v8;
template <int LOG2_G, bool SYM>
WaveCache AlignedWaves<LOG2_G, SYM>::vec;

template <typename K, typename QPtr>
cudaError_t launch_one_wave(K kernel, WaveCache& cache, int64_t units, QPtr q, const uint16_t* s, const uint8_t* zp, uint16_t* out,
                            int64_t numel, cudaStream_t st) {
    int64_t grid = resident_blocks(kernel, cache);
    const int64_t min_units_per_block = kThreads;  // small inputs: fewer, fuller blocks
    if (grid * min_units_per_block > units) grid = (units + min_units_per_block - 1) / min_units_per_block;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, q, s, zp, out, numel);
}

template <int LOG2_G, bool SYM>
cudaError_t launch_aligned(const uint8_t* q, const uint16_t* s, const uint8_t* zp, uint16_t* out, int64_t numel,
                           bool aligned32, cudaStream_t st) {
    if (aligned32)
        return launch_one_wave(decompress_v8_kernel<LOG2_G, SYM>, AlignedWaves<LOG2_G, SYM>::v8, numel >> 5, q, s, zp, out, numel, st);
    return launch_one_wave(decompress_vec_kernel<LOG2_G - 4, SYM>, AlignedWaves<LOG2_G, SYM>::vec, numel >> 4,
                           reinterpret_cast<const uint4*>(q), s, zp, out, numel, st);
}

// Loads the kernels of one group size (all three output-alignment classes) onto the current device and fills
// their wave sizes, without launching anything.
template <int LOG2_G>
cudaError_t prime_amo_variants() {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, decompress_v8_kernel<LOG2_G, false>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, decompress_vec_kernel<LOG2_G - 4, false>);
    if (e != cudaSuccess) return e;
    (void)resident_blocks(decompress_v8_kernel<LOG2_G, false>, AlignedWaves<LOG2_G, false>::v8);
    (void)resident_blocks(decompress_vec_kernel<LOG2_G - 4, false>, AlignedWaves<LOG2_G, false>::vec);
    return cudaSuccess;
}

template <int OPG, bool SYM>
cudaError_t launch_oct(const uint8_t* q, const uint16_t* s, const uint8_t* zp, uint16_t* out, int64_t numel, bool aligned32,
                       cudaStream_t st) {
    static WaveCache cache, cache32, cache32v;
    if (aligned32) {
        if constexpr (OPG == 1) {
            const bool vec_meta = (reinterpret_cast<uintptr_t>(s) & 7) == 0 && (SYM || (reinterpret_cast<uintptr_t>(zp) & 3) == 0);
            if (vec_meta)
                return launch_one_wave(decompress_v8_oct_kernel<OPG, SYM, true>, cache32v, numel >> 5, q, s, zp, out, numel, st);
        }
        return launch_one_wave(decompress_v8_oct_kernel<OPG, SYM, false>, cache32, numel >> 5, q, s, zp, out, numel, st);
    }
    return launch_one_wave(decompress_oct_kernel<OPG, SYM>, cache, numel >> 3, reinterpret_cast<const uint2*>(q), s, zp, out,
                           numel, st);
}

template <bool SYM>
int launch_any(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out, int64_t numel, int group_size,
               cudaStream_t st) {
    const uintptr_t qa = reinterpret_cast<uintptr_t>(q), oa = reinterpret_cast<uintptr_t>(out);
    const bool pow2_wide = group_size == 16 || group_size == 32 || group_size == 64 || group_size == 128;
    const bool vector_ok = pow2_wide ? ((qa | oa) & 15) == 0 : ((qa & 7) == 0 && (oa & 15) == 0);
    if (!vector_ok) {
        int64_t blocks = (numel + kThreads - 1) / kThreads;
        const int64_t cap = int64_t(tcb::sm_count()) * 16;
        decompress_scalar_kernel<SYM><<<int(blocks < cap ? blocks : cap), kThreads, 0, st>>>(q, scales, zp, out, numel, group_size);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? TCB_OK : tcb::cuda_fail(e, "decompress_scalar_kernel launch");
    }
    const bool aligned32 = ((qa | oa) & 31) == 0;
    cudaError_t e;
    switch (group_size) {
    case 8: e = launch_oct<1, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    case 24: e = launch_oct<3, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    case 48: e = launch_oct<6, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    case 16: e = launch_aligned<4, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    case 32: e = launch_aligned<5, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    case 64: e = launch_aligned<6, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    default: e = launch_aligned<7, SYM>(q, scales, zp, out, numel, aligned32, st); break;
    }
    return e == cudaSuccess ? TCB_OK : tcb::cuda_fail(e, "decompress kernel launch");
}

}  // namespace

namespace tcb {

// Makes every kernel the AMO-BQ decode of G = 16 / 32 / 64 can pick (whatever the output's alignment) resident on
// the current device, so that a later launch loads no module and asks no occupancy question.
cudaError_t prime_amo_decompress() {
    cudaFuncAttributes fa;
    cudaError_t e = prime_amo_variants<4>();
    if (e == cudaSuccess) e = prime_amo_variants<5>();
    if (e == cudaSuccess) e = prime_amo_variants<6>();
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, decompress_scalar_kernel<false>);
    (void)sm_count();
    return e;
}

// Shared by the public entry points and the streamer.  zp == nullptr selects the symmetric codec.
int launch_decompress(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out, int64_t numel,
                      int group_size, cudaStream_t st) {
    if (numel == 0) return TCB_OK;
    return zp ? launch_any<false>(q, scales, zp, out, numel, group_size, st)
              : launch_any<true>(q, scales, nullptr, out, numel, group_size, st);
}

}  // namespace tcb

extern "C" int tcb_decompress_amo(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out,
                                  int64_t numel, int group_size, void* stream) {
    if (numel < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_amo: numel %lld < 0", (long long)numel);
    if (!tcb::group_size_ok(group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "tcb_decompress_amo: group_size %d not in {8, 16, 24, 32, 48, 64, 128}", group_size);
    if (numel == 0) return TCB_OK;
    if (!q || !scales || !zp || !out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_amo: null pointer");
    if (reinterpret_cast<uintptr_t>(scales) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_amo: scales not 2-byte aligned");
    if (reinterpret_cast<uintptr_t>(out) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_amo: out not 2-byte aligned");
    return tcb::launch_decompress(q, scales, zp, out, numel, group_size, static_cast<cudaStream_t>(stream));
}

extern "C" int tcb_decompress_sym(const int8_t* q, const uint16_t* scales, uint16_t* out, int64_t numel, int group_size,
                                  void* stream) {
    if (numel < 0) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_sym: numel %lld < 0", (long long)numel);
    if (!tcb::group_size_ok(group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "tcb_decompress_sym: group_size %d not in {8, 16, 24, 32, 48, 64, 128}", group_size);
    if (numel == 0) return TCB_OK;
    if (!q || !scales || !out) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_decompress_sym: null pointer");
    if (reinterpret_cast<uintptr_t>(scales) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_sym: scales not 2-byte aligned");
    if (reinterpret_cast<uintptr_t>(out) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "tcb_decompress_sym: out not 2-byte aligned");
    return tcb::launch_decompress(reinterpret_cast<const uint8_t*>(q), scales, nullptr, out, numel, group_size,
                                  static_cast<cudaStream_t>(stream));
}
