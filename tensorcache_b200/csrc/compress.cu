// AMO-BQ encode kernels for sm_100a: per-group asymmetric min/max plus the scale
// search of the reference's CPU path, reproduced bit for bit.
//
// Three layouts of a group over the lanes share the arithmetic:
//   * "lane" kernels (compress_legacy_lane_kernel, compress_quality_lane_kernel,
//     compress_sym_lane_kernel) -- the hot path for G <= 32, and for G = 48 / 64 with
//     the candidate-table presets: ONE group per lane.  The group's values stay in the
//     thread's registers, nothing crosses lanes, the per-candidate set-up (scale, zero
//     point, reciprocal) is paid once per G values, and the squared-error sum follows
//     the reference's order with plain additions in the right sequence.
//   * "pair" kernels (compress_legacy_pair_kernel, compress_sym_pair_kernel) -- G = 128
//     with the candidate-table presets and the symmetric search: two lanes per group,
//     lane j owns columns 4j .. 4j+3 of every 8-wide vector, 64 values in registers
//     each; two shuffles per candidate chain the column totals in order.
//   * the "quad" kernel (compress_quality_kernel) -- the quality search at G = 48 / 64 /
//     128, where its three code trials per value leave no room for 64 values in one
//     thread's registers: four lanes per group.  Lane j of the quad owns
//     columns 2j and 2j+1 of every 8-wide vector of the group, so that each lane
//     accumulates its two columns privately in the reference's order and the four lanes
//     chain their totals with warp shuffles; min/max use xor-shuffles inside the quad.
//   * compress_sym_stream_kernel: the plain symmetric codec has no search and is
//     HBM-bound; 16 values per thread, one 256-bit load, one 128-bit store.
// The reference's order of the sum (its CPU reduction): vectors of 8 lanes, four partial
// accumulators per lane over runs of four vectors, left-over vectors into accumulator 0,
// accumulators combined in order, then the 8 lane totals left to right.
//
// Exactness rules (src/tensorcache/codec.py:833-893 and :721-771):
//   every operation is a separate IEEE binary32 operation -- __fdiv_rn / __fmul_rn /
//   __fadd_rn / __fsub_rn (never contracted into FMA), rintf() for
//   round-half-to-even, the first minimum wins (strict <), and the candidate
//   multipliers are the host's torch.linspace values passed in by value.
// The kernels are ALU-bound (~14 thread instructions per value and candidate).
// The reference's per-value IEEE division x / s is computed as the exact IEEE quotient
// from the candidate's reciprocal and two FMAs (exact_quotient), so the result is still the
// reference's, bit for bit.
// The kernels never synchronise with the host.
#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tcb_common.h"

namespace {

constexpr int kThreads = 256;

struct CandTable {
    float m[64];
    int n;
};

__device__ __forceinline__ bool finite_f32(float v) { return (__float_as_uint(v) & 0x7f800000u) != 0x7f800000u; }

__device__ __forceinline__ float clamp255(float v) { return fminf(fmaxf(v, 0.0f), 255.0f); }

// The correctly rounded quotient x / s without a division, for a divisor whose significand is not
// all ones (the scales of the quality search and of the symmetric codec are bf16 values: 8 bits).
// With r = rn(1 / s) and t = rn(x * r), the residual x - t * s is exact in one FMA and
// rn(t + residual * r) is the IEEE quotient (Markstein's correction step, the one a division routine
// ends with).  The residual can only underflow where the quotient is far below 2^-20, which cannot
// change the rounded code.  A cheaper reciprocal multiply with a fall-back near rounding boundaries does not do
// here: values and scales are often both short, so x / s lands exactly on k + 0.5 for a large share of the values
// and the "rare" fall-back would run all the time.
__device__ __forceinline__ float exact_quotient(float x, float s, float r) {
    const float t = __fmul_rn(x, r);
    return __fmaf_rn(__fmaf_rn(-t, s, x), r, t);
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <typename T>
__device__ __forceinline__ float widen(T v);
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float widen<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float widen<float>(float v) { return v; }

// Loads the lane's G/4 values of group `g` (zero-padded past numel), cleans
// non-finite values to 0 and records which were finite.
template <int G, typename T>
__device__ __forceinline__ void load_lane(const T* __restrict__ x, int64_t numel, int64_t base, int j, bool pair_aligned,
                                          float (&v)[G / 4], uint32_t& finmask) {
    constexpr int NVEC = G / 8;
    finmask = 0;
    const bool whole = base + G <= numel;
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
        const int64_t i = base + k * 8 + 2 * j;
        float a, b;
        if (whole && pair_aligned) {
            if (sizeof(T) == 2) {
                uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(x + i));
                uint16_t lo = uint16_t(w & 0xffffu), hi = uint16_t(w >> 16);
                a = widen<T>(*reinterpret_cast<T*>(&lo));
                b = widen<T>(*reinterpret_cast<T*>(&hi));
            } else {
                float2 w = __ldg(reinterpret_cast<const float2*>(x + i));
                a = w.x;
                b = w.y;
            }
        } else {
            a = i < numel ? widen<T>(x[i]) : 0.0f;
            b = i + 1 < numel ? widen<T>(x[i + 1]) : 0.0f;
        }
        const bool fa = finite_f32(a), fb = finite_f32(b);
        v[2 * k] = fa ? a : 0.0f;
        v[2 * k + 1] = fb ? b : 0.0f;
        finmask |= (fa ? 1u : 0u) << (2 * k);
        finmask |= (fb ? 1u : 0u) << (2 * k + 1);
    }
}

// Sum of the group's G error terms in the reference's order.  e[2k + a] is the
// term of element 8k + 2j + a.  Returns the total on every lane of the quad.
template <int G>
__device__ __forceinline__ float quad_sum(const float (&e)[G / 4], int j, int lane, uint32_t qmask) {
    // Column totals in ATen's order: complete runs of four 8-wide vectors feed four accumulators
    // (vector v of a run goes to accumulator v % 4), left-over vectors go to accumulator 0, and the
    // accumulators are combined ((a0 + a1) + a2) + a3.  All indices are compile-time constants.
    constexpr int NVEC = G / 8;
    constexpr int FULL = (NVEC / 4) * 4;
    float col[2];
#pragma unroll
    for (int a = 0; a < 2; ++a) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int vI = 0; vI < NVEC; ++vI) {
            const int t = vI < FULL ? (vI & 3) : 0;
            const bool first = vI < FULL ? vI < 4 : (FULL == 0 && vI == 0);
            acc[t] = first ? e[2 * vI + a] : __fadd_rn(acc[t], e[2 * vI + a]);
        }
        col[a] = FULL > 0 ? __fadd_rn(__fadd_rn(__fadd_rn(acc[0], acc[1]), acc[2]), acc[3]) : acc[0];
    }
    // lane totals L0..L7 are added left to right: lane 0 starts, lanes 1..3 continue
    const int q0 = lane & ~3;
    float t = __fadd_rn(col[0], col[1]);
#pragma unroll
    for (int step = 1; step < 4; ++step) {
        float prev = __shfl_sync(qmask, t, q0 + step - 1);
        if (j == step) t = __fadd_rn(__fadd_rn(prev, col[0]), col[1]);
    }
    return __shfl_sync(qmask, t, q0 + 3);
}

__device__ __forceinline__ float quad_min(float v, uint32_t qmask) {
    v = fminf(v, __shfl_xor_sync(qmask, v, 1));
    return fminf(v, __shfl_xor_sync(qmask, v, 2));
}
__device__ __forceinline__ float quad_max(float v, uint32_t qmask) {
    v = fmaxf(v, __shfl_xor_sync(qmask, v, 1));
    return fmaxf(v, __shfl_xor_sync(qmask, v, 2));
}

template <int G>
__device__ __forceinline__ void store_codes(uint8_t* __restrict__ q, int64_t numel, int64_t base, int j, bool pair_aligned,
                                            const uint8_t (&c)[G / 4]) {
    constexpr int NVEC = G / 8;
    const bool whole = base + G <= numel;
#pragma unroll
    for (int k = 0; k < NVEC; ++k) {
        const int64_t i = base + k * 8 + 2 * j;
        if (whole && pair_aligned) {
            *reinterpret_cast<uint16_t*>(q + i) = uint16_t(c[2 * k]) | (uint16_t(c[2 * k + 1]) << 8);
        } else {
            if (i < numel) q[i] = c[2 * k];
            if (i + 1 < numel) q[i + 1] = c[2 * k + 1];
        }
    }
}

// ------------------------------------------------------------------ quality mode

// min(a^2, b^2, c^2) as the square of the smallest magnitude: rounding a square is monotone in the magnitude, so the
// result is the same number with one multiplication instead of three (the arguments are finite here).
__device__ __forceinline__ float min_square(float a, float b, float c) {
    const float m = fminf(fminf(fabsf(a), fabsf(b)), fabsf(c));
    return __fmul_rn(m, m);
}

// What the three code trials of the quality mode need from a candidate.  The decoded value of code c (before its bf16
// rounding) is (c - zp) * s with c - zp an integer of at most 9 bits and s a bf16 value (8 bits): exact in fp32, and so are
// its neighbours' as that value -+ s.  s > 0, so clamping the CODE to [0, 255] and clamping the VALUE to
// [(0 - zp) s, (255 - zp) s] select the same number: t = (r - zp) s, then clamp(t), clamp(t - s), clamp(t + s) replace three
// clamps, two additions, three subtractions and three products by one of each of the latter two, two additions and
// three clamps.  (|r| stays below 600 for the candidates of the search, so t is exact; were it not, it would lie outside
// the range on the side it belongs to and clamp to the same bound.)
struct QualityCand {
    float s, zp, lo, hi;
    __device__ __forceinline__ float clampv(float v) const { return fminf(fmaxf(v, lo), hi); }
    __device__ __forceinline__ void trials(float r, float& v0, float& vm, float& vp) const {
        const float t = __fmul_rn(__fsub_rn(r, zp), s);
        v0 = clampv(t);
        vm = clampv(__fsub_rn(t, s));
        vp = clampv(__fadd_rn(t, s));
    }
};

__device__ __forceinline__ QualityCand make_quality_cand(float s, float zp) {
    QualityCand c;
    c.s = s;
    c.zp = zp;
    c.lo = __fmul_rn(__fsub_rn(0.0f, zp), s);
    c.hi = __fmul_rn(__fsub_rn(255.0f, zp), s);
    return c;
}

// The smallest decoded squared error over the codes r - 1, r, r + 1 (each clamped): what the candidate search of the
// quality mode scores.  The values are finite here (NaN / Inf were cleaned), so a plain minimum equals the reference's
// NaN-propagating one.
__device__ __forceinline__ float quality_error(float x, const QualityCand& cand, float r) {
    float v0, vm, vp;
    cand.trials(r, v0, vm, vp);
    return min_square(__fsub_rn(x, round_bf16(v0)), __fsub_rn(x, round_bf16(vm)), __fsub_rn(x, round_bf16(vp)));
}

// quality_error for two values at once: the six bf16 roundings become three packed conversions (the capture of
// the one-value form showed the conversion pipe, not the issue slots, closest to its limit).
__device__ __forceinline__ void round_bf16_pair(float a, float b, float& ra, float& rb) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);  // .x = a (low half)
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&p);
    ra = __uint_as_float(w << 16);
    rb = __uint_as_float(w & 0xffff0000u);
}
__device__ __forceinline__ void quality_error2(float x0, float x1, const QualityCand& cand, float r0, float r1, float& e0, float& e1) {
    float a0, a1, b0, b1, c0, c1, v0, vm0, vp0, v1, vm1, vp1;
    cand.trials(r0, v0, vm0, vp0);
    cand.trials(r1, v1, vm1, vp1);
    round_bf16_pair(v0, v1, a0, a1);
    round_bf16_pair(vm0, vm1, b0, b1);
    round_bf16_pair(vp0, vp1, c0, c1);
    const float da0 = __fsub_rn(x0, a0), db0 = __fsub_rn(x0, b0), dc0 = __fsub_rn(x0, c0);
    const float da1 = __fsub_rn(x1, a1), db1 = __fsub_rn(x1, b1), dc1 = __fsub_rn(x1, c1);
    e0 = min_square(da0, db0, dc0);
    e1 = min_square(da1, db1, dc1);
}

// code choice of the reference's _amo_quality_codes for one value whose rounded index r = rint(x / s + zp)
// is already known: r, r - 1 and r + 1 are tried in that order and the first smallest decoded error wins
__device__ __forceinline__ float quality_code(float x, float s, float zp, float r, float& err_out) {
    float qv = clamp255(r);
    float d = __fsub_rn(x, round_bf16(__fmul_rn(__fsub_rn(qv, zp), s)));
    float err = __fmul_rn(d, d);
    {
        const float aq = clamp255(__fadd_rn(r, -1.0f));
        const float ad = __fsub_rn(x, round_bf16(__fmul_rn(__fsub_rn(aq, zp), s)));
        const float ae = __fmul_rn(ad, ad);
        if (ae < err) {
            qv = aq;
            err = ae;
        }
    }
    {
        const float aq = clamp255(__fadd_rn(r, 1.0f));
        const float ad = __fsub_rn(x, round_bf16(__fmul_rn(__fsub_rn(aq, zp), s)));
        const float ae = __fmul_rn(ad, ad);
        if (ae < err) {
            qv = aq;
            err = ae;
        }
    }
    err_out = err;
    return qv;
}

template <int G, typename T>
__global__ void __launch_bounds__(kThreads)
compress_quality_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, uint8_t* __restrict__ q,
                        uint16_t* __restrict__ scales, uint8_t* __restrict__ zps, bool in_aligned, bool out_aligned) {
    constexpr int VPL = G / 4;
    constexpr uint32_t kAllFinite = VPL >= 32 ? 0xffffffffu : (1u << (VPL & 31)) - 1u;
    const int lane = threadIdx.x & 31;
    const int j = lane & 3;
    const uint32_t qmask = 0xFu << (lane & ~3);
    const int64_t quads_per_grid = int64_t(gridDim.x) * (kThreads / 4);

    for (int64_t g = int64_t(blockIdx.x) * (kThreads / 4) + (threadIdx.x >> 2); g < ngroups; g += quads_per_grid) {
        const int64_t base = g * G;
        float v[VPL];
        uint32_t finmask;
        load_lane<G, T>(x, numel, base, j, in_aligned, v, finmask);

        float lmin = v[0], lmax = v[0];
#pragma unroll
        for (int k = 1; k < VPL; ++k) {
            lmin = fminf(lmin, v[k]);
            lmax = fmaxf(lmax, v[k]);
        }
        const float lower = fminf(quad_min(lmin, qmask), 0.0f);
        const float upper = fmaxf(quad_max(lmax, qmask), 0.0f);
        const float scale0 = fmaxf(__fsub_rn(__fdiv_rn(upper, 255.0f), __fdiv_rn(lower, 255.0f)), float(1e-8 / 255.0));
        const int lo_bits = int(__bfloat16_as_short(__float2bfloat16_rn(__fmul_rn(scale0, 0.85f))));
        const int hi_bits = int(__bfloat16_as_short(__float2bfloat16_rn(__fmul_rn(scale0, 1.10f))));
        const float nlower = -lower;

        // Candidates are the bf16 bit patterns lo_bits .. hi_bits.  The reference
        // enumerates 64 offsets clamped to hi_bits; repeats of hi_bits can never
        // win under the strict comparison, so the loop stops after the first.
        float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
        for (int k = 0; k < 64; ++k) {
            const int bits = lo_bits + k;
            if (k > 0 && bits > hi_bits) break;
            const int use = bits < hi_bits ? bits : hi_bits;
            const float s = __uint_as_float(uint32_t(use & 0xffff) << 16);
            const float zp = clamp255(rintf(__fdiv_rn(nlower, s)));
            const float rcp = __frcp_rn(s);
            const QualityCand cand = make_quality_cand(s, zp);
            // rounded index from the exact quotient (the scale is a bf16 value), then the three-way code choice
            float e[VPL];
#pragma unroll
            for (int i = 0; i < VPL; i += 2)
                quality_error2(v[i], v[i + 1], cand, rintf(__fadd_rn(exact_quotient(v[i], s, rcp), zp)),
                               rintf(__fadd_rn(exact_quotient(v[i + 1], s, rcp), zp)), e[i], e[i + 1]);
            if (finmask != kAllFinite) {  // rare: positions that held NaN / Inf do not count
#pragma unroll
                for (int i = 0; i < VPL; ++i)
                    if (!((finmask >> i) & 1u)) e[i] = 0.0f;
            }
            const float tot = quad_sum<G>(e, j, lane, qmask);
            if (k == 0 || tot < best_err) {
                best_err = tot;
                best_s = s;
                best_zp = zp;
            }
        }

        uint8_t codes[VPL];
        const uint8_t zp8 = uint8_t(best_zp);
        const float best_rcp = __frcp_rn(best_s);
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            float err;
            const float qf = quality_code(v[i], best_s, best_zp, rintf(__fadd_rn(exact_quotient(v[i], best_s, best_rcp), best_zp)), err);
            codes[i] = ((finmask >> i) & 1u) ? uint8_t(qf) : zp8;
        }
        store_codes<G>(q, numel, base, j, out_aligned, codes);
        if (j == 0) {
            scales[g] = uint16_t(__float_as_uint(best_s) >> 16);
            zps[g] = zp8;
        }
    }
}

// ------------------------------------------------- one lane per group (G <= 32)
//
// For group sizes up to 32 a whole group fits in one thread's registers.  Then nothing is exchanged
// between lanes: no shuffles, the per-candidate set-up (scale, zero point, reciprocal) is paid once
// per G values instead of once per G / 4, and the error sum follows the reference's order with plain
// additions (for G <= 32 every one of ATen's eight lanes adds its values in index order, and the lane
// totals are added left to right).  x / s is the exact IEEE quotient from the candidate's reciprocal
// and two FMAs (exact_quotient); the two cases that construction excludes -- a significand of all
// ones, and quotients so large that the intermediate product could overflow -- take the division.

template <int G>
struct GroupMask {
    using type = uint64_t;  // one bit per value of the group
    static constexpr type kAll = G >= 64 ? ~uint64_t(0) : (uint64_t(1) << (G & 63)) - 1;
};

template <int G, typename T>
__device__ __forceinline__ void load_group(const T* __restrict__ x, int64_t numel, int64_t base, bool aligned16, float (&v)[G],
                                           uint64_t& finmask) {
    constexpr int PER16 = 16 / int(sizeof(T));  // values per 16-byte load
    if (base + G <= numel && aligned16) {
        const uint4* p = reinterpret_cast<const uint4*>(x + base);
#pragma unroll
        for (int k = 0; k < G / PER16; ++k) {
            const uint4 w = __ldg(p + k);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (sizeof(T) == 4) {
                    v[k * 4 + i] = __uint_as_float(ww[i]);
                } else {
                    uint16_t lo = uint16_t(ww[i] & 0xffffu), hi = uint16_t(ww[i] >> 16);
                    v[k * 8 + 2 * i] = widen<T>(*reinterpret_cast<T*>(&lo));
                    v[k * 8 + 2 * i + 1] = widen<T>(*reinterpret_cast<T*>(&hi));
                }
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < G; ++k) v[k] = base + k < numel ? widen<T>(x[base + k]) : 0.0f;
    }
    finmask = 0;
#pragma unroll
    for (int k = 0; k < G; ++k) {
        const bool f = finite_f32(v[k]);
        if (!f) v[k] = 0.0f;
        finmask |= uint64_t(f ? 1 : 0) << k;
    }
}

template <int G>
__device__ __forceinline__ void store_group(uint8_t* __restrict__ q, int64_t numel, int64_t base, bool aligned8, const uint32_t (&cw)[G / 4]) {
    if (base + G <= numel && aligned8) {
#pragma unroll
        for (int k = 0; k < G / 8; ++k) *reinterpret_cast<uint2*>(q + base + 8 * k) = make_uint2(cw[2 * k], cw[2 * k + 1]);
    } else {
#pragma unroll
        for (int k = 0; k < G; ++k)
            if (base + k < numel) q[base + k] = uint8_t(cw[k >> 2] >> (8 * (k & 3)));
    }
}

// The reference's running sums for the error terms of one group, fed in index order.  ATen keeps eight lanes
// (value k belongs to lane k % 8); within a lane complete runs of four 8-wide vectors go to four accumulators
// (vector v to accumulator v % 4), left-over vectors to accumulator 0, the accumulators are combined
// ((a0 + a1) + a2) + a3 and the lane totals added left to right.  For G <= 32 that is one accumulator per lane
// in index order; G = 64 needs all four.
template <int G>
struct LaneSums {
    static constexpr int NVEC = G / 8, FULL = (NVEC / 4) * 4, NACC = (FULL > 4 || (FULL == 4 && NVEC > 4)) ? 4 : 1;
    float acc[NACC][8];
    __device__ __forceinline__ void add(int k, float e) {
        const int vI = k >> 3, l = k & 7;
        if (NACC == 1) {
            acc[0][l] = vI == 0 ? e : __fadd_rn(acc[0][l], e);
        } else {
            const int t = vI < FULL ? (vI & 3) : 0;
            const bool first = vI < 4;
            acc[t][l] = first ? e : __fadd_rn(acc[t][l], e);
        }
    }
    __device__ __forceinline__ float total() const {
        float t = 0.0f;
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            const float lt = NACC == 1 ? acc[0][l] : __fadd_rn(__fadd_rn(__fadd_rn(acc[0][l], acc[1][l]), acc[2][l]), acc[3][l]);
            t = l == 0 ? lt : __fadd_rn(t, lt);
        }
        return t;
    }
};

template <int G, typename T>
__global__ void __launch_bounds__(kThreads)
compress_legacy_lane_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, CandTable tab, uint8_t* __restrict__ q,
                            uint16_t* __restrict__ scales, uint8_t* __restrict__ zps, bool in_aligned16, bool out_aligned8) {
    static_assert(G == 8 || G == 16 || G == 24 || G == 32 || G == 48 || G == 64, "group sizes with a one-group-per-lane kernel");
    constexpr uint64_t kAllFinite = GroupMask<G>::kAll;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < ngroups; g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t base = g * G;
        float v[G];
        uint64_t finmask;
        load_group<G, T>(x, numel, base, in_aligned16, v, finmask);
        float bmin = v[0], bmax = v[0];
#pragma unroll
        for (int k = 1; k < G; ++k) {
            bmin = fminf(bmin, v[k]);
            bmax = fmaxf(bmax, v[k]);
        }
        float rng = fmaxf(__fsub_rn(bmax, bmin), 1e-8f);
        if (!finite_f32(rng)) rng = 1e-8f;
        float s0 = __fdiv_rn(rng, 255.0f);
        if (!finite_f32(s0)) s0 = float(1e-8 / 255.0);
        const float nbmin = -bmin;
        const float amax = fmaxf(fabsf(bmin), fabsf(bmax));

        float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
        for (int c = 0; c < tab.n; ++c) {
            const float s = __fmul_rn(s0, tab.m[c]);
            const float zp = clamp255(rintf(__fdiv_rn(nbmin, s)));
            const float rcp = __frcp_rn(s);
            LaneSums<G> sums;
            const bool plain = (__float_as_uint(s) & 0x7fffffu) != 0x7fffffu && __fmul_rn(amax, rcp) < 1048576.0f &&
                               finmask == kAllFinite;
            if (plain) {
#pragma unroll
                for (int k = 0; k < G; ++k) {
                    const float qc = clamp255(rintf(__fadd_rn(exact_quotient(v[k], s, rcp), zp)));
                    const float d = __fsub_rn(v[k], __fmul_rn(__fsub_rn(qc, zp), s));
                    sums.add(k, __fmul_rn(d, d));
                }
            } else {  // rare: divide, and leave out the positions that held NaN / Inf
#pragma unroll
                for (int k = 0; k < G; ++k) {
                    const float qc = clamp255(rintf(__fadd_rn(__fdiv_rn(v[k], s), zp)));
                    const float d = __fsub_rn(v[k], __fmul_rn(__fsub_rn(qc, zp), s));
                    sums.add(k, ((finmask >> k) & 1u) ? __fmul_rn(d, d) : 0.0f);
                }
            }
            const float err = sums.total();
            if (c == 0 || err < best_err) {
                best_err = err;
                best_s = s;
                best_zp = zp;
            }
        }

        uint32_t cw[G / 4];
        const uint32_t zp8 = uint32_t(best_zp);
#pragma unroll
        for (int k = 0; k < G / 4; ++k) cw[k] = 0;
#pragma unroll
        for (int k = 0; k < G; ++k) {
            const float qf = clamp255(rintf(__fadd_rn(__fdiv_rn(v[k], best_s), best_zp)));
            const uint32_t code = ((finmask >> k) & 1u) ? uint32_t(qf) : zp8;
            cw[k >> 2] |= code << (8 * (k & 3));
        }
        store_group<G>(q, numel, base, out_aligned8, cw);
        scales[g] = __bfloat16_as_ushort(__float2bfloat16_rn(best_s));
        zps[g] = uint8_t(zp8);
    }
}

// ------------------------------------------------- two lanes per group (G = 128, legacy presets)
//
// 128 values do not fit one thread, but 64 do: lane j (0 / 1) of a pair owns columns 4 j .. 4 j + 3 of every 8-wide
// vector of the group.  Every running sum of the reference (accumulator v % 4 of column l, see LaneSums) then lives in
// one lane, the column totals are chained left to right through ONE shuffle (lane 0's partial total is lane 1's
// starting value), and a second shuffle hands the group's total back.  Everything else is the one-lane kernel: the
// exact two-FMA quotient, the same rare fall-backs, 64 values in registers.
constexpr int kPairG = 128;   // group size of the two-lanes-per-group kernels

// The 64 values of lane j of a pair: element 8 v + 4 j + i of group g is v[4 v + i].  Non-finite values become 0 and
// clear their bit in `finmask`.
template <typename T>
__device__ __forceinline__ void pair_load(const T* __restrict__ x, int64_t numel, int64_t g, int j, bool aligned, float (&v)[64],
                                          uint64_t& finmask) {
    const int64_t base = g * kPairG + 4 * j;
    if (g * kPairG + kPairG <= numel && aligned) {
#pragma unroll
        for (int vI = 0; vI < kPairG / 8; ++vI) {
            if (sizeof(T) == 4) {
                const uint4 w = __ldg(reinterpret_cast<const uint4*>(x + base + 8 * vI));
                v[4 * vI] = __uint_as_float(w.x), v[4 * vI + 1] = __uint_as_float(w.y);
                v[4 * vI + 2] = __uint_as_float(w.z), v[4 * vI + 3] = __uint_as_float(w.w);
            } else {
                const uint2 w = __ldg(reinterpret_cast<const uint2*>(x + base + 8 * vI));
                uint16_t h0 = uint16_t(w.x), h1 = uint16_t(w.x >> 16), h2 = uint16_t(w.y), h3 = uint16_t(w.y >> 16);
                v[4 * vI] = widen<T>(*reinterpret_cast<T*>(&h0)), v[4 * vI + 1] = widen<T>(*reinterpret_cast<T*>(&h1));
                v[4 * vI + 2] = widen<T>(*reinterpret_cast<T*>(&h2)), v[4 * vI + 3] = widen<T>(*reinterpret_cast<T*>(&h3));
            }
        }
    } else {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
            const int64_t at = base + 8 * (k >> 2) + (k & 3);
            v[k] = at < numel ? widen<T>(x[at]) : 0.0f;
        }
    }
    finmask = 0;
#pragma unroll
    for (int k = 0; k < 64; ++k) {
        const bool f = finite_f32(v[k]);
        if (!f) v[k] = 0.0f;
        finmask |= uint64_t(f ? 1 : 0) << k;
    }
}

// The reference's running sums for the four columns this lane owns (LaneSums for G = 128, split by column), and the
// group's total: columns 0..3 (lane 0) then 4..7 (lane 1), left to right, with lane 0's partial total as lane 1's
// starting value.  Both lanes of the pair return the same number.
struct PairSums {
    float acc[4][4];                    // [accumulator v % 4][column of this lane]
    __device__ __forceinline__ void add(int k, float e) {
        const int vI = k >> 2, l = k & 3;
        acc[vI & 3][l] = vI < 4 ? e : __fadd_rn(acc[vI & 3][l], e);
    }
    __device__ __forceinline__ float total(uint32_t pmask, int lane) const {
        float lt[4];
#pragma unroll
        for (int l = 0; l < 4; ++l) lt[l] = __fadd_rn(__fadd_rn(__fadd_rn(acc[0][l], acc[1][l]), acc[2][l]), acc[3][l]);
        const float left = __fadd_rn(__fadd_rn(__fadd_rn(lt[0], lt[1]), lt[2]), lt[3]);
        const float carried = __shfl_sync(pmask, left, lane & ~1);
        const float right = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(carried, lt[0]), lt[1]), lt[2]), lt[3]);
        return __shfl_sync(pmask, right, lane | 1);
    }
};

// the four codes of vector vI that this lane owns
__device__ __forceinline__ void pair_store(uint8_t* __restrict__ q, int64_t numel, int64_t g, int j, int vI, bool whole, uint32_t cw) {
    const int64_t at = g * kPairG + 4 * j + 8 * vI;
    if (whole) {
        *reinterpret_cast<uint32_t*>(q + at) = cw;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (at + i < numel) q[at + i] = uint8_t(cw >> (8 * i));
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
compress_legacy_pair_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, CandTable tab, uint8_t* __restrict__ q,
                            uint16_t* __restrict__ scales, uint8_t* __restrict__ zps, bool in_aligned8, bool out_aligned4) {
    const int lane = threadIdx.x & 31, j = lane & 1;
    const uint32_t pmask = 3u << (lane & ~1);
    const int64_t pairs_per_grid = int64_t(gridDim.x) * (blockDim.x / 2);
    for (int64_t g = int64_t(blockIdx.x) * (blockDim.x / 2) + (threadIdx.x >> 1); g < ngroups; g += pairs_per_grid) {
        float v[64];
        uint64_t finmask;
        pair_load<T>(x, numel, g, j, in_aligned8, v, finmask);
        float bmin = v[0], bmax = v[0];
#pragma unroll
        for (int k = 1; k < 64; ++k) {
            bmin = fminf(bmin, v[k]);
            bmax = fmaxf(bmax, v[k]);
        }
        bmin = fminf(bmin, __shfl_xor_sync(pmask, bmin, 1));
        bmax = fmaxf(bmax, __shfl_xor_sync(pmask, bmax, 1));
        const bool all_finite = __all_sync(pmask, finmask == ~uint64_t(0));
        float rng = fmaxf(__fsub_rn(bmax, bmin), 1e-8f);
        if (!finite_f32(rng)) rng = 1e-8f;
        float s0 = __fdiv_rn(rng, 255.0f);
        if (!finite_f32(s0)) s0 = float(1e-8 / 255.0);
        const float nbmin = -bmin;
        const float amax = fmaxf(fabsf(bmin), fabsf(bmax));

        float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
        for (int c = 0; c < tab.n; ++c) {
            const float s = __fmul_rn(s0, tab.m[c]);
            const float zp = clamp255(rintf(__fdiv_rn(nbmin, s)));
            const float rcp = __frcp_rn(s);
            PairSums sums;
            const bool plain = (__float_as_uint(s) & 0x7fffffu) != 0x7fffffu && __fmul_rn(amax, rcp) < 1048576.0f && all_finite;
            if (plain) {
#pragma unroll
                for (int k = 0; k < 64; ++k) {
                    const float qc = clamp255(rintf(__fadd_rn(exact_quotient(v[k], s, rcp), zp)));
                    const float d = __fsub_rn(v[k], __fmul_rn(__fsub_rn(qc, zp), s));
                    sums.add(k, __fmul_rn(d, d));
                }
            } else {  // rare: divide, and leave out the positions that held NaN / Inf
#pragma unroll
                for (int k = 0; k < 64; ++k) {
                    const float qc = clamp255(rintf(__fadd_rn(__fdiv_rn(v[k], s), zp)));
                    const float d = __fsub_rn(v[k], __fmul_rn(__fsub_rn(qc, zp), s));
                    sums.add(k, ((finmask >> k) & 1u) ? __fmul_rn(d, d) : 0.0f);
                }
            }
            const float err = sums.total(pmask, lane);
            if (c == 0 || err < best_err) {
                best_err = err;
                best_s = s;
                best_zp = zp;
            }
        }

        const uint32_t zp8 = uint32_t(best_zp);
        const bool whole = g * kPairG + kPairG <= numel && out_aligned4;
#pragma unroll
        for (int vI = 0; vI < kPairG / 8; ++vI) {
            uint32_t cw = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = 4 * vI + i;
                const float qf = clamp255(rintf(__fadd_rn(__fdiv_rn(v[k], best_s), best_zp)));
                const uint32_t code = ((finmask >> k) & 1u) ? uint32_t(qf) : zp8;
                cw |= code << (8 * i);
            }
            pair_store(q, numel, g, j, vI, whole, cw);
        }
        if (j == 0) {
            scales[g] = __bfloat16_as_ushort(__float2bfloat16_rn(best_s));
            zps[g] = uint8_t(zp8);
        }
    }
}

template <int G, typename T>
__global__ void __launch_bounds__(kThreads)
compress_quality_lane_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, uint8_t* __restrict__ q,
                             uint16_t* __restrict__ scales, uint8_t* __restrict__ zps, bool in_aligned16, bool out_aligned8) {
    static_assert(G == 8 || G == 16 || G == 24 || G == 32 || G == 48 || G == 64, "group sizes with a one-group-per-lane kernel");
    constexpr uint64_t kAllFinite = GroupMask<G>::kAll;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < ngroups; g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t base = g * G;
        float v[G];
        uint64_t finmask;
        load_group<G, T>(x, numel, base, in_aligned16, v, finmask);
        float lower = v[0], upper = v[0];
#pragma unroll
        for (int k = 1; k < G; ++k) {
            lower = fminf(lower, v[k]);
            upper = fmaxf(upper, v[k]);
        }
        lower = fminf(lower, 0.0f);
        upper = fmaxf(upper, 0.0f);
        const float scale0 = fmaxf(__fsub_rn(__fdiv_rn(upper, 255.0f), __fdiv_rn(lower, 255.0f)), float(1e-8 / 255.0));
        const int lo_bits = int(__bfloat16_as_short(__float2bfloat16_rn(__fmul_rn(scale0, 0.85f))));
        const int hi_bits = int(__bfloat16_as_short(__float2bfloat16_rn(__fmul_rn(scale0, 1.10f))));
        const float nlower = -lower;

        // The range contains zero, so |x| <= upper - lower and |x / s| < 255 / 0.85 + 1 for every candidate: the exact
        // quotient's intermediate product cannot overflow, and a bf16 scale never has a significand of all ones.
        float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
        for (int c = 0; c < 64; ++c) {
            const int bits = lo_bits + c;
            if (c > 0 && bits > hi_bits) break;
            const int use = bits < hi_bits ? bits : hi_bits;
            const float s = __uint_as_float(uint32_t(use & 0xffff) << 16);
            const float zp = clamp255(rintf(__fdiv_rn(nlower, s)));
            const float rcp = __frcp_rn(s);
            const QualityCand cand = make_quality_cand(s, zp);
            LaneSums<G> sums;
            if (finmask == kAllFinite) {
#pragma unroll
                for (int k = 0; k < G; k += 2) {
                    float e0, e1;
                    quality_error2(v[k], v[k + 1], cand, rintf(__fadd_rn(exact_quotient(v[k], s, rcp), zp)),
                                   rintf(__fadd_rn(exact_quotient(v[k + 1], s, rcp), zp)), e0, e1);
                    sums.add(k, e0);
                    sums.add(k + 1, e1);
                }
            } else {
#pragma unroll
                for (int k = 0; k < G; ++k) {
                    const float e = quality_error(v[k], cand, rintf(__fadd_rn(exact_quotient(v[k], s, rcp), zp)));
                    sums.add(k, ((finmask >> k) & 1u) ? e : 0.0f);
                }
            }
            const float tot = sums.total();
            if (c == 0 || tot < best_err) {
                best_err = tot;
                best_s = s;
                best_zp = zp;
            }
        }

        uint32_t cw[G / 4];
        const uint32_t zp8 = uint32_t(best_zp);
        const float best_rcp = __frcp_rn(best_s);
#pragma unroll
        for (int k = 0; k < G / 4; ++k) cw[k] = 0;
#pragma unroll
        for (int k = 0; k < G; ++k) {
            float e;
            const float qf = quality_code(v[k], best_s, best_zp, rintf(__fadd_rn(exact_quotient(v[k], best_s, best_rcp), best_zp)), e);
            const uint32_t code = ((finmask >> k) & 1u) ? uint32_t(qf) : zp8;
            cw[k >> 2] |= code << (8 * (k & 3));
        }
        store_group<G>(q, numel, base, out_aligned8, cw);
        scales[g] = uint16_t(__float_as_uint(best_s) >> 16);
        zps[g] = uint8_t(zp8);
    }
}

// ------------------------------------------------------------ symmetric codec

__device__ __forceinline__ float clamp_i8(float v) { return fminf(fmaxf(v, -128.0f), 127.0f); }


// The adaptive search of the symmetric codec with one group per lane (G <= 32), like the AMO-BQ lane kernels.
// |x| <= max|x| and every candidate scale is at least 0.9 max|x| / 127, so the quotients stay below 142.
// src/tensorcache/codec.py:530-565 (tab.n == 0: scale = bf16(max|x| / 127)) and :568-620 (tab.n > 0: the
// "adaptive" search over s0 * multiplier, scored on the raw values so that a NaN / Inf in the group
// makes every score NaN / Inf and candidate 0 wins, then the winner rounded to bf16).  Signed codes.
template <int G, typename T>
__global__ void __launch_bounds__(kThreads)
compress_sym_lane_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, CandTable tab, uint8_t* __restrict__ q,
                         uint16_t* __restrict__ scales, bool in_aligned16, bool out_aligned8) {
    static_assert(G == 8 || G == 16 || G == 24 || G == 32 || G == 48 || G == 64, "group sizes with a one-group-per-lane kernel");
    constexpr uint64_t kAllFinite = GroupMask<G>::kAll;
    for (int64_t g = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < ngroups; g += int64_t(gridDim.x) * blockDim.x) {
        const int64_t base = g * G;
        float v[G];
        uint64_t finmask;
        load_group<G, T>(x, numel, base, in_aligned16, v, finmask);
        float amax = fabsf(v[0]);
#pragma unroll
        for (int k = 1; k < G; ++k) amax = fmaxf(amax, fabsf(v[k]));
        const float s0 = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        float best_s = s0;
        if (tab.n > 0) {
            best_s = __fmul_rn(s0, tab.m[0]);  // a group that held NaN / Inf scores NaN / Inf everywhere: candidate 0
            if (finmask == kAllFinite) {
                float best_err = 0.0f;
                for (int c = 0; c < tab.n; ++c) {
                    const float s = __fmul_rn(s0, tab.m[c]);
                    const float rcp = __frcp_rn(s);
                    const bool plain = (__float_as_uint(s) & 0x7fffffu) != 0x7fffffu;
                    LaneSums<G> sums;
                    if (plain) {
#pragma unroll
                        for (int k = 0; k < G; ++k) {
                            const float d = __fsub_rn(v[k], __fmul_rn(clamp_i8(rintf(exact_quotient(v[k], s, rcp))), s));
                            sums.add(k, __fmul_rn(d, d));
                        }
                    } else {  // rare: a scale whose significand is all ones takes the division
#pragma unroll
                        for (int k = 0; k < G; ++k) {
                            const float d = __fsub_rn(v[k], __fmul_rn(clamp_i8(rintf(__fdiv_rn(v[k], s))), s));
                            sums.add(k, __fmul_rn(d, d));
                        }
                    }
                    const float err = sums.total();
                    if (c == 0 || err < best_err) {
                        best_err = err;
                        best_s = s;
                    }
                }
            }
        }
        const uint16_t sbits = __bfloat16_as_ushort(__float2bfloat16_rn(best_s));
        const float sf = __uint_as_float(uint32_t(sbits) << 16);
        uint32_t cw[G / 4];
#pragma unroll
        for (int k = 0; k < G / 4; ++k) cw[k] = 0;
#pragma unroll
        for (int k = 0; k < G; ++k) {
            const float qf = clamp_i8(rintf(__fdiv_rn(v[k], sf)));
            const uint32_t code = ((finmask >> k) & 1u) ? (uint32_t(int(qf)) & 0xffu) : 0u;
            cw[k >> 2] |= code << (8 * (k & 3));
        }
        store_group<G>(q, numel, base, out_aligned8, cw);
        scales[g] = sbits;
    }
}

// The same search with two lanes per group (G = 128): the layout of compress_legacy_pair_kernel, the arithmetic of
// compress_sym_lane_kernel.
template <typename T>
__global__ void __launch_bounds__(kThreads)
compress_sym_pair_kernel(const T* __restrict__ x, int64_t numel, int64_t ngroups, CandTable tab, uint8_t* __restrict__ q,
                         uint16_t* __restrict__ scales, bool in_aligned8, bool out_aligned4) {
    const int lane = threadIdx.x & 31, j = lane & 1;
    const uint32_t pmask = 3u << (lane & ~1);
    const int64_t pairs_per_grid = int64_t(gridDim.x) * (blockDim.x / 2);
    for (int64_t g = int64_t(blockIdx.x) * (blockDim.x / 2) + (threadIdx.x >> 1); g < ngroups; g += pairs_per_grid) {
        float v[64];
        uint64_t finmask;
        pair_load<T>(x, numel, g, j, in_aligned8, v, finmask);
        float amax = fabsf(v[0]);
#pragma unroll
        for (int k = 1; k < 64; ++k) amax = fmaxf(amax, fabsf(v[k]));
        amax = fmaxf(amax, __shfl_xor_sync(pmask, amax, 1));
        const bool all_finite = __all_sync(pmask, finmask == ~uint64_t(0));
        const float s0 = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        float best_s = s0;
        if (tab.n > 0) {
            best_s = __fmul_rn(s0, tab.m[0]);  // a group that held NaN / Inf scores NaN / Inf everywhere: candidate 0
            if (all_finite) {
                float best_err = 0.0f;
                for (int c = 0; c < tab.n; ++c) {
                    const float s = __fmul_rn(s0, tab.m[c]);
                    const float rcp = __frcp_rn(s);
                    const bool plain = (__float_as_uint(s) & 0x7fffffu) != 0x7fffffu;
                    PairSums sums;
                    if (plain) {
#pragma unroll
                        for (int k = 0; k < 64; ++k) {
                            const float d = __fsub_rn(v[k], __fmul_rn(clamp_i8(rintf(exact_quotient(v[k], s, rcp))), s));
                            sums.add(k, __fmul_rn(d, d));
                        }
                    } else {  // rare: a scale whose significand is all ones takes the division
#pragma unroll
                        for (int k = 0; k < 64; ++k) {
                            const float d = __fsub_rn(v[k], __fmul_rn(clamp_i8(rintf(__fdiv_rn(v[k], s))), s));
                            sums.add(k, __fmul_rn(d, d));
                        }
                    }
                    const float err = sums.total(pmask, lane);
                    if (c == 0 || err < best_err) {
                        best_err = err;
                        best_s = s;
                    }
                }
            }
        }
        const uint16_t sbits = __bfloat16_as_ushort(__float2bfloat16_rn(best_s));
        const float sf = __uint_as_float(uint32_t(sbits) << 16);
        const bool whole = g * kPairG + kPairG <= numel && out_aligned4;
#pragma unroll
        for (int vI = 0; vI < kPairG / 8; ++vI) {
            uint32_t cw = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = 4 * vI + i;
                const float qf = clamp_i8(rintf(__fdiv_rn(v[k], sf)));
                const uint32_t code = ((finmask >> k) & 1u) ? (uint32_t(int(qf)) & 0xffu) : 0u;
                cw |= code << (8 * i);
            }
            pair_store(q, numel, g, j, vI, whole, cw);
        }
        if (j == 0) scales[g] = sbits;
    }
}

// Plain symmetric codec (no scale search) as a streaming kernel.  One pass over the data, so it is
// bound by HBM (2 bytes read, 1 + 2/G written per bf16 value), not by arithmetic, and is laid out
// like the decoder: every thread owns 16 consecutive values (one 256-bit load for 16-bit inputs, two
// for fp32), G/16 neighbouring lanes form a group and combine their max|x| with xor-shuffles, and
// each thread writes its 16 codes with one 128-bit store.  x / scale is the exact IEEE quotient, built
// from the group's reciprocal and two FMAs per value (no division, no fallback path: with bf16 inputs
// and a bf16 scale the quotient lands exactly on k + 0.5 for a large share of the values, so a
// "rare boundary case" design does not work here); rounding to nearest-even and the conversion to
// int8 come from adding 1.5 * 2^23, whose low mantissa byte is the two's-complement code.
// Covers G in {16, 32, 64, 128}, whole groups, x 32-byte and q 16-byte aligned; everything else
// (other G, ragged tail, odd alignment, the adaptive search) runs on compress_sym_kernel.
constexpr int kSymUnroll = 2;

// Sixteen consecutive values in the registers they were loaded into (8 words for the 16-bit types,
// 16 for fp32); they are widened to fp32 where they are used, twice, which is cheaper than holding
// 16 floats per unit in flight: fewer registers, more resident warps, more loads in flight.
template <typename T>
struct Raw16;

__device__ __forceinline__ void ldg_stream_v8(const void* p, uint32_t* w) {
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}

template <>
struct Raw16<__nv_bfloat16> {
    static constexpr int kWords = 8;
    uint32_t w[kWords];
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { ldg_stream_v8(p, w); }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int k = 0; k < kWords; ++k) w[k] = 0;
    }
    // max |x| over the 16 values, computed on the packed pairs; NaN if any value is NaN, Inf if any is Inf
    __device__ __forceinline__ float amax_or_nonfinite() const {
        __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[0]));
#pragma unroll
        for (int k = 1; k < kWords; ++k) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[k])));
        return __bfloat162float(__hmax_nan(__low2bfloat16(m), __high2bfloat16(m)));
    }
    __device__ __forceinline__ void clean() {  // NaN / Inf -> 0
#pragma unroll
        for (int k = 0; k < kWords; ++k) {
            if ((w[k] & 0x7f80u) == 0x7f80u) w[k] &= 0xffff0000u;
            if ((w[k] & 0x7f800000u) == 0x7f800000u) w[k] &= 0x0000ffffu;
        }
    }
    __device__ __forceinline__ float get(int i) const {
        return __uint_as_float((i & 1) ? (w[i >> 1] & 0xffff0000u) : (w[i >> 1] << 16));
    }
};

template <>
struct Raw16<__half> {
    static constexpr int kWords = 8;
    uint32_t w[kWords];
    __device__ __forceinline__ void load(const __half* p) { ldg_stream_v8(p, w); }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int k = 0; k < kWords; ++k) w[k] = 0;
    }
    __device__ __forceinline__ float amax_or_nonfinite() const {
        __half2 m = __habs2(*reinterpret_cast<const __half2*>(&w[0]));
#pragma unroll
        for (int k = 1; k < kWords; ++k) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __half2*>(&w[k])));
        return __half2float(__hmax_nan(__low2half(m), __high2half(m)));
    }
    __device__ __forceinline__ void clean() {
#pragma unroll
        for (int k = 0; k < kWords; ++k) {
            if ((w[k] & 0x7c00u) == 0x7c00u) w[k] &= 0xffff0000u;
            if ((w[k] & 0x7c000000u) == 0x7c000000u) w[k] &= 0x0000ffffu;
        }
    }
    __device__ __forceinline__ float get(int i) const {
        const __half2 h = *reinterpret_cast<const __half2*>(&w[i >> 1]);
        return (i & 1) ? __high2float(h) : __low2float(h);
    }
};

template <>
struct Raw16<float> {
    static constexpr int kWords = 16;
    uint32_t w[kWords];
    __device__ __forceinline__ void load(const float* p) {
        ldg_stream_v8(p, w);
        ldg_stream_v8(p + 8, w + 8);
    }
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int k = 0; k < kWords; ++k) w[k] = 0;
    }
    // non-negative floats order like their bit patterns, and NaN / Inf patterns sort above every finite one
    __device__ __forceinline__ float amax_or_nonfinite() const {
        uint32_t m = 0;
#pragma unroll
        for (int k = 0; k < kWords; ++k) m = max(m, w[k] & 0x7fffffffu);
        return __uint_as_float(m);
    }
    __device__ __forceinline__ void clean() {
#pragma unroll
        for (int k = 0; k < kWords; ++k)
            if ((w[k] << 1) >= 0xff000000u) w[k] = 0;
    }
    __device__ __forceinline__ float get(int i) const { return __uint_as_float(w[i]); }
};

template <int LPG, typename T>  // LPG = lanes per group = G / 16
__global__ void __launch_bounds__(kThreads, 5)
compress_sym_stream_kernel(const T* __restrict__ x, int64_t units, uint8_t* __restrict__ q, uint16_t* __restrict__ scales) {
    // every block owns a contiguous range of 16-value units that starts and ends on a multiple of 8 units
    // (LPG divides 8), so no group is split between blocks or between warps
    const int64_t octs = units >> 3;
    const int64_t begin = (octs * blockIdx.x / gridDim.x) << 3;
    const int64_t end = blockIdx.x + 1 == gridDim.x ? units : (octs * (blockIdx.x + 1) / gridDim.x) << 3;
    const float magic = 12582912.0f;  // 1.5 * 2^23

    // the trip count is uniform across the block so that the shuffles always run with full warps
    for (int64_t u0 = begin; u0 < end; u0 += int64_t(kThreads) * kSymUnroll) {
        Raw16<T> raw[kSymUnroll];
        bool live[kSymUnroll];
#pragma unroll
        for (int k = 0; k < kSymUnroll; ++k) {
            const int64_t u = u0 + int64_t(k) * kThreads + threadIdx.x;
            live[k] = u < end;
            if (live[k]) raw[k].load(x + (u << 4));
            else raw[k].zero();
        }
#pragma unroll
        for (int k = 0; k < kSymUnroll; ++k) {
            const int64_t u = u0 + int64_t(k) * kThreads + threadIdx.x;
            float amax = raw[k].amax_or_nonfinite();
            if (!finite_f32(amax)) {  // rare: NaN / Inf count as 0 and get code 0
                raw[k].clean();
                amax = raw[k].amax_or_nonfinite();
            }
#pragma unroll
            for (int off = 1; off < LPG; off <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
            const float s0 = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
            const uint16_t sbits = __bfloat16_as_ushort(__float2bfloat16_rn(s0));
            const float sf = __uint_as_float(uint32_t(sbits) << 16);
            const float rcp = __frcp_rn(sf);
            // x / sf is the exact IEEE quotient (exact_quotient: sf has an 8-bit significand).
            // |x| <= amax and sf >= (amax / 127) (1 - 2^-9), so |x / sf| < 127.26: the reference's clamp to
            // [-128, 127] never binds and is left out.  Adding 1.5 * 2^23 rounds to nearest-even.
            uint32_t code[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                code[i] = __float_as_uint(__fadd_rn(exact_quotient(raw[k].get(i), sf, rcp), magic));
            if (live[k]) {
                uint4 o;
                o.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
                o.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
                o.z = __byte_perm(__byte_perm(code[8], code[9], 0x0040), __byte_perm(code[10], code[11], 0x0040), 0x5410);
                o.w = __byte_perm(__byte_perm(code[12], code[13], 0x0040), __byte_perm(code[14], code[15], 0x0040), 0x5410);
                __stcs(reinterpret_cast<uint4*>(q + (u << 4)), o);  // streamed once: evict-first
                if ((threadIdx.x & (LPG - 1)) == 0) scales[u / LPG] = sbits;
            }
        }
    }
}

template <int LPG, typename T>
cudaError_t launch_sym_stream(const void* x, int64_t groups, uint8_t* q, uint16_t* scales, cudaStream_t st) {
    static std::atomic<int> blocks_cache[64];   // zero-initialised; the look-up is idempotent
    int dev = 0;
    int resident = tcb::sm_count() * 4;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
        int have = blocks_cache[dev].load(std::memory_order_relaxed);
        if (have == 0) {
            int per_sm = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, compress_sym_stream_kernel<LPG, T>, kThreads, 0) != cudaSuccess ||
                per_sm < 1)
                per_sm = 4;
            have = per_sm * tcb::sm_count();
            blocks_cache[dev].store(have, std::memory_order_relaxed);
        }
        resident = have;
    }
    const int64_t units = groups * LPG;
    int64_t grid = resident;  // one wave; small inputs get fewer, fuller blocks
    if (grid * kThreads > units) grid = (units + kThreads - 1) / kThreads;
    if (grid < 1) grid = 1;
    compress_sym_stream_kernel<LPG, T><<<unsigned(grid), kThreads, 0, st>>>(static_cast<const T*>(x), units, q, scales);
    return cudaGetLastError();
}

template <int LPG>
cudaError_t launch_sym_stream_typed(const void* x, int dtype, int64_t groups, uint8_t* q, uint16_t* scales, cudaStream_t st) {
    switch (dtype) {
    case TCB_DT_BF16: return launch_sym_stream<LPG, __nv_bfloat16>(x, groups, q, scales, st);
    case TCB_DT_F16: return launch_sym_stream<LPG, __half>(x, groups, q, scales, st);
    default: return launch_sym_stream<LPG, float>(x, groups, q, scales, st);
    }
}

// -------------------------------------------------------------------- dispatch

enum class Coder { Legacy, Quality, Sym };

template <int G, typename T>
cudaError_t launch_typed(Coder coder, const void* x, int64_t numel, int64_t ngroups, const CandTable* tab, uint8_t* q,
                         uint16_t* s, uint8_t* zp, int grid, cudaStream_t st) {
    const T* xt = static_cast<const T*>(x);
    const bool in_aligned = (reinterpret_cast<uintptr_t>(x) % (2 * sizeof(T))) == 0;
    const bool out_aligned = (reinterpret_cast<uintptr_t>(q) & 1) == 0;
    // Kernels that hold 48 or more values per thread need about 180 registers: blocks of 64 threads let an SM hold ten
    // warps of them where one block of 256 would leave it with eight.
    constexpr int kLaneThreads = G >= 48 ? 64 : kThreads;
    auto blocks_for = [&](int groups_per_block) {
        const int64_t blocks = (ngroups + groups_per_block - 1) / groups_per_block;
        const int64_t cap = int64_t(grid) * (kThreads / kLaneThreads);
        return int(blocks < cap ? blocks : cap);
    };
    switch (coder) {
    case Coder::Legacy:
        if constexpr (G <= 64) {
            const bool in16 = reinterpret_cast<uintptr_t>(x) % 16 == 0 && (G * sizeof(T)) % 16 == 0;
            const bool out8 = reinterpret_cast<uintptr_t>(q) % 8 == 0;
            compress_legacy_lane_kernel<G, T><<<blocks_for(kLaneThreads), kLaneThreads, 0, st>>>(xt, numel, ngroups, *tab, q, s, zp, in16, out8);
        } else {
            static_assert(G == 128, "the two-lanes-per-group kernel is written for G = 128");
            const bool in8 = reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T)) == 0;
            const bool out4 = reinterpret_cast<uintptr_t>(q) % 4 == 0;
            compress_legacy_pair_kernel<T><<<blocks_for(kLaneThreads / 2), kLaneThreads, 0, st>>>(xt, numel, ngroups, *tab, q, s, zp, in8, out4);
        }
        break;
    case Coder::Quality:
        if constexpr (G <= 32) {
            const bool in16 = reinterpret_cast<uintptr_t>(x) % 16 == 0 && (G * sizeof(T)) % 16 == 0;
            const bool out8 = reinterpret_cast<uintptr_t>(q) % 8 == 0;
            compress_quality_lane_kernel<G, T><<<blocks_for(kLaneThreads), kLaneThreads, 0, st>>>(xt, numel, ngroups, q, s, zp, in16, out8);
        } else {
            compress_quality_kernel<G, T><<<grid, kThreads, 0, st>>>(xt, numel, ngroups, q, s, zp, in_aligned, out_aligned);
        }
        break;
    default:
        if constexpr (G <= 64) {
            const bool in16 = reinterpret_cast<uintptr_t>(x) % 16 == 0 && (G * sizeof(T)) % 16 == 0;
            const bool out8 = reinterpret_cast<uintptr_t>(q) % 8 == 0;
            compress_sym_lane_kernel<G, T><<<blocks_for(kLaneThreads), kLaneThreads, 0, st>>>(xt, numel, ngroups, *tab, q, s, in16, out8);
        } else {
            static_assert(G == 128, "the two-lanes-per-group kernel is written for G = 128");
            const bool in8 = reinterpret_cast<uintptr_t>(x) % (4 * sizeof(T)) == 0;
            const bool out4 = reinterpret_cast<uintptr_t>(q) % 4 == 0;
            compress_sym_pair_kernel<T><<<blocks_for(kLaneThreads / 2), kLaneThreads, 0, st>>>(xt, numel, ngroups, *tab, q, s, in8, out4);
        }
        break;
    }
    return cudaGetLastError();
}

template <int G>
cudaError_t launch_g(Coder coder, const void* x, int dtype, int64_t numel, int64_t ngroups, const CandTable* tab, uint8_t* q,
                     uint16_t* s, uint8_t* zp, int grid, cudaStream_t st) {
    switch (dtype) {
    case TCB_DT_BF16: return launch_typed<G, __nv_bfloat16>(coder, x, numel, ngroups, tab, q, s, zp, grid, st);
    case TCB_DT_F16: return launch_typed<G, __half>(coder, x, numel, ngroups, tab, q, s, zp, grid, st);
    default: return launch_typed<G, float>(coder, x, numel, ngroups, tab, q, s, zp, grid, st);
    }
}

int compress_common(const char* who, Coder coder, const void* x, int dtype, int64_t numel, int group_size,
                    const CandTable* tab, uint8_t* q, uint16_t* scales, uint8_t* zp, void* stream) {
    if (numel < 0) return tcb::fail(TCB_ERR_BAD_ARG, "%s: numel %lld < 0", who, (long long)numel);
    if (!tcb::group_size_ok(group_size))
        return tcb::fail(TCB_ERR_GROUP_SIZE, "%s: group_size %d not in {8, 16, 24, 32, 48, 64, 128}", who, group_size);
    if (dtype != TCB_DT_BF16 && dtype != TCB_DT_F16 && dtype != TCB_DT_F32)
        return tcb::fail(TCB_ERR_BAD_ARG, "%s: dtype %d is not bf16(0) / f16(1) / f32(2)", who, dtype);
    if (numel == 0) return TCB_OK;
    if (!x || !q || !scales || (!zp && coder != Coder::Sym)) return tcb::fail(TCB_ERR_BAD_ARG, "%s: null pointer", who);
    const size_t esz = dtype == TCB_DT_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(x) % esz) return tcb::fail(TCB_ERR_ALIGNMENT, "%s: x not aligned to its element size", who);
    if (reinterpret_cast<uintptr_t>(scales) & 1) return tcb::fail(TCB_ERR_ALIGNMENT, "%s: scales not 2-byte aligned", who);

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // plain symmetric codec: the whole groups go through the streaming kernel when the layout allows it
    if (coder == Coder::Sym && tab->n == 0 && (group_size == 16 || group_size == 32 || group_size == 64 || group_size == 128) &&
        reinterpret_cast<uintptr_t>(x) % 32 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0 && numel >= group_size) {
        const int64_t whole = numel / group_size;
        cudaError_t e;
        switch (group_size) {
        case 16: e = launch_sym_stream_typed<1>(x, dtype, whole, q, scales, st); break;
        case 32: e = launch_sym_stream_typed<2>(x, dtype, whole, q, scales, st); break;
        case 64: e = launch_sym_stream_typed<4>(x, dtype, whole, q, scales, st); break;
        default: e = launch_sym_stream_typed<8>(x, dtype, whole, q, scales, st); break;
        }
        if (e != cudaSuccess) return tcb::cuda_fail(e, who);
        const int64_t done = whole * group_size;
        if (done == numel) return TCB_OK;
        x = static_cast<const uint8_t*>(x) + done * esz;  // the ragged last group takes the general kernel
        q += done;
        scales += whole;
        numel -= done;
    }
    const int64_t ngroups = (numel + group_size - 1) / group_size;
    const int64_t blocks = (ngroups + kThreads / 4 - 1) / (kThreads / 4);
    const int64_t max_grid = int64_t(tcb::sm_count()) * 64;
    const int grid = int(blocks < max_grid ? blocks : max_grid);
    cudaError_t e;
    switch (group_size) {
    case 8: e = launch_g<8>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    case 16: e = launch_g<16>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    case 24: e = launch_g<24>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    case 32: e = launch_g<32>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    case 48: e = launch_g<48>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    case 64: e = launch_g<64>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    default: e = launch_g<128>(coder, x, dtype, numel, ngroups, tab, q, scales, zp, grid, st); break;
    }
    return e == cudaSuccess ? TCB_OK : tcb::cuda_fail(e, who);
}

}  // namespace

extern "C" int tcb_compress_amo(const void* x, int dtype, int64_t numel, int group_size, const float* multipliers,
                                int n_cand, uint8_t* q, uint16_t* scales, uint8_t* zp, void* stream) {
    if (!multipliers) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_compress_amo: multipliers is null");
    if (n_cand < 1 || n_cand > 64)
        return tcb::fail(TCB_ERR_TOO_LARGE, "tcb_compress_amo: n_cand %d outside 1..64", n_cand);
    CandTable tab;
    for (int i = 0; i < 64; ++i) tab.m[i] = i < n_cand ? multipliers[i] : 0.0f;
    tab.n = n_cand;
    return compress_common("tcb_compress_amo", Coder::Legacy, x, dtype, numel, group_size, &tab, q, scales, zp, stream);
}

extern "C" int tcb_compress_amo_quality(const void* x, int dtype, int64_t numel, int group_size, uint8_t* q,
                                        uint16_t* scales, uint8_t* zp, void* stream) {
    return compress_common("tcb_compress_amo_quality", Coder::Quality, x, dtype, numel, group_size, nullptr, q, scales, zp,
                           stream);
}

extern "C" int tcb_compress_sym(const void* x, int dtype, int64_t numel, int group_size, const float* multipliers,
                                int n_cand, int8_t* q, uint16_t* scales, void* stream) {
    if (n_cand < 0 || n_cand > 64)
        return tcb::fail(TCB_ERR_TOO_LARGE, "tcb_compress_sym: n_cand %d outside 0..64", n_cand);
    if (n_cand > 0 && !multipliers) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_compress_sym: multipliers is null");
    CandTable tab;
    for (int i = 0; i < 64; ++i) tab.m[i] = i < n_cand ? multipliers[i] : 0.0f;
    tab.n = n_cand;
    return compress_common("tcb_compress_sym", Coder::Sym, x, dtype, numel, group_size, &tab,
                           reinterpret_cast<uint8_t*>(q), scales, nullptr, stream);
}
