/*
 * CPU oracle for the AMO-BQ feature-cache hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU PyTorch
 * implementation of AMO-BQ (TensorCache v0.7.3).  It exists so that the CUDA
 * kernels can be checked bit-for-bit on a machine that does not have the
 * reference installed, and so that a CPU baseline can be timed beside the GPU
 * numbers.  Nothing in the product package links, loads or calls it; only the
 * tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status: PINNED.  Every function here is compared bit-for-bit with the
 * imported reference (CPU tensors) by oracle/check_against_reference.py, and the
 * fixtures under tests/golden/ are outputs of the reference itself.
 *
 * Reference locations (paths inside the TensorCache project):
 *   legacy presets   src/tensorcache/codec.py:833-893  (quantize_int8_amo_bq)
 *   sanitising       src/tensorcache/codec.py:254-260  (_sanitize_blocks)
 *   quality mode     src/tensorcache/codec.py:721-771  (_amo_quality_codes,
 *                                                       _quantize_amo_quality_torch)
 *   decode           src/tensorcache/codec.py:953-966  (dequantize_int8_amo_bq)
 *   symmetric codec  src/tensorcache/codec.py:530-565  (quantize_int8_g32),
 *                    src/tensorcache/codec.py:568-620  (quantize_int8_adaptive),
 *                    src/tensorcache/codec.py:685-695  (dequantize_int8_g32, CPU branch)
 *
 * Arithmetic rules that make the restatement bit-exact:
 *   - every operation is a separate IEEE-754 binary32 operation (compile with
 *     -ffp-contract=off; no FMA contraction, no fast-math);
 *   - division is the correctly rounded one, rounding to integer is
 *     round-half-to-even (nearbyintf under the default rounding mode);
 *   - the candidate multipliers are passed in (they are the values produced by
 *     torch.linspace on the CPU, which are not reproducible by a closed formula);
 *   - the squared-error sum over a group follows the order ATen's vectorised
 *     inner reduction uses on x86-64: eight lanes, four partial accumulators
 *     (see sum_group()).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TCB_ORACLE_MAX_G 256

/* ------------------------------------------------------------------ types */

static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* float -> bfloat16 with round-half-to-even; NaN becomes 0x7FC0 (what
 * c10::BFloat16's round_to_nearest_even does). */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if (f != f) return 0x7FC0;
    uint32_t bias = 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)((u + bias) >> 16);
}

static inline float round_to_bf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

static inline float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3FFu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* dtype codes shared with the C ABI of the CUDA library */
enum { TCB_DT_BF16 = 0, TCB_DT_F16 = 1, TCB_DT_F32 = 2 };

static inline float load_as_f32(const void* x, int dtype, int64_t i) {
    switch (dtype) {
    case TCB_DT_BF16: return bf16_bits_to_f32(((const uint16_t*)x)[i]);
    case TCB_DT_F16: return f16_bits_to_f32(((const uint16_t*)x)[i]);
    default: return ((const float*)x)[i];
    }
}

static inline float clamp_0_255(float v) {
    /* torch.clamp(v, 0, 255) == min(max(v, 0), 255) with NaN propagating */
    if (v != v) return v;
    if (v < 0.0f) v = 0.0f;
    if (v > 255.0f) v = 255.0f;
    return v;
}

/*
 * Sum of G floats in the order of ATen's contiguous inner-dimension reduction on
 * x86-64 (observed on torch 2.11 CPU with AVX2 and AVX-512 builds): the row is
 * cut into vectors of 8 lanes; complete runs of four vectors feed four partial
 * accumulators (vector j of a run goes to accumulator j), left-over vectors go
 * to accumulator 0; the accumulators are combined ((a0+a1)+a2)+a3 per lane; the
 * eight lane totals are then added left to right.  A tail of G % 8 scalars is
 * added last, one by one.
 */
static float sum_group(const float* e, int G) {
    int nvec = G / 8;
    int full = (nvec / 4) * 4;
    float lane_tot[8];
    for (int l = 0; l < 8; ++l) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        for (int v = 0; v < full; v += 4) {
            a0 = a0 + e[(v + 0) * 8 + l];
            a1 = a1 + e[(v + 1) * 8 + l];
            a2 = a2 + e[(v + 2) * 8 + l];
            a3 = a3 + e[(v + 3) * 8 + l];
        }
        for (int v = full; v < nvec; ++v) a0 = a0 + e[v * 8 + l];
        lane_tot[l] = ((a0 + a1) + a2) + a3;
    }
    float tot = 0.0f;
    if (nvec > 0)
        for (int l = 0; l < 8; ++l) tot = tot + lane_tot[l];
    for (int i = nvec * 8; i < G; ++i) tot = tot + e[i];
    return tot;
}

/* first index of the minimum, NaN counting as smaller than everything
 * (torch.argmin semantics) */
static inline int better_than(float cand, float best) {
    if (best != best) return 0;
    if (cand != cand) return 1;
    return cand < best;
}

/* ----------------------------------------------------------- group coders */

/* codec.py:833-893, one group of G values already widened to fp32 and
 * zero-padded.  Writes G codes, one bf16 scale, one zero point. */
static void encode_group_legacy(const float* xin, int G, const float* mult, int ncand,
                                uint8_t* q_out, uint16_t* s_out, uint8_t* zp_out) {
    float x[TCB_ORACLE_MAX_G];
    unsigned char fin[TCB_ORACLE_MAX_G];
    float e[TCB_ORACLE_MAX_G];
    float bmin = 0.0f, bmax = 0.0f;
    for (int i = 0; i < G; ++i) {
        fin[i] = isfinite(xin[i]) ? 1 : 0;
        x[i] = fin[i] ? xin[i] : 0.0f; /* codec.py:254-260 */
        if (i == 0 || x[i] < bmin) bmin = x[i];
        if (i == 0 || x[i] > bmax) bmax = x[i];
    }
    float rng = bmax - bmin; /* codec.py:847-850 */
    if (rng < 1e-8f) rng = 1e-8f;
    if (!isfinite(rng)) rng = 1e-8f;
    float s0 = rng / 255.0f;
    if (!isfinite(s0)) s0 = (float)(1e-8 / 255.0);

    float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
    for (int c = 0; c < ncand; ++c) { /* codec.py:868-882 */
        float s = s0 * mult[c];
        float zp = clamp_0_255(nearbyintf((-bmin) / s));
        for (int i = 0; i < G; ++i) {
            float t = x[i] / s;
            t = t + zp;
            float qc = clamp_0_255(nearbyintf(t));
            float rec = (qc - zp) * s;
            float d = fin[i] ? (x[i] - rec) : 0.0f;
            e[i] = d * d;
        }
        float err = sum_group(e, G);
        if (c == 0 || better_than(err, best_err)) {
            best_err = err;
            best_s = s;
            best_zp = zp;
        }
    }
    for (int i = 0; i < G; ++i) { /* codec.py:885-891 */
        float t = x[i] / best_s;
        t = t + best_zp;
        float qf = clamp_0_255(nearbyintf(t));
        q_out[i] = fin[i] ? (uint8_t)qf : (uint8_t)best_zp;
    }
    *s_out = f32_to_bf16_bits(best_s); /* codec.py:893 */
    *zp_out = (uint8_t)best_zp;
}

/* codec.py:721-734 for one value: returns the chosen code, writes its error */
static inline float quality_code(float x, float s, float zp, float* err_out) {
    float r = nearbyintf(x / s + zp);
    float q = clamp_0_255(r);
    float rec = round_to_bf16((q - zp) * s);
    float d = x - rec;
    float err = d * d;
    for (int k = 0; k < 2; ++k) {
        float delta = k == 0 ? -1.0f : 1.0f;
        float aq = clamp_0_255(r + delta);
        float arec = round_to_bf16((aq - zp) * s);
        float ad = x - arec;
        float ae = ad * ad;
        if (ae < err) q = aq;
        /* torch.minimum: NaN propagates */
        if (ae != ae || err != err) err = NAN;
        else err = ae < err ? ae : err;
    }
    *err_out = err;
    return q;
}

/* codec.py:737-771, one group */
static void encode_group_quality(const float* xin, int G, uint8_t* q_out, uint16_t* s_out,
                                 uint8_t* zp_out) {
    float x[TCB_ORACLE_MAX_G];
    unsigned char fin[TCB_ORACLE_MAX_G];
    float e[TCB_ORACLE_MAX_G];
    float qbuf[TCB_ORACLE_MAX_G], qbest[TCB_ORACLE_MAX_G];
    float lower = 0.0f, upper = 0.0f;
    for (int i = 0; i < G; ++i) {
        fin[i] = isfinite(xin[i]) ? 1 : 0;
        x[i] = fin[i] ? xin[i] : 0.0f;
        if (i == 0 || x[i] < lower) lower = x[i];
        if (i == 0 || x[i] > upper) upper = x[i];
    }
    if (lower > 0.0f) lower = 0.0f; /* codec.py:755-756 */
    if (upper < 0.0f) upper = 0.0f;
    float scale0 = upper / 255.0f - lower / 255.0f; /* codec.py:757 */
    float floor_s = (float)(1e-8 / 255.0);
    if (scale0 < floor_s) scale0 = floor_s;
    int32_t lo_bits = (int16_t)f32_to_bf16_bits(scale0 * 0.85f); /* codec.py:758-759 */
    int32_t hi_bits = (int16_t)f32_to_bf16_bits(scale0 * 1.10f);

    float best_err = 0.0f, best_s = 0.0f, best_zp = 0.0f;
    for (int k = 0; k < 64; ++k) { /* codec.py:760-765 */
        int32_t bits = lo_bits + k;
        if (bits > hi_bits) bits = hi_bits;
        float s = bf16_bits_to_f32((uint16_t)(int16_t)bits);
        float zp = clamp_0_255(nearbyintf((-lower) / s));
        for (int i = 0; i < G; ++i) {
            float err;
            qbuf[i] = quality_code(x[i], s, zp, &err);
            e[i] = fin[i] ? err : 0.0f;
        }
        float tot = sum_group(e, G);
        if (k == 0 || better_than(tot, best_err)) {
            best_err = tot;
            best_s = s;
            best_zp = zp;
            memcpy(qbest, qbuf, sizeof(float) * (size_t)G);
        }
    }
    for (int i = 0; i < G; ++i) /* codec.py:767-768 */
        q_out[i] = fin[i] ? (uint8_t)qbest[i] : (uint8_t)best_zp;
    *s_out = f32_to_bf16_bits(best_s);
    *zp_out = (uint8_t)best_zp;
}

static inline float clamp_i8(float v) {
    if (v != v) return v;
    if (v < -128.0f) v = -128.0f;
    if (v > 127.0f) v = 127.0f;
    return v;
}

/* codec.py:530-565 (ncand == 0) and codec.py:568-620 (ncand > 0, the "adaptive"
 * scale search), one group.  Signed codes, one bf16 scale, no zero point.  The
 * adaptive search scores the candidates on the RAW values (a NaN or Inf in the
 * group makes every error NaN or Inf and candidate 0 wins), then quantises the
 * cleaned values with the bf16-rounded winner. */
static void encode_group_sym(const float* xin, int G, const float* mult, int ncand,
                             int8_t* q_out, uint16_t* s_out) {
    float x[TCB_ORACLE_MAX_G];
    unsigned char fin[TCB_ORACLE_MAX_G];
    float e[TCB_ORACLE_MAX_G];
    float bmax = 0.0f;
    for (int i = 0; i < G; ++i) {
        fin[i] = isfinite(xin[i]) ? 1 : 0;
        x[i] = fin[i] ? xin[i] : 0.0f;
        float a = fabsf(x[i]);
        if (a > bmax) bmax = a;
    }
    if (bmax < 1e-8f) bmax = 1e-8f;
    float s0 = bmax / 127.0f;
    float best_s = s0;
    if (ncand > 0) {
        float best_err = 0.0f;
        for (int c = 0; c < ncand; ++c) {
            float s = s0 * mult[c];
            for (int i = 0; i < G; ++i) {
                float qc = clamp_i8(nearbyintf(xin[i] / s));
                float rec = qc * s;
                float d = xin[i] - rec;
                e[i] = d * d;
            }
            float err = sum_group(e, G);
            if (c == 0 || better_than(err, best_err)) {
                best_err = err;
                best_s = s;
            }
        }
    }
    uint16_t sb = f32_to_bf16_bits(best_s);
    float sf = bf16_bits_to_f32(sb);
    for (int i = 0; i < G; ++i) {
        float qf = clamp_i8(nearbyintf(x[i] / sf));
        q_out[i] = fin[i] ? (int8_t)qf : 0;
    }
    *s_out = sb;
}

/* -------------------------------------------------------------- threading */

typedef void (*range_fn)(void* ctx, int64_t lo, int64_t hi);

typedef struct {
    range_fn fn;
    void* ctx;
    int64_t lo, hi;
} work_t;

static void* work_trampoline(void* p) {
    work_t* w = (work_t*)p;
    w->fn(w->ctx, w->lo, w->hi);
    return NULL;
}

/* splits [0, n) into nthreads contiguous ranges, aligned to `align` items */
static void parallel_for(int64_t n, int64_t align, int nthreads, range_fn fn, void* ctx) {
    if (nthreads < 1) nthreads = 1;
    if (nthreads > 256) nthreads = 256;
    if (nthreads == 1 || n < 2 * align) {
        fn(ctx, 0, n);
        return;
    }
    pthread_t th[256];
    work_t w[256];
    int64_t units = (n + align - 1) / align;
    int64_t per = (units + nthreads - 1) / nthreads;
    int started = 0;
    for (int t = 0; t < nthreads; ++t) {
        int64_t lo = (int64_t)t * per * align;
        int64_t hi = lo + per * align;
        if (lo >= n) break;
        if (hi > n) hi = n;
        w[t].fn = fn;
        w[t].ctx = ctx;
        w[t].lo = lo;
        w[t].hi = hi;
        if (pthread_create(&th[t], NULL, work_trampoline, &w[t]) != 0) {
            fn(ctx, lo, hi);
            th[t] = 0;
        }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t)
        if (th[t]) pthread_join(th[t], NULL);
}

/* ------------------------------------------------------------ public API */

typedef struct {
    const uint8_t* q;
    const uint16_t* s;
    const uint8_t* zp;
    uint16_t* out;
    int64_t numel;
    int G;
} dec_ctx;

static void dec_range(void* p, int64_t lo, int64_t hi) {
    dec_ctx* c = (dec_ctx*)p;
    int G = c->G;
    /* lo is a multiple of G */
    for (int64_t base = lo; base < hi; base += G) {
        int64_t g = base / G;
        float s = bf16_bits_to_f32(c->s[g]);
        float z = (float)c->zp[g];
        int64_t end = base + G < hi ? base + G : hi;
        for (int64_t i = base; i < end; ++i)
            c->out[i] = f32_to_bf16_bits(((float)c->q[i] - z) * s); /* codec.py:959-965 */
    }
}

/* out[i] = bf16((f32(q[i]) - f32(zp[i / G])) * f32(scale[i / G])) */
void tcb_oracle_decompress(const uint8_t* q, const uint16_t* scales, const uint8_t* zp,
                           uint16_t* out, int64_t numel, int group_size, int nthreads) {
    dec_ctx c = {q, scales, zp, out, numel, group_size};
    parallel_for(numel, group_size, nthreads, dec_range, &c);
}

typedef struct {
    const void* x;
    int dtype;
    int64_t numel;
    int G;
    const float* mult;
    int ncand; /* 0 selects quality mode */
    uint8_t* q;
    uint16_t* s;
    uint8_t* zp;
} enc_ctx;

static void enc_range(void* p, int64_t lo, int64_t hi) {
    enc_ctx* c = (enc_ctx*)p;
    int G = c->G;
    float xin[TCB_ORACLE_MAX_G];
    uint8_t qtmp[TCB_ORACLE_MAX_G];
    for (int64_t base = lo; base < hi; base += G) {
        int64_t g = base / G;
        int64_t n_here = c->numel - base < G ? c->numel - base : G;
        for (int i = 0; i < G; ++i)
            xin[i] = i < n_here ? load_as_f32(c->x, c->dtype, base + i) : 0.0f; /* F.pad */
        if (c->ncand > 0)
            encode_group_legacy(xin, G, c->mult, c->ncand, qtmp, &c->s[g], &c->zp[g]);
        else
            encode_group_quality(xin, G, qtmp, &c->s[g], &c->zp[g]);
        memcpy(c->q + base, qtmp, (size_t)n_here);
    }
}

/* Legacy presets (fast / balanced / accurate / max, or any custom candidate
 * table).  Returns 0, or -1 for an unsupported group size. */
int tcb_oracle_compress(const void* x, int dtype, int64_t numel, int group_size,
                        const float* multipliers, int n_cand, uint8_t* q, uint16_t* scales,
                        uint8_t* zp, int nthreads) {
    if (group_size <= 0 || group_size > TCB_ORACLE_MAX_G || n_cand <= 0) return -1;
    enc_ctx c = {x, dtype, numel, group_size, multipliers, n_cand, q, scales, zp};
    parallel_for(numel, group_size, nthreads, enc_range, &c);
    return 0;
}

/* Mode "quality": search over consecutive bf16 scales, decoded-error scoring. */
int tcb_oracle_compress_quality(const void* x, int dtype, int64_t numel, int group_size,
                                uint8_t* q, uint16_t* scales, uint8_t* zp, int nthreads) {
    if (group_size <= 0 || group_size > TCB_ORACLE_MAX_G) return -1;
    enc_ctx c = {x, dtype, numel, group_size, NULL, 0, q, scales, zp};
    parallel_for(numel, group_size, nthreads, enc_range, &c);
    return 0;
}

typedef struct {
    const void* x;
    int dtype;
    int64_t numel;
    int G;
    const float* mult;
    int ncand;
    int8_t* q;
    uint16_t* s;
} sym_ctx;

static void sym_enc_range(void* p, int64_t lo, int64_t hi) {
    sym_ctx* c = (sym_ctx*)p;
    int G = c->G;
    float xin[TCB_ORACLE_MAX_G];
    int8_t qtmp[TCB_ORACLE_MAX_G];
    for (int64_t base = lo; base < hi; base += G) {
        int64_t n_here = c->numel - base < G ? c->numel - base : G;
        for (int i = 0; i < G; ++i)
            xin[i] = i < n_here ? load_as_f32(c->x, c->dtype, base + i) : 0.0f;
        encode_group_sym(xin, G, c->mult, c->ncand, qtmp, &c->s[base / G]);
        memcpy(c->q + base, qtmp, (size_t)n_here);
    }
}

/* Symmetric int8 codec: n_cand == 0 is quantize_int8_g32, n_cand > 0 is
 * quantize_int8_adaptive with the given multipliers (torch.linspace(0.90, 1.05, n)). */
int tcb_oracle_compress_sym(const void* x, int dtype, int64_t numel, int group_size,
                            const float* multipliers, int n_cand, int8_t* q, uint16_t* scales,
                            int nthreads) {
    if (group_size <= 0 || group_size > TCB_ORACLE_MAX_G || n_cand < 0) return -1;
    sym_ctx c = {x, dtype, numel, group_size, multipliers, n_cand, q, scales};
    parallel_for(numel, group_size, nthreads, sym_enc_range, &c);
    return 0;
}

static void sym_dec_range(void* p, int64_t lo, int64_t hi) {
    dec_ctx* c = (dec_ctx*)p;
    int G = c->G;
    for (int64_t base = lo; base < hi; base += G) {
        float s = bf16_bits_to_f32(c->s[base / G]);
        int64_t end = base + G < hi ? base + G : hi;
        for (int64_t i = base; i < end; ++i)
            c->out[i] = f32_to_bf16_bits((float)(int8_t)c->q[i] * s); /* codec.py:691-694 */
    }
}

/* out[i] = bf16(f32(int8 q[i]) * f32(scale[i / G])) */
void tcb_oracle_decompress_sym(const int8_t* q, const uint16_t* scales, uint16_t* out,
                               int64_t numel, int group_size, int nthreads) {
    dec_ctx c = {(const uint8_t*)q, scales, NULL, out, numel, group_size};
    parallel_for(numel, group_size, nthreads, sym_dec_range, &c);
}

typedef struct {
    const uint16_t* dense; /* [R_d, K] bf16 */
    const uint8_t* q;      /* [R_q, K] codes */
    const uint16_t* s;
    const uint8_t* zp; /* NULL: codes are signed int8, no zero point */
    const uint16_t* bias;
    float* out; /* [R_d, R_q] fp32 (not rounded) */
    int64_t R_d, R_q, K;
    int G;
} mm_ctx;

static void mm_range(void* p, int64_t lo, int64_t hi) {
    mm_ctx* c = (mm_ctx*)p;
    float* w = (float*)malloc(sizeof(float) * (size_t)c->K);
    for (int64_t n = lo; n < hi; ++n) {
        for (int64_t k = 0; k < c->K; ++k) {
            int64_t g = (n * c->K + k) / c->G;
            float sc = bf16_bits_to_f32(c->s[g]);
            float v = c->zp ? (float)c->q[n * c->K + k] - (float)c->zp[g]
                            : (float)(int8_t)c->q[n * c->K + k];
            w[k] = v * sc;
        }
        for (int64_t m = 0; m < c->R_d; ++m) {
            const uint16_t* a = c->dense + m * c->K;
            double acc = 0.0;
            for (int64_t k = 0; k < c->K; ++k) acc += (double)bf16_bits_to_f32(a[k]) * (double)w[k];
            if (c->bias) acc += (double)bf16_bits_to_f32(c->bias[n]);
            c->out[m * c->R_q + n] = (float)acc;
        }
    }
    free(w);
}

/* out[m, n] = sum_k dense[m, k] * (q[n, k] - zp[n*K/G + k/G]) * scale[..] (+ bias[n]),
 * accumulated in double, returned as fp32 without rounding to bf16.  This is the
 * "fp32 dequant-then-matmul" the fused GEMM is compared with (tolerance test). */
void tcb_oracle_dequant_matmul(const uint16_t* dense, const uint8_t* q, const uint16_t* scales,
                               const uint8_t* zp_or_null, const uint16_t* bias_or_null, float* out,
                               int64_t R_d, int64_t R_q, int64_t K, int group_size, int nthreads) {
    mm_ctx c = {dense, q, scales, zp_or_null, bias_or_null, out, R_d, R_q, K, group_size};
    parallel_for(R_q, 1, nthreads, mm_range, &c);
}

/* Sum of one row in the pinned order; exported so a test can compare it with
 * torch.sum on the machine the tests run on. */
float tcb_oracle_sum_group(const float* e, int group_size) { return sum_group(e, group_size); }
