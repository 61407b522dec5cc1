/*
 * tcb200 -- C ABI of the B200 (sm_100a) AMO-BQ feature-cache hot path.
 *
 * The reference project (TensorCache v0.7.3) is pure Python; it has no FFI of its
 * own.  Each entry point below therefore names the Python function (path inside
 * the TensorCache project, file:line) whose device work it replaces.  The Python
 * package `tensorcache_b200` binds these symbols with ctypes and keeps the
 * reference's Python signatures on top of them.
 *
 * Conventions
 *   - plain pointers and sizes only; bf16 values travel as uint16_t bit patterns;
 *   - device pointers belong to the CUDA device that is current when the call is
 *     made; `stream` is a cudaStream_t (NULL = the legacy default stream);
 *   - every device entry point only enqueues work on `stream` (no host
 *     synchronisation, so the calls can be captured into a CUDA graph);
 *   - every function returns a TCB_* status; 0 is success.  On failure a
 *     human-readable message is kept per host thread, see tcb_last_error();
 *   - nothing aborts, traps or waits without a bound.
 */
#ifndef TCB200_H_
#define TCB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCB_VERSION 100

#if defined(__GNUC__)
#define TCB_API __attribute__((visibility("default")))
#else
#define TCB_API
#endif

enum tcb_status {
    TCB_OK = 0,
    TCB_ERR_BAD_ARG = 1,       /* null pointer, negative size, bad enum            */
    TCB_ERR_GROUP_SIZE = 2,    /* group size outside the supported set             */
    TCB_ERR_CUDA = 3,          /* a CUDA runtime / driver call failed              */
    TCB_ERR_TIMEOUT = 4,       /* a bounded device-side wait ran out               */
    TCB_ERR_ALIGNMENT = 5,     /* pointer or extent not aligned as the entry needs */
    TCB_ERR_TOO_LARGE = 6,     /* size beyond what the entry point supports        */
    TCB_ERR_IO = 7,            /* host-side file / mapping problem                 */
    TCB_ERR_SUM_ORDER = 8      /* tcb_selftest_sum_order: the host adds in another order */
};

/* element types accepted by the compressor */
enum tcb_dtype { TCB_DT_BF16 = 0, TCB_DT_F16 = 1, TCB_DT_F32 = 2 };

/* Library version (TCB_VERSION of the build). */
TCB_API int tcb_version(void);

/* Message of the last failure on the calling host thread ("" if none). */
TCB_API const char* tcb_last_error(void);

/*
 * Host-only self-test of the one ISA-dependent assumption of the encoders: the order in
 * which the G squared errors of a group are added (cand_err.sum(dim=-1),
 * src/tensorcache/codec.py:877; torch's CPU reduction: 8 lanes x 4 accumulators, lane totals
 * left to right).  `rows` holds n_rows x group_size fp32 terms, `host_sums` the n_rows sums
 * the host's torch computed for them; the function adds each row in the order the encode
 * kernels use and compares the bits.  Returns TCB_OK, or TCB_ERR_SUM_ORDER with the first
 * differing row in tcb_last_error().  Touches no GPU.
 */
TCB_API int tcb_selftest_sum_order(const float* rows, int64_t n_rows, int group_size, const float* host_sums);

/*
 * AMO-BQ decode:  out[i] = bf16_rne((f32(q[i]) - f32(zp[i / G])) * f32(scale[i / G])).
 * Replaces the device branch of dequantize_int8_amo_bq
 * (src/tensorcache/codec.py:896-966; Triton kernel codec.py:186-211) and serves
 * BlockwiseInt8Codec.dequantize (codec.py:1024-1041) and utils.decompress
 * (src/tensorcache/utils.py:142-152).
 *   q       [numel]            uint8 codes
 *   scales  [ceil(numel / G)]  bf16 bit patterns
 *   zp      [ceil(numel / G)]  uint8 zero points
 *   out     [numel]            bf16 bit patterns (may be a caller-owned out_buffer)
 * G must be 8, 16, 24, 32, 48, 64 or 128 (the reference's CPU path takes any G;
 * these are the sizes its tests and presets use).  numel may be 0 and need not be
 * a multiple of G.  The fast path needs q and out 16-byte aligned; other
 * alignments take a slower element-wise kernel with identical results.
 */
TCB_API int tcb_decompress_amo(const uint8_t* q, const uint16_t* scales, const uint8_t* zp, uint16_t* out,
                       int64_t numel, int group_size, void* stream);

/*
 * Decode of codes that sit in HOST memory, for callers that must not allocate on
 * the device.  This entry point has no counterpart in the reference.  It exists
 * for processes that run under a fixed device-memory plan -- an allocator that
 * took the whole GPU at start-up, or code that runs while another thread captures
 * a CUDA graph, when cudaMalloc is off limits -- and therefore cannot provide the
 * device staging buffers the batch readers ask their caller for.  The staging
 * lives inside the library instead: a fixed array of about 4.75 MiB in the device
 * memory of every GPU that loads the library, held until the process exits.
 *   q_host / scales_host / zp_host   host arrays laid out as for tcb_decompress_amo
 *                                    (page-locked memory makes the copies asynchronous)
 *   out_dev                          device output, [numel] bf16 bit patterns
 * At most TCB_NOALLOC_MAX_VALUES values per call; larger sizes are refused with
 * TCB_ERR_TOO_LARGE (split the tensor at a multiple of the group size).
 * The call enqueues three host-to-device copies and the decode kernel on `stream`
 * and calls no cudaMalloc / cudaFree or any other allocating routine.  The first
 * call on each device is the set-up call: it looks up the array's device address
 * (cudaGetSymbolAddress) and makes the decode kernels of all three group sizes and
 * every output alignment resident there.  Under CUDA's lazy module loading that is
 * the moment the array and the kernel code take their device memory, so make this
 * first call -- any size, numel = 32 will do -- per device while allocation is still
 * allowed: before the process freezes its memory plan and outside any stream
 * capture.  Later calls load nothing.  `stream` must belong to the device that is
 * current when the call is made (its copy of the array is the one used).
 * All calls on one device share
 * the one array, which keeps the previous call's bytes: every byte a call reads
 * it has overwritten first, so nothing needs clearing, but two calls whose work
 * overlaps on the GPU (different streams, no ordering between them) race on it.
 */
#define TCB_NOALLOC_MAX_VALUES (4 * 1024 * 1024)
TCB_API int tcb_decompress_amo_host_noalloc(const uint8_t* q_host, const uint16_t* scales_host, const uint8_t* zp_host,
                                            uint16_t* out_dev, int64_t numel, int group_size, void* stream);

/*
 * AMO-BQ encode, candidate-table presets (fast / balanced / accurate / max or a
 * custom table).  Replaces quantize_int8_amo_bq's search
 * (src/tensorcache/codec.py:774-893; Triton kernel src/tensorcache/fused_ops.py:95-143)
 * and reproduces the CPU path's results bit for bit.
 *   x            [numel] values of `dtype` (enum tcb_dtype), flattened row-major
 *   multipliers  HOST array of n_cand fp32 scale multipliers (1 <= n_cand <= 64):
 *                the values of torch.linspace(lo, hi, n_cand) computed on the CPU
 *                (codec.py:852); they are passed by value to the kernel
 *   q, scales, zp  outputs laid out as for tcb_decompress_amo
 * G must be 8, 16, 24, 32, 48, 64 or 128; the last group is zero-padded as the
 * reference pads.
 */
TCB_API int tcb_compress_amo(const void* x, int dtype, int64_t numel, int group_size, const float* multipliers,
                     int n_cand, uint8_t* q, uint16_t* scales, uint8_t* zp, void* stream);

/*
 * AMO-BQ encode, mode "quality": search over up to 64 consecutive bf16 scales
 * scored on the decoded bf16 values.  Replaces _quantize_amo_quality_torch
 * (src/tensorcache/codec.py:721-771; Triton kernel fused_ops.py:146-207),
 * bit-exact with the CPU path.  Arguments as for tcb_compress_amo.
 */
TCB_API int tcb_compress_amo_quality(const void* x, int dtype, int64_t numel, int group_size, uint8_t* q,
                             uint16_t* scales, uint8_t* zp, void* stream);

/*
 * Symmetric int8 codec (signed codes, one bf16 scale per group, no zero point).
 * n_cand == 0 replaces quantize_int8_g32 (src/tensorcache/codec.py:530-565):
 * scale = bf16(max|x| / 127), q = clamp(rne(x / scale), -128, 127).
 * n_cand > 0 replaces quantize_int8_adaptive (src/tensorcache/codec.py:568-620):
 * the scale is searched over (max|x| / 127) * multipliers[c], the host values of
 * torch.linspace(0.90, 1.05, n_cand), scored by squared error, first minimum wins.
 * Both reproduce the CPU path bit for bit; non-finite inputs become code 0.
 * These are also the codes FusedDequantLinear takes with zp == NULL.
 *   q       [numel]            int8 codes          scales  [ceil(numel / G)] bf16 bits
 * Group sizes as for tcb_compress_amo; 0 <= n_cand <= 64.
 */
TCB_API int tcb_compress_sym(const void* x, int dtype, int64_t numel, int group_size, const float* multipliers,
                             int n_cand, int8_t* q, uint16_t* scales, void* stream);

/*
 * Symmetric decode: out[i] = bf16( int8(q[i]) * scale[i / G] ), bit-exact (the
 * product is exact in fp32).  Replaces dequantize_int8_g32
 * (src/tensorcache/codec.py:623-697; Triton kernel codec.py:214-231) and
 * utils.decompress with zero_points=None (src/tensorcache/utils.py:150-152).
 * Sizes, alignment and group sizes as for tcb_decompress_amo.
 */
TCB_API int tcb_decompress_sym(const int8_t* q, const uint16_t* scales, uint16_t* out, int64_t numel, int group_size,
                               void* stream);

/*
 * Fused dequantise + GEMM on the tcgen05 tensor cores:
 *     out[m, n] = bf16( sum_k dense[m, k] * deq(q)[n, k]  + bias )
 * with deq(q)[n, k] = (q[n, k] - zp[n, k / G]) * scale[n, k / G]   (zp != NULL, uint8 codes)
 *                or    int8(q[n, k])           * scale[n, k / G]   (zp == NULL, signed codes).
 * Replaces FusedDequantLinear.forward / _fused_dequant_matmul_kernel
 * (src/tensorcache/fused_ops.py:1338-1461).
 *   dense  [R_d, K] bf16, K contiguous        q  [R_q, K] codes, K contiguous
 *   scales / zp  [R_q * K / G]                out [R_d, R_q] bf16 when quant_is_rhs != 0
 *   quant_is_rhs != 0:  out = dense . deq(q)^T   (quantised weight; bias has R_q entries)
 *   quant_is_rhs == 0:  out[R_q, R_d] = deq(q) . dense^T  (the reference's layout: quantised
 *                       activation, dense weight; bias has R_d entries)
 * Requirements: G in {16, 32, 64, 128}, K a positive multiple of G (the kernel steps K by
 * 64 and zero-fills a ragged last step); dense and q 16-byte aligned.  R_d and R_q
 * are arbitrary (edge tiles are masked).
 * Every wait inside the kernel is bounded; if one runs out the kernel records it
 * in a per-device status word that tcb_fused_dequant_linear_check() reads.
 */
TCB_API int tcb_fused_dequant_linear(const uint16_t* dense, const uint8_t* q, const uint16_t* scales,
                             const uint8_t* zp_or_null, const uint16_t* bias_or_null, uint16_t* out,
                             int64_t R_d, int64_t R_q, int64_t K, int group_size, int quant_is_rhs,
                             void* stream);

/* Reads (and clears) the per-device status word the fused GEMM writes when a
 * bounded wait runs out.  Synchronises `stream`.  Returns TCB_OK or TCB_ERR_TIMEOUT. */
TCB_API int tcb_fused_dequant_linear_check(void* stream);

/* Launches a tiny kernel whose only work is a bounded wait on a barrier that nothing
 * ever signals, with a budget of `budget_ms` milliseconds (1..1000).  The kernel
 * gives up when the budget is spent, releases its second waiter through the abort
 * flag and returns; tcb_fused_dequant_linear_check() then reports TCB_ERR_TIMEOUT.
 * Exercises the time-out path every wait of the fused GEMM uses, without hanging or
 * faulting the device.  (No counterpart in the reference, which has no device waits.) */
TCB_API int tcb_selftest_bounded_wait(int budget_ms, void* stream);

/*
 * Host-side row gather used by the batch readers: copies n rows of row_bytes
 * bytes, dst[i] = src_base[idx[i]] (idx == NULL: rows first_row .. first_row+n-1,
 * i.e. one contiguous block), using up to nthreads worker threads.  Replaces
 * the np.copyto(mmap -> pinned) steps of ZeroCopyTensorStreamer
 * (src/tensorcache/streamer.py:280-327, 434-457) and FeatureCacheDataset.iter_batches
 * (src/tensorcache/feature_cache.py:1018-1021, 1075-1078).
 */
TCB_API int tcb_gather_rows(void* dst, const void* src_base, int64_t row_bytes, const int64_t* idx,
                    int64_t first_row, int64_t n, int nthreads);

/*
 * Host-side block copy used by the cache writer: copies `bytes` bytes from `src`
 * (page-locked landing buffer of a chunk of codes) to `dst`, a range of a writable
 * mapping of a cache file, on up to nthreads worker threads.  Each worker has the
 * kernel populate its part of a still sparse file in one call before it copies, so
 * the copy does not take one page fault per 4 KB.  Replaces the row assignments into
 * np.memmap of FeatureCacheWriter.append (src/tensorcache/feature_cache.py:364-424).
 */
TCB_API int tcb_write_block(void* dst, const void* src, int64_t bytes, int nthreads);

/*
 * Native double-buffered batch pipeline behind ZeroCopyTensorStreamer
 * (src/tensorcache/streamer.py:430-495): worker threads gather rows from the
 * three memory-mapped arrays of one cache shard into pinned staging, a copy
 * stream moves them to device staging, and the decode kernel is enqueued on the
 * consumer's stream; events order both directions (host never overwrites pinned
 * memory still being read by a copy, the copy stream never overwrites device
 * staging still being decoded).
 *
 * All buffers are caller-allocated (the Python shim uses torch for that).  A
 * streamer reads one shard or several (the reference's "all shards on one GPU"
 * mode, streamer.py:114-156); n_slots = 1 is the reference's low_vram mode,
 * n_slots = 2 its double-buffered ring.
 */
typedef struct tcb_streamer tcb_streamer;

typedef struct tcb_streamer_desc {
    int n_shards;                  /* >= 1; samples are numbered shard after shard           */
    const void* const* q_bases;    /* [n_shards] mapped [size, values_per_sample] codes      */
    const void* const* s_bases;    /* [n_shards] mapped [size, groups_per_sample] bf16 bits  */
    const void* const* zp_bases;   /* [n_shards] mapped [size, groups_per_sample] zero points;
                                      NULL for a cache of the symmetric codec (int8 codes, no
                                      zero points): pinned_zp / dev_zp are then unused and may be NULL */
    const int64_t* shard_sizes;    /* [n_shards] samples per shard                           */
    int64_t values_per_sample;     /* seq_len * dim, a multiple of group_size                */
    int64_t groups_per_sample;     /* values_per_sample / group_size                         */
    int group_size;
    int batch_size;
    int n_slots;                   /* 1 (serial) .. 8 ring slots                             */
    int n_threads;                 /* gather workers (>= 1)                                  */
    void* const* pinned_q;         /* [n_slots] page-locked, batch_size rows each            */
    void* const* pinned_s;
    void* const* pinned_zp;
    void* const* dev_q;            /* [n_slots] device staging                               */
    void* const* dev_s;
    void* const* dev_zp;
    void* const* dev_out;          /* [n_slots] bf16 [batch_size, values_per_sample]         */
    int direct_dma;                /* != 0: the shard mappings are page-locked (tcb_pin_host_range);
                                      copies go straight from them, no staging copy of the codes    */
} tcb_streamer_desc;

/* Page-locks a host range so that the copy engine can read it directly (wraps
 * cudaHostRegister), and undoes it.  Used for the "resident shard" mode of the
 * readers: the shard files are mapped privately (copy-on-write) and writable --
 * the driver refuses read-only and shared file mappings -- and pinned once, which
 * costs about 0.4 s per GB and as much host memory as the shard; afterwards no
 * CPU touches the codes again.  The reference always copies rows on the CPU
 * (src/tensorcache/streamer.py:434-457). */
TCB_API int tcb_pin_host_range(void* p, int64_t bytes);
TCB_API int tcb_unpin_host_range(void* p);

/* Creates the pipeline on the current device.  The tables of the descriptor are
 * copied; the buffers and mappings they name must stay valid until destroy. */
TCB_API int tcb_streamer_create(const tcb_streamer_desc* desc, tcb_streamer** out);

/* Total number of samples over all shards of the streamer. */
TCB_API int tcb_streamer_num_samples(const tcb_streamer* s, int64_t* out);

/* Starts a pass over `n_indices` samples in the given order of global sample ids
 * (order == NULL: 0 .. n_indices-1).  The array is copied.  An unfinished pass is
 * abandoned.  The producer thread starts fetching at once. */
TCB_API int tcb_streamer_begin(tcb_streamer* s, const int64_t* order, int64_t n_indices);

/* Decode the next batch: makes `consumer_stream` wait for the batch's copies,
 * enqueues the decode kernel into dev_out[*slot] on it, and hands the slot's
 * staging back to the producer (ordered after the decode).  *batch_rows == 0
 * means the pass is finished. */
TCB_API int tcb_streamer_next(tcb_streamer* s, void* consumer_stream, int* slot, int* batch_rows);

/* The two halves of tcb_streamer_next for callers that want the raw codes
 * (iter_batches(dequantize=False), src/tensorcache/feature_cache.py:1031-1037):
 * acquire makes `consumer_stream` wait until dev_q/dev_s/dev_zp[*slot] hold the
 * batch; release (after the caller has enqueued its reads of the staging on the
 * same stream) lets the producer overwrite the slot once those reads are done. */
TCB_API int tcb_streamer_acquire(tcb_streamer* s, void* consumer_stream, int* slot, int* batch_rows);
TCB_API int tcb_streamer_release(tcb_streamer* s, void* consumer_stream);

/* Stops the producer, waits for its copies and frees the pipeline's own objects
 * (never the caller's buffers). */
TCB_API int tcb_streamer_destroy(tcb_streamer* s);

#ifdef __cplusplus
}
#endif
#endif /* TCB200_H_ */
