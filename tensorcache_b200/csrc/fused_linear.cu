// Fused AMO-BQ dequantise + GEMM for sm_100a on the tcgen05 tensor cores.
//
//     D[r_q, r_d] = sum_k deq(q)[r_q, k] * dense[r_d, k]        (fp32 accumulation in TMEM)
//
// with deq(q)[r, k] = (q[r, k] - zp[r, k / G]) * scale[r, k / G].  The quantised
// operand never exists in global memory in bf16: producer warps read the uint8
// codes, dequantise them in registers and write bf16 straight into the shared
// memory tile the tensor core reads (the canonical K-major, 128-byte-swizzled
// UMMA operand layout).  The dense operand arrives by TMA into the same layout.
//
// One CTA per SM, persistent over output tiles of 128 (quantised rows) x 256
// (dense rows); K advances 64 at a time through a 3-stage ring.
//   warp 0      TMA producer: dense tile [256 x 64] bf16 and raw code tile [128 x 64]
//               uint8 per stage (one thread)
//   warp 1      MMA issuer: 4 x tcgen05.mma (M128 N256 K16) per stage, commits
//               the stage back to the producers and the finished accumulator to
//               the epilogue (one thread); also owns the TMEM allocation
//   warps 2-9   dequantising producers: read the raw codes from shared memory,
//               write 128 rows x 64 bf16 per stage; scales / zero points come from a
//               double-buffered shared-memory chunk (32 groups per row) that the
//               producers refill themselves one chunk ahead.  (Fetching codes and
//               scales with per-thread global loads instead capped the kernel at
//               ~740 TFLOP/s: the LSU miss path, not the math, was the limit.)
//   warps 10-13 epilogue: tcgen05.ld -> (+bias) -> bf16 -> global
// The 512 TMEM columns hold two 128 x 256 fp32 accumulators, so the epilogue of
// one tile overlaps the main loop of the next.  No TMA multicast, no cluster.
//
// The dequantised value is bf16((q - zp) * scale): q - zp is formed exactly in
// fp32, rounded to bf16 without error (|q - zp| <= 255 fits 8 significant bits)
// and multiplied by the bf16 scale with one correctly rounded bf16 multiply, i.e.
// it is the same number the decode kernel produces.
//
// Every wait on an mbarrier is bounded by a clock budget.  When one runs out the
// thread raises a CTA-wide abort flag and a device status word; all roles leave
// their loops, the CTA synchronises, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include "tcb_common.h"

namespace {

constexpr int kTileQ = 128;      // rows of the quantised operand per tile (MMA M)
constexpr int kTileD = 256;      // rows of the dense operand per tile (MMA N)
constexpr int kBlockK = 64;      // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr int kNumProducerWarps = 8;
constexpr int kNumEpilogueWarps = 4;
constexpr int kThreads = 32 * (2 + kNumProducerWarps + kNumEpilogueWarps);  // 448
constexpr int kFirstProducerWarp = 2;
constexpr int kFirstEpilogueWarp = 2 + kNumProducerWarps;                   // 10
constexpr uint32_t kStageBytesA = kTileQ * kBlockK * 2;                      // 16 KB
constexpr uint32_t kStageBytesB = kTileD * kBlockK * 2;                      // 32 KB
constexpr uint32_t kStageBytesC = kTileQ * kBlockK;                          // 8 KB of raw codes
constexpr int kChunkGroups = 32;                                             // groups per row per scale chunk
constexpr uint32_t kChunkBytesS = kTileQ * kChunkGroups * 2;                 // 8 KB of bf16 scales
constexpr uint32_t kChunkBytesZ = kTileQ * kChunkGroups;                     // 4 KB of zero points
constexpr uint32_t kSmemTiles = kStages * (kStageBytesA + kStageBytesB + kStageBytesC) + 2 * (kChunkBytesS + kChunkBytesZ);
constexpr uint32_t kSmemBytes = kSmemTiles + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr long long kWaitBudgetClocks = 4000000000LL;  // ~2 s at 2 GHz
constexpr uint32_t kSuspendHintNs = 20000;              // a waiting thread may sleep this long inside one try_wait
                                                       // (it is woken when the phase completes), so waiters do not
                                                       // burn issue slots the producer warps need

__device__ int g_status = 0;  // 0 ok; otherwise (role << 8 | barrier id) of the first wait that ran out

// ----------------------------------------------------------------------- PTX

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the CTA is aborting (or this wait ran out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int who,
                                          long long budget = kWaitBudgetClocks) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > budget) {
            *abort_flag = 1;
            atomicCAS(&g_status, 0, who);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3FFFF) >> 4);  // start address, 16-byte units
    d |= uint64_t(1) << 16;                     // leading byte offset (unused with swizzle), 16-byte units
    d |= uint64_t(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                     // descriptor version for sm_100
    d |= uint64_t(2) << 61;                     // layout: 128-byte swizzle
    return d;
}

// bf16 x bf16 -> fp32, A and B K-major, M = 128, N = 256
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(kTileD >> 3) << 17) | (uint32_t(kTileQ >> 4) << 24);

// ------------------------------------------------------------------- dequant

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// 4 code bytes -> 4 bf16 values (q - zp) * scale, packed as two bf16x2
__device__ __forceinline__ void dequant_word(uint32_t w, float zmagic, uint32_t scale2, uint32_t& o0, uint32_t& o1) {
    const uint32_t magic = 0x4B000000u;  // 2^23: the byte lands in the low mantissa bits
    const float f0 = __fsub_rn(__uint_as_float(__byte_perm(w, magic, 0x7650)), zmagic);
    const float f1 = __fsub_rn(__uint_as_float(__byte_perm(w, magic, 0x7651)), zmagic);
    const float f2 = __fsub_rn(__uint_as_float(__byte_perm(w, magic, 0x7652)), zmagic);
    const float f3 = __fsub_rn(__uint_as_float(__byte_perm(w, magic, 0x7653)), zmagic);
    // |q - zp| <= 255 has at most 8 significant bits, so the upper half of the fp32
    // pattern IS the bf16 value: pack by byte permute, no conversion instruction
    const uint32_t p0 = __byte_perm(__float_as_uint(f0), __float_as_uint(f1), 0x7632);
    const uint32_t p1 = __byte_perm(__float_as_uint(f2), __float_as_uint(f3), 0x7632);
    o0 = bf16x2_mul(p0, scale2);
    o1 = bf16x2_mul(p1, scale2);
}

struct Params {
    const uint8_t* q;         // [R_q, K]
    const uint16_t* scales;   // [R_q * K / G]
    const uint8_t* zp;        // same, or null: codes are signed int8
    const uint16_t* bias;     // null, or [R_d] (natural layout) / [R_q] (transposed output)
    uint16_t* out;            // natural: [R_q, R_d]; transposed: [R_d, R_q]
    int64_t R_q, R_d, K;
    int64_t gpr;              // groups per row = K / G
    int chunk_vec_ok;         // scales / zero points of a chunk can be fetched with 16-byte loads
    int log2_g;
    int transpose_out;
    int tiles_q, tiles_d;
};

// Scales and zero points reach the producers through a small shared-memory
// buffer that covers 32 groups per row ("a chunk": 512 / 1024 / 2048 values of K for
// G = 16 / 32 / 64).  Thread (row, half) of the 256 producers fetches groups
// [16 * half, 16 * half + 16) of its row into registers one chunk ahead and spills
// them into the other half of the double buffer when the chunk turns over.  Per
// stage the producers then need only two shared-memory reads instead of two
// sector-wasting global loads, which keeps the LSU miss path almost idle.
struct ChunkRegs {
    uint4 s0, s1;  // 16 bf16 scales
    uint4 z;       // 16 zero points
};

__device__ __forceinline__ void chunk_fetch(const Params& p, int64_t grow, int64_t g_first, bool row_ok, ChunkRegs& c) {
    c.s0 = c.s1 = c.z = make_uint4(0, 0, 0, 0);
    if (!row_ok || g_first >= p.gpr) return;
    const int64_t base = grow * p.gpr + g_first;
    if (p.chunk_vec_ok && g_first + 16 <= p.gpr) {
        const uint4* sp = reinterpret_cast<const uint4*>(p.scales + base);
        c.s0 = __ldg(sp);
        c.s1 = __ldg(sp + 1);
        if (p.zp) c.z = __ldg(reinterpret_cast<const uint4*>(p.zp + base));
        return;
    }
    uint32_t sw[8] = {0, 0, 0, 0, 0, 0, 0, 0}, zw[4] = {0, 0, 0, 0};
#pragma unroll
    for (int e = 0; e < 16; ++e)
        if (g_first + e < p.gpr) {
            sw[e >> 1] |= uint32_t(__ldg(p.scales + base + e)) << (16 * (e & 1));
            if (p.zp) zw[e >> 2] |= uint32_t(__ldg(p.zp + base + e)) << (8 * (e & 3));
        }
    c.s0 = make_uint4(sw[0], sw[1], sw[2], sw[3]);
    c.s1 = make_uint4(sw[4], sw[5], sw[6], sw[7]);
    c.z = make_uint4(zw[0], zw[1], zw[2], zw[3]);
}

__device__ __forceinline__ void chunk_spill(uint8_t* sbuf, uint8_t* zbuf, int row, int half, const ChunkRegs& c) {
    uint4* sd = reinterpret_cast<uint4*>(sbuf + row * (kChunkGroups * 2) + half * 32);
    sd[0] = c.s0;
    sd[1] = c.s1;
    *reinterpret_cast<uint4*>(zbuf + row * kChunkGroups + half * 16) = c.z;
}

// One producer thread's share of a stage: row `row` of the tile, codes [32 * half, 32 * half + 32).
// Reads the raw codes the TMA delivered (rows of 64 bytes), dequantises them and writes four
// 16-byte chunks of bf16 into the 128-byte-swizzled A tile.  All addresses are a per-thread base
// (computed once, outside the main loop) plus compile-time offsets; `srow` / `zrow` point at the
// scale / zero point of the thread's first code in the current chunk buffer.
template <int LOG2_G, bool HAS_ZP>
__device__ __forceinline__ void producer_convert(const uint8_t* c_thread, uint8_t* a_row, const uint32_t (&chunk_off)[4],
                                                 const uint16_t* srow, const uint8_t* zrow) {
    const uint4 c0 = *reinterpret_cast<const uint4*>(c_thread);
    const uint4 c1 = *reinterpret_cast<const uint4*>(c_thread + 16);
    uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    constexpr bool kTwoGroups = LOG2_G == 4;  // G = 16: the thread's 32 codes span two groups
    uint32_t sb[2], zv[2];
    sb[0] = srow[0];
    sb[1] = kTwoGroups ? uint32_t(srow[1]) : sb[0];
    if (HAS_ZP) {
        zv[0] = zrow[0];
        zv[1] = kTwoGroups ? uint32_t(zrow[1]) : zv[0];
    } else {  // signed codes: flip the sign bit and subtract 128
#pragma unroll
        for (int i = 0; i < 8; ++i) words[i] ^= 0x80808080u;
        zv[0] = zv[1] = 128;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {  // chunk j of this half: codes 8j .. 8j+7
        const int h = j >> 1;
        const float zmagic = __uint_as_float(0x4B000000u | zv[h]);  // 2^23 + zp, exact
        const uint32_t s2 = __byte_perm(sb[h], sb[h], 0x1010);      // the scale in both halves
        uint4 o;
        dequant_word(words[2 * j], zmagic, s2, o.x, o.y);
        dequant_word(words[2 * j + 1], zmagic, s2, o.z, o.w);
        *reinterpret_cast<uint4*>(a_row + chunk_off[j]) = o;
    }
}

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&b);
}

// -------------------------------------------------------------------- kernel

template <int LOG2_G, bool HAS_ZP>
__global__ void __launch_bounds__(kThreads, 1)
fused_dequant_gemm_kernel(const __grid_constant__ CUtensorMap dense_map, const __grid_constant__ CUtensorMap code_map, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_a = smem;                                   // kStages x 16 KB, dequantised operand
    uint8_t* smem_b = smem + kStages * kStageBytesA;          // kStages x 32 KB, dense operand (TMA)
    uint8_t* smem_c = smem_b + kStages * kStageBytesB;        // kStages x 8 KB, raw codes (TMA)
    uint8_t* smem_s = smem_c + kStages * kStageBytesC;        // 2 x 8 KB, scales of the current / next chunk
    uint8_t* smem_z = smem_s + 2 * kChunkBytesS;              // 2 x 4 KB, zero points
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
    // barrier ids: [0,S) full_b, [S,2S) full_a, [2S,3S) empty, [3S,4S) full_c, 4S+{0,1} tmem_full, 4S+{2,3} tmem_empty,
    // 4S+4 chunk turn-over among the producers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kStages + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int id) { return bar0 + 8u * uint32_t(id); };
    const int FULL_B = 0, FULL_A = kStages, EMPTY = 2 * kStages, FULL_C = 3 * kStages, TFULL = 4 * kStages, TEMPTY = 4 * kStages + 2,
              CHUNK = 4 * kStages + 4;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(FULL_B + s), 1);
            mbar_init(bar(FULL_A + s), kNumProducerWarps * 32);
            mbar_init(bar(EMPTY + s), 1);
            mbar_init(bar(FULL_C + s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar(TFULL + b), 1);
            mbar_init(bar(TEMPTY + b), kNumEpilogueWarps * 32);
        }
        mbar_init(bar(CHUNK), kNumProducerWarps * 32);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = int((p.K + kBlockK - 1) / kBlockK);  // a ragged last K block is zero-filled by the TMA (dense tile and
                                                            // codes) and gets zero scales from the chunk fetch
    const int num_tiles = p.tiles_q * p.tiles_d;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (dense operand and raw codes)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                const int td = tile % p.tiles_d, tq = tile / p.tiles_d;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(bar(EMPTY + s), ph ^ 1, abort_flag, (1 << 8) | (EMPTY + s)))) break;
                    mbar_arrive_expect_tx(bar(FULL_C + s), kStageBytesC);
                    tma_load_2d(smem_u32(smem_c + s * kStageBytesC), &code_map, kb * kBlockK, tq * kTileQ, bar(FULL_C + s));
                    mbar_arrive_expect_tx(bar(FULL_B + s), kStageBytesB);
                    tma_load_2d(smem_u32(smem_b + s * kStageBytesB), &dense_map, kb * kBlockK, td * kTileD, bar(FULL_B + s));
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
                const int buf = local_tile & 1;
                const uint32_t tph = (local_tile >> 1) & 1;
                if (!(ok = mbar_wait(bar(TEMPTY + buf), tph ^ 1, abort_flag, (2 << 8) | (TEMPTY + buf)))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + uint32_t(buf * kTileD);
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(bar(FULL_B + s), ph, abort_flag, (2 << 8) | (FULL_B + s)))) break;
                    if (!(ok = mbar_wait(bar(FULL_A + s), ph, abort_flag, (2 << 8) | (FULL_A + s)))) break;
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem_a + s * kStageBytesA);
                    const uint32_t b_addr = smem_u32(smem_b + s * kStageBytesB);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)
                        umma_bf16(d_tmem, make_smem_desc(a_addr + k * 32), make_smem_desc(b_addr + k * 32), kInstrDesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(bar(EMPTY + s));  // the stage may be refilled once these MMAs have read it
                }
                if (ok) umma_commit(bar(TFULL + buf));  // accumulator complete
            }
        }
    } else if (warp < kFirstEpilogueWarp) {
        // ------------------------------------------------ dequantising producers
        // Per stage: wait for the raw codes (which the TMA thread only requests once the
        // stage's previous MMAs have released it), convert, publish.  Scales and zero
        // points come from the chunk buffer; the registers for the next chunk are
        // fetched one chunk ahead, across tile boundaries too.
        const int pt = threadIdx.x - kFirstProducerWarp * 32;  // 0..255
        const int row = pt >> 1, half = pt & 1;
        constexpr int kLog2Cs = LOG2_G - 1;                    // stages per chunk = 32 * G / 64
        constexpr int kCsMask = (1 << kLog2Cs) - 1;
        const int chunks_per_tile = (num_kb + kCsMask) >> kLog2Cs;
        // per-thread addresses, fixed for the whole kernel
        const uint8_t* c_thread = smem_c + row * kBlockK + half * 32;               // + stage * kStageBytesC
        uint8_t* a_row = smem_a + (row >> 3) * 1024 + (row & 7) * 128;               // + stage * kStageBytesA
        uint32_t chunk_off[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) chunk_off[j] = uint32_t(((half * 4 + j) ^ (row & 7)) * 16);
        // group (inside a chunk) of the thread's first code at stage j of the chunk:
        // G16: 4 j + 2 half, G32: 2 j + half, G64: j
        constexpr int kGroupsPerStage = 64 >> LOG2_G;                                // 4, 2, 1
        const int g_half = LOG2_G == 4 ? 2 * half : (LOG2_G == 5 ? half : 0);
        const uint8_t* s_thread = smem_s + row * (kChunkGroups * 2) + g_half * 2;   // + buf * kChunkBytesS + j * groups * 2
        const uint8_t* z_thread = smem_z + row * kChunkGroups + g_half;             // + buf * kChunkBytesZ + j * groups
        // cursor of the chunk prefetch: (tile, chunk inside the tile)
        int pf_tile = blockIdx.x, pf_chunk = 0;
        ChunkRegs regs;
        auto fetch_next_chunk = [&]() {
            if (pf_tile < num_tiles) {
                const int64_t grow = int64_t(pf_tile / p.tiles_d) * kTileQ + row;
                chunk_fetch(p, grow, int64_t(pf_chunk) * kChunkGroups + half * 16, grow < p.R_q, regs);
            }
            if (++pf_chunk == chunks_per_tile) {
                pf_chunk = 0;
                pf_tile += gridDim.x;
            }
        };
        fetch_next_chunk();
        const int my_tiles = blockIdx.x < num_tiles ? (num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
        const int64_t total = int64_t(my_tiles) * num_kb;
        uint32_t gc = 0;      // chunks published so far
        uint32_t ph = 0;      // parity of the stage ring, flips once per kStages steps
        int kb = 0;           // k-block inside the current tile
        bool ok = true;
        for (int64_t i0 = 0; ok && i0 < total; i0 += kStages, ph ^= 1) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) {  // the stage index is a compile-time constant in here
                if (i0 + s >= total) break;
                const int j = kb & kCsMask;      // stage inside the chunk
                if (j == 0) {
                    // chunk turn-over: publish the prefetched registers, start fetching the next chunk
                    const int nb = gc & 1;
                    chunk_spill(smem_s + nb * kChunkBytesS, smem_z + nb * kChunkBytesZ, row, half, regs);
                    fetch_next_chunk();
                    // every producer must have spilled before anyone reads the new chunk (bounded, like all waits)
                    mbar_arrive(bar(CHUNK));
                    if (!(ok = mbar_wait(bar(CHUNK), gc & 1, abort_flag, (3 << 8) | CHUNK))) break;
                    ++gc;
                }
                const int buf = (gc - 1) & 1;
                if (!(ok = mbar_wait(bar(FULL_C + s), ph, abort_flag, (3 << 8) | (FULL_C + s)))) break;
                producer_convert<LOG2_G, HAS_ZP>(
                    c_thread + s * kStageBytesC, a_row + s * kStageBytesA, chunk_off,
                    reinterpret_cast<const uint16_t*>(s_thread + buf * kChunkBytesS + j * (kGroupsPerStage * 2)),
                    z_thread + buf * kChunkBytesZ + j * kGroupsPerStage);
                fence_proxy_async();  // make the generic-proxy stores visible to the tensor core
                mbar_arrive(bar(FULL_A + s));
                if (++kb == num_kb) kb = 0;
            }
        }
    } else {
        // ------------------------------------------------ epilogue
        const int ew = warp & 3;                 // TMEM lane quadrant this warp may read
        const int r_in_tile = ew * 32 + lane;    // accumulator row = quantised-operand row
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++local_tile) {
            const int tq = tile / p.tiles_d, td = tile % p.tiles_d;
            const int buf = local_tile & 1;
            const uint32_t tph = (local_tile >> 1) & 1;
            if (!(ok = mbar_wait(bar(TFULL + buf), tph, abort_flag, (4 << 8) | (TFULL + buf)))) break;
            tc_fence_after();
            const int64_t rq = int64_t(tq) * kTileQ + r_in_tile;
            const uint32_t taddr0 = tmem_base + (uint32_t(ew * 32) << 16) + uint32_t(buf * kTileD);
            float bias_row = 0.0f;
            if (p.bias && p.transpose_out && rq < p.R_q) bias_row = __uint_as_float(uint32_t(p.bias[rq]) << 16);
#pragma unroll 1
            for (int c = 0; c < kTileD / 32; ++c) {
                uint32_t v[32];
                tmem_ld32(taddr0 + uint32_t(c * 32), v);
                tmem_ld_wait();
                const int64_t rd0 = int64_t(td) * kTileD + c * 32;
                if (p.transpose_out) {
                    // out[r_d, r_q]: for a fixed register the 32 lanes write 32 consecutive r_q
                    if (rq < p.R_q) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (rd0 + i < p.R_d) p.out[(rd0 + i) * p.R_q + rq] = f32_to_bf16_bits(__uint_as_float(v[i]) + bias_row);
                    }
                } else if (rq < p.R_q) {
                    // out[r_q, r_d]: each lane owns 32 consecutive r_d of its row
                    uint16_t* dst = p.out + rq * p.R_d + rd0;
                    if (rd0 + 32 <= p.R_d && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float a = __uint_as_float(v[2 * i]), b = __uint_as_float(v[2 * i + 1]);
                            if (p.bias) {
                                a += __uint_as_float(uint32_t(p.bias[rd0 + 2 * i]) << 16);
                                b += __uint_as_float(uint32_t(p.bias[rd0 + 2 * i + 1]) << 16);
                            }
                            w[i] = uint32_t(f32_to_bf16_bits(a)) | (uint32_t(f32_to_bf16_bits(b)) << 16);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (rd0 + i < p.R_d) {
                                float a = __uint_as_float(v[i]);
                                if (p.bias) a += __uint_as_float(uint32_t(p.bias[rd0 + i]) << 16);
                                dst[i] = f32_to_bf16_bits(a);
                            }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar(TEMPTY + buf));  // this accumulator may be overwritten
        }
    }

    // common exit: normal completion or abort
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// Self-test of the bounded wait: warp 0 waits on a barrier nobody ever arrives on, with a short
// clock budget; warp 1 waits on a second such barrier with the full budget and must be released by
// the abort flag.  The kernel always terminates; the status word records who gave up.
__global__ void bounded_wait_selftest_kernel(long long budget_clocks) {
    __shared__ uint64_t bars[2];
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) {
        if (warp == 0)
            (void)mbar_wait(smem_u32(&bars[0]), 0, abort_flag, (9 << 8) | 0, budget_clocks);
        else
            (void)mbar_wait(smem_u32(&bars[1]), 0, abort_flag, (9 << 8) | 1);
    }
    __syncthreads();
}

// -------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

}  // namespace

extern "C" int tcb_fused_dequant_linear(const uint16_t* dense, const uint8_t* q, const uint16_t* scales, const uint8_t* zp_or_null,
                                        const uint16_t* bias_or_null, uint16_t* out, int64_t R_d, int64_t R_q, int64_t K,
                                        int group_size, int quant_is_rhs, void* stream) {
    const char* who = "tcb_fused_dequant_linear";
    if (R_d < 0 || R_q < 0 || K < 0) return tcb::fail(TCB_ERR_BAD_ARG, "%s: negative size", who);
    if (!tcb::core_group_size_ok(group_size)) return tcb::fail(TCB_ERR_GROUP_SIZE, "%s: group_size %d not in {16, 32, 64}", who, group_size);
    if (R_d == 0 || R_q == 0) return TCB_OK;
    if (K <= 0 || K % group_size != 0)
        return tcb::fail(TCB_ERR_BAD_ARG, "%s: K = %lld must be a positive multiple of the group size %d", who, (long long)K, group_size);
    if (!dense || !q || !scales || !out) return tcb::fail(TCB_ERR_BAD_ARG, "%s: null pointer", who);
    if ((reinterpret_cast<uintptr_t>(dense) | reinterpret_cast<uintptr_t>(q)) & 15)
        return tcb::fail(TCB_ERR_ALIGNMENT, "%s: dense and q must be 16-byte aligned", who);
    if ((reinterpret_cast<uintptr_t>(scales) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias_or_null)) & 1)
        return tcb::fail(TCB_ERR_ALIGNMENT, "%s: scales, bias and out must be 2-byte aligned", who);
    if (R_d > (int64_t(1) << 31) - 1 || R_q > (int64_t(1) << 31) - 1 || K > (int64_t(1) << 31) - 1)
        return tcb::fail(TCB_ERR_TOO_LARGE, "%s: dimension beyond 2^31 - 1", who);
    const int64_t tiles_q = (R_q + kTileQ - 1) / kTileQ, tiles_d = (R_d + kTileD - 1) / kTileD;
    if (tiles_q * tiles_d > (int64_t(1) << 30)) return tcb::fail(TCB_ERR_TOO_LARGE, "%s: too many output tiles", who);

    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
    CUtensorMap map;
    const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(R_d)};
    const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
    const cuuint32_t box[2] = {cuuint32_t(kBlockK), cuuint32_t(kTileD)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(dense), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with %d", who, int(cr));
    // raw codes: [R_q, K] bytes, 64-byte rows in shared memory, no swizzle (read by the producer warps)
    CUtensorMap cmap;
    const cuuint64_t cdims[2] = {cuuint64_t(K), cuuint64_t(R_q)};
    const cuuint64_t cstrides[1] = {cuuint64_t(K)};
    const cuuint32_t cbox[2] = {cuuint32_t(kBlockK), cuuint32_t(kTileQ)};
    cr = encode(&cmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(q), cdims, cstrides, cbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled (codes) failed with %d", who, int(cr));

    // one instantiation per (group size, zero points or not): those are compile-time in the producer warps
    typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const Params);
    static const KernelFn kernels[3][2] = {
        {fused_dequant_gemm_kernel<4, false>, fused_dequant_gemm_kernel<4, true>},
        {fused_dequant_gemm_kernel<5, false>, fused_dequant_gemm_kernel<5, true>},
        {fused_dequant_gemm_kernel<6, false>, fused_dequant_gemm_kernel<6, true>}};
    const int gi = group_size == 16 ? 0 : group_size == 32 ? 1 : 2;
    const KernelFn kernel = kernels[gi][zp_or_null ? 1 : 0];
    static bool attr_set[64][3][2] = {};
    int dev = 0;
    TCB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev][gi][zp_or_null ? 1 : 0]) {
        TCB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
        attr_set[dev][gi][zp_or_null ? 1 : 0] = true;
    }
    Params p;
    p.q = q;
    p.scales = scales;
    p.zp = zp_or_null;
    p.bias = bias_or_null;
    p.out = out;
    p.R_q = R_q;
    p.R_d = R_d;
    p.K = K;
    p.log2_g = group_size == 16 ? 4 : group_size == 32 ? 5 : 6;
    p.gpr = K / group_size;
    p.chunk_vec_ok = p.gpr % 16 == 0 && (reinterpret_cast<uintptr_t>(scales) & 15) == 0 &&
                     (zp_or_null == nullptr || (reinterpret_cast<uintptr_t>(zp_or_null) & 15) == 0);
    p.transpose_out = quant_is_rhs ? 1 : 0;
    p.tiles_q = int(tiles_q);
    p.tiles_d = int(tiles_d);
    const int64_t num_tiles = tiles_q * tiles_d;
    const int sms = tcb::sm_count();
    const int grid = int(num_tiles < sms ? num_tiles : sms);
    kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(map, cmap, p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TCB_OK : tcb::cuda_fail(e, who);
}

extern "C" int tcb_selftest_bounded_wait(int budget_ms, void* stream) {
    if (budget_ms < 1 || budget_ms > 1000) return tcb::fail(TCB_ERR_BAD_ARG, "tcb_selftest_bounded_wait: budget %d ms outside 1..1000", budget_ms);
    int dev = 0, khz = 0;
    TCB_CUDA_TRY(cudaGetDevice(&dev));
    TCB_CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<long long>(khz) * budget_ms);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TCB_OK : tcb::cuda_fail(e, "tcb_selftest_bounded_wait");
}

extern "C" int tcb_fused_dequant_linear_check(void* stream) {
    TCB_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    int status = 0;
    TCB_CUDA_TRY(cudaMemcpyFromSymbol(&status, g_status, sizeof(int)));
    if (status == 0) return TCB_OK;
    const int zero = 0;
    TCB_CUDA_TRY(cudaMemcpyToSymbol(g_status, &zero, sizeof(int)));
    return tcb::fail(TCB_ERR_TIMEOUT, "tcb_fused_dequant_linear: a bounded wait ran out (role %d, barrier %d)", status >> 8, status & 0xff);
}
