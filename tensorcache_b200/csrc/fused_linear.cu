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
// The kernel runs as pairs of CTAs (a cluster of two, one CTA per SM of a TPC) that
// issue tcgen05.mma.cta_group::2.  A pair owns an output tile of 256 rows of the
// quantised operand x 512 rows of the dense one; K advances 64 at a time through a
// 3-stage ring.  Each CTA dequantises 128 rows of q and loads 256 dense rows per stage;
// per K step the leader issues two groups of four MMAs (M 256, N 256, K 16), one group
// per half of the CTAs' dense rows, into the two 256-column accumulators that fill
// the 512 TMEM columns.
//
// Why this shape.  What bounds a kernel of this kind is the shared-memory data pipe of
// the SM (one 128-byte wavefront per clock): it serves the tensor core's operand reads,
// the TMA's writes and the producers' loads and stores.  A single-CTA 128 x 256 tile
// needs about 1150 wavefronts per 512 clocks of MMA work, a pair on a 256 x 256 tile
// 730 (the tensor cores of the two SMs exchange the halves of the N-side operand, so
// each CTA stages half of it), and this tile 1110 per 1024 clocks: every dequantised
// tile, the expensive one to make, is used against twice as many dense rows.  The price
// is that both accumulators belong to one tile, so the epilogue no longer overlaps the
// next tile's MMAs; the eight epilogue warps hand the accumulators back as soon as they
// have read them.  Tiles that would make up a last, less than half full round of the CTA
// pairs (and an odd last 256-row unit of the dense operand) run as 256 x 256 tiles on one
// accumulator instead, side by side on twice as many pairs.
//
// Which operand is the M side depends on the wanted output layout, so that every
// epilogue store is a row-contiguous vector store:
//     quant_is_rhs (out = dense . deq(q)^T, [R_d, R_q]):  A = dense, B = dequantised
//     otherwise    (out = deq(q) . dense^T, [R_q, R_d]):  A = dequantised, B = dense
// The per-CTA work is the same in both cases.
//
// Warp roles, per CTA:
//   warp 0      TMA producer (one thread): raw code tile [128 x 64] uint8 into the CTA's
//               own barrier, dense tile [256 x 64] bf16 (128-byte swizzle) into the
//               leader CTA's barrier (cp.async.bulk.tensor with cta_group::2, no multicast)
//   warp 1      leader CTA only, one thread: per stage ONE barrier wait (dense rows of both
//               CTAs landed + all 16 producer warps of the pair done), 8 x tcgen05.mma and
//               ONE tcgen05.commit that arrives on the stage barrier of both CTAs; after the
//               last K step one more on both accumulator barriers.  This thread's serial
//               latency per stage is on the critical path, hence the merged barrier and the
//               single commit.  In both CTAs this warp owns the TMEM allocation.
//   warps 2-9   dequantising producers: 16 rows per warp.  A warp instruction reads 512
//               contiguous bytes of codes and writes 16-byte pieces that cover all 32
//               banks per quarter warp, so neither side has bank conflicts.  Scales and
//               zero points sit merged (scale << 16 | zp) in a per-warp shared-memory
//               table of 32 groups per row that the warp refills itself one table ahead
//               (global -> registers -> table), so a turn-over needs only a warp sync.
//   warps 10-17 epilogue, one per TMEM lane quadrant and accumulator:
//               tcgen05.ld -> (+bias) -> bf16 -> global (32-byte stores)
// No TMA multicast anywhere.
//
// The dequantised value is bf16((q - zp) * scale), the number the decode kernel produces:
// the code byte is spliced into the mantissa of 2^15, one FMA with the exact constant
// -(2^15 + zp) * scale yields (q - zp) * scale exactly in fp32 (16 x 8 significant
// bits), and cvt.rn.bf16x2.f32 rounds two of them once.
//
// Every wait on an mbarrier is bounded by a clock budget.  When one runs out the
// thread raises the abort flag of both CTAs of the pair and a device status word; all
// roles leave their loops, the pair synchronises, frees its TMEM and returns.  Nothing
// in the kernel blocks without such a bound (in particular no setmaxnreg, whose .inc
// form waits for registers another warp group has to give up).
#include <atomic>
#include <type_traits>

#include <cuda.h>
#include <cuda_bf16.h>

#include "tcb_common.h"

namespace {

constexpr int kTileRows = 128;   // rows of each operand per CTA and tile
constexpr int kPairRows = 256;   // rows of each operand per CTA pair and tile (MMA M = N = 256)
constexpr int kBlockK = 64;      // K per stage: 64 bf16 = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr int kDenseRows = 256;  // dense rows per CTA and tile: two MMA groups of 128
constexpr int kNumProducerWarps = 8;
constexpr int kNumEpilogueWarps = 8;
constexpr int kThreads = 32 * (2 + kNumProducerWarps + kNumEpilogueWarps);  // 576
constexpr int kFirstProducerWarp = 2;
constexpr int kFirstEpilogueWarp = 2 + kNumProducerWarps;                   // 10
constexpr uint32_t kStageBytesQ = kTileRows * kBlockK * 2;                   // 16 KB dequantised operand
constexpr uint32_t kStageBytesD = kDenseRows * kBlockK * 2;                  // 32 KB dense operand
constexpr uint32_t kStageBytesC = kTileRows * kBlockK;                       // 8 KB of raw codes
constexpr int kTableGroups = 32;                                             // groups per row in the scale table
constexpr uint32_t kTableRowBytes = kTableGroups * 4 + 16;                   // 144: the pad spreads 8 rows over all banks
constexpr uint32_t kTableBytes = kTileRows * kTableRowBytes;                 // 18 KB
constexpr uint32_t kSmemTiles = kStages * (kStageBytesQ + kStageBytesD + kStageBytesC) + kTableBytes;
constexpr uint32_t kSmemBytes = kSmemTiles + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr long long kWaitBudgetClocks = 2000000000LL;  // ~1 s at 2 GHz

__device__ int g_status = 0;  // 0 ok; otherwise (role << 8 | barrier id) of the first wait that ran out

// ----------------------------------------------------------------------- PTX

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Arrival on a barrier that may live in the other CTA of the pair (shared::cluster address).  The plain form: with
// .release.cluster on every arrival the arriving warp stalled for about a thousand clocks per stage.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll of a barrier phase.  Cluster-scope acquire: most of these barriers take arrivals from the other CTA of
// the pair or from MMAs both CTAs take part in.  No suspend-time hint: it made no difference here.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the CTA pair is aborting (or this wait ran out).  `abort_peer` is the
// shared::cluster address of the other CTA's abort flag (0: no pair).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t abort_peer, int who,
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
            if (abort_peer) st_cluster_u32(abort_peer, 1u);
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
// Load into this CTA's shared memory that signals a barrier of either CTA of the pair
// (`cluster_bar` is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            dst),
        "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The four MMAs (K = 16 each) of one 64-wide K step on one accumulator, issued back to back from one asm block: the
// descriptors advance by 32 bytes (2 in their 16-byte address field) per MMA, only the first one may overwrite the
// accumulator.  hi words of the descriptors are the same for every operand tile of this kernel.
__device__ __forceinline__ void umma_bf16_pair_x4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                                  uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, t;\n\t.reg .b64 a, b;\n\t.reg .b32 al, bl;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.eq.b32 t, %5, %5;\n\t"
        "mov.b64 a, {%1, %3};\n\tmov.b64 b, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %4, p;\n\t"
        "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 a, {al, %3};\n\tmov.b64 b, {bl, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %4, t;\n\t"
        "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 a, {al, %3};\n\tmov.b64 b, {bl, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %4, t;\n\t"
        "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 a, {al, %3};\n\tmov.b64 b, {bl, %3};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %4, t;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate_first)
        : "memory");
}
// Arrival on the barrier at offset `bar` of BOTH CTAs of the pair once every MMA this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(uint16_t(3))
                 : "memory");
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

__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

// Shared-memory operand descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes apart.
// Low word: start address in 16-byte units (14 bits) and the (unused) leading byte offset 1 at bit 16; high word: stride
// byte offset 1024 >> 4, descriptor version 1 (bit 46 of the 64), layout type 2 = 128-byte swizzle (bits 61..63).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16); }

// bf16 x bf16 -> fp32, A and B K-major, M = 256 (128 rows per CTA of the pair), N = 256
constexpr uint32_t kInstrDesc =
    (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(kPairRows >> 3) << 17) | (uint32_t(kPairRows >> 4) << 24);

// ------------------------------------------------------------------- dequant

struct Params {
    const uint8_t* q;         // [R_q, K]
    const uint16_t* scales;   // [R_q * K / G]
    const uint8_t* zp;        // same, or null: codes are signed int8
    const uint16_t* bias;     // null, or one entry per output column
    uint16_t* out;            // [rows of the A operand, rows of the B operand]
    int64_t R_q, R_d, K;
    int64_t gpr;              // groups per row = K / G
    int table_vec_ok;         // scales / zero points of a table can be fetched with 16-byte loads
    int quant_is_a;           // the dequantised operand is the M side (output rows); otherwise the dense one is
    // Tile list of a launch.  Dense rows are counted in units of 256.  Tiles [0, n_wide) are wide (256 x 512: dense units
    // 2j, 2j + 1); the next 2 n_conv tiles are the halves (256 x 256) of the wide tiles that would have made up a last,
    // less than half full round of the CTA pairs; if the number of dense units is odd, one half tile per row of tiles
    // covers the last unit.
    int tiles_q;              // 256-row tiles along the quantised operand
    int units_d;              // 256-row units along the dense operand
    int wide_cols;            // units_d / 2
    int n_wide, n_conv, n_odd;
    int num_tiles;            // n_wide + 2 n_conv + n_odd
};

// Scales and zero points reach the producers through a shared-memory table that covers
// 32 groups per row (512 / 1024 / 2048 values of K for G = 16 / 32 / 64), one 32-bit word
// (scale << 16 | zp) per group.  Each producer warp owns the 16 rows it converts: lane
// (row = lane / 2, half = lane % 2) fetches groups [16 * half, 16 * half + 16) of its row
// into registers one table ahead and writes them out when the table turns over.
struct TableRegs {
    uint4 s0, s1;  // 16 bf16 scales
    uint4 z;       // 16 zero points
};

__device__ __forceinline__ void table_fetch(const Params& p, int64_t grow, int64_t g_first, bool row_ok, TableRegs& c) {
    c.s0 = c.s1 = c.z = make_uint4(0, 0, 0, 0);
    if (!row_ok || g_first >= p.gpr) return;
    const int64_t base = grow * p.gpr + g_first;
    if (p.table_vec_ok && g_first + 16 <= p.gpr) {
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

// Writes the 16 (scale, zero point) pairs a lane holds as 16 merged words: bytes 3..2 = scale, byte 0 = zp.
__device__ __forceinline__ void table_spill(uint8_t* dst, const TableRegs& c) {
    const uint32_t sw[8] = {c.s0.x, c.s0.y, c.s0.z, c.s0.w, c.s1.x, c.s1.y, c.s1.z, c.s1.w};
    const uint32_t zw[4] = {c.z.x, c.z.y, c.z.z, c.z.w};
    uint32_t m[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        // selector nibbles, low to high: zp byte (e & 3) of zw, the same again, scale bytes (2 (e & 1), 2 (e & 1) + 1) of sw
        const uint32_t zsel = 4 + (e & 3), ssel = 2 * (e & 1);
        m[e] = __byte_perm(sw[e >> 1], zw[e >> 2], zsel | (zsel << 4) | (ssel << 8) | ((ssel + 1) << 12));
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) reinterpret_cast<uint4*>(dst)[v] = make_uint4(m[4 * v], m[4 * v + 1], m[4 * v + 2], m[4 * v + 3]);
}

// 16 codes of one row -> 16 bf16 values, written as two 16-byte pieces of the 128-byte-swizzled operand row.
// Per code: one byte permute (the byte into the mantissa of 2^15), one FMA, half a cvt.rn.bf16x2.f32.
template <bool HAS_ZP>
__device__ __forceinline__ void convert16(uint4 c, uint32_t sz_word, uint8_t* piece0, uint8_t* piece1) {
    uint32_t w[4] = {c.x, c.y, c.z, c.w};
    const float scale = __uint_as_float(sz_word & 0xFFFF0000u);
    float base;
    if (HAS_ZP) {
        base = __uint_as_float(__byte_perm(sz_word, 0x47000000u, 0x7604));
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) w[i] ^= 0x80808080u;
        base = __uint_as_float(0x47008000u);
    }
    const float cc = -__fmul_rn(base, scale);
    const uint32_t magic = 0x47000000u;
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float f0 = __fmaf_rn(__uint_as_float(__byte_perm(w[i], magic, 0x7604)), scale, cc);
        const float f1 = __fmaf_rn(__uint_as_float(__byte_perm(w[i], magic, 0x7614)), scale, cc);
        const float f2 = __fmaf_rn(__uint_as_float(__byte_perm(w[i], magic, 0x7624)), scale, cc);
        const float f3 = __fmaf_rn(__uint_as_float(__byte_perm(w[i], magic, 0x7634)), scale, cc);
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[2 * i]) : "f"(f1), "f"(f0));
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[2 * i + 1]) : "f"(f3), "f"(f2));
    }
    *reinterpret_cast<uint4*>(piece0) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(piece1) = make_uint4(o[4], o[5], o[6], o[7]);
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    __nv_bfloat16 b = __float2bfloat16_rn(v);
    return *reinterpret_cast<uint16_t*>(&b);
}

struct Tile {
    int tq;       // tile row along the quantised operand
    int d_unit;   // first 256-row unit of the dense operand
    int half;     // 1: a 256 x 256 tile (one accumulator, 128 dense rows per CTA)
};

__device__ __forceinline__ Tile decode_tile(const Params& p, int t) {
    Tile r;
    if (t < p.n_wide) {
        r.half = 0;
        r.tq = t / p.wide_cols;
        r.d_unit = 2 * (t % p.wide_cols);
    } else if (t < p.n_wide + 2 * p.n_conv) {
        const int u = t - p.n_wide, w = p.n_wide + (u >> 1);
        r.half = 1;
        r.tq = w / p.wide_cols;
        r.d_unit = 2 * (w % p.wide_cols) + (u & 1);
    } else {
        r.half = 1;
        r.tq = t - p.n_wide - 2 * p.n_conv;
        r.d_unit = p.units_d - 1;
    }
    return r;
}

// -------------------------------------------------------------------- kernel

template <int LOG2_G, bool HAS_ZP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fused_dequant_gemm_kernel(const __grid_constant__ CUtensorMap dense_map, const __grid_constant__ CUtensorMap dense_map_half,
                          const __grid_constant__ CUtensorMap code_map, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                                   // kStages x 16 KB, dequantised operand
    uint8_t* smem_d = smem + kStages * kStageBytesQ;          // kStages x 16 KB, dense operand (TMA)
    uint8_t* smem_c = smem_d + kStages * kStageBytesD;        // kStages x 8 KB, raw codes (TMA)
    uint8_t* smem_t = smem_c + kStages * kStageBytesC;        // 18 KB, scale / zero point tables of the 8 producer warps
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
    // barrier ids: [0,S) full, [S,2S) empty, [2S,3S) full_c, 3S+{0,1} tmem_full, 3S+{2,3} tmem_empty.
    // full and tmem_empty are used in the leader CTA only (the other CTA arrives on them remotely).
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kStages + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();   // 0: leader (issues the MMAs)
    const bool leader = rank == 0;
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int id) { return bar0 + 8u * uint32_t(id); };
    auto leader_bar = [&](int id) { return map_to_cta(bar(id), 0); };
    const uint32_t abort_peer = map_to_cta(smem_u32(const_cast<int*>(abort_flag)), rank ^ 1);
    const int FULL = 0, EMPTY = kStages, FULL_C = 2 * kStages, TFULL = 3 * kStages, TEMPTY = 3 * kStages + 1;

    // both CTAs of the pair are resident before either touches the other's shared or tensor memory
    cluster_sync_all();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar(FULL + s), 2 + 2 * kNumProducerWarps);
            mbar_init(bar(EMPTY + s), 1);
            mbar_init(bar(FULL_C + s), 1);
        }
        mbar_init(bar(TFULL), 1);
        mbar_init(bar(TEMPTY), 2 * kNumEpilogueWarps * 32);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(tmem_slot), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_kb = int((p.K + kBlockK - 1) / kBlockK);  // a ragged last K block is zero-filled by the TMA (dense tile and
                                                            // codes) and gets zero scales from the table fetch
    const int num_tiles = p.num_tiles;
    const int first_tile = int(blockIdx.x >> 1), tile_step = int(gridDim.x >> 1);

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (dense operand and raw codes)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
                const Tile t = decode_tile(p, tile);
                const int q_row = t.tq * kPairRows + int(rank) * kTileRows;
                const int d_row = t.d_unit * kPairRows + int(rank) * (t.half ? kTileRows : kDenseRows);
                const CUtensorMap* dmap = t.half ? &dense_map_half : &dense_map;
                const uint32_t d_bytes = t.half ? kStageBytesD / 2 : kStageBytesD;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(bar(EMPTY + s), ph ^ 1, abort_flag, abort_peer, (1 << 8) | (EMPTY + s));
                    if (!ok) break;
                    mbar_arrive_expect_tx(bar(FULL_C + s), kStageBytesC);
                    tma_load_2d(smem_u32(smem_c + s * kStageBytesC), &code_map, kb * kBlockK, q_row, bar(FULL_C + s));
                    const uint32_t fd = leader_bar(FULL + s);
                    tma_load_2d_pair(smem_u32(smem_d + s * kStageBytesD), dmap, kb * kBlockK, d_row, fd);
                    if (leader)
                        mbar_arrive_expect_tx(bar(FULL + s), 2 * d_bytes);
                    else
                        mbar_arrive_cluster(fd);
                    if (++s == kStages) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            int s = 0;
            uint32_t ph = 0, local_tile = 0;
            bool ok = true;
            for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++local_tile) {
                // both accumulators (TMEM columns [0,256) and [256,512)) belong to this tile: wait until the epilogue has
                // moved the previous tile out
                ok = mbar_wait(bar(TEMPTY), (local_tile & 1) ^ 1, abort_flag, abort_peer, (2 << 8) | TEMPTY);
                if (!ok) break;
                tc_fence_after();
                // the K loop, once per tile kind, so that the issue sequence of a stage has no branch in it
                const uint32_t q_lo0 = smem_desc_lo(smem_u32(smem_q)), d_lo0 = smem_desc_lo(smem_u32(smem_d));
                auto k_loop = [&](auto groups_tag, auto quant_is_a_tag) {
                    constexpr int kGroups = decltype(groups_tag)::value;   // MMA groups per stage: 2 (wide tile) or 1
                    constexpr bool kQuantIsA = decltype(quant_is_a_tag)::value;
                    for (int kb = 0; kb < num_kb; ++kb) {
                        ok = mbar_wait(bar(FULL + s), ph, abort_flag, abort_peer, (2 << 8) | (FULL + s));
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t q_lo = q_lo0 + uint32_t(s) * (kStageBytesQ >> 4);
                        const uint32_t d_lo = d_lo0 + uint32_t(s) * (kStageBytesD >> 4);
#pragma unroll
                        for (int h = 0; h < kGroups; ++h) {   // dense rows [128 h, 128 h + 128) of each CTA -> accumulator h
                            const uint32_t dh = d_lo + uint32_t(h) * ((128u * kBlockK * 2u) >> 4);
                            umma_bf16_pair_x4(tmem_base + uint32_t(h * kPairRows), kQuantIsA ? q_lo : dh, kQuantIsA ? dh : q_lo, kDescHi,
                                              kInstrDesc, kb > 0 ? 1u : 0u);
                        }
                        // the stage may be refilled, in both CTAs, once these MMAs have read it
                        umma_commit_both(bar(EMPTY + s));
                        if (++s == kStages) { s = 0; ph ^= 1; }
                    }
                };
                const bool half = decode_tile(p, tile).half != 0;
                if (p.quant_is_a) {
                    if (half) k_loop(std::integral_constant<int, 1>(), std::true_type());
                    else k_loop(std::integral_constant<int, 2>(), std::true_type());
                } else {
                    if (half) k_loop(std::integral_constant<int, 1>(), std::false_type());
                    else k_loop(std::integral_constant<int, 2>(), std::false_type());
                }
                if (ok) umma_commit_both(bar(TFULL));  // accumulators complete: each CTA's epilogue reads its own 128 lanes
            }
        }
    } else if (warp < kFirstEpilogueWarp) {
        // ------------------------------------------------ dequantising producers
        // Per stage: wait for the raw codes (which the TMA thread only requests once the stage's
        // previous MMAs have released it), convert, publish to the leader's barrier.
        const int pw = warp - kFirstProducerWarp;              // 0..7: rows [16 pw, 16 pw + 16) of the CTA's tile
        constexpr int kLog2Ts = LOG2_G - 1;                    // stages per table = 32 * G / 64
        constexpr int kTsMask = (1 << kLog2Ts) - 1;
        constexpr int kGroupsPerStage = LOG2_G <= 6 ? (64 >> LOG2_G) : 1;   // 4, 2, 1; G = 128: one group per TWO stages
        constexpr int kStagesPerGroupLog2 = LOG2_G <= 6 ? 0 : LOG2_G - 6;
        const int tables_per_tile = (num_kb + kTsMask) >> kLog2Ts;
        // conversion role of this lane: 16 codes at quarter kq of rows ra and ra + 8
        const int ra = pw * 16 + (lane >> 2), kq = lane & 3;
        const uint8_t* c_lane = smem_c + ra * kBlockK + kq * 16;                        // + stage * kStageBytesC; second row: + 512
        uint8_t* q_row = smem_q + (ra >> 3) * 1024 + (ra & 7) * 128;                    // + stage * kStageBytesQ; second row: + 1024
        const uint32_t piece0 = uint32_t(((2 * kq) ^ (ra & 7)) * 16), piece1 = piece0 ^ 16u;
        const int g_sel = LOG2_G == 4 ? kq : (LOG2_G == 5 ? (kq >> 1) : 0);             // group of the lane's codes inside a stage
        const uint8_t* t_lane = smem_t + ra * kTableRowBytes + g_sel * 4;               // + 4 * groups per stage * stage in table
        // fetch role of this lane: row fr, groups [16 fh, 16 fh + 16) of the table
        const int fr = pw * 16 + (lane >> 1), fh = lane & 1;
        uint8_t* t_spill = smem_t + fr * kTableRowBytes + fh * 64;
        int pf_tile = first_tile, pf_table = 0;
        TableRegs regs;
        auto fetch_next_table = [&]() {
            if (pf_tile < num_tiles) {
                const int64_t grow = int64_t(decode_tile(p, pf_tile).tq) * kPairRows + int64_t(rank) * kTileRows + fr;
                table_fetch(p, grow, int64_t(pf_table) * kTableGroups + fh * 16, grow < p.R_q, regs);
            }
            if (++pf_table == tables_per_tile) {
                pf_table = 0;
                pf_tile += tile_step;
            }
        };
        fetch_next_table();
        const int my_tiles = first_tile < num_tiles ? (num_tiles - 1 - first_tile) / tile_step + 1 : 0;
        const int64_t total = int64_t(my_tiles) * num_kb;
        uint32_t ph = 0;      // parity of the stage ring, flips once per kStages steps
        int kb = 0;           // k-block inside the current tile
        bool ok = true;
        for (int64_t i0 = 0; ok && i0 < total; i0 += kStages, ph ^= 1) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) {  // the stage index is a compile-time constant in here
                if (i0 + s >= total) break;
                const int j = kb & kTsMask;      // stage inside the table
                if (j == 0) {
                    // table turn-over, inside the warp: everybody has read the old words, write the prefetched
                    // ones, start fetching the next table
                    __syncwarp();
                    table_spill(t_spill, regs);
                    fetch_next_table();
                    __syncwarp();
                }
                const int t_word = (j >> kStagesPerGroupLog2) * (kGroupsPerStage * 4);   // byte offset of the stage's first group
                const uint32_t sz_a = *reinterpret_cast<const uint32_t*>(t_lane + t_word);
                const uint32_t sz_b = *reinterpret_cast<const uint32_t*>(t_lane + 8 * kTableRowBytes + t_word);
                // the verdict of the wait is made warp-uniform: the warp-level syncs below need every lane
                ok = __all_sync(0xffffffffu, mbar_wait(bar(FULL_C + s), ph, abort_flag, abort_peer, (3 << 8) | (FULL_C + s)));
                if (!ok) break;
                const uint4 ca = *reinterpret_cast<const uint4*>(c_lane + s * kStageBytesC);
                const uint4 cb = *reinterpret_cast<const uint4*>(c_lane + s * kStageBytesC + 8 * kBlockK);
                uint8_t* qa = q_row + s * kStageBytesQ;
                convert16<HAS_ZP>(ca, sz_a, qa + piece0, qa + piece1);
                convert16<HAS_ZP>(cb, sz_b, qa + 1024 + piece0, qa + 1024 + piece1);
                fence_proxy_async();  // make this lane's generic-proxy stores visible to the tensor cores
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_bar(FULL + s));
                if (++kb == num_kb) kb = 0;
            }
        }
    } else {
        // ------------------------------------------------ epilogue
        // Accumulator h (TMEM columns [256 h, 256 h + 256)) holds, per CTA, 128 rows of the A operand against 256 rows of the
        // B operand.  Dense rows of a tile are split as CTA r: [256 r, 256 r + 256), of which MMA group h took [128 h, +128).
        const int ew = warp & 3;                 // TMEM lane quadrant this warp may read
        const int r_in_tile = ew * 32 + lane;
        const int64_t rows_a = p.quant_is_a ? p.R_q : p.R_d, rows_b = p.quant_is_a ? p.R_d : p.R_q;
        const bool out_vec = (rows_b % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 31) == 0) &&
                             ((reinterpret_cast<uintptr_t>(p.bias) & 3) == 0);
        uint32_t local_tile = 0;
        bool ok = true;
        for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++local_tile) {
            const Tile t = decode_tile(p, tile);
            // warp-uniform verdict: tcgen05.ld is a warp-wide instruction
            ok = __all_sync(0xffffffffu, mbar_wait(bar(TFULL), local_tile & 1, abort_flag, abort_peer, (4 << 8) | TFULL));
            if (!ok) break;
            tc_fence_after();
            {
                const int h = (warp - kFirstEpilogueWarp) >> 2;   // one warp per lane quadrant and accumulator
                // output row of this lane and first output column of accumulator column 0 / 128
                int64_t row, col_lo, col_hi;
                const int dense_per_cta = t.half ? kTileRows : kDenseRows;
                if (p.quant_is_a) {
                    row = int64_t(t.tq) * kPairRows + int64_t(rank) * kTileRows + r_in_tile;
                    col_lo = int64_t(t.d_unit) * kPairRows + 128 * h;      // B rows held by CTA 0
                    col_hi = col_lo + dense_per_cta;                        // B rows held by CTA 1
                } else {
                    row = int64_t(t.d_unit) * kPairRows + int64_t(rank) * dense_per_cta + 128 * h + r_in_tile;
                    col_lo = int64_t(t.tq) * kPairRows;
                    col_hi = col_lo + kTileRows;
                }
                const uint32_t taddr0 = tmem_base + (uint32_t(ew * 32) << 16) + uint32_t(h * kPairRows);
#pragma unroll 1
                for (int c = 0; c < kPairRows / 32; ++c) {
                    const int64_t col0 = (c < 4 ? col_lo : col_hi) + (c & 3) * 32;
                    if (col0 >= rows_b || h >= (t.half ? 1 : 2)) continue;   // warp-uniform: outside the output, or an unused accumulator
                    uint32_t v[32];
                    tmem_ld32(taddr0 + uint32_t(c * 32), v);
                    tmem_ld_wait();
                    if (row < rows_a) {
                        uint16_t* dst = p.out + row * rows_b + col0;
                        if (out_vec && col0 + 32 <= rows_b) {
#pragma unroll
                            for (int hh = 0; hh < 2; ++hh) {
                                uint32_t w[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) {
                                    float a = __uint_as_float(v[16 * hh + 2 * i]), b = __uint_as_float(v[16 * hh + 2 * i + 1]);
                                    if (p.bias) {
                                        const uint32_t bb = __ldg(reinterpret_cast<const uint32_t*>(p.bias + col0) + 8 * hh + i);
                                        a += __uint_as_float(bb << 16);
                                        b += __uint_as_float(bb & 0xFFFF0000u);
                                    }
                                    w[i] = pack_bf16(a, b);
                                }
                                st_global_v8(dst + 16 * hh, w);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (col0 + i < rows_b) {
                                    float a = __uint_as_float(v[i]);
                                    if (p.bias) a += __uint_as_float(uint32_t(p.bias[col0 + i]) << 16);
                                    dst[i] = f32_to_bf16_bits(a);
                                }
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(leader_bar(TEMPTY));  // the accumulators may be overwritten
        }
    }

    // common exit: normal completion or abort.  Neither CTA leaves while the other may still arrive on its
    // barriers or have its shared memory read by an MMA.
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
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
            (void)mbar_wait(smem_u32(&bars[0]), 0, abort_flag, 0u, (9 << 8) | 0, budget_clocks);
        else
            (void)mbar_wait(smem_u32(&bars[1]), 0, abort_flag, 0u, (9 << 8) | 1);
    }
    __syncthreads();
}

// -------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(sym);
            cached.store(fn, std::memory_order_release);
        }
    }
    return fn;
}

}  // namespace

extern "C" int tcb_fused_dequant_linear(const uint16_t* dense, const uint8_t* q, const uint16_t* scales, const uint8_t* zp_or_null,
                                        const uint16_t* bias_or_null, uint16_t* out, int64_t R_d, int64_t R_q, int64_t K,
                                        int group_size, int quant_is_rhs, void* stream) {
    const char* who = "tcb_fused_dequant_linear";
    if (R_d < 0 || R_q < 0 || K < 0) return tcb::fail(TCB_ERR_BAD_ARG, "%s: negative size", who);
    if (!tcb::core_group_size_ok(group_size) && group_size != 128)
        return tcb::fail(TCB_ERR_GROUP_SIZE, "%s: group_size %d not in {16, 32, 64, 128}", who, group_size);
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
    const int64_t tiles_q = (R_q + kPairRows - 1) / kPairRows, units_d = (R_d + kPairRows - 1) / kPairRows;
    if (tiles_q * units_d > (int64_t(1) << 30)) return tcb::fail(TCB_ERR_TOO_LARGE, "%s: too many output tiles", who);

    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
    // dense operand: [R_d, K] bf16, one box = the 256 rows x 64 columns a CTA stages per K step of a wide tile
    // (a second map with 128-row boxes serves the 256 x 256 tiles)
    CUtensorMap map, map_half;
    const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(R_d)};
    const cuuint64_t strides[1] = {cuuint64_t(K) * 2};
    const cuuint32_t box[2] = {cuuint32_t(kBlockK), cuuint32_t(kDenseRows)};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(dense), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with %d", who, int(cr));
    const cuuint32_t box_half[2] = {cuuint32_t(kBlockK), cuuint32_t(kTileRows)};
    cr = encode(&map_half, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(dense), dims, strides, box_half, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled (half tiles) failed with %d", who, int(cr));
    // raw codes: [R_q, K] bytes, 64-byte rows in shared memory, no swizzle (read by the producer warps)
    CUtensorMap cmap;
    const cuuint64_t cdims[2] = {cuuint64_t(K), cuuint64_t(R_q)};
    const cuuint64_t cstrides[1] = {cuuint64_t(K)};
    const cuuint32_t cbox[2] = {cuuint32_t(kBlockK), cuuint32_t(kTileRows)};
    cr = encode(&cmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(q), cdims, cstrides, cbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return tcb::fail(TCB_ERR_CUDA, "%s: cuTensorMapEncodeTiled (codes) failed with %d", who, int(cr));

    // one instantiation per (group size, zero points or not): those are compile-time in the producer warps
    typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const Params);
    static const KernelFn kernels[4][2] = {
        {fused_dequant_gemm_kernel<4, false>, fused_dequant_gemm_kernel<4, true>},
        {fused_dequant_gemm_kernel<5, false>, fused_dequant_gemm_kernel<5, true>},
        {fused_dequant_gemm_kernel<6, false>, fused_dequant_gemm_kernel<6, true>},
        {fused_dequant_gemm_kernel<7, false>, fused_dequant_gemm_kernel<7, true>}};
    const int gi = group_size == 16 ? 0 : group_size == 32 ? 1 : group_size == 64 ? 2 : 3;
    const int zi = zp_or_null ? 1 : 0;
    const KernelFn kernel = kernels[gi][zi];
    static std::atomic<bool> attr_set[64][4][2] = {};
    int dev = 0;
    TCB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev][gi][zi].load(std::memory_order_acquire)) {
        TCB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes)));
        if (dev >= 0 && dev < 64) attr_set[dev][gi][zi].store(true, std::memory_order_release);
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
    p.gpr = K / group_size;
    p.table_vec_ok = p.gpr % 16 == 0 && (reinterpret_cast<uintptr_t>(scales) & 15) == 0 &&
                     (zp_or_null == nullptr || (reinterpret_cast<uintptr_t>(zp_or_null) & 15) == 0);
    p.quant_is_a = quant_is_rhs ? 0 : 1;
    // The tile list: wide (256 x 512) tiles as far as they fill whole rounds of the CTA pairs; if what is left of them
    // would occupy at most half of the pairs for a last round, those become twice as many 256 x 256 tiles, which run
    // side by side in half the time; an odd last dense unit is covered by 256 x 256 tiles as well.
    const int pairs = tcb::sm_count() / 2 > 0 ? tcb::sm_count() / 2 : 1;
    const int64_t wide_cols = units_d / 2, wide_total = tiles_q * wide_cols;
    const int64_t last_round = wide_total % pairs;
    const int64_t n_conv = (last_round > 0 && 2 * last_round <= pairs) ? last_round : 0;
    p.tiles_q = int(tiles_q);
    p.units_d = int(units_d);
    p.wide_cols = int(wide_cols);
    p.n_wide = int(wide_total - n_conv);
    p.n_conv = int(n_conv);
    p.n_odd = (units_d & 1) ? int(tiles_q) : 0;
    p.num_tiles = p.n_wide + 2 * p.n_conv + p.n_odd;
    const int grid = 2 * (p.num_tiles < pairs ? p.num_tiles : pairs);   // a cluster of two CTAs per tile in flight
    kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(map, map_half, cmap, p);
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

