// Fused quantize kernel on the 5th-generation tensor cores (tcgen05 + TMEM) for fp16 rows with d = 128:
//   norm -> rotation (128 x 128 x 128 contraction per tile of 128 rows) -> Lloyd-Max boundary search -> bit-pack.
//
// The rotation has to be float32-accurate (a code flips whenever a rotated value crosses a boundary), so the
// fp16 rows are used UN-normalised as exact MMA operands and R is split into two fp16 matrices,
// R = R_hi + 2^-11 * R_lo; both products are exact in the fp32 accumulators, and the normalisation by the
// row norm is applied afterwards.  Per tile: 2 x 8 tcgen05.mma (M = 128, N = 128, K = 16) into two TMEM
// accumulators, double-buffered so that the epilogue of tile i overlaps the loads and MMAs of tile i+1.
//
// Warp roles in a persistent CTA (one per SM, 800 threads):
//   warps 0-15  epilogue: thread <-> one row (TMEM lane) and one quarter of the coordinates; tcgen05.ld, boundary
//               search (up to 3 bits: binary search over boundaries held in registers; 4 bits: a 513-bin lookup
//               table, bin -> nearest boundary + count below it; both exact, see build_bins), packing, 128-bit stores
//   warp  16    allocates TMEM, issues the MMAs (one elected thread) and commits them to mbarriers
//   warps 17-24 producers: 128-bit global loads of the rows, sum of squares for the norm, stores into the
//               128-byte-swizzled K-major shared-memory layout the MMA descriptors expect
// Two ways to fill the operand stages.  TMA (the default when the driver offers tensor maps): one thread issues two
// cp.async.bulk.tensor copies per tile with the 128-byte swizzle the MMA descriptors expect - three stages of rows
// in flight per SM at no register cost - and warps 17-24 only read the tile back from shared memory for the norms.
// Otherwise warps 17-24 load the rows themselves (one tile's worth of registers in flight).
// Every mbarrier wait is bounded: on a timeout the kernel raises a status word, drains and frees its TMEM.
#include <algorithm>
#include <cstdlib>

#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace tq {

namespace tc {

constexpr int D = 128, TM = 128;                 // head_dim, rows per tile
constexpr int A_STAGES = 3, ACC_STAGES = 2;
constexpr int N_EPI = 512, N_PROD = 256;         // threads per role
constexpr int EPI_WARPS = N_EPI / 32;            // 16: TMEM lane quadrant = warp % 4, coordinate quarter = warp / 4
constexpr int NT = N_EPI + 32 + N_PROD;          // 800
constexpr int N_NORM = 128;                       // TMA variant: threads that read the rows back for the norms (one row each)
constexpr int NT_TMA = N_EPI + 32 + N_NORM + 32; // 704: the last warp's first lane feeds the operand stages by TMA
constexpr int BIN_REP = 8;                       // copies of every lookup-table entry (lane & 7 picks one): fewer bank conflicts
constexpr int KBLK_BYTES = TM * 128;             // one 64-column K-block of a 128-row operand: 16 KB
constexpr int OPER_BYTES = 2 * KBLK_BYTES;       // 32 KB per operand tile
constexpr int NBINS = 516;                       // 513 used + guard
constexpr uint32_t WAIT_LIMIT = 4u << 20;        // bounded spin: a few hundred milliseconds at most

// shared memory map (bytes)
constexpr int OFF_A = 0;                                   // A_STAGES x 32 KB, 1024-byte aligned
constexpr int OFF_RHI = OFF_A + A_STAGES * OPER_BYTES;     // 32 KB
constexpr int OFF_RLO = OFF_RHI + OPER_BYTES;              // 32 KB
constexpr int OFF_BINS = OFF_RLO + OPER_BYTES;             // NBINS x BIN_REP x 8 B: the table of the 4-bit codebook (only bits_hi can be 4)
constexpr int OFF_BND = OFF_BINS + NBINS * BIN_REP * 8;    // 2 x 16 floats: raw boundaries
constexpr int OFF_NSQ = OFF_BND + 128;                     // A_STAGES x 2 x 128 floats: partial sums of squares
constexpr int OFF_BAR = OFF_NSQ + A_STAGES * 2 * TM * 4;   // mbarriers
constexpr int OFF_MISC = OFF_BAR + 16 * 8;                 // tmem base, abort flag (barriers: 3 + 3 + 2 + 2 + 3 norm-ready)
constexpr int SMEM_BYTES = OFF_MISC + 64;

struct Params {
    const __half* x; int64_t n_lanes, n_rows, x_lane_stride, x_row_stride;
    const float* rot;
    const float* bnd_hi; const float* bnd_lo; int bits_hi, bits_lo;
    uint8_t* p_hi; uint8_t* p_lo; float* norms; int64_t out_lane_stride;
    int64_t n_tiles;
    int64_t tiles_per_lane;      // TMA variant: tiles never cross cache lanes; tile = lane * tiles_per_lane + tile in lane
    int* status;
};

__device__ int g_status = 0;   // 0 ok, otherwise the code of the first wait that timed out

#ifdef TQ_TIMING
// Development builds only: globaltimer stamps of CTA 0, [role][iteration][slot].
__device__ unsigned long long g_tc_timing[3 * 64 * 4 + 8];
__device__ __forceinline__ void tstamp(int idx) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_tc_timing[idx] = t;
}
#define TC_STAMP(cond, role, it, slot) do { if ((cond) && blockIdx.x == 0 && (it) < 64) tstamp(((role) * 64 + (it)) * 4 + (slot)); } while (0)
#define TC_STAMP0(cond, slot) do { if ((cond) && blockIdx.x == 0) tstamp(3 * 64 * 4 + (slot)); } while (0)
#else
#define TC_STAMP(cond, role, it, slot)
#define TC_STAMP0(cond, slot)
#endif

// ---- PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false after WAIT_LIMIT polls (or when another role already gave up).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = code;
    atomicCAS(&g_status, 0, code);
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
// Tiled TMA load of a (64 columns x 128 rows x 1 lane) box; the innermost coordinate is 0 or 64 halves (0 or 128 bytes).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory, 128-byte swizzle: row r of K-block b at  b*16 KB + r*128 B, its 16-byte
// chunk c stored at chunk position c ^ (r & 7).  Descriptor for the 16-column slab `ks` (0..3) of K-block b.
__device__ __forceinline__ uint64_t smem_desc(uint32_t tile_addr, int kblk, int ks) {
    const uint32_t addr = tile_addr + kblk * KBLK_BYTES + ks * 32;
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);          // start address
    d |= uint64_t(1) << 16;                       // leading byte offset (ignored for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;               // stride byte offset: 8 rows x 128 B
    d |= uint64_t(1) << 46;                       // descriptor version (Blackwell)
    d |= uint64_t(2) << 61;                       // SWIZZLE_128B
    return d;
}
// kind::f16: fp16 A and B, fp32 accumulate, both K-major, N = 128, M = 128
constexpr uint32_t IDESC = (1u << 4) | (uint32_t(D >> 3) << 17) | (uint32_t(TM >> 4) << 24);

// Lookup table for the boundary search.  Bin k covers normalised values around (k - 256) / 256 (width 1/256);
// entry = (boundary to test, number of boundaries below the bin's neighbourhood) where the neighbourhood is the
// bin widened by one bin on each side, so that a bin index that is off by one through rounding still gives the
// exact count.  A neighbourhood holding two boundaries is marked (a flag bit in the count) and handled by the plain
// counting loop.
constexpr int MARKED = 0x100;
#ifndef TQ_DIRECT_MAX_BITS
#define TQ_DIRECT_MAX_BITS 3
#endif
constexpr int DIRECT_MAX_BITS = TQ_DIRECT_MAX_BITS;   // up to this width the boundaries are searched in registers, above it through the
                                                      // bin table (at 4 bits the register search costs more issue slots than the table's bank conflicts)
static_assert(DIRECT_MAX_BITS <= 3, "the register search is written for at most seven boundaries");
__device__ void build_bins(float2* bins, const float* bnd, int n_bnd, int tid, int nthreads) {
    for (int k = tid; k < NBINS; k += nthreads) {
        const float lo = (float(k) - 256.f - 1.5f) / 256.f, hi = (float(k) - 256.f + 1.5f) / 256.f;
        int below = 0, inside = 0;
        float b_in = 2.0f;                    // no boundary near this bin: |y| <= 1 never exceeds the sentinel
        for (int i = 0; i < n_bnd; ++i) {
            const float b = bnd[i];
            if (b < lo) ++below;
            else if (b <= hi) { ++inside; b_in = b; }
        }
        const float2 e = make_float2(b_in, __int_as_float(inside > 1 ? (below | MARKED) : below));
#pragma unroll
        for (int r = 0; r < BIN_REP; ++r) bins[k * BIN_REP + r] = e;
    }
}

// Up to three bits the code is never formed: the boundaries live in registers, a binary search (one compare per bit)
// decides how many of them the value exceeds - the number the counting loop gives for a non-decreasing boundary
// list, NaN included (0) - and each level's outcome adds its bit, already shifted into place, to the group word
// (eight codes per group, so a code never straddles two words while it is being built).
template <int BITS>
__device__ __forceinline__ void add_code(uint32_t& grp, float y, const float (&b)[15], int sh) {
    if (BITS == 1) {
        if (y > b[0]) grp += 1u << sh;
    } else if (BITS == 2) {
        const bool p1 = y > b[1];
        const bool p2 = y > (p1 ? b[2] : b[0]);
        if (p1) grp += 2u << sh;
        if (p2) grp += 1u << sh;
    } else {
        const bool p1 = y > b[3];
        const bool p2 = y > (p1 ? b[5] : b[1]);
        const float lo = p2 ? b[2] : b[0], hi = p2 ? b[6] : b[4];
        const bool p3 = y > (p1 ? hi : lo);
        if (p1) grp += 4u << sh;
        if (p2) grp += 2u << sh;
        if (p3) grp += 1u << sh;
    }
}
// Plain counting loop, kept out of line: only reached when two boundaries share a bin neighbourhood.
__device__ __noinline__ uint32_t code_slow(float y, const float* raw_bnd, int n_bnd) {
    uint32_t c = 0;
    for (int i = 0; i < n_bnd; ++i) c += (y > raw_bnd[i]) ? 1u : 0u;
    return c;
}

struct EpiCtx {
    const Params& p; unsigned char* smem; uint32_t tmem_base, bar_accfull, bar_accfree, bar_afree, bar_nrm;
    volatile int* abort_flag; int64_t total_rows; int warp, lane;
};

// One chunk of 16 coordinates (TMEM columns col .. col + 15 of the hi and lo accumulators) at BITS bits: the codes go into
// g0 / g1 (eight codes each; plain 4-bit words on the table path).
template <int BITS>
__device__ __forceinline__ void epilogue_chunk(uint32_t taddr, float rinv, float rbin, const float (&bnd)[15], const float2* bins,
                                               const float* raw_bnd, uint32_t& g0, uint32_t& g1) {
    constexpr int n_bnd = (1 << BITS) - 1;
    uint32_t vh[16], vl[16];
    tmem_ld16(taddr, vh);
    tmem_ld16(taddr + 128, vl);
    tmem_ld_wait();
    if (BITS <= DIRECT_MAX_BITS) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float yp = fmaf(__uint_as_float(vl[i]), 1.f / 2048.f, __uint_as_float(vh[i]));
            add_code<BITS>(i < 8 ? g0 : g1, yp, bnd, BITS * (i & 7));                 // bnd: boundaries times the row's norm
        }
    } else {
        // table path: count-below times 16^k goes in with one multiply-add, the compare adds its bit in place
        uint32_t seen = 0;
        const uint32_t w0 = g0, w1 = g1;                                        // restored if the group has to be redone
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float yp = fmaf(__uint_as_float(vl[i]), 1.f / 2048.f, __uint_as_float(vh[i]));
            vh[i] = __float_as_uint(yp);
            // bin index from the mantissa of (y * 256 + 256 + 2^23): exact rounding to nearest, no convert instruction.
            // |y| <= 1 keeps the index below 513; NaN and infinity give index 0 (ten low mantissa bits are zero).
            const float tt = fmaf(yp, rbin, 8388608.f + 256.f);
            const float2 en = bins[(__float_as_uint(tt) & 0x3FFu) * BIN_REP];
            seen |= __float_as_uint(en.y);
            uint32_t& w = i < 8 ? g0 : g1;
            w += __float_as_uint(en.y) * (1u << (4 * (i & 7)));
            if ((yp * rinv) > en.x) w += 1u << (4 * (i & 7));                  // strict >, codebook.py:220-223
        }
        if (__any_sync(0xffffffffu, (seen & MARKED) != 0)) {     // a marked bin was hit: redo the group with the counting loop
            g0 = w0; g1 = w1;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                (i < 8 ? g0 : g1) |= code_slow(__uint_as_float(vh[i]) * rinv, raw_bnd, n_bnd) << (4 * (i & 7));
        }
    }
}

// 2 * BITS bytes: the sixteen codes of one chunk as the little-endian bit stream, stored at dst (2-byte aligned at least)
template <int BITS>
__device__ __forceinline__ void store_chunk(uint8_t* dst, uint32_t g0, uint32_t g1) {
    if (BITS == 4) {
        if ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) *reinterpret_cast<uint2*>(dst) = make_uint2(g0, g1);
        else { reinterpret_cast<uint16_t*>(dst)[0] = uint16_t(g0); reinterpret_cast<uint16_t*>(dst)[1] = uint16_t(g0 >> 16);
               reinterpret_cast<uint16_t*>(dst)[2] = uint16_t(g1); reinterpret_cast<uint16_t*>(dst)[3] = uint16_t(g1 >> 16); }
    } else if (BITS == 3) {
        const uint32_t w0 = g0 | (g1 << 24), w1 = g1 >> 8;
        reinterpret_cast<uint16_t*>(dst)[0] = uint16_t(w0); reinterpret_cast<uint16_t*>(dst)[1] = uint16_t(w0 >> 16);
        reinterpret_cast<uint16_t*>(dst)[2] = uint16_t(w1);
    } else if (BITS == 2) {
        const uint32_t w0 = g0 | (g1 << 16);
        if ((reinterpret_cast<uintptr_t>(dst) & 3) == 0) *reinterpret_cast<uint32_t*>(dst) = w0;
        else { reinterpret_cast<uint16_t*>(dst)[0] = uint16_t(w0); reinterpret_cast<uint16_t*>(dst)[1] = uint16_t(w0 >> 16); }
    } else {
        *reinterpret_cast<uint16_t*>(dst) = uint16_t(g0 | (g1 << 8));
    }
}

// Fractional widths, balanced: every warp takes sixteen coordinates of the high-bit half and sixteen of the low-bit half
// (coordinate quarter q: [16 q, 16 q + 16) and [64 + 16 q, 64 + 16 q + 16)), so no warp is left with only the
// costlier width while the others wait at the accumulator barrier.
template <int BH, int BL, bool TMA>
__device__ __forceinline__ void epilogue_loop_frac(const EpiCtx& e) {
    const Params& p = e.p;
    const int quad = e.warp & 3, quarter = e.warp >> 2, row_in_tile = quad * 32 + e.lane;
    const float2* bins = reinterpret_cast<const float2*>(e.smem + OFF_BINS) + (e.lane & (BIN_REP - 1));      // 4-bit side only
    const float* raw_h = reinterpret_cast<const float*>(e.smem + OFF_BND);
    const float* raw_l = raw_h + 16;
    float bnd_h[15], bnd_l[15];
#pragma unroll
    for (int i = 0; i < 15; ++i) { bnd_h[i] = raw_h[i < (1 << BH) - 1 ? i : 0]; bnd_l[i] = raw_l[i < (1 << BL) - 1 ? i : 0]; }
    const int64_t stride_rows = int64_t(gridDim.x) * TM;
    const int64_t step_o = TMA ? int64_t(gridDim.x) / p.tiles_per_lane : stride_rows / p.n_rows;
    const int64_t step_r = TMA ? (int64_t(gridDim.x) - step_o * p.tiles_per_lane) * TM : stride_rows - step_o * p.n_rows;
    const int64_t wrap_r = TMA ? p.tiles_per_lane * TM : p.n_rows;
    int64_t lane_o = 0, lane_r = 0;
    int it = 0;
    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        const int a = it % ACC_STAGES, s = it % A_STAGES;
        if (!mbar_wait(e.bar_accfull + 8 * a, (it / ACC_STAGES) & 1, e.abort_flag, 3)) break;
        if (TMA && !mbar_wait(e.bar_nrm + 8 * s, (it / A_STAGES) & 1, e.abort_flag, 5)) break;     // sums of squares written
        tc_fence_after();
        const float* nsq = reinterpret_cast<const float*>(e.smem + OFF_NSQ) + s * 2 * TM;
        const float nrm = sqrtf(nsq[row_in_tile] + nsq[TM + row_in_tile]);
        mbar_arrive(e.bar_afree + 8 * s);                       // norm slots of this stage are free again
        const float nden = fmaxf(nrm, 1e-10f);                  // cache.py:237-238 guards the zero vector the same way
        const float rinv = 1.f / nden;
        const float rbin = rinv * 256.f;
        // register search: y / |x| > b is tested as y > b * |x| (one multiply per boundary and row instead of one per coordinate)
        float sb_h[15], sb_l[15];
#pragma unroll
        for (int i = 0; i < 15; ++i) { sb_h[i] = bnd_h[i] * nden; sb_l[i] = bnd_l[i] * nden; }
        if (it == 0) {      // one division at the start, then advanced by the grid stride
            if (TMA) { lane_o = tile / p.tiles_per_lane; lane_r = (tile - lane_o * p.tiles_per_lane) * TM + row_in_tile; }
            else { const int64_t row = tile * TM + row_in_tile; lane_o = row / p.n_rows; lane_r = row - lane_o * p.n_rows; }
        }
        const bool live = TMA ? lane_r < p.n_rows : tile * TM + row_in_tile < e.total_rows;
        int64_t orow = 0;
        if (live) {
            orow = lane_o * p.out_lane_stride + lane_r;
            if (quarter == 0) p.norms[orow] = nrm;
        }
        lane_r += step_r; lane_o += step_o;
        if (lane_r >= wrap_r + (TMA ? row_in_tile : 0)) { lane_r -= wrap_r; ++lane_o; }
        const uint32_t t_row = e.tmem_base + (uint32_t(quad * 32) << 16) + a * 256;
        uint32_t h0 = 0, h1 = 0, l0 = 0, l1 = 0;
        epilogue_chunk<BH>(t_row + quarter * 16, rinv, rbin, sb_h, bins, raw_h, h0, h1);
        epilogue_chunk<BL>(t_row + 64 + quarter * 16, rinv, rbin, sb_l, bins, raw_l, l0, l1);
        tc_fence_before();
        mbar_arrive(e.bar_accfree + 8 * a);                     // accumulators may be overwritten
        if (live) {
            store_chunk<BH>(p.p_hi + orow * (8 * BH) + quarter * (2 * BH), h0, h1);      // a row of the half: 64 codes = 8 * bits bytes
            store_chunk<BL>(p.p_lo + orow * (8 * BL) + quarter * (2 * BL), l0, l1);
        }
    }
}

template <int BITS, bool TMA>
__device__ __forceinline__ void epilogue_loop(const EpiCtx& e) {
    const Params& p = e.p;
    const int quad = e.warp & 3, quarter = e.warp >> 2, row_in_tile = quad * 32 + e.lane;
    const bool second = p.bits_lo && quarter >= 2;              // fractional mode: coordinates [64, 128) use the low-bit codebook
    const float2* bins = reinterpret_cast<const float2*>(e.smem + OFF_BINS) + (e.lane & (BIN_REP - 1));      // 4-bit side only
    const float* raw_bnd = reinterpret_cast<const float*>(e.smem + OFF_BND) + (second ? 16 : 0);
    constexpr int n_bnd = (1 << BITS) - 1;
    constexpr int WBYTES = 32 * BITS / 8;                       // bytes this thread produces per row (32 coordinates)
    float bnd[15];
#pragma unroll
    for (int i = 0; i < 15; ++i) bnd[i] = raw_bnd[i < n_bnd ? i : 0];
    // the tile stride in (lane, row) form.  TMA variant: a tile is (lane, tile in lane), rows past the lane's end are
    // zero-filled by the copy and dropped here; otherwise tiles run over the flattened rows of all lanes.
    const int64_t stride_rows = int64_t(gridDim.x) * TM;
    const int64_t step_o = TMA ? int64_t(gridDim.x) / p.tiles_per_lane : stride_rows / p.n_rows;
    const int64_t step_r = TMA ? (int64_t(gridDim.x) - step_o * p.tiles_per_lane) * TM : stride_rows - step_o * p.n_rows;
    const int64_t wrap_r = TMA ? p.tiles_per_lane * TM : p.n_rows;
    int64_t lane_o = 0, lane_r = 0;
    int it = 0;
    for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
        const int a = it % ACC_STAGES, s = it % A_STAGES;
        TC_STAMP(e.warp == 0 && e.lane == 0, 2, it, 0);
        if (!mbar_wait(e.bar_accfull + 8 * a, (it / ACC_STAGES) & 1, e.abort_flag, 3)) break;
        if (TMA && !mbar_wait(e.bar_nrm + 8 * s, (it / A_STAGES) & 1, e.abort_flag, 5)) break;     // sums of squares written
        tc_fence_after();
        TC_STAMP(e.warp == 0 && e.lane == 0, 2, it, 1);
        const float* nsq = reinterpret_cast<const float*>(e.smem + OFF_NSQ) + s * 2 * TM;
        const float nrm = sqrtf(nsq[row_in_tile] + nsq[TM + row_in_tile]);
        mbar_arrive(e.bar_afree + 8 * s);                       // norm slots of this stage are free again
        const float nden = fmaxf(nrm, 1e-10f);                  // cache.py:237-238 guards the zero vector the same way
        const float rinv = 1.f / nden;
        const float rbin = rinv * 256.f;
        // register search: y / |x| > b is tested as y > b * |x| (one multiply per boundary and row instead of one per coordinate)
        float sb[15];
#pragma unroll
        for (int i = 0; i < 15; ++i) sb[i] = bnd[i] * nden;
        if (it == 0) {      // one division at the start, then advanced by the grid stride
            if (TMA) { lane_o = tile / p.tiles_per_lane; lane_r = (tile - lane_o * p.tiles_per_lane) * TM + row_in_tile; }
            else { const int64_t row = tile * TM + row_in_tile; lane_o = row / p.n_rows; lane_r = row - lane_o * p.n_rows; }
        }
        const bool live = TMA ? lane_r < p.n_rows : tile * TM + row_in_tile < e.total_rows;
        int64_t orow = 0;
        if (live) {
            orow = lane_o * p.out_lane_stride + lane_r;
            if (quarter == 0) p.norms[orow] = nrm;
        }
        lane_r += step_r; lane_o += step_o;
        if (lane_r >= wrap_r + (TMA ? row_in_tile : 0)) { lane_r -= wrap_r; ++lane_o; }
        const uint32_t t_hi = e.tmem_base + (uint32_t(quad * 32) << 16) + a * 256 + quarter * 32;
        uint32_t words[4], groups[4];                           // 32 codes x at most 4 bits; eight codes per group
#pragma unroll
        for (int i = 0; i < 4; ++i) words[i] = groups[i] = 0;
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {                        // 16 coordinates at a time
            uint32_t vh[16], vl[16];
            tmem_ld16(t_hi + cb * 16, vh);
            tmem_ld16(t_hi + 128 + cb * 16, vl);
            tmem_ld_wait();
            if (BITS <= DIRECT_MAX_BITS) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float yp = fmaf(__uint_as_float(vl[i]), 1.f / 2048.f, __uint_as_float(vh[i]));
                    add_code<BITS>(groups[cb * 2 + (i >> 3)], yp, sb, BITS * (i & 7));
                }
            } else {
                // table path: count-below times 16^k goes in with one multiply-add, the compare adds its bit in place
                uint32_t seen = 0;
                const uint32_t w0 = words[cb * 2], w1 = words[cb * 2 + 1];      // restored if the group has to be redone
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float yp = fmaf(__uint_as_float(vl[i]), 1.f / 2048.f, __uint_as_float(vh[i]));
                    vh[i] = __float_as_uint(yp);
                    // bin index from the mantissa of (y * 256 + 256 + 2^23): exact rounding to nearest, no convert instruction.
                    // |y| <= 1 keeps the index below 513; NaN and infinity give index 0 (ten low mantissa bits are zero).
                    const float tt = fmaf(yp, rbin, 8388608.f + 256.f);
                    const float2 en = bins[(__float_as_uint(tt) & 0x3FFu) * BIN_REP];
                    seen |= __float_as_uint(en.y);
                    uint32_t& w = words[cb * 2 + (i >> 3)];
                    w += __float_as_uint(en.y) * (1u << (4 * (i & 7)));
                    if ((yp * rinv) > en.x) w += 1u << (4 * (i & 7));          // strict >, codebook.py:220-223
                }
                if (__any_sync(0xffffffffu, (seen & MARKED) != 0)) {     // a marked bin was hit: redo the group with the counting loop
                    words[cb * 2] = w0; words[cb * 2 + 1] = w1;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        words[cb * 2 + (i >> 3)] |= code_slow(__uint_as_float(vh[i]) * rinv, raw_bnd, n_bnd) << (4 * (i & 7));
                }
            }
        }
        if (BITS <= DIRECT_MAX_BITS) {
            // groups[g] holds codes 8g .. 8g+7 in 8 * BITS bits: lay them out as the little-endian bit stream
            if (BITS == 3) {
                words[0] = groups[0] | (groups[1] << 24);
                words[1] = (groups[1] >> 8) | (groups[2] << 16);
                words[2] = (groups[2] >> 16) | (groups[3] << 8);
            } else if (BITS == 2) {
                words[0] = groups[0] | (groups[1] << 16);
                words[1] = groups[2] | (groups[3] << 16);
            } else {
                words[0] = groups[0] | (groups[1] << 8) | (groups[2] << 16) | (groups[3] << 24);
            }
        }
        tc_fence_before();
        mbar_arrive(e.bar_accfree + 8 * a);                     // accumulators may be overwritten
        TC_STAMP(e.warp == 0 && e.lane == 0, 2, it, 2);
        if (live) {
            const bool frac = p.bits_lo != 0;
            // integer mode: the row holds 4 quarters; fractional mode: packed_hi and packed_lo hold 2 quarters each
            uint8_t* dst = second ? p.p_lo + orow * (2 * WBYTES) + (quarter - 2) * WBYTES
                                  : p.p_hi + orow * ((frac ? 2 : 4) * WBYTES) + quarter * WBYTES;
            if ((WBYTES & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                for (int i = 0; i < WBYTES / 16; ++i)
                    reinterpret_cast<uint4*>(dst)[i] = make_uint4(words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3]);
            } else if ((WBYTES & 7) == 0 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
#pragma unroll
                for (int i = 0; i < WBYTES / 8; ++i) reinterpret_cast<uint2*>(dst)[i] = make_uint2(words[2 * i], words[2 * i + 1]);
            } else if ((WBYTES & 3) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
#pragma unroll
                for (int i = 0; i < WBYTES / 4; ++i) reinterpret_cast<uint32_t*>(dst)[i] = words[i];
            } else {
#pragma unroll
                for (int i = 0; i < WBYTES; ++i) dst[i] = uint8_t(words[i >> 2] >> (8 * (i & 3)));
            }
        }
    }
}

// FRAC: the balanced epilogue for the reference's fractional widths (bits_lo == bits_hi - 1); a kernel of its own so that the
// integer-width kernel keeps its register allocation
template <bool TMA, bool FRAC>
__global__ void __launch_bounds__(TMA ? NT_TMA : NT, 1) quantize_tc_kernel(Params p, const __grid_constant__ CUtensorMap tmap) {
    constexpr int NTHREADS = TMA ? NT_TMA : NT;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    // barriers: full[A_STAGES] (producers -> MMA), a_free[A_STAGES] (MMA commit + epilogue's norm read -> producers),
    //           acc_full[ACC_STAGES] (MMA commit -> epilogue), acc_free[ACC_STAGES] (epilogue -> MMA)
    const uint32_t bar_full = sbase + OFF_BAR, bar_afree = bar_full + 8 * A_STAGES;
    const uint32_t bar_accfull = bar_afree + 8 * A_STAGES, bar_accfree = bar_accfull + 8 * ACC_STAGES;
    const uint32_t bar_nrm = bar_accfree + 8 * ACC_STAGES;       // TMA variant: sums of squares of a stage are written

    TC_STAMP0(tid == 0, 0);
    if (sbase & 1023u) {                  // the swizzled operand tiles need 1024-byte alignment (uniform across the CTA)
        if (tid == 0) atomicCAS(&g_status, 0, 9);
        return;
    }
    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < A_STAGES; ++s) {
            // TMA: one arrival (the issuing thread, with the byte count) fills a stage; it is free again once the MMAs have
            // committed, the epilogue has read the norms and the norm warps have read the rows
            mbar_init(bar_full + 8 * s, TMA ? 1 : N_PROD);
            mbar_init(bar_afree + 8 * s, TMA ? 1 + N_EPI + N_NORM : 1 + N_EPI);
            mbar_init(bar_nrm + 8 * s, N_NORM);
        }
        for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(bar_accfull + 8 * a, 1); mbar_init(bar_accfree + 8 * a, N_EPI); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // R -> fp16 hi / lo operand tiles (swizzled K-major): B[n = j][k] = R[j][k]
    for (int idx = tid; idx < D * (D / 8); idx += NTHREADS) {
        const int j = idx / (D / 8), c = idx - j * (D / 8);      // row j, 16-byte chunk c (8 halves) of the row
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p.rot + j * D + c * 8));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p.rot + j * D + c * 8 + 4));
        const float v[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
        __align__(16) __half hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            hi[i] = __float2half_rn(v[i]);
            lo[i] = __float2half_rn((v[i] - __half2float(hi[i])) * 2048.f);
        }
        const int kblk = c >> 3, cc = c & 7;
        const int off = kblk * KBLK_BYTES + j * 128 + ((cc ^ (j & 7)) << 4);
        *reinterpret_cast<uint4*>(smem + OFF_RHI + off) = *reinterpret_cast<const uint4*>(hi);
        *reinterpret_cast<uint4*>(smem + OFF_RLO + off) = *reinterpret_cast<const uint4*>(lo);
    }
    {
        float* raw = reinterpret_cast<float*>(smem + OFF_BND);
        if (tid < 32) {
            const int side = tid >> 4, i = tid & 15;
            const float* src = side ? p.bnd_lo : p.bnd_hi;
            const int nb = (1 << (side ? p.bits_lo : p.bits_hi)) - 1;
            raw[tid] = (src != nullptr && i < nb) ? src[i] : INFINITY;
        }
        __syncthreads();
        if (p.bits_hi > DIRECT_MAX_BITS) build_bins(reinterpret_cast<float2*>(smem + OFF_BINS), raw, (1 << p.bits_hi) - 1, tid, NTHREADS);
    }
    if (warp == EPI_WARPS) {              // one warp owns the TMEM allocation: 2 stages x (hi + lo) x 128 columns
        tmem_alloc(sbase + OFF_MISC, 512);
        tmem_relinquish();
    }
    fence_proxy_async();                  // the operand tiles written above are read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int64_t total_rows = p.n_lanes * p.n_rows;
    TC_STAMP0(tid == 0, 1);

    if (warp < EPI_WARPS) {
        // ======================= epilogue: row = 32*(warp%4) + lane, coordinate quarter = warp/4 =======================
        const int bits = (p.bits_lo && (warp >> 3)) ? p.bits_lo : p.bits_hi;
        EpiCtx e{p, smem, tmem_base, bar_accfull, bar_accfree, bar_afree, bar_nrm, abort_flag, total_rows, warp, lane};
        if (FRAC) {                                             // 3.5, 2.5, 1.5 bits
            if (p.bits_hi == 4) epilogue_loop_frac<4, 3, TMA>(e);
            else if (p.bits_hi == 3) epilogue_loop_frac<3, 2, TMA>(e);
            else epilogue_loop_frac<2, 1, TMA>(e);
        } else if (bits == 4) epilogue_loop<4, TMA>(e);
        else if (bits == 3) epilogue_loop<3, TMA>(e);
        else if (bits == 2) epilogue_loop<2, TMA>(e);
        else epilogue_loop<1, TMA>(e);
    } else if (warp == EPI_WARPS) {
        // ======================= MMA issue: one elected thread =======================
        if (lane == 0) {
            int it = 0;
            for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
                const int a = it % ACC_STAGES, s = it % A_STAGES;
                if (it >= ACC_STAGES && !mbar_wait(bar_accfree + 8 * a, ((it / ACC_STAGES) - 1) & 1, abort_flag, 2)) break;
                TC_STAMP(true, 1, it, 0);
                if (!mbar_wait(bar_full + 8 * s, (it / A_STAGES) & 1, abort_flag, 1)) break;
                tc_fence_after();
                TC_STAMP(true, 1, it, 1);
                const uint32_t a_tile = sbase + OFF_A + s * OPER_BYTES;
                const uint32_t d_hi = tmem_base + a * 256, d_lo = d_hi + 128;
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t da = smem_desc(a_tile, kb, ks);
                        const uint32_t acc = (kb | ks) ? 1u : 0u;
                        umma_f16(d_hi, da, smem_desc(sbase + OFF_RHI, kb, ks), IDESC, acc);
                        umma_f16(d_lo, da, smem_desc(sbase + OFF_RLO, kb, ks), IDESC, acc);
                    }
                }
                umma_commit(bar_afree + 8 * s);      // rows of this stage consumed: producers may refill it
                umma_commit(bar_accfull + 8 * a);    // both accumulators complete: epilogue may read them
                TC_STAMP(true, 1, it, 2);
            }
        }
        __syncwarp();
    } else if (TMA && warp == EPI_WARPS + 1 + N_NORM / 32) {
        // ======================= TMA issue: one thread keeps the operand stages full =======================
        if (lane == 0) {
            int64_t o = int64_t(blockIdx.x) / p.tiles_per_lane, tl = int64_t(blockIdx.x) - o * p.tiles_per_lane;
            const int64_t so = int64_t(gridDim.x) / p.tiles_per_lane, st = int64_t(gridDim.x) - so * p.tiles_per_lane;
            int it = 0;
            for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
                const int s = it % A_STAGES;
                if (it >= A_STAGES && !mbar_wait(bar_afree + 8 * s, ((it / A_STAGES) - 1) & 1, abort_flag, 6)) break;
                const uint32_t a_tile = sbase + OFF_A + s * OPER_BYTES;
                mbar_expect_tx(bar_full + 8 * s, OPER_BYTES);
                tma_load_3d(a_tile, &tmap, 0, int(tl * TM), int(o), bar_full + 8 * s);                    // columns 0..63
                tma_load_3d(a_tile + KBLK_BYTES, &tmap, 64, int(tl * TM), int(o), bar_full + 8 * s);      // columns 64..127
                o += so; tl += st;
                if (tl >= p.tiles_per_lane) { tl -= p.tiles_per_lane; ++o; }
            }
        }
        __syncwarp();
    } else if (TMA) {
        // ======================= norm warps: sum of squares of every row, read back from the stage =======================
        // thread -> row 32 nw + lane, both 64-column blocks: eight consecutive rows hit eight different 16-byte columns
        // of the swizzled tile, so the 128-bit reads are free of bank conflicts
        const int nw = warp - (EPI_WARPS + 1), r = nw * 32 + lane;
        int it = 0;
        for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
            const int s = it % A_STAGES;
            if (!mbar_wait(bar_full + 8 * s, (it / A_STAGES) & 1, abort_flag, 7)) break;
            const unsigned char* rowp = smem + OFF_A + s * OPER_BYTES + r * 128;
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = *reinterpret_cast<const uint4*>(rowp + ((c ^ (r & 7)) << 4));
                const uint4 w = *reinterpret_cast<const uint4*>(rowp + KBLK_BYTES + ((c ^ (r & 7)) << 4));
                const __half2* h = reinterpret_cast<const __half2*>(&v);
                const __half2* g = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 f = __half22float2(h[u]), e = __half22float2(g[u]);
                    a = fmaf(f.x, f.x, a); a = fmaf(f.y, f.y, a);
                    b = fmaf(e.x, e.x, b); b = fmaf(e.y, e.y, b);
                }
            }
            float* nsq = reinterpret_cast<float*>(smem + OFF_NSQ) + s * 2 * TM;
            nsq[r] = a; nsq[TM + r] = b;
            mbar_arrive(bar_nrm + 8 * s);        // release: the epilogue reads the sums after waiting on this barrier
            mbar_arrive(bar_afree + 8 * s);      // this thread is done reading the stage
        }
    } else {
        // ======================= producers =======================
        // Warp pw owns rows [16*pw, 16*pw + 16) of the tile; one warp-wide 128-bit load covers two whole rows
        // (lane = 16*(row & 1) + chunk), i.e. 512 contiguous bytes when rows are contiguous.
        const int pt = tid - (N_EPI + 32);
        const int pw = pt >> 5, chunk = lane & 15, rsub = lane >> 4;
        const int kblk = chunk >> 3, cc = chunk & 7;
        // (lane, row) of this thread's first row of the tile, advanced by the grid stride: no 64-bit division per row
        const bool wide = p.n_rows >= TM;            // a tile then spans at most two lanes
        const int64_t stride_rows = int64_t(gridDim.x) * TM;
        const int64_t step_o = stride_rows / p.n_rows, step_r = stride_rows - step_o * p.n_rows;
        int64_t base_o = (int64_t(blockIdx.x) * TM + pw * 16 + rsub) / p.n_rows;
        int64_t base_r = (int64_t(blockIdx.x) * TM + pw * 16 + rsub) - base_o * p.n_rows;
        int it = 0;
        for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
            const int s = it % A_STAGES;
            uint4 v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t row = tile * TM + pw * 16 + i * 2 + rsub;
                v[i] = make_uint4(0, 0, 0, 0);
                if (row < total_rows) {
                    int64_t o, rr;
                    if (wide) {
                        o = base_o; rr = base_r + i * 2;
                        if (rr >= p.n_rows) { rr -= p.n_rows; ++o; }
                    } else {
                        o = row / p.n_rows; rr = row - o * p.n_rows;
                    }
                    v[i] = __ldg(reinterpret_cast<const uint4*>(p.x + o * p.x_lane_stride + rr * p.x_row_stride) + chunk);
                }
            }
            base_r += step_r; base_o += step_o;
            if (base_r >= p.n_rows) { base_r -= p.n_rows; ++base_o; }
            TC_STAMP(pt == 0, 0, it, 0);
            float ss[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half2* h = reinterpret_cast<const __half2*>(&v[i]);
                float a = 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float2 f = __half22float2(h[u]);
                    a = fmaf(f.x, f.x, a);
                    a = fmaf(f.y, f.y, a);
                }
#pragma unroll
                for (int off = 8; off; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
                ss[i] = a;
            }
            TC_STAMP(pt == 0, 0, it, 1);
            // the stage and its norm slots must be free: MMAs of tile it - A_STAGES done, its epilogue has read the norms
            if (it >= A_STAGES && !mbar_wait(bar_afree + 8 * s, ((it / A_STAGES) - 1) & 1, abort_flag, 4)) break;
            TC_STAMP(pt == 0, 0, it, 2);
            unsigned char* stage = smem + OFF_A + s * OPER_BYTES + kblk * KBLK_BYTES;
            float* nsq = reinterpret_cast<float*>(smem + OFF_NSQ) + s * 2 * TM;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = pw * 16 + i * 2 + rsub;
                *reinterpret_cast<uint4*>(stage + r * 128 + ((cc ^ (r & 7)) << 4)) = v[i];
                if (chunk == 0) { nsq[r] = ss[i]; nsq[TM + r] = 0.f; }
            }
            fence_proxy_async();                     // generic-proxy stores -> visible to the tensor core
            mbar_arrive(bar_full + 8 * s);
            TC_STAMP(pt == 0, 0, it, 3);
        }
    }
    // ---- teardown: every loop above is bounded, so every thread gets here ----
    tc_fence_before();
    __syncthreads();
    if (warp == EPI_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (tid == 0 && *abort_flag && p.status) *p.status = *abort_flag;
}

}  // namespace tc

}  // namespace tq

using namespace tq;

static int g_quantize_tma = 1;     // tq_set_tuning("quantize_tma", 0 / 1)
namespace tq { void set_quantize_tma(int on) { g_quantize_tma = on ? 1 : 0; } }

// Takes the call when it fits the tensor-core kernel: fp16 rows, d = 128, 16-byte aligned rows, no QJL sketch,
// no rotated-row output.  Otherwise reports "not handled" and the caller uses the general CUDA-core kernel.
int tq_quantize_pack_tc(const tq_quantize_args* q, cudaStream_t s, bool* handled) {
    *handled = false;
    if (q->d != tc::D || q->x_dtype != TQ_F16 || q->qjl_bits || q->y_out) return TQ_OK;
    if (q->bits_lo > tc::DIRECT_MAX_BITS) return TQ_OK;      // the kernel keeps one bin table: only the high-bit half may need it
    if (!aligned(q->x, 16) || q->x_row_stride % 8 || q->x_lane_stride % 8 || !aligned(q->rot, 16)) return TQ_OK;
    static int disabled = -1;
    if (disabled < 0) {
        const char* e = getenv("TQ_DISABLE_TC");
        disabled = (e && e[0] == '1') ? 1 : 0;
    }
    if (disabled) return TQ_OK;
    const int64_t total = q->n_lanes * q->n_rows;
    if (total < 4 * tc::TM) return TQ_OK;            // tiny inputs: not worth a persistent launch
    static bool attr_set[16] = {false};
    static int sms[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return TQ_OK;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tc::quantize_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_quantize_pack: shared memory %d B: %s", tc::SMEM_BYTES, cudaGetErrorString(e));
        if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0) sms[dev] = 148;
        attr_set[dev] = true;
    }
    tc::Params p{};
    p.x = static_cast<const __half*>(q->x);
    p.n_lanes = q->n_lanes; p.n_rows = q->n_rows; p.x_lane_stride = q->x_lane_stride; p.x_row_stride = q->x_row_stride;
    p.rot = q->rot; p.bnd_hi = q->bnd_hi; p.bnd_lo = q->bnd_lo; p.bits_hi = q->bits_hi; p.bits_lo = q->bits_lo;
    p.p_hi = q->packed_hi; p.p_lo = q->packed_lo; p.norms = q->norms; p.out_lane_stride = q->out_lane_stride;
    p.status = nullptr;

    // Tensor map over the rows as (column, row, lane): boxes of 64 columns x 128 rows x 1 lane land in shared memory in
    // the 128-byte-swizzled layout the MMA descriptors describe; rows past a lane's end read as zeros.
    CUtensorMap tmap{};
    bool use_tma = false;
    static int env_off = -1;
    if (env_off < 0) {
        const char* e = getenv("TQ_DISABLE_TMA");
        env_off = (e && e[0] == '1') ? 1 : 0;
    }
    const bool tma_off = env_off || !g_quantize_tma;
    static PFN_cuTensorMapEncodeTiled encode = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
        looked_up = true;
    }
    if (!tma_off && encode && q->n_rows < (int64_t(1) << 31) && q->n_lanes < (int64_t(1) << 31)) {
        const cuuint64_t dims[3] = {cuuint64_t(tc::D), cuuint64_t(q->n_rows), cuuint64_t(q->n_lanes)};
        const cuuint64_t strides[2] = {cuuint64_t(q->x_row_stride) * 2, cuuint64_t(q->x_lane_stride) * 2};     // bytes, multiples of 16
        const cuuint32_t box[3] = {64, cuuint32_t(tc::TM), 1};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(q->x), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        use_tma = (r == CUDA_SUCCESS);
    }
    const bool frac = q->bits_lo != 0 && q->bits_hi == q->bits_lo + 1;     // balanced epilogue of the fractional widths
    if (use_tma) {
        p.tiles_per_lane = (q->n_rows + tc::TM - 1) / tc::TM;
        p.n_tiles = q->n_lanes * p.tiles_per_lane;
        const unsigned grid = unsigned(std::min<int64_t>(p.n_tiles, sms[dev]));
        if (frac) tc::quantize_tc_kernel<true, true><<<grid, tc::NT_TMA, tc::SMEM_BYTES, s>>>(p, tmap);
        else tc::quantize_tc_kernel<true, false><<<grid, tc::NT_TMA, tc::SMEM_BYTES, s>>>(p, tmap);
    } else {
        p.tiles_per_lane = 0;
        p.n_tiles = (total + tc::TM - 1) / tc::TM;
        const unsigned grid = unsigned(std::min<int64_t>(p.n_tiles, sms[dev]));
        if (frac) tc::quantize_tc_kernel<false, true><<<grid, tc::NT, tc::SMEM_BYTES, s>>>(p, tmap);
        else tc::quantize_tc_kernel<false, false><<<grid, tc::NT, tc::SMEM_BYTES, s>>>(p, tmap);
    }
    *handled = true;
    return check_launch("tq_quantize_pack (tensor core)");
}

// 0 if no tensor-core quantize launch on the current device has reported a timed-out wait, else its code.
// Synchronises the device.
#ifdef TQ_TIMING
extern "C" int tq_debug_tc_timing(unsigned long long* host_out, int n) {
    return int(cudaMemcpyFromSymbol(host_out, tc::g_tc_timing, sizeof(unsigned long long) * n));
}
#endif

namespace tq { int decode_status_host(); int decode_status_clear(); }   // decode_direct.cu

extern "C" int tq_device_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tc::g_status, sizeof(int)) != cudaSuccess) return -1;
    return v ? v : decode_status_host();
}

extern "C" int tq_device_status_clear(void) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(tc::g_status, &zero, sizeof(int)) != cudaSuccess) return -1;
    return decode_status_clear();
}
