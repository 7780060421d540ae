// Fused quantize kernel on the 5th-generation tensor cores (tcgen05 + TMEM) for fp16 / bf16 rows with d in {64, 96, 128}:
//   norm -> rotation (128 rows x d x d contraction per tile) -> Lloyd-Max boundary search -> bit-pack (+ QJL sketch).
//
// The rotation has to be float32-accurate (a code flips whenever a rotated value crosses a boundary), so the rows are
// used UN-normalised as exact MMA operands and R is split into terms that are exact operands too:
//   fp16 rows: R = R_hi + 2^-11 R_lo (fp16 each): one MMA of N = 2 d per k-step against [R_hi ; 2^11 R_lo] fills a
//              high and a low accumulator (two chains of d / 16 dependent MMAs would take as long as one: a dependent
//              step costs about 70 ns whatever its width); the epilogue adds them.  With the sketch on there is room
//              for one accumulator per tile only: the low products are accumulated first and the first high MMA takes
//              the accumulator scaled by 2^-11 (the instruction's scale-input-d).
//   bf16 rows: R = R_1 + R_2 + R_3 (bf16 each, 24 bits together; bf16 has float32's exponent range, so no scaling) into
//              one accumulator.
// Every product is exact in the fp32 accumulator; the normalisation by the row norm is applied afterwards.
//
// Warp roles in a persistent CTA (one per SM; 704 threads, 448 with the sketch on).  Epilogue warps come first (E of them),
// then one MMA warp, four norm warps, one TMA warp:
//   warps 0..E-1 epilogue; thread <-> one row (TMEM lane) and a share of its sixteen-coordinate chunks (tcgen05.ld).
//                fp16 rows: all sixteen warps work on the same tile in step, a quarter of the row each, reading the
//                high and the low accumulator and combining them; two accumulator stages, so the MMAs of the next tile
//                run meanwhile.  bf16 rows: two groups of eight warps take alternate tiles (two stages each), half a row
//                per thread.  With the QJL sketch on, a thread owns a whole row (E = 8: two groups of four warps, two
//                stages each): it forms the quantization residual of every coordinate and accumulates its 32
//                projections (the projection matrix is read from shared memory as warp-wide broadcasts).
//                Up to 3 bits a binary search over boundaries (times the row's norm) held in registers adds its
//                outcome bits straight into the packed word; at 4 bits one lookup in a 513-bin table (bin -> nearest
//                boundary + count below; see build_bins).  Fractional widths: the threads of a row take chunks of
//                either width, so they finish together.
//   warp  E      allocates TMEM, issues the MMAs (one elected thread) and commits them to mbarriers
//   next four    norms: read each tile back from shared memory for the rows' sums of squares
//   last warp    one thread keeps the operand stages full with tiled TMA copies (cp.async.bulk.tensor, 3-D tensor map
//                (column, row, lane), 128-byte swizzle as the MMA descriptors expect; rows past a lane's end and
//                columns past d read as zeros)
// Every mbarrier wait is bounded: on a timeout the kernel raises a status word, drains and frees its TMEM.
#include <algorithm>
#include <cstdlib>

#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace tq {

namespace tc {

constexpr int DMAX = 128, TM = 128;              // largest head_dim, rows per tile
constexpr int A_STAGES_MAX = 3, ACC_STAGES = 4;
constexpr int N_NORM = 128;                      // threads that read the rows back for the norms
// epilogue warps: 16, or 8 with the QJL sketch on (its 32 running projections per thread need the registers); then the
// MMA warp, the norm warps, the TMA warp
// (twelve warps in three groups were measured too: the compiler then has 96 registers per thread, spills 300 bytes, and the
// launch takes the same time - the sketch variant is bound by its instruction count, some 30-37 per coordinate, not by how
// many warps issue them)
#ifndef TQ_QJL_EPI_WARPS
#define TQ_QJL_EPI_WARPS 8
#endif
__host__ __device__ constexpr int epi_warps(bool qjl) { return qjl ? TQ_QJL_EPI_WARPS : 16; }
__host__ __device__ constexpr int n_threads(bool qjl) { return epi_warps(qjl) * 32 + 32 + N_NORM + 32; }     // 704 / 448
constexpr int BIN_REP = 8;                       // copies of every lookup-table entry (lane & 7 picks one): fewer bank conflicts
constexpr int KBLK_BYTES = TM * 128;             // one 64-column K-block of a 128-row operand: 16 KB
constexpr int OPER_BYTES = 2 * KBLK_BYTES;       // 32 KB per operand tile
constexpr int NBINS = 516;                       // 513 used + guard
constexpr int QM = 32;                           // projections of the QJL sketch
constexpr uint32_t WAIT_LIMIT = 4u << 20;        // bounded spin: a few hundred milliseconds at most

// shared memory map (bytes).  fp16 rows: three row stages and two terms of R; bf16 rows: two row stages and three terms.
constexpr int OFF_A = 0;                                   // stage s at s * 32 KB, 1024-byte aligned
constexpr int OFF_R3 = OFF_A + 2 * OPER_BYTES;             // bf16: third term of R (fp16: the third row stage)
constexpr int OFF_R1 = OFF_A + 3 * OPER_BYTES;             // R_hi / R_1
constexpr int OFF_R2 = OFF_R1 + OPER_BYTES;                // R_lo / R_2
constexpr int OFF_BINS = OFF_R2 + OPER_BYTES;              // NBINS x BIN_REP x 8 B: the table of the 4-bit codebook (only bits_hi can be 4)
constexpr int OFF_PT = OFF_BINS + NBINS * BIN_REP * 8;     // QJL: (S R^T) as fp16 high / low parts in mma B-fragment order: [d / 16][4 n-tiles][hi | lo][32 lanes] x 8 bytes
constexpr int OFF_BND = OFF_PT + DMAX * QM * 4;            // 2 x 16 floats raw boundaries, 2 x 16 floats centroids
constexpr int OFF_NSQ = OFF_BND + 256;                     // A_STAGES_MAX x 2 x 128 floats: partial sums of squares
constexpr int OFF_BAR = OFF_NSQ + A_STAGES_MAX * 2 * TM * 4;   // mbarriers: 3 full, 3 a_free, 3 norm-ready, 4 acc_full, 4 acc_free
constexpr int OFF_MISC = OFF_BAR + 24 * 8;                 // tmem base, abort flag
constexpr int SK_LD = 32;                                  // QJL: bytes per staged row of 16 fp16 residuals; the two 16-byte halves of rows 4-7 (mod 8) swap places, so the eight rows of an 8 x 8 matrix land in distinct banks
constexpr int OFF_SKETCH = (OFF_MISC + 64 + 127) / 128 * 128;   // QJL: one 32-row staging buffer per epilogue warp
constexpr int SMEM_BYTES = OFF_SKETCH + TQ_QJL_EPI_WARPS * 32 * SK_LD;
static_assert(SMEM_BYTES <= 227 * 1024, "shared-memory plan");

struct Params {
    int d, bf16, a_stages;
    int64_t n_rows, n_tiles, tiles_per_lane;     // tiles never cross cache lanes; tile = lane * tiles_per_lane + tile in lane
    const float* rot;
    const float* bnd_hi; const float* bnd_lo; int bits_hi, bits_lo;
    uint8_t* p_hi; uint8_t* p_lo; float* norms; int64_t out_lane_stride;
    const float* qjl_proj_rot; const float* cent_hi; const float* cent_lo; uint32_t* qjl_bits; float* qjl_gamma;
};

__device__ int g_status = 0;   // 0 ok, otherwise the code of the first wait that timed out

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
// Tiled TMA load of a (64 columns x 128 rows x 1 lane) box; the innermost coordinate is 0 or 64 elements (0 or 128 bytes).
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
// D = A.B (+ D when accumulate != 0)
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    const uint32_t zero = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero), "r"(zero), "r"(zero), "r"(zero) : "memory");
}
// D = A.B + 2^-11 D
__device__ __forceinline__ void umma_f16_scaled11(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
    const uint32_t zero = 0, one = 1;
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p, 11;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(one), "r"(zero), "r"(zero), "r"(zero), "r"(zero) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
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
// kind::f16 instruction descriptor: fp32 accumulate, A and B both fp16 or both bf16, both K-major, M = 128, N = d
__device__ __forceinline__ uint32_t make_idesc(int d, bool bf16) {
    return (1u << 4) | (bf16 ? ((1u << 7) | (1u << 10)) : 0u) | (uint32_t(d >> 3) << 17) | (uint32_t(TM >> 4) << 24);
}

// Lookup table for the boundary search.  Bin k covers normalised values around (k - 256) / 256 (width 1/256);
// entry = (boundary to test, number of boundaries below the bin's neighbourhood) where the neighbourhood is the
// bin widened by one bin on each side, so that a bin index that is off by one through rounding still gives the
// exact count.  A neighbourhood holding two boundaries is marked (a flag bit in the count) and handled by the plain
// counting loop.
constexpr int MARKED = 0x100;
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

// Up to three bits the code is never formed: the boundaries (times the row's norm) live in registers, a binary search
// (one compare per bit) decides how many of them the value exceeds - the number the counting loop gives for a
// non-decreasing boundary list, NaN included (0) - and each level's outcome adds its bit, already shifted into place,
// to the group word (eight codes per group, so a code never straddles two words while it is being built).
template <int BITS>
__device__ __forceinline__ void add_code(uint32_t& grp, float y, const float (&b)[7], int sh) {
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

// What a thread needs to know about its row while it walks the coordinates.
struct RowCtx {
    float rinv, rbin;              // 1 / max(|x|, 1e-10) and 256 times that
    const float2* bins;            // this lane's copy of the 4-bit table
};

// Sixteen coordinates (TMEM columns taddr .. + 15) at BITS bits: the codes go into g0 / g1 (eight codes each, BITS bits
// per code).  sb: boundaries times the row's norm (register search); raw: unscaled boundaries (table path's fallback).
template <int BITS>
__device__ __forceinline__ void quantize16(const uint32_t* v, const RowCtx& rc, const float (&sb)[7], const float* raw, uint32_t& g0, uint32_t& g1) {
    g0 = g1 = 0;
    if (BITS <= 3) {
#pragma unroll
        for (int i = 0; i < 16; ++i) add_code<BITS>(i < 8 ? g0 : g1, __uint_as_float(v[i]), sb, BITS * (i & 7));
    } else {
        // table path: count-below times 16^k goes in with one multiply-add, the compare adds its bit in place
        uint32_t seen = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float yp = __uint_as_float(v[i]);
            // bin index from the mantissa of (y * 256 + 256 + 2^23): exact rounding to nearest, no convert instruction.
            // |y| <= 1 keeps the index below 513; NaN and infinity give index 0 (ten low mantissa bits are zero).
            const float tt = fmaf(yp, rc.rbin, 8388608.f + 256.f);
            const float2 en = rc.bins[min(__float_as_uint(tt) & 0x3FFu, uint32_t(NBINS - 1)) * BIN_REP];     // (the clamp only matters for |y| > |x|, i.e. never)
            seen |= __float_as_uint(en.y);
            uint32_t& w = i < 8 ? g0 : g1;
            w += __float_as_uint(en.y) * (1u << (4 * (i & 7)));
            if ((yp * rc.rinv) > en.x) w += 1u << (4 * (i & 7));                  // strict >, codebook.py:220-223
        }
        if (__any_sync(0xffffffffu, (seen & MARKED) != 0)) {     // a marked bin was hit: redo the group with the counting loop
            g0 = g1 = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i)
                (i < 8 ? g0 : g1) |= code_slow(__uint_as_float(v[i]) * rc.rinv, raw, 15) << (4 * (i & 7));
        }
    }
}

// Appends a group of eight codes (8 * BITS bits) to a row's bit stream held in words[]: group k sits at bit 8 * BITS * k.
template <int BITS, int NW>
__device__ __forceinline__ void put_group(uint32_t (&words)[NW], int k, uint32_t g) {
    constexpr int GB = 8 * BITS;
    const int bit = GB * k, w = bit >> 5, sh = bit & 31;                          // all compile-time after unrolling
    words[w] |= g << sh;
    if (sh + GB > 32 && w + 1 < NW) words[w + 1] |= g >> (32 - sh);
}

// nbytes of words[] to dst with the widest stores the address and the size allow (both known per row only)
template <int NW>
__device__ __forceinline__ void store_words(uint8_t* dst, const uint32_t (&words)[NW], int nbytes) {
    const uint32_t al = uint32_t(reinterpret_cast<uintptr_t>(dst)) | uint32_t(nbytes);
    if ((al & 15u) == 0) {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i)
            if (16 * i < nbytes) reinterpret_cast<uint4*>(dst)[i] = make_uint4(words[4 * i], words[4 * i + 1], words[4 * i + 2], words[4 * i + 3]);
    } else if ((al & 7u) == 0) {
#pragma unroll
        for (int i = 0; i < NW / 2; ++i)
            if (8 * i < nbytes) reinterpret_cast<uint2*>(dst)[i] = make_uint2(words[2 * i], words[2 * i + 1]);
    } else if ((al & 3u) == 0) {
#pragma unroll
        for (int i = 0; i < NW; ++i)
            if (4 * i < nbytes) reinterpret_cast<uint32_t*>(dst)[i] = words[i];
    } else {                                                                      // rows of 6 or 18 bytes: 2-byte aligned
#pragma unroll
        for (int i = 0; i < 2 * NW; ++i)
            if (2 * i < nbytes) reinterpret_cast<uint16_t*>(dst)[i] = uint16_t(words[i >> 1] >> (16 * (i & 1)));
    }
}

struct EpiCtx {
    const Params& p; unsigned char* smem; uint32_t tmem_base, bar_accfull, bar_accfree, bar_afree, bar_nrm;
    volatile int* abort_flag; int warp, lane;
};

// QJL: the residual of sixteen coordinates (normalised rotated value minus its centroid) enters the 32 projections and
// the residual's sum of squares.  A thread owns a row, a warp 32 rows: the projections of the warp's rows are a
// 32 x 16 by 16 x 32 product per call, done with mma.sync (a CUDA-core version cost 32 multiply-adds and 8 shared-memory
// reads per coordinate and thread: two thirds of the kernel's instructions).  Only the SIGN of a projection is kept, so
// the residual is scaled by 2^8 (clear of fp16 subnormals) and split into fp16 high and low parts, as is S R^T:
// acc += hi x hi + lo x hi + hi x lo reproduces the float32 product to about 2^-21.  The operands go through a
// 32-row staging buffer of the warp (row = lane) and come back as fragments with ldmatrix.
struct Sketch {
    float acc[2][4][4];        // [16-row half of the warp][8 projections][mma accumulator]: rows g / g + 8, projections 2t, 2t + 1
    uint32_t stage;            // shared-window address of the warp's staging buffer
    const uint2* bfrag;        // B fragments of S R^T (OFF_PT)
    int lane;
};
__device__ __forceinline__ void sk_mma(float (&c)[4], const uint32_t (&a)[4], uint2 b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b.x), "r"(b.y));
}
__device__ __forceinline__ void sk_ldsm(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void sk_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
template <int BITS>
__device__ __forceinline__ void sketch16(const uint32_t* v, uint32_t g0, uint32_t g1, float rinv, const float* cent, int col0, Sketch& sk, float& ee) {
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float e2[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint32_t code = (((i + u) < 8 ? g0 : g1) >> (BITS * ((i + u) & 7))) & ((1u << BITS) - 1u);
            const float e = fmaf(__uint_as_float(v[i + u]), rinv, -cent[code]);       // 2^8 times the residual (rinv and the centroids carry the factor)
            ee = fmaf(e, e, ee);
            e2[u] = e;
        }
        const __half2 h = __floats2half2_rn(e2[0], e2[1]);
        const float2 hf = __half22float2(h);
        const __half2 l = __floats2half2_rn(e2[0] - hf.x, e2[1] - hf.y);
        hi[i >> 1] = *reinterpret_cast<const uint32_t*>(&h);
        lo[i >> 1] = *reinterpret_cast<const uint32_t*>(&l);
    }
    const uint32_t swz = uint32_t((sk.lane >> 2) & 1) * 16;                                            // rows 4-7 (mod 8): halves swapped
    const uint32_t row = sk.stage + uint32_t(sk.lane) * SK_LD;
    const uint32_t frag = sk.stage + uint32_t(sk.lane & 15) * SK_LD + ((uint32_t(sk.lane >> 4) * 16) ^ swz);   // ldmatrix row of this lane (second half: + 16 rows)
    uint32_t ah[2][4], al[2][4];
    sk_sts128(row + swz, hi[0], hi[1], hi[2], hi[3]);
    sk_sts128(row + (16 ^ swz), hi[4], hi[5], hi[6], hi[7]);
    __syncwarp();
    sk_ldsm(ah[0], frag);
    sk_ldsm(ah[1], frag + 16 * SK_LD);
    __syncwarp();
    sk_sts128(row + swz, lo[0], lo[1], lo[2], lo[3]);
    sk_sts128(row + (16 ^ swz), lo[4], lo[5], lo[6], lo[7]);
    __syncwarp();
    sk_ldsm(al[0], frag);
    sk_ldsm(al[1], frag + 16 * SK_LD);
    __syncwarp();
    const uint2* bf = sk.bfrag + (col0 >> 4) * (4 * 2 * 32) + sk.lane;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const uint2 bh = bf[(nt * 2 + 0) * 32], bl = bf[(nt * 2 + 1) * 32];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            sk_mma(sk.acc[mt][nt], ah[mt], bh);
            sk_mma(sk.acc[mt][nt], al[mt], bh);
            sk_mma(sk.acc[mt][nt], ah[mt], bl);
        }
    }
}
// The sign word of this thread's row (row = lane) from the warp's accumulators: bit p set iff projection p >= 0.
__device__ __forceinline__ uint32_t sketch_bits(const Sketch& sk) {
    const int g = sk.lane >> 2, t = sk.lane & 3;
    uint32_t w[4];                                         // rows g, g + 8, 16 + g, 24 + g: this lane's two bits per n-tile
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint32_t x = 0;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
                x |= ((sk.acc[mt][nt][2 * h] >= 0.f ? 1u : 0u) | (sk.acc[mt][nt][2 * h + 1] >= 0.f ? 2u : 0u)) << (8 * nt + 2 * t);
            x |= __shfl_xor_sync(0xffffffffu, x, 1);
            x |= __shfl_xor_sync(0xffffffffu, x, 2);
            w[mt * 2 + h] = x;
        }
    // row r = lane is held by the lanes of group g = r & 7 as word (r >> 3)
    const int src = (sk.lane & 7) * 4;
    const uint32_t w0 = __shfl_sync(0xffffffffu, w[0], src), w1 = __shfl_sync(0xffffffffu, w[1], src);
    const uint32_t w2 = __shfl_sync(0xffffffffu, w[2], src), w3 = __shfl_sync(0xffffffffu, w[3], src);
    const int k = sk.lane >> 3;
    (void)g;
    return k == 0 ? w0 : k == 1 ? w1 : k == 2 ? w2 : w3;
}

// A run of a row's coordinates ([col0, col0 + 16 * nch) at BITS bits) in rolled steps of 32 coordinates; the step's codes
// (32 * BITS bits) are assembled in registers and stored at once.  Keeping the loop rolled keeps its body within the
// instruction cache.  SPLITACC: the high and low products sit in two accumulators lo_off columns apart and are combined
// here (y = hi + 2^-11 lo), sixteen coordinates per pair of loads; otherwise one 32-column load per step.
// NCH: the number of chunks when it is known at compile time (1 or 2: a single step whose shape folds), 0 = nch_rt.
template <int BITS, bool QJL, bool SPLITACC, int NCH>
__device__ __forceinline__ void quantize_part(uint32_t t_row, int col0, int nch_rt, int lo_off, const RowCtx& rc, const float (&sb)[7], const float* raw,
                                              const float* cent, uint8_t* dst, bool live, Sketch& sk, float& ee) {
    constexpr int NW = 2 * 16 * BITS / 32;                                          // words of a step: BITS
    const int nch = NCH ? NCH : nch_rt;
#pragma unroll 1
    for (int c0 = 0; c0 < nch; c0 += 2) {
        uint32_t v[32], w[NW];
#pragma unroll
        for (int i = 0; i < NW; ++i) w[i] = 0;
        const int nc = min(2, nch - c0);                                            // a run may end on a half step
        if (!SPLITACC && !QJL) {
            tmem_ld32(t_row + col0 + c0 * 16, v);
            tmem_ld_wait();
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            if (c < nc) {
                uint32_t g0, g1;
                uint32_t* vc = v + ((SPLITACC || QJL) ? 0 : 16 * c);
                if (QJL && !SPLITACC) {                                         // (the sketch keeps 32 accumulators: sixteen columns at a time)
                    tmem_ld16(t_row + col0 + (c0 + c) * 16, *reinterpret_cast<uint32_t (*)[16]>(v));
                    tmem_ld_wait();
                }
                if (SPLITACC) {
                    uint32_t (&hi)[16] = *reinterpret_cast<uint32_t (*)[16]>(v);
                    uint32_t (&lo)[16] = *reinterpret_cast<uint32_t (*)[16]>(v + 16);
                    tmem_ld16(t_row + col0 + (c0 + c) * 16, hi);
                    tmem_ld16(t_row + lo_off + col0 + (c0 + c) * 16, lo);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(fmaf(__uint_as_float(v[16 + i]), 1.f / 2048.f, __uint_as_float(v[i])));
                }
                quantize16<BITS>(vc, rc, sb, raw, g0, g1);
                put_group<BITS, NW>(w, 2 * c, g0);
                put_group<BITS, NW>(w, 2 * c + 1, g1);
                if constexpr (QJL) sketch16<BITS>(vc, g0, g1, rc.rinv * 256.f, cent, col0 + (c0 + c) * 16, sk, ee);
            }
        }
        if (live) store_words<NW>(dst + c0 * 2 * BITS, w, nc * 2 * BITS);
    }
}

// BH bits for coordinates [0, half), BL for [half, d) (BL == 0: BH for all of them, half = d).  Three shapes:
//   fp16 rows (SPLITACC): two accumulators per tile (high and low products: two independent chains of MMAs instead of
//     one twice as long) leave room for two stages, so all sixteen warps work on the same tile in step - thread <-> one
//     row and a quarter of its sixteen-coordinate chunks (of either width) - while the MMAs of the next tile run.
//   bf16 rows: one accumulator per tile, four stages; two groups of eight warps take alternate tiles (two stages each),
//     a thread owns one row and half of its chunks.
//   QJL sketch: a thread needs the whole row (32 running projections) and the registers for it: eight epilogue warps,
//     two groups of four that take alternate tiles, one accumulator per tile, two stages per group.
template <bool QJL, bool SPLITACC> struct EpiShape {
    static constexpr int EW = epi_warps(QJL), NT = n_threads(QJL), N_EPI = EW * 32;
    static constexpr int GROUPS = SPLITACC ? 1 : QJL ? epi_warps(true) / 4 : 2;     // groups of warps that take tiles in turn
    static constexpr int WPG = EW / GROUPS;                                         // warps per group: 4 row quadrants x SPLIT shares of the columns
    static constexpr int SPLIT = WPG / 4;
    static constexpr int STAGES = SPLITACC ? 2 : 4;                                 // accumulator stages
    static constexpr int STAGE_COLS = SPLITACC ? 2 * DMAX : DMAX;
};
// DC: head_dim when it is known at compile time (the chunk shares, row widths and store shapes then fold), 0 = read it
// from the parameters.
template <int BH, int BL, bool QJL, bool SPLITACC, int DC>
__device__ __forceinline__ void epilogue_loop(const EpiCtx& e) {
    using Sh = EpiShape<QJL, SPLITACC>;
    const Params& p = e.p;
    const int group = e.warp / Sh::WPG, quad = e.warp & 3, part = (e.warp % Sh::WPG) >> 2, row_in_tile = quad * 32 + e.lane;
    const int d = DC ? DC : p.d, half = BL ? d / 2 : d;
    const int nch_h = half / 16, nch_l = BL ? (d - half) / 16 : 0;                   // chunks of sixteen coordinates per bit width
    // this thread's chunks: [h0, h1) of the first width, [l0, l1) of the second
    // (share q of n chunks: [ceil(q n / SPLIT), ceil((q + 1) n / SPLIT)); the second width is dealt from the other end so
    // that the shares of a fractional row add up evenly)
    const int h0 = (part * nch_h + Sh::SPLIT - 1) / Sh::SPLIT, h1 = ((part + 1) * nch_h + Sh::SPLIT - 1) / Sh::SPLIT;
    const int l0 = part * nch_l / Sh::SPLIT, l1 = (part + 1) * nch_l / Sh::SPLIT;
    const float* raw_h = reinterpret_cast<const float*>(e.smem + OFF_BND);
    const float* raw_l = raw_h + 16;
    const float* cent_h = raw_h + 32;
    const float* cent_l = raw_h + 48;
    Sketch sk;
    sk.stage = static_cast<uint32_t>(__cvta_generic_to_shared(e.smem + OFF_SKETCH)) + uint32_t(e.warp) * 32 * SK_LD;
    sk.bfrag = reinterpret_cast<const uint2*>(e.smem + OFF_PT);
    sk.lane = e.lane;
    RowCtx rc;
    rc.bins = reinterpret_cast<const float2*>(e.smem + OFF_BINS) + (e.lane & (BIN_REP - 1));      // 4-bit side only
    float bnd_h[7], bnd_l[7];
#pragma unroll
    for (int i = 0; i < 7; ++i) { bnd_h[i] = raw_h[(BH <= 3 && i < (1 << BH) - 1) ? i : 0]; bnd_l[i] = raw_l[(BL >= 1 && BL <= 3 && i < (1 << BL) - 1) ? i : 0]; }
    const uint32_t tpl = uint32_t(p.tiles_per_lane);
    const int a_stages = p.a_stages;
    const int nb_h = half * BH / 8, nb_l = BL ? (d - half) * BL / 8 : 0;            // bytes of a packed row (per width)
    int s = group % a_stages;                                                       // operand stage of iteration `it`
    // (cache lane, tile inside the lane) of the group's current tile, advanced by the group's tile stride: one division here
    const uint32_t first_tile = blockIdx.x + uint32_t(group) * gridDim.x, stride_tiles = uint32_t(Sh::GROUPS) * gridDim.x;
    uint32_t lane_o = first_tile / tpl, tl = first_tile - lane_o * tpl;
    const uint32_t step_o = stride_tiles / tpl, step_t = stride_tiles - step_o * tpl;
    for (int64_t tile = first_tile, it = group; tile < p.n_tiles; tile += stride_tiles, it += Sh::GROUPS) {
        const int a = int(it % Sh::STAGES);
        if (!mbar_wait(e.bar_accfull + 8 * a, uint32_t(it / Sh::STAGES) & 1u, e.abort_flag, 3)) break;
        if (!mbar_wait(e.bar_nrm + 8 * s, uint32_t(it / a_stages) & 1u, e.abort_flag, 5)) break;     // sums of squares written
        tc_fence_after();
        const float* nsq = reinterpret_cast<const float*>(e.smem + OFF_NSQ) + s * 2 * TM;
        const float nrm = sqrtf(nsq[row_in_tile] + nsq[TM + row_in_tile]);
        mbar_arrive(e.bar_afree + 8 * s);                       // norm slots of this stage are free again
        s = (s + Sh::GROUPS) % a_stages;
        const float nden = fmaxf(nrm, 1e-10f);                  // cache.py:237-238 guards the zero vector the same way
        rc.rinv = 1.f / nden;
        rc.rbin = rc.rinv * 256.f;
        // register search: y / |x| > b is tested as y > b * |x| (one multiply per boundary and row instead of one per coordinate)
        float sb_h[7], sb_l[7];
#pragma unroll
        for (int i = 0; i < 7; ++i) { sb_h[i] = bnd_h[i] * nden; sb_l[i] = bnd_l[i] * nden; }
        const int64_t lane_r = int64_t(tl) * TM + row_in_tile;
        const bool live = lane_r < p.n_rows;                    // rows past the lane's end were zero-filled by the copy
        const int64_t orow = int64_t(lane_o) * p.out_lane_stride + lane_r;
        lane_o += step_o; tl += step_t;
        if (tl >= tpl) { tl -= tpl; ++lane_o; }
        const uint32_t t_row = e.tmem_base + (uint32_t(quad * 32) << 16) + a * Sh::STAGE_COLS;
        float ee = 0.f;
        if (QJL) {
#pragma unroll
            for (int i = 0; i < 32; ++i) (&sk.acc[0][0][0])[i] = 0.f;
        }
        // with head_dim 128 and quarter shares every thread has two chunks of an integer width, or one of each fractional width
        constexpr int NCH_H = (DC == 128 && Sh::SPLIT == 4) ? (BL ? 1 : 2) : 0, NCH_L = (DC == 128 && Sh::SPLIT == 4) ? 1 : 0;
        quantize_part<BH, QJL, SPLITACC, NCH_H>(t_row, h0 * 16, h1 - h0, d, rc, sb_h, raw_h, cent_h, p.p_hi + orow * nb_h + h0 * 2 * BH, live, sk, ee);
        if (BL) quantize_part<(BL ? BL : 1), QJL, SPLITACC, NCH_L>(t_row, half + l0 * 16, l1 - l0, d, rc, sb_l, raw_l, cent_l, p.p_lo + orow * nb_l + l0 * 2 * BL, live, sk, ee);
        tc_fence_before();
        mbar_arrive(e.bar_accfree + 8 * a);                     // the accumulator may be overwritten
        uint32_t zb = 0;
        if (QJL) zb = sketch_bits(sk);                          // (every lane of the warp takes part)
        if (live && part == 0) {
            p.norms[orow] = nrm;
            if (QJL) {
                if (nrm == 0.f) zb = 0xffffffffu;               // zero row: the reference's residual is exactly 0, and 0 >= 0
                p.qjl_bits[orow] = zb;
                p.qjl_gamma[orow] = nrm * sqrtf(ee) * (1.f / 256.f);   // |x - dequant(x)| = |x| |y_n - c| (the rotation is orthogonal); ee sums 2^16 times the squares
            }
        }
    }
}

// SPLITACC (fp16 rows without the sketch): high and low products in two accumulators, one MMA of N = 2 d per k-step
// against [R_hi ; R_lo].  Otherwise one accumulator: fp16 low products first and the scale-input-d trick, bf16 three terms.
template <bool QJL, bool SPLITACC, int DC>
__global__ void __launch_bounds__(n_threads(QJL), 1) quantize_tc_kernel(Params p, const __grid_constant__ CUtensorMap tmap) {
    using Sh = EpiShape<QJL, SPLITACC>;
    constexpr int ACCS = Sh::STAGES, NT = Sh::NT, EPI_WARPS = Sh::EW, N_EPI = Sh::N_EPI;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    const int d = DC ? DC : p.d, a_stages = p.a_stages;
    const bool bf16 = p.bf16 != 0;
    // barriers: full[3] (TMA -> MMA, norms), a_free[3] (MMA commit + norm warps + the epilogue's norm read -> TMA),
    //           nrm[3] (norm warps -> epilogue), acc_full[4] (MMA commit -> epilogue group), acc_free[4] (epilogue group -> MMA)
    const uint32_t bar_full = sbase + OFF_BAR, bar_afree = bar_full + 8 * A_STAGES_MAX, bar_nrm = bar_afree + 8 * A_STAGES_MAX;
    const uint32_t bar_accfull = bar_nrm + 8 * A_STAGES_MAX, bar_accfree = bar_accfull + 8 * ACC_STAGES;      // (ACCS of the 4 slots are used)

    if (sbase & 1023u) {                  // the swizzled operand tiles need 1024-byte alignment (uniform across the CTA)
        if (tid == 0) atomicCAS(&g_status, 0, 9);
        return;
    }
    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < A_STAGES_MAX; ++s) {
            // one arrival (the issuing thread, with the byte count) fills a stage; it is free again once the MMAs have
            // committed, the norm warps have read the rows and the tile's epilogue group has read the norms
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_afree + 8 * s, 1 + N_NORM + N_EPI / Sh::GROUPS);
            mbar_init(bar_nrm + 8 * s, N_NORM);
        }
        for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(bar_accfull + 8 * a, 1); mbar_init(bar_accfree + 8 * a, N_EPI / Sh::GROUPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // R -> operand tiles (swizzled K-major): B[n = j][k] = R[j][k], rows j < d, 16-byte chunks c < d / 8
    for (int idx = tid; idx < d * (d / 8); idx += NT) {
        const int j = idx / (d / 8), c = idx - j * (d / 8);      // row j, chunk c (8 elements) of the row
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p.rot + j * d + c * 8));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p.rot + j * d + c * 8 + 4));
        const float v[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
        const int kblk = c >> 3, cc = c & 7;
        const int off = kblk * KBLK_BYTES + j * 128 + ((cc ^ (j & 7)) << 4);
        if (SPLITACC) {
            // one operand of 2 d rows per K-block: row j = R_hi[j], row d + j = 2^11 R_lo[j] (K-blocks 32 KB apart)
            __align__(16) __half hi[8], lo[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hi[i] = __float2half_rn(v[i]);
                lo[i] = __float2half_rn((v[i] - __half2float(hi[i])) * 2048.f);
            }
            const int jl = d + j;
            *reinterpret_cast<uint4*>(smem + OFF_R1 + kblk * (2 * KBLK_BYTES) + j * 128 + ((cc ^ (j & 7)) << 4)) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(smem + OFF_R1 + kblk * (2 * KBLK_BYTES) + jl * 128 + ((cc ^ (jl & 7)) << 4)) = *reinterpret_cast<const uint4*>(lo);
        } else if (!bf16) {
            __align__(16) __half hi[8], lo[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                hi[i] = __float2half_rn(v[i]);
                lo[i] = __float2half_rn((v[i] - __half2float(hi[i])) * 2048.f);
            }
            *reinterpret_cast<uint4*>(smem + OFF_R1 + off) = *reinterpret_cast<const uint4*>(hi);
            *reinterpret_cast<uint4*>(smem + OFF_R2 + off) = *reinterpret_cast<const uint4*>(lo);
        } else {
            __align__(16) __nv_bfloat16 t1[8], t2[8], t3[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                t1[i] = __float2bfloat16_rn(v[i]);
                const float r1 = v[i] - __bfloat162float(t1[i]);               // exact
                t2[i] = __float2bfloat16_rn(r1);
                t3[i] = __float2bfloat16_rn(r1 - __bfloat162float(t2[i]));     // exact remainder, 8 bits left at most
            }
            *reinterpret_cast<uint4*>(smem + OFF_R1 + off) = *reinterpret_cast<const uint4*>(t1);
            *reinterpret_cast<uint4*>(smem + OFF_R2 + off) = *reinterpret_cast<const uint4*>(t2);
            *reinterpret_cast<uint4*>(smem + OFF_R3 + off) = *reinterpret_cast<const uint4*>(t3);
        }
    }
    {
        float* raw = reinterpret_cast<float*>(smem + OFF_BND);
        if (tid < 64) {
            const int which = tid >> 4, i = tid & 15;                    // 0 / 1: boundaries hi / lo, 2 / 3: centroids hi / lo
            const int bits = (which & 1) ? p.bits_lo : p.bits_hi;
            float val = which < 2 ? INFINITY : 0.f;
            if (which < 2) {
                const float* src = which ? p.bnd_lo : p.bnd_hi;
                if (src != nullptr && bits > 0 && i < (1 << bits) - 1) val = src[i];
            } else if (QJL) {
                const float* src = (which & 1) ? p.cent_lo : p.cent_hi;
                if (src != nullptr && bits > 0 && i < (1 << bits)) val = src[i] * 256.f;     // (the sketch works on 2^8 times the residual)
            }
            raw[tid] = val;
        }
        if (QJL) {
            // (S R^T) is (32, d): as mma B fragments (k = coordinate, n = projection), fp16 high and low parts;
            // lane (g, t) of fragment (k-step ks, n-tile nt): b0 = coordinates 16 ks + 2t, + 1 of projection 8 nt + g, b1 = the same + 8
            uint2* bf = reinterpret_cast<uint2*>(smem + OFF_PT);
            for (int idx = tid; idx < (d / 16) * 4 * 32; idx += NT) {
                const int ks = idx >> 7, nt = (idx >> 5) & 3, ln = idx & 31, g = ln >> 2, t = ln & 3;
                const float* srow = p.qjl_proj_rot + (8 * nt + g) * d + 16 * ks + 2 * t;
                uint32_t hw[2], lw[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float x0 = __ldg(srow + 8 * u), x1 = __ldg(srow + 8 * u + 1);
                    const __half2 h = __floats2half2_rn(x0, x1);
                    const float2 hf = __half22float2(h);
                    const __half2 l = __floats2half2_rn(x0 - hf.x, x1 - hf.y);
                    hw[u] = *reinterpret_cast<const uint32_t*>(&h);
                    lw[u] = *reinterpret_cast<const uint32_t*>(&l);
                }
                bf[((ks * 4 + nt) * 2 + 0) * 32 + ln] = make_uint2(hw[0], hw[1]);
                bf[((ks * 4 + nt) * 2 + 1) * 32 + ln] = make_uint2(lw[0], lw[1]);
            }
        }
        __syncthreads();
        if (p.bits_hi == 4) build_bins(reinterpret_cast<float2*>(smem + OFF_BINS), raw, 15, tid, NT);
    }
    if (warp == EPI_WARPS) {              // one warp owns the TMEM allocation: 4 stages x 128 columns
        tmem_alloc(sbase + OFF_MISC, 512);
        tmem_relinquish();
    }
    fence_proxy_async();                  // the operand tiles written above are read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t oper_bytes = d > 64 ? OPER_BYTES : KBLK_BYTES;        // bytes one tile's copies deliver

    if (warp < EPI_WARPS) {
        // ======================= epilogue: row = 32 * (warp % 4) + lane; groups and column halves as in EpiShape =======================
        EpiCtx e{p, smem, tmem_base, bar_accfull, bar_accfree, bar_afree, bar_nrm, abort_flag, warp, lane};
        const int key = p.bits_hi * 8 + p.bits_lo;
        switch (key) {
            case 4 * 8 + 0: epilogue_loop<4, 0, QJL, SPLITACC, DC>(e); break;
            case 3 * 8 + 0: epilogue_loop<3, 0, QJL, SPLITACC, DC>(e); break;
            case 2 * 8 + 0: epilogue_loop<2, 0, QJL, SPLITACC, DC>(e); break;
            case 1 * 8 + 0: epilogue_loop<1, 0, QJL, SPLITACC, DC>(e); break;
            case 4 * 8 + 3: epilogue_loop<4, 3, QJL, SPLITACC, DC>(e); break;
            case 3 * 8 + 2: epilogue_loop<3, 2, QJL, SPLITACC, DC>(e); break;
            case 2 * 8 + 1: epilogue_loop<2, 1, QJL, SPLITACC, DC>(e); break;
            default: break;               // the host only launches the combinations above
        }
    } else if (warp == EPI_WARPS) {
        // ======================= MMA issue: one elected thread =======================
        if (lane == 0) {
            const uint32_t idesc = make_idesc(SPLITACC ? 2 * d : d, bf16);
            const int ksteps = d / 16;
            int it = 0;
            for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
                const int a = it % ACCS, s = it % a_stages;
                if (it >= ACCS && !mbar_wait(bar_accfree + 8 * a, uint32_t((it / ACCS) - 1) & 1u, abort_flag, 2)) break;
                if (!mbar_wait(bar_full + 8 * s, uint32_t(it / a_stages) & 1u, abort_flag, 1)) break;
                tc_fence_after();
                const uint32_t a_tile = sbase + OFF_A + s * OPER_BYTES;
                const uint32_t d_acc = tmem_base + a * Sh::STAGE_COLS;
                if (SPLITACC) {
                    // columns [0, d): x.R_hi, columns [d, 2 d): 2^11 x.R_lo; the operand's K-blocks are 32 KB apart
#ifdef EXP_TWO_MMA
                    const uint32_t idesc1 = make_idesc(d, bf16);
                    for (int ks = 0; ks < ksteps; ++ks) {
                        const uint64_t da = smem_desc(a_tile, ks >> 2, ks & 3);
                        const uint32_t rb = sbase + OFF_R1 + (ks >> 2) * KBLK_BYTES;
                        umma_f16(d_acc, da, smem_desc(rb, ks >> 2, ks & 3), idesc1, ks ? 1u : 0u);
                        umma_f16(d_acc + d, da, smem_desc(rb + d * 128, ks >> 2, ks & 3), idesc1, ks ? 1u : 0u);
                    }
#else
                    for (int ks = 0; ks < ksteps; ++ks)
                        umma_f16(d_acc, smem_desc(a_tile, ks >> 2, ks & 3), smem_desc(sbase + OFF_R1 + (ks >> 2) * KBLK_BYTES, ks >> 2, ks & 3), idesc, ks ? 1u : 0u);
#endif
                } else if (!bf16) {
                    for (int ks = 0; ks < ksteps; ++ks)            // 2^11-scaled low products first
                        umma_f16(d_acc, smem_desc(a_tile, ks >> 2, ks & 3), smem_desc(sbase + OFF_R2, ks >> 2, ks & 3), idesc, ks ? 1u : 0u);
                    umma_f16_scaled11(d_acc, smem_desc(a_tile, 0, 0), smem_desc(sbase + OFF_R1, 0, 0), idesc);    // acc = x.R_hi + 2^-11 acc
                    for (int ks = 1; ks < ksteps; ++ks)
                        umma_f16(d_acc, smem_desc(a_tile, ks >> 2, ks & 3), smem_desc(sbase + OFF_R1, ks >> 2, ks & 3), idesc, 1u);
                } else {
                    const int r_off[3] = {OFF_R3, OFF_R2, OFF_R1};   // smallest term first
                    for (int term = 0; term < 3; ++term)
                        for (int ks = 0; ks < ksteps; ++ks)
                            umma_f16(d_acc, smem_desc(a_tile, ks >> 2, ks & 3), smem_desc(sbase + r_off[term], ks >> 2, ks & 3), idesc, (term | ks) ? 1u : 0u);
                }
                umma_commit(bar_afree + 8 * s);      // rows of this stage consumed
                umma_commit(bar_accfull + 8 * a);    // the accumulator is complete: its epilogue group may read it
            }
        }
        __syncwarp();
    } else if (warp == EPI_WARPS + 1 + N_NORM / 32) {
        // ======================= TMA issue: one thread keeps the operand stages full =======================
        if (lane == 0) {
            const uint32_t tpl = uint32_t(p.tiles_per_lane);
            int it = 0;
            for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
                const int s = it % a_stages;
                if (it >= a_stages && !mbar_wait(bar_afree + 8 * s, uint32_t((it / a_stages) - 1) & 1u, abort_flag, 6)) break;
                const uint32_t t32 = uint32_t(tile), o = t32 / tpl, tl = t32 - o * tpl;
                const uint32_t a_tile = sbase + OFF_A + s * OPER_BYTES;
                mbar_expect_tx(bar_full + 8 * s, oper_bytes);
                tma_load_3d(a_tile, &tmap, 0, int(tl * TM), int(o), bar_full + 8 * s);                              // columns 0..63
                if (d > 64) tma_load_3d(a_tile + KBLK_BYTES, &tmap, 64, int(tl * TM), int(o), bar_full + 8 * s);    // columns 64..127 (zeros past d)
            }
        }
        __syncwarp();
    } else {
        // ======================= norm warps: sum of squares of every row, read back from the stage =======================
        // thread -> row 32 nw + lane, both 64-column blocks: eight consecutive rows hit eight different 16-byte columns
        // of the swizzled tile, so the 128-bit reads are free of bank conflicts
        const int nw = warp - (EPI_WARPS + 1), r = nw * 32 + lane;
        int it = 0;
        for (int64_t tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
            const int s = it % a_stages;
            if (!mbar_wait(bar_full + 8 * s, uint32_t(it / a_stages) & 1u, abort_flag, 7)) break;
            const unsigned char* rowp = smem + OFF_A + s * OPER_BYTES + r * 128;
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = *reinterpret_cast<const uint4*>(rowp + ((c ^ (r & 7)) << 4));
                uint4 w = make_uint4(0, 0, 0, 0);
                if (d > 64) w = *reinterpret_cast<const uint4*>(rowp + KBLK_BYTES + ((c ^ (r & 7)) << 4));
                if (!bf16) {
                    const __half2* h = reinterpret_cast<const __half2*>(&v);
                    const __half2* g = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float2 f = __half22float2(h[u]), e = __half22float2(g[u]);
                        a = fmaf(f.x, f.x, a); a = fmaf(f.y, f.y, a);
                        b = fmaf(e.x, e.x, b); b = fmaf(e.y, e.y, b);
                    }
                } else {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
                    const __nv_bfloat162* g = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float2 f = __bfloat1622float2(h[u]), e = __bfloat1622float2(g[u]);
                        a = fmaf(f.x, f.x, a); a = fmaf(f.y, f.y, a);
                        b = fmaf(e.x, e.x, b); b = fmaf(e.y, e.y, b);
                    }
                }
            }
            float* nsq = reinterpret_cast<float*>(smem + OFF_NSQ) + s * 2 * TM;
            nsq[r] = a; nsq[TM + r] = b;
            mbar_arrive(bar_nrm + 8 * s);        // release: the epilogue reads the sums after waiting on this barrier
            mbar_arrive(bar_afree + 8 * s);      // this thread is done reading the stage
        }
    }
    // ---- teardown: every loop above is bounded, so every thread gets here ----
    tc_fence_before();
    __syncthreads();
    if (warp == EPI_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace tc

}  // namespace tq

using namespace tq;

// Takes the call when it fits the tensor-core kernel: fp16 / bf16 rows, d in {64, 96, 128}, 16-byte aligned rows, no
// rotated-row output, a bit-width pair the epilogue is compiled for.  Otherwise reports "not handled" and the caller uses
// the general CUDA-core kernel.
int tq_quantize_pack_tc(const tq_quantize_args* q, cudaStream_t s, bool* handled) {
    *handled = false;
    const int d = q->d;
    if ((d != 64 && d != 96 && d != 128) || (q->x_dtype != TQ_F16 && q->x_dtype != TQ_BF16) || q->y_out) return TQ_OK;
    const bool frac = q->bits_lo != 0;
    if (frac && (q->bits_hi != q->bits_lo + 1)) return TQ_OK;                  // the reference's fractional widths only
    if (!aligned(q->x, 16) || q->x_row_stride % 8 || q->x_lane_stride % 8 || !aligned(q->rot, 16)) return TQ_OK;
    if (q->n_rows >= (int64_t(1) << 31) || q->n_lanes >= (int64_t(1) << 31)) return TQ_OK;
    static int disabled = -1;
    if (disabled < 0) {
        const char* e = getenv("TQ_DISABLE_TC");
        disabled = (e && e[0] == '1') ? 1 : 0;
    }
    if (disabled) return TQ_OK;
    const int64_t total = q->n_lanes * q->n_rows;
    if (total < 4 * tc::TM) return TQ_OK;            // tiny inputs: not worth a persistent launch
    const bool qjl = q->qjl_bits != nullptr;
    static bool attr_set[16] = {false};
    static int sms[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) return TQ_OK;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(tc::quantize_tc_kernel<false, true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<false, true, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<false, false, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(tc::quantize_tc_kernel<true, false, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::SMEM_BYTES);
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_quantize_pack: shared memory %d B: %s", tc::SMEM_BYTES, cudaGetErrorString(e));
        if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0) sms[dev] = 148;
        attr_set[dev] = true;
    }
    static PFN_cuTensorMapEncodeTiled encode = nullptr;
    static bool looked_up = false;
    if (!looked_up) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
        looked_up = true;
    }
    if (!encode) return TQ_OK;
    // Tensor map over the rows as (column, row, lane): boxes of 64 columns x 128 rows x 1 lane land in shared memory in
    // the 128-byte-swizzled layout the MMA descriptors describe; rows past a lane's end and columns past d read as zeros.
    CUtensorMap tmap{};
    const cuuint64_t dims[3] = {cuuint64_t(d), cuuint64_t(q->n_rows), cuuint64_t(q->n_lanes)};
    const cuuint64_t strides[2] = {cuuint64_t(q->x_row_stride) * 2, cuuint64_t(q->x_lane_stride ? q->x_lane_stride : q->x_row_stride * q->n_rows) * 2};   // bytes, multiples of 16
    const cuuint32_t box[3] = {64, cuuint32_t(tc::TM), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(&tmap, q->x_dtype == TQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(q->x),
                              dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TQ_OK;

    tc::Params p{};
    p.d = d; p.bf16 = q->x_dtype == TQ_BF16 ? 1 : 0; p.a_stages = p.bf16 ? 2 : 3;
    p.n_rows = q->n_rows;
    p.tiles_per_lane = (q->n_rows + tc::TM - 1) / tc::TM;
    p.n_tiles = q->n_lanes * p.tiles_per_lane;
    if (p.n_tiles >= (int64_t(1) << 31)) return TQ_OK;
    p.rot = q->rot; p.bnd_hi = q->bnd_hi; p.bnd_lo = q->bnd_lo; p.bits_hi = q->bits_hi; p.bits_lo = q->bits_lo;
    p.p_hi = q->packed_hi; p.p_lo = q->packed_lo; p.norms = q->norms; p.out_lane_stride = q->out_lane_stride;
    p.qjl_proj_rot = q->qjl_proj_rot; p.cent_hi = q->cent_hi; p.cent_lo = q->cent_lo; p.qjl_bits = q->qjl_bits; p.qjl_gamma = q->qjl_gamma;
    const unsigned grid = unsigned(std::min<int64_t>(p.n_tiles, sms[dev]));
    if (qjl) tc::quantize_tc_kernel<true, false, 0><<<grid, tc::n_threads(true), tc::SMEM_BYTES, s>>>(p, tmap);
    else if (p.bf16) tc::quantize_tc_kernel<false, false, 0><<<grid, tc::n_threads(false), tc::SMEM_BYTES, s>>>(p, tmap);
    else if (d == 128) tc::quantize_tc_kernel<false, true, 128><<<grid, tc::n_threads(false), tc::SMEM_BYTES, s>>>(p, tmap);
    else tc::quantize_tc_kernel<false, true, 0><<<grid, tc::n_threads(false), tc::SMEM_BYTES, s>>>(p, tmap);
    *handled = true;
    return check_launch("tq_quantize_pack (tensor core)");
}

namespace tq { int decode_status_host(); int decode_status_clear(); }   // decode_direct.cu

// 0 if no kernel on the current device has reported a timed-out wait, else the code of the first one.
// Synchronises the device.
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
