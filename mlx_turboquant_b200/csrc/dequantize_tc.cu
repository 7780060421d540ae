// Dequantize on the fifth-generation tensor cores: unpack -> centroid -> inverse rotation -> scale
// (TurboQuantMSE.dequantize / cache._dequantize_kv(_fractional) / metal_dequantize: quantizer.py:87-109,
// cache.py:276-343, kernels.py:313-360) for head_dim 64 / 96 / 128, any bit width 1-4, fractional splits; rows with a
// QJL correction, head_dim 256 and unaligned outputs stay with the CUDA-core row kernel (rowops.cu).
//
//   out[t][j] = norm[t] * sum_k c[code(t, k)] R[k][j]          (y @ R, rotation.py:68-78)
//
// is a dense 128 x d x d contraction per 128 rows.  To stay float32-faithful on fp16 operands both factors are split,
// c = c_hi + 2^-11 c_lo and R = R_hi + 2^-11 R_lo, and three products are kept: c_hi R_hi in one accumulator,
// c_hi R_lo + c_lo R_hi in a second one that the epilogue adds with weight 2^-11 (the fourth product is below float32
// resolution).
//
// Persistent CTAs (one per SM) walk the 128-row tiles, warp-specialised:
//   * warps 4-7 and 9-12 (two groups, alternating tiles) unpack a tile's codes into two fp16 A-operand tiles (hi / lo parts of the centroids; K-major, 128-byte
//     swizzle), buffer t & 1, and stage the rows' norms and output offsets;
//   * one thread of warp 8 issues the 2 x d/16 tcgen05.mma of the tile (c_hi [R_hi | R_lo] with N 256, c_lo R_hi with N 128;
//     M 128, K 16) into accumulator pair t & 1
//     of tensor memory - R sits in shared memory as two MN-major B tiles built once per CTA - and commits to mbarriers;
//   * warps 0-3 own the 128 accumulator lanes (a row per thread): tcgen05.ld of both accumulators, combine, scale by the
//     norm, convert, and write out through a small per-warp staging area so that stores cover whole 128-byte lines.
// Every mbarrier wait is bounded (status 105); tensor memory is freed on every path.
#include <algorithm>

#include "common.cuh"

namespace tq {

int* decode_status_ptr();

namespace dqtc {

constexpr int TM = 128, NT = 416, ROW_T = 128, PROD_T = 128;          // warps 0-3 rows, 4-7 and 9-12 two producer groups, 8 MMA issue
constexpr uint32_t KBLK = 16384, TILE_BYTES = 2 * KBLK;                     // a 128 x 128 fp16 operand tile: two 64-column blocks
constexpr uint32_t OFF_RHI = 0, OFF_RLO = TILE_BYTES;                       // R as B operands (rows = k, columns = j)
constexpr uint32_t OFF_A = 2 * TILE_BYTES;                                  // [2 buffers][hi, lo] A tiles
constexpr uint32_t OFF_NRM = 6 * TILE_BYTES;                                // float   [4][128] row norms (slot = tile & 3)
constexpr uint32_t OFF_OFFS = OFF_NRM + 2048;                               // int64   [4][128] output element offsets (-1: no such row)
constexpr uint32_t OFF_CTAB = OFF_OFFS + 4096;                              // uint32  [2][16] centroids as {hi, lo} fp16 pairs: first half's table, second half's
constexpr uint32_t STAGE_LD = 144;                                          // bytes per staged row: 128 + 16 (rows start four banks apart)
constexpr uint32_t OFF_STAGE = OFF_CTAB + 128;                              // [4 warps][32 rows][STAGE_LD] results on their way out
constexpr uint32_t OFF_BAR = OFF_STAGE + 4 * 32 * STAGE_LD;
constexpr uint32_t OFF_SLOT = OFF_BAR + 64;                                 // [0] tensor-memory base, [1] abort
constexpr uint32_t SMEM_USED = OFF_SLOT + 16;
constexpr size_t SMEM_BYTES = SMEM_USED + 1024;
static_assert(SMEM_BYTES <= 227u * 1024u, "shared-memory plan");
constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_WAIT = 105;
constexpr int PF_AHEAD = 4;                                                 // a tile's packed rows are asked for in L2 this many tiles early
constexpr uint32_t TMEM_COLS = 512;                                         // buffer b: c_hi R_hi at 256 b, the mixed products at 256 b + 128
enum Bars { A_FULL = 0, A_FREE = 2, ACC_FULL = 4, ACC_FREE = 6 };

struct Params {
    const uint8_t* packed_hi; const uint8_t* packed_lo; const float* norms;
    int64_t n_rows, in_lane_stride, total;          // rows per lane, lane stride (rows), lanes x rows
    int d, half, bits_hi, bits_lo, w_hi, w_lo;      // half: coordinates in packed_hi; w: bytes per packed row
    const float* cent_hi; const float* cent_lo; const float* rot;
    void* out; int out_dtype; int64_t out_lane_stride, out_row_stride;
    int n_tiles;
    int* status;
};

// ---- PTX wrappers -----------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
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
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }
__device__ __forceinline__ uint32_t h2_bits(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Operand tiles: 128 rows of 128 fp16 as two blocks of 64 columns (16 KB each); row r of a block at r * 128 B, its
// 16-byte chunk c at chunk position c ^ (r & 7) (128-byte swizzle; tiles are 1024-byte aligned).
__device__ __forceinline__ uint32_t chunk_off(int r, int c16) {
    return uint32_t(c16 >> 3) * KBLK + uint32_t(r) * 128u + (uint32_t((c16 & 7) ^ (r & 7)) << 4);
}
// K-major descriptor (rows = M index, 64-column blocks along K): the 16-column slab `ks` of the tile
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int ks) {
    const uint32_t addr = tile_addr + uint32_t(ks >> 2) * KBLK + uint32_t(ks & 3) * 32u;
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);
    d |= uint64_t(1) << 16;
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// MN-major descriptor of a tile whose rows are the K index and whose 128 columns are the N index: the 16-row slab `ks`
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int ks) {
    const uint32_t addr = tile_addr + uint32_t(ks) * 2048u;
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);
    d |= uint64_t(KBLK >> 4) << 16;               // leading byte offset: the second block of 64 columns
    d |= uint64_t(1024 >> 4) << 32;               // stride byte offset: the next 8 rows
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// kind::f16: fp32 accumulate, fp16 A (K-major) and B (MN-major), M = 128, N = 128
constexpr uint32_t IDESC = (1u << 4) | (1u << 16) | (uint32_t(128 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
constexpr uint32_t IDESC_N256 = (1u << 4) | (1u << 16) | (uint32_t(256 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
static_assert(OFF_RLO == OFF_RHI + TILE_BYTES, "the N = 256 product reads R_hi and R_lo as one operand");

// Eight codes of BITS bits each: BITS bytes of a packed row (4 bits: one aligned word; 2 bits: an aligned half-word).
template <int BITS> __device__ __forceinline__ uint32_t load_codes(const uint8_t* src) {
    if (BITS == 4) return __ldg(reinterpret_cast<const uint32_t*>(src));
    if (BITS == 2) return __ldg(reinterpret_cast<const uint16_t*>(src));
    if (BITS == 1) return __ldg(src);
    return uint32_t(__ldg(src)) | (uint32_t(__ldg(src + 1)) << 8) | (uint32_t(__ldg(src + 2)) << 16);
}

// BH / BL: bits of the first / second half of the coordinates (BL = 0: one width for the whole row); compile-time so that the
// code extraction is immediate shifts and masks.
template <int BH, int BL>
__global__ void __launch_bounds__(NT, 1) dequantize_tc_kernel(Params p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t raw_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t sbase = (raw_addr + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw_addr);
    float* s_nrm = reinterpret_cast<float*>(smem + OFF_NRM);
    long long* s_off = reinterpret_cast<long long*>(smem + OFF_OFFS);
    uint32_t* ctab = reinterpret_cast<uint32_t*>(smem + OFF_CTAB);
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_SLOT);
    auto bar = [&](int which) -> uint32_t { return sbase + OFF_BAR + 8u * uint32_t(which); };
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int d = p.d;

    // ---------------- set-up: barriers, tensor memory, centroid tables, R as two fp16 B tiles ------------------------
    if (tid == 0) {
        mbar_init(bar(A_FULL), PROD_T); mbar_init(bar(A_FULL + 1), PROD_T);
        mbar_init(bar(A_FREE), 1); mbar_init(bar(A_FREE + 1), 1);
        mbar_init(bar(ACC_FULL), 1); mbar_init(bar(ACC_FULL + 1), 1);
        mbar_init(bar(ACC_FREE), ROW_T); mbar_init(bar(ACC_FREE + 1), ROW_T);
        fence_barrier_init();
        slot[1] = 0u;
    }
    if (warp == 8) {
        tmem_alloc(sbase + OFF_SLOT, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid < 32) {
        const int which = tid >> 4, k = tid & 15;
        const float* src = which ? p.cent_lo : p.cent_hi;
        const int bits = which ? p.bits_lo : p.bits_hi;
        float c = 0.f;
        if (src != nullptr && bits > 0 && k < (1 << bits)) c = src[k];
        const __half hi = __float2half_rn(c);
        const __half lo = __float2half_rn((c - __half2float(hi)) * 2048.f);
        ctab[tid] = uint32_t(__half_as_ushort(hi)) | (uint32_t(__half_as_ushort(lo)) << 16);
    }
    for (int i = tid; i < 128 * 16; i += NT) {                               // chunk (row k, columns 8 c .. 8 c + 7) of R
        const int k = i >> 4, c = i & 15;
        uint32_t hi[4] = {0u, 0u, 0u, 0u}, lo[4] = {0u, 0u, 0u, 0u};
        if (k < d && c * 8 < d) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(p.rot + int64_t(k) * d + c * 8));
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.rot + int64_t(k) * d + c * 8 + 4));
            const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __half2 h = __floats2half2_rn(x[2 * u], x[2 * u + 1]);
                const float2 hf = __half22float2(h);
                hi[u] = *reinterpret_cast<const uint32_t*>(&h);
                lo[u] = h2_bits((x[2 * u] - hf.x) * 2048.f, (x[2 * u + 1] - hf.y) * 2048.f);
            }
        }
        *reinterpret_cast<uint4*>(smem + OFF_RHI + chunk_off(k, c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(smem + OFF_RLO + chunk_off(k, c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slot[0];

    auto wait_bar = [&](uint32_t addr, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
            if (mbar_try(addr, parity)) return true;
            if ((i & 1023u) == 1023u && slot[1]) return false;
        }
        slot[1] = 1u;
        atomicCAS(p.status, 0, ERR_WAIT);
        return false;
    };
    const int n_mine = p.n_tiles > int(blockIdx.x) ? (p.n_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;   // tiles blockIdx.x, + gridDim.x, ...
    const int ksteps = d / 16;

    if ((warp >= 4 && warp < 8) || warp >= 9) {
        // ======================= producers: two groups of four warps; group g takes the tiles with it & 1 == g (and so always
        // fills A buffer g); warp w of a group unpacks rows 32 w .. 32 w + 31 of the tile.  Two groups keep two tiles' worth
        // of global loads in flight per SM: one group alone was bound by their latency. =======================
        const int grp = warp >= 9 ? 1 : 0;
        const int pw = warp - (grp ? 9 : 4);
        // A tile's packed words, norms and row offsets are requested one tile ahead, before the previous tile is converted:
        // their latency passes under that work.  Chunk c = lane + 32 k of the warp's 32 rows: row c >> 4,
        // coordinates 8 (c & 15) ...; eight codes are `bits` bytes of the packed row.
        uint32_t w[16], wn[16];
        long long off_cur = -1, off_next = -1;
        float nrm_cur = 0.f, nrm_next = 0.f;
        auto request = [&](int it, uint32_t (&w)[16]) {
            const int64_t row0 = (int64_t(blockIdx.x) + int64_t(it) * gridDim.x) * TM;
            const int64_t gr = row0 + pw * 32 + lane;                         // this lane's row of the tile
            long long in_row = -1;
            off_next = -1; nrm_next = 0.f;
            if (gr < p.total) {
                const int64_t ln = gr / p.n_rows, rw = gr - ln * p.n_rows;
                in_row = ln * p.in_lane_stride + rw;
                off_next = ln * p.out_lane_stride + rw * p.out_row_stride;
                nrm_next = __ldg(p.norms + in_row);
            }
            {   // the same row of the tile PF_AHEAD tiles further on: asked for in L2 now (a packed row is at most 64 bytes, so
                // every 128-byte line of the tile holds the start of some row)
                const int64_t gp = gr + int64_t(PF_AHEAD) * gridDim.x * TM;
                if (gp < p.total) {
                    const int64_t ln = gp / p.n_rows, rw = gp - ln * p.n_rows;
                    const int64_t ir = ln * p.in_lane_stride + rw;
                    prefetch_l2(p.packed_hi + ir * p.w_hi);
                    if (BL != 0) prefetch_l2(p.packed_lo + ir * p.w_lo);
                    if ((lane & 31) == 0 || rw == 0) prefetch_l2(p.norms + ir);
                }
            }
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int c = lane + 32 * k, rl = c >> 4, j8 = c & 15;
                const long long src_row = __shfl_sync(0xffffffffu, in_row, rl);
                const bool second = BL != 0 && j8 * 8 >= p.half;
                uint32_t x = 0u;
                if (src_row >= 0 && j8 * 8 < d) {
                    if (!second) x = load_codes<BH>(p.packed_hi + src_row * p.w_hi + j8 * BH);
                    else x = load_codes<BL>(p.packed_lo + src_row * p.w_lo + (j8 - p.half / 8) * BL);
                }
                w[k] = x;
            }
        };
        if (n_mine > grp) request(grp, w);
        off_cur = off_next; nrm_cur = nrm_next;
        for (int it = grp; it < n_mine; it += 2) {
            const int bf = it & 1;
            bool ok = true;
            // the MMAs of tile it - 2 have read the A buffer (the norm / offset slots are four deep: the rows of tile it - 4
            // finished before those MMAs could start)
            if (it >= 2) ok = wait_bar(bar(A_FREE + bf), uint32_t(((it >> 1) - 1) & 1));
            if (!__all_sync(0xffffffffu, ok)) break;
            unsigned char* a_hi = smem + OFF_A + bf * 2 * TILE_BYTES;
            unsigned char* a_lo = a_hi + TILE_BYTES;
            if (it + 2 < n_mine) request(it + 2, wn);                         // in flight while this tile is converted
            s_nrm[(it & 3) * TM + pw * 32 + lane] = nrm_cur;
            s_off[(it & 3) * TM + pw * 32 + lane] = off_cur;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
                const int c = lane + 32 * k, rl = c >> 4, j8 = c & 15;
                if (j8 * 8 >= d) continue;
                const bool second = BL != 0 && j8 * 8 >= p.half;
                uint32_t e[8];
                if (!second) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) e[u] = ctab[(w[k] >> (BH * u)) & ((1u << BH) - 1u)];
                } else {
#pragma unroll
                    for (int u = 0; u < 8; ++u) e[u] = ctab[16 + ((w[k] >> (BL * u)) & ((1u << (BL ? BL : 1)) - 1u))];
                }
                const int r = pw * 32 + rl;
                *reinterpret_cast<uint4*>(a_hi + chunk_off(r, j8)) =
                    make_uint4(__byte_perm(e[0], e[1], 0x5410), __byte_perm(e[2], e[3], 0x5410), __byte_perm(e[4], e[5], 0x5410), __byte_perm(e[6], e[7], 0x5410));
                *reinterpret_cast<uint4*>(a_lo + chunk_off(r, j8)) =
                    make_uint4(__byte_perm(e[0], e[1], 0x7632), __byte_perm(e[2], e[3], 0x7632), __byte_perm(e[4], e[5], 0x7632), __byte_perm(e[6], e[7], 0x7632));
            }
            fence_proxy_async();
            mbar_arrive(bar(A_FULL + bf));
#pragma unroll
            for (int k = 0; k < 16; ++k) w[k] = wn[k];
            off_cur = off_next; nrm_cur = nrm_next;
        }
    } else if (warp == 8) {
        // ======================= MMA issue: one thread =======================
        if (lane == 0) {
            for (int it = 0; it < n_mine; ++it) {
                const int bf = it & 1;
                if (!wait_bar(bar(A_FULL + bf), uint32_t((it >> 1) & 1))) break;
                if (it >= 2 && !wait_bar(bar(ACC_FREE + bf), uint32_t(((it >> 1) - 1) & 1))) break;
                tc_fence_after();
                const uint32_t a_hi = sbase + OFF_A + bf * 2 * TILE_BYTES, a_lo = a_hi + TILE_BYTES;
                const uint32_t acc = tmem_base + uint32_t(bf) * 256u;
                // c_hi [R_hi | R_lo]: one N = 256 product per K step fills both accumulators (the two R tiles are adjacent: four
                // blocks of 64 columns); then c_lo R_hi joins the second one
                for (int ks = 0; ks < ksteps; ++ks)
                    umma_f16(acc, desc_kmajor(a_hi, ks), desc_mnmajor(sbase + OFF_RHI, ks), IDESC_N256, ks > 0 ? 1u : 0u);
                for (int ks = 0; ks < ksteps; ++ks)
                    umma_f16(acc + 128u, desc_kmajor(a_lo, ks), desc_mnmajor(sbase + OFF_RHI, ks), IDESC, 1u);
                umma_commit(bar(A_FREE + bf));
                umma_commit(bar(ACC_FULL + bf));
            }
        }
    } else {
        // ======================= rows: combine, scale, convert, store =======================
        const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16);
        for (int it = 0; it < n_mine; ++it) {
            const int bf = it & 1;
            // (the norms and offsets were written before the producers' arrival that the MMA thread waited for before it issued
            //  the products this barrier tracks; the rows must not wait on A_FULL themselves: its next phase may complete - the
            //  next tile for the buffer only needs the MMAs, not the rows - before a late row thread has looked)
            if (!wait_bar(bar(ACC_FULL + bf), uint32_t((it >> 1) & 1))) break;
            tc_fence_after();
            const float nrm = s_nrm[(it & 3) * TM + tid];
            const long long* offs = s_off + (it & 3) * TM + warp * 32;       // output offsets of this warp's 32 rows
            const uint32_t acc = t_row + uint32_t(bf) * 256u;
            unsigned char* stg = smem + OFF_STAGE + warp * (32 * STAGE_LD);   // this warp's [32 rows][128 bytes + pad]
            // 32 columns at a time: this thread's row out of tensor memory, combined, scaled and converted into the warp's staging
            // rows; once a row's 128 staged bytes are full (64 columns of a 16-bit type, 32 of float32) the warp writes them out
            // with eight lanes per row, so that a store instruction covers four whole 128-byte lines instead of 32 half-sectors
            const int es = p.out_dtype == TQ_F32 ? 4 : 2;
#pragma unroll 1
            for (int c0 = 0; c0 < d; c0 += 32) {
                uint32_t hi[32], lo[32];
                tmem_ld32(acc + c0, hi);
                tmem_ld32(acc + 128u + c0, lo);
                tmem_ld_wait();
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = fmaf(__uint_as_float(lo[j]), 1.f / 2048.f, __uint_as_float(hi[j])) * nrm;
                if (es == 4) {
                    float4* dst = reinterpret_cast<float4*>(stg + lane * STAGE_LD);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(stg + lane * STAGE_LD + ((c0 >> 5) & 1) * 64);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t w[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float x0 = v[8 * j + 2 * u], x1 = v[8 * j + 2 * u + 1];
                            if (p.out_dtype == TQ_F16) w[u] = h2_bits(x0, x1);
                            else {
                                const __nv_bfloat162 bb = __floats2bfloat162_rn(x0, x1);
                                w[u] = *reinterpret_cast<const uint32_t*>(&bb);
                            }
                        }
                        dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                const bool flush = es == 4 || ((c0 >> 5) & 1) == 1 || c0 + 32 >= d;     // the staged rows are complete (or the row ends)
                if (flush) {
                    __syncwarp();
                    const int col0 = es == 4 ? c0 : (c0 & ~63);                        // first column of the staged bytes
                    const int n_bytes = (min(c0 + 32, d) - col0) * es;                 // staged bytes per row: 128, or 64 at the end of a 96-column 16-bit row
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int r = 4 * k + (lane >> 3), ch = lane & 7;
                        const long long o = offs[r];
                        if (o >= 0 && ch * 16 < n_bytes)
                            *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.out) + (o + col0) * es + ch * 16) =
                                *reinterpret_cast<const uint4*>(stg + r * STAGE_LD + ch * 16);
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            mbar_arrive(bar(ACC_FREE + bf));
        }
    }
    // ---------------- teardown: every loop above is bounded, so every thread gets here ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace dqtc

// Dequantize on the tensor cores when the shape allows; *handled = false leaves the call to the row kernel.
int tq_dequantize_tc(const tq_dequantize_args* q, cudaStream_t s, bool* handled) {
    *handled = false;
    const int d = q->d;
    if (d != 64 && d != 96 && d != 128) return TQ_OK;
    if (q->qjl_bits) return TQ_OK;
    if (q->bits_lo && q->bits_lo != q->bits_hi - 1) return TQ_OK;              // the reference's fractional widths are (b, b - 1)
    const int half = q->bits_lo ? d / 2 : d;
    if (half % 8 || (d - half) % 8) return TQ_OK;
    const int es = q->out_dtype == TQ_F32 ? 4 : 2;
    const int64_t vec = 16 / es;                                               // elements per 16-byte store
    if (!aligned(q->out, 16) || q->out_lane_stride % vec || q->out_row_stride % vec || q->out_row_stride < d) return TQ_OK;
    if (!aligned(q->rot, 16)) return TQ_OK;
    // packed rows are read as 4-byte words (4 bits), 2-byte words (2 bits) or bytes
    const int w_hi = half * q->bits_hi / 8, w_lo = q->bits_lo ? (d - half) * q->bits_lo / 8 : 0;
    auto words_ok = [](const void* ptr, int bits, int w) {
        const size_t a = bits == 4 ? 4 : bits == 2 ? 2 : 1;
        return aligned(ptr, a) && w % int(a) == 0;
    };
    if (!words_ok(q->packed_hi, q->bits_hi, w_hi) || (q->bits_lo && !words_ok(q->packed_lo, q->bits_lo, w_lo))) return TQ_OK;
    const int64_t total = q->n_lanes * q->n_rows;
    const int64_t tiles = (total + dqtc::TM - 1) / dqtc::TM;
    if (tiles > 0x7fffffff) return TQ_OK;
    *handled = true;
    dqtc::Params p{};
    p.packed_hi = q->packed_hi; p.packed_lo = q->packed_lo; p.norms = q->norms;
    p.n_rows = q->n_rows; p.in_lane_stride = q->in_lane_stride; p.total = total;
    p.d = d; p.half = half; p.bits_hi = q->bits_hi; p.bits_lo = q->bits_lo; p.w_hi = w_hi; p.w_lo = w_lo;
    p.cent_hi = q->cent_hi; p.cent_lo = q->cent_lo; p.rot = q->rot;
    p.out = q->out; p.out_dtype = q->out_dtype; p.out_lane_stride = q->out_lane_stride; p.out_row_stride = q->out_row_stride;
    p.n_tiles = int(tiles);
    if (!(p.status = decode_status_ptr())) return fail(TQ_ERR_LAUNCH, "tq_dequantize: cannot locate the status word");
    static bool set[16] = {false};
    static int sms[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 16) dev = 0;
    using Kernel = void (*)(dqtc::Params);
    const Kernel kernels[7] = {dqtc::dequantize_tc_kernel<1, 0>, dqtc::dequantize_tc_kernel<2, 0>, dqtc::dequantize_tc_kernel<3, 0>, dqtc::dequantize_tc_kernel<4, 0>,
                               dqtc::dequantize_tc_kernel<2, 1>, dqtc::dequantize_tc_kernel<3, 2>, dqtc::dequantize_tc_kernel<4, 3>};
    if (!set[dev]) {
        for (Kernel k : kernels) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dqtc::SMEM_BYTES));
            if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_dequantize: shared memory %zu B: %s", dqtc::SMEM_BYTES, cudaGetErrorString(e));
        }
        if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0) sms[dev] = 148;
        set[dev] = true;
    }
    const unsigned grid = unsigned(std::min<int64_t>(tiles, sms[dev]));
    kernels[q->bits_lo ? 2 + q->bits_hi : q->bits_hi - 1]<<<grid, dqtc::NT, dqtc::SMEM_BYTES, s>>>(p);
    return check_launch("tq_dequantize");
}

}  // namespace tq
