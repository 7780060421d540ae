// Causal attention for several query tokens per sequence over the compressed cache, on the fifth-generation tensor
// cores: the large-tile form of prefill.cu for head_dim 128 (same contract, same
// arithmetic: what the reference does as dense reassembly, cache.py:674-706, followed by the consumer's masked
// attention; sketched for packed keys in kernels.py:558-590 and docs/FUSED_ATTENTION_DESIGN.md:281-283).
//
// A CTA owns 128 rows = 128 / GP query tokens x the GP (1, 2, 4 or 8) query heads of one GQA group, and walks the cache
// in tiles of 128 tokens, warp-specialised:
//   * warps 4-7 (producers) unpack tile g into key / value buffer g & 1: fp16, keys and values both token-major, in the
//     128-byte-swizzled layout the tensor core's shared-memory descriptors describe (keys: the K-major B operand of
//     S = Q K^T; values: the MN-major B operand of O += P V, so no transpose is ever materialised), plus the tile's norms
//     and positions;
//   * one thread of warp 8 issues S_g = Q K_g^T as eight tcgen05.mma (M 128, N 128, K 16) into score columns g & 1 of
//     tensor memory, then O += P_{g-1} V_{g-1}, each followed by tcgen05.commit to mbarriers: the scores of tile g are
//     computed while the rows are still busy with tile g - 1;
//   * warps 0-3 own the 128 accumulator lanes (one row per thread): they read S back (tcgen05.ld), apply key norms,
//     causal mask (skipped on tiles every row sees in full) and the running-maximum softmax in one sweep, and write
//     P (weights x value norms, fp16) as the next A operand; when a row's reference maximum or the value-norm scale
//     moves, its O rows in tensor memory are rescaled (tcgen05.ld / st) and the sweep is repeated (rare).
// Packed tokens accumulate in rotated space under the rotated query; sink / recent tokens form a second region under
// the raw query (which takes the rotated one's place in shared memory) with a second accumulator.  At the end the
// rotation of the packed part is undone once (y @ R, rotation.py:68-78), the parts are added, divided by the softmax
// denominators and stored.  Tensor memory: S twice 128 columns, O (packed) 128, O (uncompressed) 128.
//
// Every mbarrier wait is bounded; a wait that runs out leaves status 104 (tq_device_status) and raises a flag that ends
// every other wait, the threads meet at the end of the region, and the tensor memory is freed on every path.
#include <algorithm>

#include "decode_dev.cuh"

namespace tq {

int* decode_status_ptr();

namespace pftc {

constexpr int D = 128, TM = 128, TN = 128;
constexpr int NT = 288;                               // warps 0-3: one accumulator row per thread; 4-7: unpack; 8: MMA issue
constexpr int ROW_T = 128, PROD_T = 128;
constexpr uint32_t KBLK = 16384, TILE_BYTES = 2 * KBLK;                     // a 128 x 128 fp16 operand tile: two 64-column blocks
constexpr uint32_t OFF_Q = 0;                                               // the query tile: rotated, later raw
constexpr uint32_t OFF_K = TILE_BYTES, OFF_V = 3 * TILE_BYTES;              // two key tiles, two value tiles
constexpr uint32_t OFF_P = 5 * TILE_BYTES;
constexpr uint32_t OFF_KN = 6 * TILE_BYTES;                                 // float [2][128] key norms (or inverse staging scales)
constexpr uint32_t OFF_VN = OFF_KN + 1024;                                  // float [2][128]
constexpr uint32_t OFF_POS = OFF_VN + 1024;                                 // int   [2][128] absolute positions of the tile's tokens
constexpr int TREP = 8;                                                     // copies of every table entry (lane l reads copy l mod 8)
constexpr uint32_t OFF_T4 = OFF_POS + 1024;                                 // uint  [256][TREP] byte of two 4-bit codes -> half2
constexpr uint32_t OFF_T2 = OFF_T4 + 1024 * TREP;                           // uint2 [256][TREP] byte of four 2-bit codes -> 4 halves
constexpr uint32_t OFF_CTAB = OFF_T2 + 2048 * TREP;                         // half  [64]: key centroids (first half, second half), value centroids (first, second)
constexpr uint32_t OFF_BAR = OFF_CTAB + 128 + 256;                                 // mbarriers (see Bars)
constexpr uint32_t OFF_SLOT = OFF_BAR + 128;                                // words: [0] tensor-memory base, [1] abort, [4..5] "every row sees every token" of tile buffer 0 / 1, [8..15] largest value norm per buffer and producer warp
constexpr uint32_t SMEM_USED = OFF_SLOT + 64;
constexpr size_t SMEM_BYTES = SMEM_USED + 1024;                             // + slack to align the tiles to 1024 bytes
static_assert(SMEM_BYTES <= 227u * 1024u, "shared-memory plan");
// the finish reuses the tiles: two [128][129] float arrays
constexpr uint32_t FIN_LD = 129, OFF_FD = 0, OFF_FP = 66560;
static_assert(OFF_FP + 128 * FIN_LD * 4 <= OFF_KN && 128 * FIN_LD * 4 <= OFF_FP, "finish scratch");
constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_WAIT = 104;
constexpr uint32_t TMEM_COLS = 512, COL_S = 0, COL_OP = 256, COL_OD = 384;  // S twice (tile parity), O of the packed part, O of the uncompressed part
// mbarriers, 8 bytes each from OFF_BAR
enum Bars { KV_FULL = 0, KV_FREE = 2, S_FULL = 4, S_FREE = 6, P_FULL = 8, PV_DONE = 9, N_BARS = 10 };

struct Params {
    DecodeParams c;
    const void* q; int q_dtype;
    void* out; int out_dtype;
    int Tq;
    int64_t q_pos0;
    int GP, QT;
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
// D = A.B (+ D when accumulate != 0); A and B through shared-memory descriptors
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
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Operand tiles: 128 rows of 128 fp16, stored as two blocks of 64 columns (16 KB each); row r of a block at r * 128 B,
// its 16-byte chunk c at chunk position c ^ (r & 7) (128-byte swizzle; the tile is 1024-byte aligned).
__device__ __forceinline__ uint32_t chunk_off(int r, int c16) {            // c16: 16-byte chunk of the row, 0 .. 15
    return uint32_t(c16 >> 3) * KBLK + uint32_t(r) * 128u + (uint32_t((c16 & 7) ^ (r & 7)) << 4);
}
// K-major descriptor (rows = M or N index, 64-column blocks along K): the 16-column slab `ks` (0 .. 7) of the tile
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int ks) {
    const uint32_t addr = tile_addr + uint32_t(ks >> 2) * KBLK + uint32_t(ks & 3) * 32u;
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);
    d |= uint64_t(1) << 16;                       // leading byte offset (not used by swizzled K-major layouts)
    d |= uint64_t(1024 >> 4) << 32;               // stride byte offset: 8 rows x 128 B
    d |= uint64_t(1) << 46;                       // descriptor version
    d |= uint64_t(2) << 61;                       // 128-byte swizzle
    return d;
}
// MN-major descriptor of the same physical tile read the other way round (rows = K index, i.e. tokens; the 128 columns =
// N index in two blocks of 64): the 16-row slab `ks` (0 .. 7).  Eight rows form a 1024-byte atom (stride byte offset),
// the second block of 64 columns sits 16 KB further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int ks) {
    const uint32_t addr = tile_addr + uint32_t(ks) * 2048u;
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFF);
    d |= uint64_t(KBLK >> 4) << 16;
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulate, fp16 A and B, A K-major, M = 128, N = 128; B K-major or MN-major
__device__ __forceinline__ uint32_t make_idesc(bool b_mn_major) {
    return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (uint32_t(TN >> 3) << 17) | (uint32_t(TM >> 4) << 24);
}

__global__ void __launch_bounds__(NT, 1) prefill_tc_kernel(Params P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t raw_addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_raw));
    const uint32_t sbase = (raw_addr + 1023u) & ~1023u;
    unsigned char* smem = smem_raw + (sbase - raw_addr);
    const DecodeParams& p = P.c;
    float* s_kn = reinterpret_cast<float*>(smem + OFF_KN);                   // [2][128]
    float* s_vn = reinterpret_cast<float*>(smem + OFF_VN);
    int* s_pos = reinterpret_cast<int*>(smem + OFF_POS);
    uint32_t* t4 = reinterpret_cast<uint32_t*>(smem + OFF_T4);
    uint2* t2 = reinterpret_cast<uint2*>(smem + OFF_T2);
    __half* ctab = reinterpret_cast<__half*>(smem + OFF_CTAB);
    uint32_t* ctab32 = reinterpret_cast<uint32_t*>(smem + OFF_CTAB + 128);   // the same 64 centroids, one per 32-bit word (code-by-code unpack)
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_SLOT);
    auto bar = [&](int which) -> uint32_t { return sbase + OFF_BAR + 8u * uint32_t(which); };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t cp = uint32_t(lane) & (TREP - 1);
    const int hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int tq0 = blockIdx.x * P.QT, GP = P.GP;
    auto row_valid = [&](int m) { return (m % GP) < heads_here && tq0 + m / GP < P.Tq; };
    auto row_q_index = [&](int m) -> int64_t {
        const int h = hkv * p.G + hg * HPG + (m % GP);
        return ((int64_t(b) * p.Hq + h) * P.Tq + (tq0 + m / GP)) * D;
    };

    // ---------------- set-up: barriers, tensor memory, tables ------------------------------------------------------
    if (tid == 0) {
        mbar_init(bar(KV_FULL), PROD_T); mbar_init(bar(KV_FULL + 1), PROD_T);
        mbar_init(bar(KV_FREE), 1); mbar_init(bar(KV_FREE + 1), 1);
        mbar_init(bar(S_FULL), 1); mbar_init(bar(S_FULL + 1), 1);
        mbar_init(bar(S_FREE), ROW_T); mbar_init(bar(S_FREE + 1), ROW_T);
        mbar_init(bar(P_FULL), ROW_T);
        mbar_init(bar(PV_DONE), 1);
        fence_barrier_init();
        slot[1] = 0u;
    }
    if (warp == 8) {
        tmem_alloc(sbase + OFF_SLOT, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid < 64) {
        const int which = tid >> 4, k = tid & 15;
        const float* src = which == 0 ? p.kc_hi : which == 1 ? p.kc_lo : which == 2 ? p.vc_hi : p.vc_lo;
        const int bits = which == 0 ? p.kb_hi : which == 1 ? p.kb_lo : which == 2 ? p.vb_hi : p.vb_lo;
        const float sc = which == 2 ? p.v_scale_hi : which == 3 ? p.v_scale_lo : 1.f;     // value tables: fp16 under a table-wide scale, divided out at the end
        ctab[tid] = __float2half_rn((src != nullptr && bits > 0 && k < (1 << bits)) ? src[k] * sc : 0.f);
        ctab32[tid] = uint32_t(__half_as_ushort(ctab[tid]));
    }
    __syncthreads();
    // whole-byte tables for the commonest widths (4-bit keys, 2-bit values, not fractional, word-aligned rows): a tile is then
    // unpacked a 32-bit word at a time; every other width goes code by code through the 16-entry tables
    const bool fast_unpack = p.kb_hi == 4 && p.kb_lo == 0 && p.vb_hi == 2 && p.vb_lo == 0 && p.words_ok;
    if (tid < 256) {
        const int e = tid;
        const __half2 hk = __halves2half2(ctab[e & 15], ctab[e >> 4]);
        const __half2 v01 = __halves2half2(ctab[32 + (e & 3)], ctab[32 + ((e >> 2) & 3)]);
        const __half2 v23 = __halves2half2(ctab[32 + ((e >> 4) & 3)], ctab[32 + (e >> 6)]);
#pragma unroll
        for (int r = 0; r < TREP; ++r) {
            t4[e * TREP + r] = *reinterpret_cast<const uint32_t*>(&hk);
            t2[e * TREP + r] = make_uint2(*reinterpret_cast<const uint32_t*>(&v01), *reinterpret_cast<const uint32_t*>(&v23));
        }
    }

    // ---------------- the query block, rotated and scaled, as the fp16 A-operand tile -------------------------------
    const float f = p.scale * LOG2E;
    {
        float* qf = reinterpret_cast<float*>(smem + OFF_K);                  // [128][D] float32 (the key tiles' space)
        float* rs = reinterpret_cast<float*>(smem + OFF_P);                  // [32][D + 1] slab of R
        for (int e = tid; e < TM * D; e += NT) {
            const int m = e / D, k = e - m * D;
            qf[e] = row_valid(m) ? load_as_f32(P.q, P.q_dtype, row_q_index(m) + k) * f : 0.f;
        }
        // q_rot[m][j] = sum_k q[m][k] R[j][k] (rotation.py:81-110): 32 rows of R at a time; thread = (row j of the slab, 16 query rows)
        constexpr int RS = D + 1;
        const int jl = tid & 31, cg = tid >> 5;
        for (int j0 = 0; j0 < D; j0 += 32) {
            __syncthreads();
            for (int e = tid; e < 32 * D; e += NT) {
                const int r = e / D, k = e - r * D;
                rs[r * RS + k] = __ldg(p.rot + int64_t(j0 + r) * D + k);
            }
            __syncthreads();
            if (cg < 8) {
                float acc[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) acc[u] = 0.f;
                for (int k = 0; k < D; k += 4) {
                    const float r0 = rs[jl * RS + k], r1 = rs[jl * RS + k + 1], r2 = rs[jl * RS + k + 2], r3 = rs[jl * RS + k + 3];
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const float4 x = *reinterpret_cast<const float4*>(qf + (cg * 16 + u) * D + k);
                        acc[u] = fmaf(x.x, r0, fmaf(x.y, r1, fmaf(x.z, r2, fmaf(x.w, r3, acc[u]))));
                    }
                }
                const int j = j0 + jl;
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const int m = cg * 16 + u;
                    *reinterpret_cast<__half*>(smem + OFF_Q + chunk_off(m, j >> 3) + (j & 7) * 2) = __float2half_rn(acc[u]);
                }
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slot[0];

    const int64_t cta_q_max = P.q_pos0 + min(tq0 + P.QT, P.Tq) - 1;               // the latest position any row sees
    const int64_t min_q_pos = P.q_pos0 + tq0;                                      // the earliest position any (valid) row sits at
    const uint32_t idesc_qk = make_idesc(false), idesc_pv = make_idesc(true);

    // bounded wait on an mbarrier; a thread that runs out raises the abort flag for everybody
    auto wait_bar = [&](uint32_t addr, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
            if (mbar_try(addr, parity)) return true;
            if ((i & 1023u) == 1023u && slot[1]) return false;
        }
        slot[1] = 1u;
        atomicCAS(P.status, 0, ERR_WAIT);
        return false;
    };

    // per-row softmax state (threads 0 .. 127 own rows)
    const int q_pos = (tid < ROW_T && row_valid(tid)) ? int(P.q_pos0 + tq0 + tid / GP) : -1;   // the latest position this row sees
    float m_ref = -1e30f, l_sum = 0.f, vsc = 1.f, vthr = 0.f;                   // (vthr 0: the first tile with a non-zero value norm picks the scale)
    float lvsc = 0.f, bias = 0.f, t_thr = MAX_SLACK;                             // log2(vsc); lvsc - m_ref (0 until the first tile has set the reference); MAX_SLACK + lvsc
    const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    bool have_op = false, have_od = false;        // the accumulators hold sums (same in every thread)

    // Tiles are numbered g = 0, 1, ... across both regions; tile g uses key / value / norm buffer g & 1 and score columns
    // COL_S + 128 (g & 1).  Barrier phases follow from g: the per-buffer barriers complete once per two tiles, P_FULL and
    // PV_DONE once per tile.
    int g0 = 0;                                   // number of the region's first tile
    for (int region = 0; region < 2; ++region) {
        const bool dense_region = region == 1;
        const int64_t n_dense = p.sink_len + p.res_len;
        // tokens of the region some row of the CTA sees: packed token t sits at position sink_len + t; uncompressed token t at
        // t (sink) or c_len + t (recent)
        const int64_t vis = dense_region ? min(n_dense, max(p.sink_len, cta_q_max - p.c_len + 1)) : min(p.c_len, cta_q_max - p.sink_len + 1);
        const int n_tiles = vis > 0 ? int((vis + TN - 1) / TN) : 0;
        if (dense_region) {
            // the raw query takes the rotated one's place (every product of the packed region has completed)
            for (int i = tid; i < TM * 16; i += NT) {
                const int m = i >> 4, c = i & 15;
                uint32_t h[4] = {0u, 0u, 0u, 0u};
                if (row_valid(m)) {
                    const int64_t e = row_q_index(m) + c * 8;
#pragma unroll
                    for (int u = 0; u < 4; ++u) h[u] = pack_h2(load_as_f32(P.q, P.q_dtype, e + 2 * u) * f, load_as_f32(P.q, P.q_dtype, e + 2 * u + 1) * f);
                }
                *reinterpret_cast<uint4*>(smem + OFF_Q + chunk_off(m, c)) = make_uint4(h[0], h[1], h[2], h[3]);
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
            tc_fence_after();
        }

        if (warp >= 4 && warp < 8) {
            // ======================= producers: unpack tile g into buffer g & 1 =======================
            const int pt = tid - ROW_T;                                       // 0 .. 127
            // packed region: the words and norms of a tile are requested one tile ahead, so that their latency passes while
            // the thread waits for the buffer and converts the previous tile
            uint32_t kx[16], vx[8];
            float nk = 0.f, nv = 0.f;
            auto request_packed = [&](int it) {
                const int64_t tok0 = int64_t(it) * TN;
                const int rows = int(min(int64_t(TN), p.c_len - tok0));
                const uint32_t* ksrc = reinterpret_cast<const uint32_t*>(p.k_hi + (kvl * p.c_ls + tok0) * (D / 2));
                const uint32_t* vsrc = reinterpret_cast<const uint32_t*>(p.v_hi + (kvl * p.c_ls + tok0) * (D / 4));
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int i = pt + PROD_T * k, r = i >> 4;
                    kx[k] = r < rows ? __ldg(ksrc + i) : 0u;
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int i = pt + PROD_T * k, r = i >> 3;
                    vx[k] = r < rows ? __ldg(vsrc + i) : 0u;
                }
                const bool live = pt < rows;
                const int64_t n = kvl * p.c_ls + tok0 + (live ? pt : 0);
                nk = live ? __ldg(p.k_norms + n) : 0.f;
                nv = live ? __ldg(p.v_norms + n) : 0.f;
            };
            if (!dense_region && fast_unpack && n_tiles > 0) request_packed(0);
            for (int it = 0; it < n_tiles; ++it) {
                const int g = g0 + it, bf = g & 1;
                if (g >= 2 && !wait_bar(bar(KV_FREE + bf), uint32_t(((g >> 1) - 1) & 1))) break;     // the products of tile g - 2 have read the buffer
                const int64_t tok0 = int64_t(it) * TN;
                unsigned char* kt = smem + OFF_K + bf * TILE_BYTES;
                unsigned char* vt = smem + OFF_V + bf * TILE_BYTES;
                float* kn = s_kn + bf * TN; float* vn = s_vn + bf * TN; int* ps = s_pos + bf * TN;
                float my_vn = 0.f;
                if (!dense_region && !fast_unpack) {
                    // any width 1-4, fractional splits: chunk c = pt + 128 k of a tensor is row c >> 4, coordinates 8 (c & 15) ...;
                    // eight codes are `bits` bytes of the packed row (read bytewise: no alignment asked of the rows)
                    const int rows = int(min(int64_t(TN), p.c_len - tok0));
                    if (pt == 0) slot[4 + bf] = (rows == TN && p.sink_len + tok0 + TN - 1 <= min_q_pos) ? 1u : 0u;
                    {
                        const bool live = pt < rows;
                        const int64_t n = kvl * p.c_ls + tok0 + (live ? pt : 0);
                        const float a = live ? __ldg(p.k_norms + n) : 0.f;
                        my_vn = live ? __ldg(p.v_norms + n) : 0.f;
                        kn[pt] = a; vn[pt] = my_vn;
                        ps[pt] = live ? int(p.sink_len + tok0 + pt) : 0x7fffffff;
                    }
#pragma unroll 1
                    for (int side = 0; side < 2; ++side) {
                        const int b_hi = side ? p.vb_hi : p.kb_hi, b_lo = side ? p.vb_lo : p.kb_lo;
                        const int half = b_lo ? D / 2 : D;
                        const int w_hi = half * b_hi / 8, w_lo = b_lo ? (D - half) * b_lo / 8 : 0;
                        const uint8_t* base_hi = (side ? p.v_hi : p.k_hi) + (kvl * p.c_ls + tok0) * w_hi;
                        const uint8_t* base_lo = b_lo ? (side ? p.v_lo : p.k_lo) + (kvl * p.c_ls + tok0) * w_lo : nullptr;
                        unsigned char* dst = side ? vt : kt;
                        // packed rows can be read as aligned 32-bit words when every row starts on a 4-byte boundary
                        const bool words = (reinterpret_cast<uintptr_t>(base_hi) & 3u) == 0 && (w_hi & 3) == 0 &&
                                           (b_lo == 0 || ((reinterpret_cast<uintptr_t>(base_lo) & 3u) == 0 && (w_lo & 3) == 0));
#pragma unroll 8
                        for (int k = 0; k < 16; ++k) {
                            const int c = pt + PROD_T * k, r = c >> 4, j8 = c & 15;
                            const bool second = b_lo != 0 && j8 * 8 >= half;
                            const int bits = second ? b_lo : b_hi;
                            uint32_t w = 0u;
                            if (r < rows) {
                                const uint8_t* src = second ? base_lo + int64_t(r) * w_lo + (j8 - half / 8) * bits : base_hi + int64_t(r) * w_hi + j8 * bits;
                                if (words) {          // aligned words around the `bits` bytes, shifted into place
                                    const uint32_t sh = uint32_t(reinterpret_cast<uintptr_t>(src)) & 3u;
                                    const uint32_t* a4 = reinterpret_cast<const uint32_t*>(src - sh);
                                    const uint32_t lo = __ldg(a4), hi = sh + uint32_t(bits) > 4u ? __ldg(a4 + 1) : 0u;
                                    w = __funnelshift_r(lo, hi, sh * 8u);
                                } else {
                                    for (int u = 0; u < bits; ++u) w |= uint32_t(__ldg(src + u)) << (8 * u);
                                }
                            }
                            const uint32_t mask = (1u << bits) - 1u;
                            const uint32_t* tb = ctab32 + side * 32 + (second ? 16 : 0);
                            uint32_t e[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) e[u] = tb[(w >> (bits * u)) & mask];
                            *reinterpret_cast<uint4*>(dst + chunk_off(r, j8)) =
                                make_uint4(__byte_perm(e[0], e[1], 0x5410), __byte_perm(e[2], e[3], 0x5410), __byte_perm(e[4], e[5], 0x5410), __byte_perm(e[6], e[7], 0x5410));
                        }
                    }
                } else if (!dense_region) {
                    const int rows = int(min(int64_t(TN), p.c_len - tok0));
                    if (pt == 0) slot[4 + bf] = (rows == TN && p.sink_len + tok0 + TN - 1 <= min_q_pos) ? 1u : 0u;
                    my_vn = nv;
                    kn[pt] = nk; vn[pt] = nv;
                    ps[pt] = pt < rows ? int(p.sink_len + tok0 + pt) : 0x7fffffff;
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        const int i = pt + PROD_T * k, r = i >> 4, w = i & 15;
                        const uint32_t x = kx[k];
                        *reinterpret_cast<uint4*>(kt + chunk_off(r, w)) =
                            make_uint4(t4[(x & 255u) * TREP + cp], t4[((x >> 8) & 255u) * TREP + cp], t4[((x >> 16) & 255u) * TREP + cp], t4[(x >> 24) * TREP + cp]);
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int i = pt + PROD_T * k, r = i >> 3, w = i & 7;
                        const uint32_t x = vx[k];
                        const uint2 a = t2[(x & 255u) * TREP + cp], bb = t2[((x >> 8) & 255u) * TREP + cp], cc = t2[((x >> 16) & 255u) * TREP + cp], ee = t2[(x >> 24) * TREP + cp];
                        *reinterpret_cast<uint4*>(vt + chunk_off(r, 2 * w)) = make_uint4(a.x, a.y, bb.x, bb.y);
                        *reinterpret_cast<uint4*>(vt + chunk_off(r, 2 * w + 1)) = make_uint4(cc.x, cc.y, ee.x, ee.y);
                    }
                    if (it + 1 < n_tiles) request_packed(it + 1);
                } else {
                    // one thread per token row; float32 / bfloat16 rows under a per-token power-of-two scale (largest magnitude into
                    // [2^7, 2^8)) whose inverse goes where the packed tokens have their norms: a pass for the maximum, a pass to convert
                    const int r = pt;
                    const int64_t tok = tok0 + r;
                    const bool live = tok < n_dense;
                    const bool in_sink = tok < p.sink_len;
                    const int64_t e0 = live ? (in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len)) * D : 0;
                    if (pt == 0) {
                        const int64_t tl = tok0 + TN - 1;                     // the tile's last token, if it has 128
                        slot[4 + bf] = (tl < n_dense && (tl < p.sink_len ? tl : p.c_len + tl) <= min_q_pos) ? 1u : 0u;
                    }
                    float inv[2] = {0.f, 0.f};
#pragma unroll 1
                    for (int side = 0; side < 2; ++side) {
                        const void* base = side == 0 ? (in_sink ? p.sink_k : p.res_k) : (in_sink ? p.sink_v : p.res_v);
                        unsigned char* dst = side == 0 ? kt : vt;
                        float sc = 1.f;
                        if (p.dense_dtype == TQ_F16) {
#pragma unroll 4
                            for (int c = 0; c < 16; ++c)
                                *reinterpret_cast<uint4*>(dst + chunk_off(r, c)) =
                                    live ? __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + e0) + c) : make_uint4(0, 0, 0, 0);
                        } else if (p.dense_dtype == TQ_BF16) {
                            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + e0);
                            uint32_t mxb = 0u;
                            if (live) {
#pragma unroll 4
                                for (int c = 0; c < 16; ++c) {
                                    const uint4 x = __ldg(src + c);
                                    const uint32_t mm = 0x7fff7fffu;
                                    const uint32_t a = __vmaxu2(__vmaxu2(x.x & mm, x.y & mm), __vmaxu2(x.z & mm, x.w & mm));
                                    mxb = max(mxb, max(a & 0xffffu, a >> 16) << 16);
                                }
                            }
                            sc = stage_scale(mxb);
                            auto two = [&](uint32_t w) -> uint32_t { return pack_h2(__uint_as_float(w << 16) * sc, __uint_as_float(w & 0xffff0000u) * sc); };
#pragma unroll 4
                            for (int c = 0; c < 16; ++c) {
                                const uint4 x = live ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
                                *reinterpret_cast<uint4*>(dst + chunk_off(r, c)) = make_uint4(two(x.x), two(x.y), two(x.z), two(x.w));
                            }
                        } else {
                            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const float*>(base) + e0);
                            uint32_t mxb = 0u;
                            if (live) {
#pragma unroll 4
                                for (int c = 0; c < 32; ++c) {
                                    const uint4 x = __ldg(src + c);
                                    const uint32_t mm = 0x7fffffffu;
                                    mxb = max(mxb, max(max(x.x & mm, x.y & mm), max(x.z & mm, x.w & mm)));
                                }
                            }
                            sc = stage_scale(mxb);
#pragma unroll 4
                            for (int c = 0; c < 16; ++c) {
                                const uint4 x = live ? __ldg(src + 2 * c) : make_uint4(0, 0, 0, 0), y = live ? __ldg(src + 2 * c + 1) : make_uint4(0, 0, 0, 0);
                                *reinterpret_cast<uint4*>(dst + chunk_off(r, c)) =
                                    make_uint4(pack_h2(__uint_as_float(x.x) * sc, __uint_as_float(x.y) * sc), pack_h2(__uint_as_float(x.z) * sc, __uint_as_float(x.w) * sc),
                                               pack_h2(__uint_as_float(y.x) * sc, __uint_as_float(y.y) * sc), pack_h2(__uint_as_float(y.z) * sc, __uint_as_float(y.w) * sc));
                            }
                        }
                        inv[side] = live ? 1.f / sc : 0.f;
                    }
                    kn[r] = inv[0]; vn[r] = inv[1];
                    ps[r] = live ? int(in_sink ? tok : p.c_len + tok) : 0x7fffffff;
                    my_vn = inv[1];
                }
#pragma unroll
                for (int off = 16; off; off >>= 1) my_vn = fmaxf(my_vn, __shfl_xor_sync(0xffffffffu, my_vn, off));
                if (lane == 0) slot[8 + bf * 4 + (warp - 4)] = __float_as_uint(fmaxf(my_vn, 0.f));     // this warp's largest value norm
                fence_proxy_async();                                          // the tiles (generic-proxy stores) before the tensor core reads them
                mbar_arrive(bar(KV_FULL + bf));
            }
        } else if (warp == 8) {
            // ======================= MMA issue: one thread =======================
            if (lane == 0) {
                auto issue_pv = [&](int g) -> bool {                          // O += P V of tile g
                    const int bf = g & 1;
                    if (!wait_bar(bar(P_FULL), uint32_t(g & 1))) return false;
                    tc_fence_after();
                    const uint32_t col = dense_region ? COL_OD : COL_OP;
                    const bool first = g == g0;                               // the region's first product starts its accumulator
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        umma_f16(tmem_base + col, desc_kmajor(sbase + OFF_P, ks), desc_mnmajor(sbase + OFF_V + bf * TILE_BYTES, ks), idesc_pv,
                                 (!first || ks > 0) ? 1u : 0u);
                    umma_commit(bar(KV_FREE + bf));
                    umma_commit(bar(PV_DONE));
                    return true;
                };
                bool ok = true;
                for (int it = 0; it < n_tiles && ok; ++it) {
                    const int g = g0 + it, bf = g & 1;
                    ok = wait_bar(bar(KV_FULL + bf), uint32_t((g >> 1) & 1));
                    if (ok && g >= 2) ok = wait_bar(bar(S_FREE + bf), uint32_t(((g >> 1) - 1) & 1));     // the rows have read the scores of tile g - 2
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        umma_f16(tmem_base + COL_S + bf * TN, desc_kmajor(sbase + OFF_Q, ks), desc_kmajor(sbase + OFF_K + bf * TILE_BYTES, ks), idesc_qk, ks > 0 ? 1u : 0u);
                    umma_commit(bar(S_FULL + bf));
                    if (it > 0) ok = issue_pv(g - 1);                         // the scores of tile g are under way while the rows finish tile g - 1
                }
                if (ok && n_tiles > 0) issue_pv(g0 + n_tiles - 1);
            }
        } else {
            // ======================= rows: softmax of tile g, P for its second product =======================
            for (int it = 0; it < n_tiles; ++it) {
                const int g = g0 + it, bf = g & 1;
                // the tile's norms, positions and flags come from the producers directly; the scores from the tensor core
                if (!wait_bar(bar(KV_FULL + bf), uint32_t((g >> 1) & 1))) break;
                if (!wait_bar(bar(S_FULL + bf), uint32_t((g >> 1) & 1))) break;
                // P and the O rows are free once the second product of tile g - 1 has finished
                if (g >= 1 && !wait_bar(bar(PV_DONE), uint32_t((g - 1) & 1))) break;
                tc_fence_after();
                const float* kn_t = s_kn + bf * TN; const float* vn_t = s_vn + bf * TN; const int* ps_t = s_pos + bf * TN;
                const float vmax = fmaxf(fmaxf(__uint_as_float(slot[8 + bf * 4]), __uint_as_float(slot[9 + bf * 4])),
                                         fmaxf(__uint_as_float(slot[10 + bf * 4]), __uint_as_float(slot[11 + bf * 4])));
                const bool masked = slot[4 + bf] == 0u;                       // some token of the tile is hidden from some row (or dead)
                const uint32_t s_col = t_row + COL_S + bf * TN;
                // Reference maximum / value scale: refreshed for the whole warp when any row needs it (the tensor-memory loads
                // and stores are warp-wide).  mx: the row's largest visible score of this tile.
                auto refresh = [&](float mx) {
                    const float mn = fmaxf(fmaxf(m_ref, mx), -1e30f);
                    float a = ex2(m_ref - mn);
                    m_ref = mn;
                    if (vmax > vthr) {
                        int eb = (__float_as_int(vmax) >> 23) & 0xff;
                        eb = min(max(eb, 16), 240);
                        const float nsc = __int_as_float((261 - eb) << 23);
                        a *= nsc / vsc;
                        vsc = nsc;
                        vthr = VSC_CAP / nsc;
                        lvsc = float(134 - eb);                            // log2 of the scale
                    }
                    l_sum *= a;                                           // the denominator carries the value scale like the sums do
                    bias = lvsc - m_ref;
                    t_thr = MAX_SLACK + lvsc;
#pragma unroll 1
                    for (int acc = 0; acc < 2; ++acc) {
                        // an accumulator holds sums once a product of its region has completed: the packed one from the second packed
                        // tile on, the other from the second uncompressed tile on (the region's first product overwrites)
                        const bool holds = acc == 0 ? have_op : have_od;
                        if (!holds) continue;
                        const uint32_t col = acc == 0 ? COL_OP : COL_OD;
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t v[32];
                            tmem_ld32(t_row + col + c0, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * a);
                            tmem_st32(t_row + col + c0, v);
                        }
                        tmem_st_wait();
                    }
                };
                // One sweep over the row's 128 scores: weights against the current reference, P = p * value norm * scale as fp16
                // into the A-operand tile (row = this thread), the row's largest score alongside.  write = false: the maximum only.
                auto sweep = [&](bool write, float& mx, float& lsum) {
                    mx = -INFINITY; lsum = 0.f;
                    auto chunk = [&](const uint32_t (&v)[32], int c0) {       // 32 scores: columns c0 .. c0 + 31
                        uint32_t h[16];
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            // t = score * key norm - reference + log2(value scale): one multiply-add per score; the weight ex2(t)
                            // already carries the value scale, and so does the denominator it is summed into
                            const float4 kn = *reinterpret_cast<const float4*>(kn_t + c0 + j);
                            float s0 = fmaf(__uint_as_float(v[j]), kn.x, bias), s1 = fmaf(__uint_as_float(v[j + 1]), kn.y, bias);
                            float s2 = fmaf(__uint_as_float(v[j + 2]), kn.z, bias), s3 = fmaf(__uint_as_float(v[j + 3]), kn.w, bias);
                            if (masked) {
                                const int4 ps = *reinterpret_cast<const int4*>(ps_t + c0 + j);
                                s0 = ps.x <= q_pos ? s0 : -INFINITY; s1 = ps.y <= q_pos ? s1 : -INFINITY;
                                s2 = ps.z <= q_pos ? s2 : -INFINITY; s3 = ps.w <= q_pos ? s3 : -INFINITY;
                            }
                            mx = fmaxf(fmaxf(mx, fmaxf(s0, s1)), fmaxf(s2, s3));
                            if (write) {
                                const float4 vn = *reinterpret_cast<const float4*>(vn_t + c0 + j);
                                const float p0 = ex2(s0), p1 = ex2(s1), p2 = ex2(s2), p3 = ex2(s3);
                                lsum += (p0 + p1) + (p2 + p3);
                                h[j >> 1] = pack_h2(p0 * vn.x, p1 * vn.y);
                                h[(j >> 1) + 1] = pack_h2(p2 * vn.z, p3 * vn.w);
                            }
                        }
                        if (write) {
#pragma unroll
                            for (int c = 0; c < 4; ++c)
                                *reinterpret_cast<uint4*>(smem + OFF_P + chunk_off(tid, (c0 >> 3) + c)) = make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
                        }
                    };
                    // the next 32 columns are on their way from tensor memory while the current ones are worked on
                    uint32_t va[32], vb[32];
                    tmem_ld32(s_col, va);
                    tmem_ld_wait();
#pragma unroll 1
                    for (int c0 = 0; c0 < TN; c0 += 64) {
                        tmem_ld32(s_col + c0 + 32, vb);
                        chunk(va, c0);
                        tmem_ld_wait();
                        if (c0 + 64 < TN) tmem_ld32(s_col + c0 + 64, va);
                        chunk(vb, c0 + 32);
                        tmem_ld_wait();
                    }
                };
                have_op = dense_region ? have_op : it >= 1;
                have_od = dense_region && it >= 1;
                float mx, lsum;
                // the very first tile (no reference yet; every valid row sees its first token) and a tile that moves the value
                // scale: settle the references first
                // (sweep returns the row's largest t; the score itself is t - bias)
                if (g == 0 || vmax > vthr) {
                    sweep(false, mx, lsum);
                    refresh(mx - bias);
                }
                sweep(true, mx, lsum);
                if (__any_sync(0xffffffffu, mx > t_thr)) {    // a score beyond the slack: new reference, weights again (rare)
                    refresh(mx - bias);
                    sweep(true, mx, lsum);
                }
                l_sum += lsum;
                tc_fence_before();                                            // this thread's tensor-memory loads of the scores are complete
                mbar_arrive(bar(S_FREE + bf));
                fence_proxy_async();                                          // P (generic-proxy stores) before the tensor core reads it
                mbar_arrive(bar(P_FULL));
            }
        }
        // ---- end of the region: every product has completed before anything is reused ----
        if (n_tiles > 0) wait_bar(bar(PV_DONE), uint32_t((g0 + n_tiles - 1) & 1));
        tc_fence_after();
        if (n_tiles > 0) { if (dense_region) have_od = true; else have_op = true; }
        g0 += n_tiles;
        tc_fence_before();
        if (__syncthreads_or(int(slot[1]))) break;                            // leave together after a failed wait
    }

    // ---------------- finish: value scales, rotation of the packed part, normalise, store ---------------------------
    __syncthreads();                                                              // the tiles are dead
    tc_fence_after();
    float* fd = reinterpret_cast<float*>(smem + OFF_FD);                          // [128][129] sums of the uncompressed part
    float* fp = reinterpret_cast<float*>(smem + OFF_FP);                          // [128][129] sums of the packed part, rotated space
    const bool failed = slot[1] != 0u;
    if (tid < ROW_T) {
        const float ip_hi = 1.f / p.v_scale_hi, ip_lo = 1.f / (p.vb_lo ? p.v_scale_lo : p.v_scale_hi), id = 1.f;   // (sums and denominator carry the same value scale)
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t v[32];
            if (have_op) { tmem_ld32(t_row + COL_OP + c0, v); tmem_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) fp[tid * FIN_LD + c0 + j] = have_op ? __uint_as_float(v[j]) * (c0 < D / 2 ? ip_hi : ip_lo) : 0.f;
            if (have_od) { tmem_ld32(t_row + COL_OD + c0, v); tmem_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) fd[tid * FIN_LD + c0 + j] = have_od ? __uint_as_float(v[j]) * id : 0.f;
        }
        s_kn[tid] = l_sum;
    }
    tc_fence_before();
    __syncthreads();
    if (warp < 8) {
        // out[m][j] = (sum_k fp[m][k] R[k][j] + fd[m][j]) / l[m]  (y @ R, rotation.py:68-78): warp -> 16 rows, lane -> j = lane + 32 i
        float acc[16][4];
#pragma unroll
        for (int u = 0; u < 16; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[u][i] = 0.f;
        if (have_op) {
            for (int k = 0; k < D; ++k) {
                float r[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) r[i] = __ldg(p.rot + int64_t(k) * D + lane + 32 * i);
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const float a = fp[(warp * 16 + u) * FIN_LD + k];
#pragma unroll
                    for (int i = 0; i < 4; ++i) acc[u][i] = fmaf(a, r[i], acc[u][i]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int m = warp * 16 + u;
            if (!row_valid(m) || failed) continue;
            const float il = 1.f / s_kn[m];
            const int64_t o = row_q_index(m);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = lane + 32 * i;
                store_from_f32(P.out, P.out_dtype, o + j, (acc[u][i] + fd[m * FIN_LD + j]) * il);
            }
        }
    }
    // ---------------- teardown --------------------------------------------------------------------------------------
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace pftc

// Whether the tensor-core kernel takes this call; the caller has validated the arguments.
bool prefill_tc_applicable(const tq_decode_args* a, int t_q) {
    if (a->d != 128) return false;
    // fractional widths split the coordinates in halves of 64: (b, b - 1) bits as the reference does (cache.py:232-274)
    if (a->c_len > 0 && ((a->k_bits_lo && a->k_bits_lo != a->k_bits_hi - 1) || (a->v_bits_lo && a->v_bits_lo != a->v_bits_hi - 1))) return false;
    if (a->c_len + a->sink_len + a->res_len >= 0x7fffffff) return false;       // positions are kept as 32-bit integers
    // uncompressed rows are read as 16-byte chunks
    if ((a->sink_len > 0 && (!aligned(a->sink_k, 16) || !aligned(a->sink_v, 16))) || (a->res_len > 0 && (!aligned(a->res_k, 16) || !aligned(a->res_v, 16))))
        return false;
    const int g = std::min(a->n_q_heads / a->n_kv_heads, HPG);
    const int gp = g <= 1 ? 1 : g <= 2 ? 2 : g <= 4 ? 4 : 8;
    return int64_t(t_q) * gp >= 64;                                             // at least half a tile of rows
}

int launch_prefill_tc(const DecodeParams& c, const void* q, int q_dtype, void* out, int out_dtype, int t_q, int64_t q_pos0, cudaStream_t s) {
    pftc::Params P{};
    P.c = c;
    P.q = q; P.q_dtype = q_dtype; P.out = out; P.out_dtype = out_dtype; P.Tq = t_q; P.q_pos0 = q_pos0;
    const int gmin = std::min(c.G, HPG);
    P.GP = gmin <= 1 ? 1 : gmin <= 2 ? 2 : gmin <= 4 ? 4 : 8;
    P.QT = pftc::TM / P.GP;
    if (!(P.status = decode_status_ptr())) return fail(TQ_ERR_LAUNCH, "tq_prefill_attn: cannot locate the status word");
    static bool set[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(pftc::prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(pftc::SMEM_BYTES));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_prefill_attn: shared memory %zu B: %s", pftc::SMEM_BYTES, cudaGetErrorString(e));
        set[dev] = true;
    }
    const dim3 grid(unsigned((t_q + P.QT - 1) / P.QT), unsigned(c.Hkv * c.HG), unsigned(c.B));
    pftc::prefill_tc_kernel<<<grid, pftc::NT, pftc::SMEM_BYTES, s>>>(P);
    return check_launch("tq_prefill_attn");
}

}  // namespace tq
