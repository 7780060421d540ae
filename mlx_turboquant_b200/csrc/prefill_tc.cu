// Causal attention for several query tokens per sequence over the compressed cache, on the fifth-generation tensor
// cores: the large-tile form of prefill.cu for head_dim 128 with 4-bit keys and 2-bit values (same contract, same
// arithmetic: what the reference does as dense reassembly, cache.py:674-706, followed by the consumer's masked
// attention; sketched for packed keys in kernels.py:558-590 and docs/FUSED_ATTENTION_DESIGN.md:281-283).
//
// A CTA owns 128 rows = 128 / GP query tokens x the GP (1, 2, 4 or 8) query heads of one GQA group, and walks the cache
// in tiles of 128 tokens.  Per tile:
//   1. all 8 warps unpack the tile to fp16 in shared memory - keys and values both token-major, in the 128-byte-swizzled
//      layout the tensor core's shared-memory descriptors describe (keys: the K-major B operand of S = Q K^T; values:
//      the MN-major B operand of O += P V, so no transpose is ever materialised) - and stage the tile's norms;
//   2. one thread issues S = Q K^T as eight tcgen05.mma (M 128, N 128, K 16) into tensor memory and commits to an
//      mbarrier;
//   3. the four warps that own the 128 accumulator lanes (one row per thread) read S back (tcgen05.ld), apply key
//      norms, causal mask and the running-maximum softmax, and write P (weights x value norms, fp16) as the next A
//      operand; when a row's reference maximum or the value-norm scale moves, its O rows in tensor memory are rescaled
//      (tcgen05.ld / st);
//   4. one thread issues O += P V (eight more MMAs) into the accumulator of the region: packed tokens accumulate in
//      rotated space under the rotated query, sink / recent tokens under the raw query in a second accumulator.
// At the end the rotation of the packed part is undone once (y @ R, rotation.py:68-78), the parts are added, divided by
// the softmax denominators and stored.  Tensor memory: S 128 columns, O (packed) 128, O (uncompressed) 128.
//
// Every mbarrier wait is bounded; a wait that runs out leaves status 104 (tq_device_status), every thread leaves the
// tile loop at the next barrier, and the tensor memory is freed on every path.
#include <algorithm>

#include "decode_dev.cuh"

namespace tq {

int* decode_status_ptr();

namespace pftc {

constexpr int D = 128, TM = 128, TN = 128, NT = 256;
constexpr uint32_t KBLK = 16384, TILE_BYTES = 2 * KBLK;                     // a 128 x 128 fp16 operand tile: two 64-column blocks
constexpr uint32_t OFF_QR = 0, OFF_QD = TILE_BYTES, OFF_K = 2 * TILE_BYTES, OFF_V = 3 * TILE_BYTES, OFF_P = 4 * TILE_BYTES;
constexpr uint32_t OFF_KN = 5 * TILE_BYTES;                                 // float [128] key norms (or inverse staging scales)
constexpr uint32_t OFF_VN = OFF_KN + 512;                                   // float [128]
constexpr uint32_t OFF_POS = OFF_VN + 512;                                  // int   [128] absolute positions of the tile's tokens
constexpr uint32_t OFF_T4 = OFF_POS + 512;                                  // uint  [256][TREP] byte of two 4-bit codes -> half2
constexpr int TREP = 8;                                                      // copies of every table entry (lane l reads copy l mod 8)
constexpr uint32_t OFF_T2 = OFF_T4 + 1024 * TREP;                           // uint2 [256][TREP] byte of four 2-bit codes -> 4 halves
constexpr uint32_t OFF_CTAB = OFF_T2 + 2048 * TREP;                                // half  [32]
constexpr uint32_t OFF_BAR = OFF_CTAB + 64;                                 // two mbarriers
constexpr uint32_t OFF_SLOT = OFF_BAR + 16;                                 // tensor-memory base, largest value norm of the tile, abort flag
constexpr uint32_t SMEM_USED = OFF_SLOT + 16;
constexpr size_t SMEM_BYTES = SMEM_USED + 1024;                             // + slack to align the tiles to 1024 bytes
// the finish reuses the tiles: two [128][129] float arrays
constexpr uint32_t FIN_LD = 129, OFF_FD = 0, OFF_FP = 66560;
static_assert(OFF_FP + 128 * FIN_LD * 4 <= OFF_KN && 128 * FIN_LD * 4 <= OFF_FP, "finish scratch");
constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_WAIT = 104;
constexpr uint32_t TMEM_COLS = 512, COL_S = 0, COL_OP = 128, COL_OD = 256;

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
    float* s_kn = reinterpret_cast<float*>(smem + OFF_KN);
    float* s_vn = reinterpret_cast<float*>(smem + OFF_VN);
    int* s_pos = reinterpret_cast<int*>(smem + OFF_POS);
    uint32_t* t4 = reinterpret_cast<uint32_t*>(smem + OFF_T4);
    uint2* t2 = reinterpret_cast<uint2*>(smem + OFF_T2);
    __half* ctab = reinterpret_cast<__half*>(smem + OFF_CTAB);
    volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem + OFF_SLOT);   // [0] tmem base, [1] tile's largest value norm (bits), [2] abort, [3] every row sees every token of the tile
    const uint32_t bar_s = sbase + OFF_BAR, bar_o = bar_s + 8;

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
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        fence_barrier_init();
        slot[2] = 0u;
    }
    if (warp == 4) {
        tmem_alloc(sbase + OFF_SLOT, TMEM_COLS);
        tmem_relinquish();
    }
    if (tid < 32) {
        const int which = tid >> 4, k = tid & 15;
        const float* src = which == 0 ? p.kc_hi : p.vc_hi;
        const float sc = which == 1 ? p.v_scale_hi : 1.f;
        ctab[tid] = __float2half_rn((src != nullptr && k < (which ? 4 : 16)) ? src[k] * sc : 0.f);
    }
    __syncthreads();
    {
        const int e = tid;      // NT == 256 entries
        const __half2 hk = __halves2half2(ctab[e & 15], ctab[e >> 4]);
        const __half2 v01 = __halves2half2(ctab[16 + (e & 3)], ctab[16 + ((e >> 2) & 3)]);
        const __half2 v23 = __halves2half2(ctab[16 + ((e >> 4) & 3)], ctab[16 + (e >> 6)]);
#pragma unroll
        for (int r = 0; r < TREP; ++r) {
            t4[e * TREP + r] = *reinterpret_cast<const uint32_t*>(&hk);
            t2[e * TREP + r] = make_uint2(*reinterpret_cast<const uint32_t*>(&v01), *reinterpret_cast<const uint32_t*>(&v23));
        }
    }

    // ---------------- the query block: raw (scaled) and rotated (scaled), fp16 operand tiles ------------------------
    const float f = p.scale * LOG2E;
    {
        float* qf = reinterpret_cast<float*>(smem + OFF_K);                  // [128][D] float32 (the K and V tiles' space)
        float* rs = reinterpret_cast<float*>(smem + OFF_P);                  // [32][D + 1] slab of R
        for (int e = tid; e < TM * D; e += NT) {
            const int m = e / D, k = e - m * D;
            qf[e] = row_valid(m) ? load_as_f32(P.q, P.q_dtype, row_q_index(m) + k) * f : 0.f;
        }
        __syncthreads();
        for (int i = tid; i < TM * 16; i += NT) {                            // raw query tile: 16-byte chunks
            const int m = i >> 4, c = i & 15;
            const float4 a = *reinterpret_cast<const float4*>(qf + m * D + c * 8), bb = *reinterpret_cast<const float4*>(qf + m * D + c * 8 + 4);
            *reinterpret_cast<uint4*>(smem + OFF_QD + chunk_off(m, c)) =
                make_uint4(pack_h2(a.x, a.y), pack_h2(a.z, a.w), pack_h2(bb.x, bb.y), pack_h2(bb.z, bb.w));
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
                *reinterpret_cast<__half*>(smem + OFF_QR + chunk_off(m, j >> 3) + (j & 7) * 2) = __float2half_rn(acc[u]);
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = slot[0];

    // ---------------- per-row softmax state (threads 0 .. 127 own rows) ---------------------------------------------
    const bool row_thread = tid < TM;
    const int q_pos = (row_thread && row_valid(tid)) ? int(P.q_pos0 + tq0 + tid / GP) : -1;   // the latest position this row sees
    const int64_t cta_q_max = P.q_pos0 + min(tq0 + P.QT, P.Tq) - 1;
    const int64_t min_q_pos = P.q_pos0 + tq0;                                      // the earliest position any (valid) row sits at
    float m_ref = -1e30f, m_thr = -1e30f, l_sum = 0.f, vsc = 1.f, vthr = VSC_CAP;
    const uint32_t t_row = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t idesc_qk = make_idesc(false), idesc_pv = make_idesc(true);
    bool have_op = false, have_od = false;        // the accumulators hold sums (uniform over the CTA)
    uint32_t ph_s = 0, ph_o = 0;
    bool pv_pending = false;

    // bounded wait of every thread on an mbarrier; a thread that runs out raises the abort flag for everybody
    auto wait_bar = [&](uint32_t bar, uint32_t parity) {
        for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
            if (mbar_try(bar, parity)) return;
            if ((i & 1023u) == 1023u && slot[2]) return;
        }
        slot[2] = 1u;
        atomicCAS(P.status, 0, ERR_WAIT);
    };

    // One tile whose K / V / norms / positions are in shared memory: S, softmax, P, O += P V.
    auto run_tile = [&](bool dense_region) {
        // (1) scores
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_tile = sbase + (dense_region ? OFF_QD : OFF_QR);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_f16(tmem_base + COL_S, desc_kmajor(a_tile, ks), desc_kmajor(sbase + OFF_K, ks), idesc_qk, ks > 0 ? 1u : 0u);
            umma_commit(bar_s);
        }
        wait_bar(bar_s, ph_s);
        ph_s ^= 1u;
        tc_fence_after();
        if (row_thread) {
            const float vmax = __uint_as_float(slot[1]);
            const bool masked = slot[3] == 0u;                                // some token of the tile is hidden from some row (or dead)
            // Reference maximum / value scale: refreshed for the whole warp when any row needs it (the tensor-memory loads
            // and stores are warp-wide).  mx: the row's largest visible score of this tile.
            auto refresh = [&](float mx) {
                const float mn = fmaxf(fmaxf(m_ref, mx), -1e30f);
                float a = ex2(m_ref - mn);
                m_ref = mn; m_thr = mn + MAX_SLACK;
                l_sum *= a;
                if (vmax > vthr) {
                    int eb = (__float_as_int(vmax) >> 23) & 0xff;
                    eb = min(max(eb, 16), 240);
                    const float nsc = __int_as_float((261 - eb) << 23);
                    a *= nsc / vsc;
                    vsc = nsc;
                    vthr = VSC_CAP / nsc;
                }
#pragma unroll 1
                for (int acc = 0; acc < 2; ++acc) {
                    if (acc == 0 ? !have_op : !have_od) continue;
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
            // into the A-operand tile (row = this thread), the row's largest score alongside.  WRITE = false: the maximum only.
            auto sweep = [&](bool write, float& mx, float& lsum) {
                mx = -INFINITY; lsum = 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < TN; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(t_row + COL_S + c0, v);
                    tmem_ld_wait();
                    uint32_t h[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 kn = *reinterpret_cast<const float4*>(s_kn + c0 + j);
                        float s0 = __uint_as_float(v[j]) * kn.x, s1 = __uint_as_float(v[j + 1]) * kn.y;
                        float s2 = __uint_as_float(v[j + 2]) * kn.z, s3 = __uint_as_float(v[j + 3]) * kn.w;
                        if (masked) {
                            const int4 ps = *reinterpret_cast<const int4*>(s_pos + c0 + j);
                            s0 = ps.x <= q_pos ? s0 : -INFINITY; s1 = ps.y <= q_pos ? s1 : -INFINITY;
                            s2 = ps.z <= q_pos ? s2 : -INFINITY; s3 = ps.w <= q_pos ? s3 : -INFINITY;
                        }
                        mx = fmaxf(fmaxf(mx, fmaxf(s0, s1)), fmaxf(s2, s3));
                        if (write) {
                            const float4 vn = *reinterpret_cast<const float4*>(s_vn + c0 + j);
                            const float p0 = ex2(s0 - m_ref), p1 = ex2(s1 - m_ref), p2 = ex2(s2 - m_ref), p3 = ex2(s3 - m_ref);
                            lsum += (p0 + p1) + (p2 + p3);
                            h[j >> 1] = pack_h2(p0 * (vn.x * vsc), p1 * (vn.y * vsc));
                            h[(j >> 1) + 1] = pack_h2(p2 * (vn.z * vsc), p3 * (vn.w * vsc));
                        }
                    }
                    if (write) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4*>(smem + OFF_P + chunk_off(tid, (c0 >> 3) + c)) = make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
                    }
                }
            };
            float mx, lsum;
            // the very first tile (no reference yet) and a tile that moves the value scale: settle the references first
            if (__any_sync(0xffffffffu, m_ref <= -1e30f || vmax > vthr)) {
                sweep(false, mx, lsum);
                refresh(mx);
            }
            sweep(true, mx, lsum);
            if (__any_sync(0xffffffffu, mx > m_thr)) {        // a score beyond the slack: new reference, weights again (rare)
                refresh(mx);
                sweep(true, mx, lsum);
            }
            l_sum += lsum;
        }
        fence_proxy_async();        // P (generic-proxy stores) before the tensor core reads it
        tc_fence_before();
        __syncthreads();
        // (5) values
        if (tid == 0) {
            tc_fence_after();
            const uint32_t col = dense_region ? COL_OD : COL_OP;
            const bool have = dense_region ? have_od : have_op;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
                umma_f16(tmem_base + col, desc_kmajor(sbase + OFF_P, ks), desc_mnmajor(sbase + OFF_V, ks), idesc_pv, (have || ks > 0) ? 1u : 0u);
            umma_commit(bar_o);
        }
        if (dense_region) have_od = true; else have_op = true;
        pv_pending = true;
    };
    // before the tiles are overwritten (and before O is touched): the previous tile's second product has finished
    auto drain_pv = [&]() {
        if (pv_pending) {
            wait_bar(bar_o, ph_o);
            ph_o ^= 1u;
            tc_fence_after();
            pv_pending = false;
        }
    };

    // ---------------- packed tokens: absolute positions sink_len .. sink_len + c_len - 1 -----------------------------
    {
        const int64_t vis = min(p.c_len, cta_q_max - p.sink_len + 1);
        for (int64_t tok0 = 0; tok0 < vis; tok0 += TN) {
            drain_pv();
            if (__syncthreads_or(int(slot[2]))) break;                        // everybody is past the previous tile; leave together after a failed wait
            const int rows = int(min(int64_t(TN), p.c_len - tok0));
            if (tid == 0) {
                slot[1] = 0u;
                slot[3] = (rows == TN && p.sink_len + tok0 + TN - 1 <= min_q_pos) ? 1u : 0u;
            }
            {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.k_hi + (kvl * p.c_ls + tok0) * (D / 2));
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int i = tid + NT * k, r = i >> 4, w = i & 15;
                    const uint32_t x = r < rows ? __ldg(src + i) : 0u;
                    *reinterpret_cast<uint4*>(smem + OFF_K + chunk_off(r, w)) =
                        make_uint4(t4[(x & 255u) * TREP + cp], t4[((x >> 8) & 255u) * TREP + cp], t4[((x >> 16) & 255u) * TREP + cp], t4[(x >> 24) * TREP + cp]);
                }
            }
            {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.v_hi + (kvl * p.c_ls + tok0) * (D / 4));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = tid + NT * k, r = i >> 3, w = i & 7;
                    const uint32_t x = r < rows ? __ldg(src + i) : 0u;
                    const uint2 a = t2[(x & 255u) * TREP + cp], bb = t2[((x >> 8) & 255u) * TREP + cp], cc = t2[((x >> 16) & 255u) * TREP + cp], ee = t2[(x >> 24) * TREP + cp];
                    *reinterpret_cast<uint4*>(smem + OFF_V + chunk_off(r, 2 * w)) = make_uint4(a.x, a.y, bb.x, bb.y);
                    *reinterpret_cast<uint4*>(smem + OFF_V + chunk_off(r, 2 * w + 1)) = make_uint4(cc.x, cc.y, ee.x, ee.y);
                }
            }
            __syncthreads();                                                  // slot[1] reset before the maxima below
            if (tid < TN) {
                const bool live = tid < rows;
                const int64_t n = kvl * p.c_ls + tok0 + (live ? tid : 0);
                const float kn = live ? __ldg(p.k_norms + n) : 0.f, vn = live ? __ldg(p.v_norms + n) : 0.f;
                s_kn[tid] = kn; s_vn[tid] = vn;
                s_pos[tid] = live ? int(p.sink_len + tok0 + tid) : 0x7fffffff;
                float vm = vn;
#pragma unroll
                for (int off = 16; off; off >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, off));
                if (lane == 0) atomicMax(const_cast<uint32_t*>(slot + 1), __float_as_uint(fmaxf(vm, 0.f)));
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
            run_tile(false);
        }
    }

    // ---------------- uncompressed tokens: sink (positions 0 ..), recent (positions sink_len + c_len ..), raw query ----------------
    {
        const int64_t n_dense = p.sink_len + p.res_len;
        // dense index t -> position: t < sink_len ? t : c_len + t; tokens past the CTA's last position are not visited
        const int64_t vis_d = min(n_dense, max(p.sink_len, cta_q_max - p.c_len + 1));
        for (int64_t tok0 = 0; tok0 < vis_d; tok0 += TN) {
            drain_pv();
            if (__syncthreads_or(int(slot[2]))) break;
            if (tid == 0) {
                slot[1] = 0u;
                const int64_t tl = tok0 + TN - 1;                             // the tile's last token, if it has 128
                slot[3] = (tl < n_dense && (tl < p.sink_len ? tl : p.c_len + tl) <= min_q_pos) ? 1u : 0u;
            }
            __syncthreads();
            // two threads per token row: each converts 64 coordinates of the key row and of the value row; float32 /
            // bfloat16 rows under a per-token power-of-two scale (largest magnitude into [2^7, 2^8)) whose inverse goes
            // where the packed tokens have their norms
            {
                const int r = tid >> 1, hf = tid & 1;
                const int64_t tok = tok0 + r;
                const bool live = tok < n_dense;
                const bool in_sink = tok < p.sink_len;
                const int64_t e0 = live ? (in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len)) * D + hf * (D / 2) : 0;
                float inv_k = 0.f, inv_v = 0.f;
#pragma unroll 1
                for (int side = 0; side < 2; ++side) {
                    const void* base = side == 0 ? (in_sink ? p.sink_k : p.res_k) : (in_sink ? p.sink_v : p.res_v);
                    const uint32_t dst = side == 0 ? OFF_K : OFF_V;
                    float sc = 1.f;
                    if (p.dense_dtype == TQ_F16) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint4 x = live ? __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + e0) + c) : make_uint4(0, 0, 0, 0);
                            *reinterpret_cast<uint4*>(smem + dst + chunk_off(r, hf * 8 + c)) = x;
                        }
                    } else if (p.dense_dtype == TQ_BF16) {
                        uint4 x[8];
                        uint32_t mxb = 0u;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            x[c] = live ? __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + e0) + c) : make_uint4(0, 0, 0, 0);
                            const uint32_t mm = 0x7fff7fffu;
                            const uint32_t a = __vmaxu2(__vmaxu2(x[c].x & mm, x[c].y & mm), __vmaxu2(x[c].z & mm, x[c].w & mm));
                            mxb = max(mxb, max(a & 0xffffu, a >> 16) << 16);
                        }
                        mxb = max(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
                        sc = stage_scale(mxb);
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            auto two = [&](uint32_t w) -> uint32_t { return pack_h2(__uint_as_float(w << 16) * sc, __uint_as_float(w & 0xffff0000u) * sc); };
                            *reinterpret_cast<uint4*>(smem + dst + chunk_off(r, hf * 8 + c)) = make_uint4(two(x[c].x), two(x[c].y), two(x[c].z), two(x[c].w));
                        }
                    } else {
                        uint4 x[16];
                        uint32_t mxb = 0u;
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            x[c] = live ? __ldg(reinterpret_cast<const uint4*>(static_cast<const float*>(base) + e0) + c) : make_uint4(0, 0, 0, 0);
                            const uint32_t mm = 0x7fffffffu;
                            mxb = max(mxb, max(max(x[c].x & mm, x[c].y & mm), max(x[c].z & mm, x[c].w & mm)));
                        }
                        mxb = max(mxb, __shfl_xor_sync(0xffffffffu, mxb, 1));
                        sc = stage_scale(mxb);
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(smem + dst + chunk_off(r, hf * 8 + c)) =
                                make_uint4(pack_h2(__uint_as_float(x[2 * c].x) * sc, __uint_as_float(x[2 * c].y) * sc),
                                           pack_h2(__uint_as_float(x[2 * c].z) * sc, __uint_as_float(x[2 * c].w) * sc),
                                           pack_h2(__uint_as_float(x[2 * c + 1].x) * sc, __uint_as_float(x[2 * c + 1].y) * sc),
                                           pack_h2(__uint_as_float(x[2 * c + 1].z) * sc, __uint_as_float(x[2 * c + 1].w) * sc));
                    }
                    if (side == 0) inv_k = live ? 1.f / sc : 0.f; else inv_v = live ? 1.f / sc : 0.f;
                }
                if (hf == 0) {
                    s_kn[r] = inv_k; s_vn[r] = inv_v;
                    const int64_t pos = in_sink ? tok : p.c_len + tok;
                    s_pos[r] = live ? int(pos) : 0x7fffffff;
                }
                float vm = inv_v;
#pragma unroll
                for (int off = 16; off; off >>= 1) vm = fmaxf(vm, __shfl_xor_sync(0xffffffffu, vm, off));
                if (lane == 0) atomicMax(const_cast<uint32_t*>(slot + 1), __float_as_uint(vm));
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
            run_tile(true);
        }
    }
    drain_pv();

    // ---------------- finish: value scales, rotation of the packed part, normalise, store ---------------------------
    __syncthreads();                                                              // the tiles are dead
    float* fd = reinterpret_cast<float*>(smem + OFF_FD);                          // [128][129] sums of the uncompressed part
    float* fp = reinterpret_cast<float*>(smem + OFF_FP);                          // [128][129] sums of the packed part, rotated space
    if (row_thread) {
        const float ip = 1.f / (vsc * p.v_scale_hi), id = 1.f / vsc;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t v[32];
            if (have_op) { tmem_ld32(t_row + COL_OP + c0, v); tmem_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) fp[tid * FIN_LD + c0 + j] = have_op ? __uint_as_float(v[j]) * ip : 0.f;
            if (have_od) { tmem_ld32(t_row + COL_OD + c0, v); tmem_ld_wait(); }
#pragma unroll
            for (int j = 0; j < 32; ++j) fd[tid * FIN_LD + c0 + j] = have_od ? __uint_as_float(v[j]) * id : 0.f;
        }
        s_kn[tid] = l_sum;
    }
    tc_fence_before();
    __syncthreads();
    {
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
        const bool failed = slot[2] != 0u;
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
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace pftc

// Whether the tensor-core kernel takes this call; the caller has validated the arguments.
bool prefill_tc_applicable(const tq_decode_args* a, int t_q) {
    if (a->d != 128) return false;
    if (a->c_len > 0 && (a->k_bits_hi != 4 || a->k_bits_lo != 0 || a->v_bits_hi != 2 || a->v_bits_lo != 0 || !aligned(a->k_hi, 4) || !aligned(a->v_hi, 4)))
        return false;
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
