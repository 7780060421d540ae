// Decode attention over a cache with 4-bit keys and 2-bit values at d = 128: the specialised kernel.
//
// Same decomposition as the general kernel of decode.cu (grid (splits, kv_heads * head_groups, batch); warps own
// 16-token tiles; S = K.Q^T, online softmax, O^T += V^T.P^T with mma.sync.m16n8k16; last-arrival merge), with the
// following differences, all aimed at the instruction count per tile and at the fixed cost per CTA:
//
//   * Raw packed tiles (1024 B of keys, 512 B of values) arrive in a per-warp ring of five stages through bulk
//     asynchronous copies (cp.async.bulk, completion on an mbarrier); a warp owns a contiguous run of tiles, so
//     the norms of four tiles come in one pair of copies.  One lane issues 2.5 copies per tile and nobody
//     computes addresses per 16-byte chunk.  (The copy engine accepts a copy every ~20 cycles whatever its
//     size: 64-byte copies of norms per tile made the first tiles of sixteen warps queue for microseconds.)
//   * Operand fragments come straight from lookup tables: byte of two 4-bit codes -> half2 of two key centroids;
//     byte of the 2-bit codes of a token pair -> two half2 value fragments.  The tables sit at shared-window
//     address 0x10000 with one 256-byte slot per byte value (32 conflict-free copies of the key entry, 16 of the
//     value entry), so the address of an entry is ONE byte-permute of (packed word, per-lane constant).
//   * The query is rotated on the tensor cores: before the kernel waits for its predecessor on the stream, every
//     CTA splits R into two fp16 matrices, R = R_hi + 2^-11 R_lo (both products with an fp16 query are exact in the
//     fp32 accumulators), so that after the wait the rotation is 16-24 MMAs in eight warps.  The 64 KB the split
//     matrix occupies become two more ring stages per warp once the query is rotated.
//   * Partials stay in rotated space; the CTA that merges a (sequence, KV head) undoes the rotation once, in fp32,
//     reading R from global memory while the partials are in flight.
//
// Every mbarrier wait is bounded; if one runs out the kernel records a status code (tq_device_status), waits
// (bounded again) for the copies it still has in flight and finishes with whatever it has.
#include "decode_dev.cuh"

namespace tq {

namespace dd {

constexpr int D = 128, NW = DIRECT_WARPS, NT = NW * 32;
constexpr int STAGES = 5;
constexpr uint32_t KT = TILE * (D / 2), VT = TILE * (D / 4), STG = KT + VT;                  // 1024 + 512
constexpr int NCH = 4;                                         // tiles per chunk of norms (256 B of key norms + 256 B of value norms)
constexpr uint32_t NBUF = 2 * NCH * TILE * 4;                  // one norm buffer: 512 B

// Absolute shared-window addresses.  The dynamic allocation starts at `sbase` (reserved system bytes come first)
// and the tables must start on a 64 KB boundary.  Below the tables: R_lo (row j at j * 256, except the first rows,
// whose natural address would be below sbase: those go to RLO_TAIL) and R_hi; after the query is rotated the upper
// 52 KB of that space are ring stages 3 and 4 of every warp.
constexpr uint32_t RHI = 0x8000u;                              // 128 rows x 256 B
constexpr uint32_t XRING = 0x10000u - NW * 2 * STG;            // 16384: NW x 2 x STG, ends at the tables
constexpr uint32_t LUT_BASE = 0x10000u;                        // 256 slots of 256 B
constexpr uint32_t C_BASE = 0x20000u;
constexpr uint32_t RLO_TAIL = C_BASE;                          // rows 0 .. j0-1 of R_lo (j0 <= 8)
constexpr uint32_t RING = RLO_TAIL + 2048;                     // NW x 3 x STG: ring stages 0..2
constexpr uint32_t NORMS = RING + NW * 3 * STG;                // NW x 2 norm buffers
constexpr uint32_t BARS = NORMS + NW * 2 * NBUF;               // per warp: STAGES ring barriers + 2 norm barriers
constexpr uint32_t QS = BARS + 1024;                           // [8][D] half: scaled fp16 query (rotated or raw)
constexpr uint32_t CTAB = QS + HPG * D * 2;                    // 2 x 16 halves: key / value centroids
constexpr uint32_t MISC = CTAB + 128;                          // a few scalars
constexpr uint32_t SMEM_END = MISC + 64;
constexpr uint32_t MAX_SBASE = 2048;
constexpr int NBAR = STAGES + 2;
static_assert(NW * NBAR * 8 <= 1024, "ring barriers");
// phases after the main loop reuse the ring (CTA reduction) and the tables (merge)
constexpr int DS = D + 8, RWF = HPG * DS + 2 * HPG;            // floats per warp in the reduction buffer (2 DS = 16 mod 32: heads 2t, 2t+2 on different banks)
static_assert(uint32_t(NW) * RWF * 4 <= NW * 3 * STG, "reduction scratch must fit in the ring");
constexpr uint32_t M_ACC = LUT_BASE;                           // float [8][D]: merged packed part, rotated space
constexpr uint32_t M_AD = M_ACC + HPG * D * 4;                 // float [8][D]: merged part of the uncompressed tokens
constexpr uint32_t M_IL = M_AD + HPG * D * 4;                  // float [8]: 1 / softmax denominator
constexpr uint32_t M_ML = M_IL + 64;                           // float2 [NW][32]: (max, sum) pairs, one staging row per warp
static_assert(M_ML + NW * 32 * 8 <= C_BASE, "merge scratch must fit in the table region");
constexpr uint32_t M_PP = RING;                                // float [NW][8][D]: partial products with 8 rows of R each
static_assert(NW * HPG * D * 4 <= NW * 3 * STG, "partial products must fit in the ring");
// CTAs that own uncompressed tokens stage fp16 tiles from LUT_BASE on
static_assert(LUT_BASE + uint32_t(NW) * 2 * TILE * stage_ld<D>() * 2 <= BARS, "dense staging must end before the barriers");

constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_RING = 101, ERR_LAYOUT = 103, ERR_GATHER_WAIT = 201;

__device__ int g_status = 0;
__device__ unsigned g_probe_base = 0;

#ifdef TQ_TIMING
__device__ unsigned long long g_timing[4096 * 16];
__device__ __forceinline__ void stamp(int slot) {
    const int cta = int(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    if (threadIdx.x == 0 && cta < 4096) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_timing[cta * 16 + slot] = t;
    }
}
#define DD_STAMP(slot) stamp(slot)
#else
#define DD_STAMP(slot)
#endif

// ---- PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Bulk copy global -> this CTA's shared memory; bytes a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void ldsm_x4_at(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// Row j of the fp16 halves of R: 256 B, 16-byte chunk ch stored at chunk position (ch & 8) | ((ch ^ j) & 7), so
// that ldmatrix (eight rows, one chunk column) and the row-wise stores are both free of bank conflicts.
__device__ __forceinline__ uint32_t rhi_row(int j) { return RHI + uint32_t(j) * 256u; }
__device__ __forceinline__ uint32_t rlo_row(int j, int j0) { return j >= j0 ? uint32_t(j) * 256u : RLO_TAIL + uint32_t(j) * 256u; }
__device__ __forceinline__ uint32_t r_chunk(int j, int ch) { return uint32_t((ch & 8) | ((ch ^ j) & 7)) * 16u; }
__device__ __forceinline__ uint32_t h2_bits(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void smem_base_probe() {
    extern __shared__ __align__(16) unsigned char smem[];
    if (threadIdx.x == 0) g_probe_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
}

// Softmax step of the direct path: the validity masks only matter in the last tile of the cache, so the common
// case multiplies by the norms unconditionally.  Rows past the end of the cache hold arbitrary bytes.
__device__ __forceinline__ void softmax_direct(float (&s)[4], float kn0, float kn1, float vn0, float vn1, bool partial, bool ok0,
                                               bool ok1, WarpAcc<D>& st, uint32_t (&bp)[2]) {
    if (partial) {
        kn0 = ok0 ? kn0 : 0.f; kn1 = ok1 ? kn1 : 0.f; vn0 = ok0 ? vn0 : 0.f; vn1 = ok1 ? vn1 : 0.f;
        s[0] = ok0 ? s[0] * kn0 : -INFINITY; s[1] = ok0 ? s[1] * kn0 : -INFINITY;
        s[2] = ok1 ? s[2] * kn1 : -INFINITY; s[3] = ok1 ? s[3] * kn1 : -INFINITY;
    } else {
        s[0] *= kn0; s[1] *= kn0; s[2] *= kn1; s[3] *= kn1;
    }
    float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
    if (__any_sync(0xffffffffu, mx0 > st.mt[0] || mx1 > st.mt[1])) {
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        }
        const float mn0 = fmaxf(fmaxf(st.m[0], mx0), -1e30f), mn1 = fmaxf(fmaxf(st.m[1], mx1), -1e30f);
        const float a0 = ex2(st.m[0] - mn0), a1 = ex2(st.m[1] - mn1);
        st.m[0] = mn0; st.m[1] = mn1;
        st.mt[0] = mn0 + MAX_SLACK; st.mt[1] = mn1 + MAX_SLACK;
        st.l[0] *= a0; st.l[1] *= a1;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
            st.o[mt][0] *= a0; st.o[mt][1] *= a1; st.o[mt][2] *= a0; st.o[mt][3] *= a1;
        }
    }
    const float p0 = ex2(s[0] - st.m[0]), p1 = ex2(s[1] - st.m[1]), p2 = ex2(s[2] - st.m[0]), p3 = ex2(s[3] - st.m[1]);
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    const uint32_t h0 = pack_h2(fminf(p0 * vn0, 65504.f), fminf(p1 * vn0, 65504.f));
    const uint32_t h1 = pack_h2(fminf(p2 * vn1, 65504.f), fminf(p3 * vn1, 65504.f));
    bp[0] = movm_t(h0);
    bp[1] = movm_t(h1);
}

// NH: query heads per group the rotations are compiled for (4 or 8); heads_here <= NH.
template <int NH>
__global__ void __launch_bounds__(NT, 1) decode_direct_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    auto gp = [&](uint32_t abs_addr) -> unsigned char* { return smem + (abs_addr - sbase); };   // generic pointer of a window address
    const int j0 = int((sbase + 255u) >> 8);           // rows of R_lo below j0 live in RLO_TAIL
    __half* qs = reinterpret_cast<__half*>(gp(QS));
    __half* ctab = reinterpret_cast<__half*>(gp(CTAB));
    float* s_misc = reinterpret_cast<float*>(gp(MISC));

    DD_STAMP(0);
    pdl_trigger();     // the next launch on the stream may become resident and run its own prologue
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;        // lane of the cache arrays
    const bool dense = split >= p.n_ps;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int64_t qbase = (int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG) * D;   // first query head of this group
    const int S = p.n_ps + p.n_ds;
    const uint32_t my_bars = BARS + warp * (NBAR * 8), my_nbars = my_bars + STAGES * 8;
    if (sbase > MAX_SBASE || (sbase & 15u)) {            // cannot happen after the host-side probe; never run on a bad plan
        if (tid == 0) atomicCAS(&g_status, 0, ERR_LAYOUT);
        return;
    }

    // ---------------- prologue on constants only (runs before the previous launch has finished) -----------
    float4 rr[D * D / 4 / NT];         // this thread's 32 entries of R, in flight across the prologue
    if (!dense) {
        if (tid < NW * NBAR) {
            mbar_init(BARS + tid * 8, 1);
            fence_barrier_init();
        }
        // R (one row per warp and pass, coalesced 128-bit loads) is split into fp16 halves further down, once the
        // query loads are on their way; the tables are built while it is in flight
#pragma unroll
        for (int i = 0; i < D * D / 4 / NT; ++i) rr[i] = __ldg(reinterpret_cast<const float4*>(p.rot) + tid + i * NT);
        if (tid < 32) {
            const int which = tid >> 4, k = tid & 15;
            float c = 0.f;
            if (k < (which ? 4 : 16)) c = p.cent_by_value ? (which ? p.vc4[k & 3] : p.kc16[k]) : (which ? p.vc_hi : p.kc_hi)[k];
            ctab[which * 16 + k] = __float2half_rn(c * (which ? p.v_scale_hi : 1.f));
        }
        __syncthreads();
        DD_STAMP(9);
        // tables: slot e at LUT_BASE + e * 256: +0 32 copies of half2(kc[e & 15], kc[e >> 4]);
        // +128 16 copies of the value entry (two half2: one per coordinate, each pairing the two tokens); copies r with
        // (r & 2) serve lanes that read the token pair in swapped order
        uint4* lut = reinterpret_cast<uint4*>(gp(LUT_BASE));
        for (int idx = tid; idx < 256 * 16; idx += NT) {
            const int e = idx >> 4, q = idx & 15;
            uint4 v;
            if (q < 8) {
                const __half2 h = __halves2half2(ctab[e & 15], ctab[e >> 4]);
                const uint32_t u = *reinterpret_cast<const uint32_t*>(&h);
                v = make_uint4(u, u, u, u);
            } else {
                // entry e: low nibble = two adjacent 2-bit codes of the first word read, high nibble = the same two
                // coordinates of the second word; tokens (A, B) = (first, second), or (second, first) for swapped copies
                const bool sw = (q & 1) != 0;            // copies 2(q-8), 2(q-8)+1: bit 1 of the copy index is (q & 1)
                const int na = sw ? e >> 4 : e & 15, nb = sw ? e & 15 : e >> 4;
                const __half2 h0 = __halves2half2(ctab[16 + (na & 3)], ctab[16 + (nb & 3)]);      // first coordinate: (token A, token B)
                const __half2 h1 = __halves2half2(ctab[16 + (na >> 2)], ctab[16 + (nb >> 2)]);    // second coordinate
                const uint32_t u0 = *reinterpret_cast<const uint32_t*>(&h0), u1 = *reinterpret_cast<const uint32_t*>(&h1);
                v = make_uint4(u0, u1, u0, u1);
            }
            lut[idx] = v;
        }
    }
    DD_STAMP(1);
    pdl_wait();        // from here on: the query, the cache and the workspace of the previous launch are settled
    DD_STAMP(2);

    // ---------------- ring of packed tiles --------------------------------------------------------------
    // warp w owns a contiguous run of the CTA's tiles: n_my tiles from tile `first`
    const int n_tiles = int((p.c_len + TILE - 1) / TILE);
    const int tile_lo = int(split * p.p_tps);
    const int tile_hi = dense ? 0 : min(tile_lo + int(p.p_tps), n_tiles);
    const int n_cta = max(tile_hi - tile_lo, 0), t_base = n_cta / NW, t_extra = n_cta - t_base * NW;
    const int n_my = t_base + (warp < t_extra ? 1 : 0);
    const int first = tile_lo + warp * t_base + min(warp, t_extra);
    // stage s of this warp: 0..2 in RING, 3..4 in XRING (usable once the query is rotated)
    const uint32_t ring_lo = RING + warp * (3 * STG), ring_hi = XRING + warp * (2 * STG) - 3 * STG;
    const uint32_t nbuf0 = NORMS + warp * (2 * NBUF);
    auto stage_addr = [&](int stage) -> uint32_t { return (stage < 3 ? ring_lo : ring_hi) + stage * STG; };
    auto issue = [&](int stage, int i) {                 // one lane; local tile i; the whole tile lies inside the lane's allocation
        const uint32_t sb = stage_addr(stage), bar = my_bars + stage * 8;
        const int64_t tok0 = int64_t(first + i) * TILE;
        mbar_expect_tx(bar, STG);
        bulk_g2s(sb, p.k_hi + (kvl * p.c_ls + tok0) * (D / 2), KT, bar);
        bulk_g2s(sb + KT, p.v_hi + (kvl * p.c_ls + tok0) * (D / 4), VT, bar);
    };
    auto issue_norms = [&](int chunk) {                  // one lane; norms of local tiles [chunk * NCH, + NCH) into buffer chunk & 1
        const uint32_t nb = nbuf0 + (chunk & 1) * NBUF, bar = my_nbars + (chunk & 1) * 8;
        const int64_t tok0 = int64_t(first + chunk * NCH) * TILE;
        const uint32_t bytes = uint32_t(min(NCH, n_my - chunk * NCH)) * (TILE * 4);
        mbar_expect_tx(bar, 2 * bytes);
        bulk_g2s(nb, p.k_norms + kvl * p.c_ls + tok0, bytes, bar);
        bulk_g2s(nb + NBUF / 2, p.v_norms + kvl * p.c_ls + tok0, bytes, bar);
    };
    if (!dense && lane == 0 && n_my > 0) {               // the first tile only: the copy engine's queue is short and the
        issue_norms(0);                                  // query rotation must not wait behind sixteen warps' prefetches
        issue(0, 0);
    }

    // ---------------- the query heads of this group: (rotated) scaled fp16 ------------------------------------
    const float f = p.scale * LOG2E;
    bool failed = false;
    // query fragments (B operand of the rotation) for the eight warps that rotate: loads issued here, used after
    // the split of R below
    const bool q16 = p.q_dtype == TQ_F16;
    uint32_t bh[D / 16][2], bl[D / 16][2];
    if (!dense && warp < D / 16) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            bh[ks][0] = bh[ks][1] = bl[ks][0] = bl[ks][1] = 0u;
            if (g < heads_here) {
                const int64_t e = qbase + g * D + ks * 16 + 2 * t;
                if (q16) {
                    bh[ks][0] = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __half*>(p.q) + e));
                    bh[ks][1] = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __half*>(p.q) + e + 8));
                } else {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float x0 = load_as_f32(p.q, p.q_dtype, e + 8 * u), x1 = load_as_f32(p.q, p.q_dtype, e + 8 * u + 1);
                        const __half2 h = __floats2half2_rn(x0, x1);
                        const float2 hf = __half22float2(h);
                        bh[ks][u] = *reinterpret_cast<const uint32_t*>(&h);
                        bl[ks][u] = h2_bits((x0 - hf.x) * 2048.f, (x1 - hf.y) * 2048.f);
                    }
                }
            }
        }
    }
    if (!dense) {
        // R -> fp16 halves, R = R_hi + 2^-11 R_lo
#pragma unroll
        for (int i = 0; i < D * D / 4 / NT; ++i) {
            const int j = warp + i * NW, c4 = lane;       // float4 c4 of row j: coordinates 4 c4 .. 4 c4 + 3
            const float4 x = rr[i];
            const __half2 h01 = __floats2half2_rn(x.x, x.y), h23 = __floats2half2_rn(x.z, x.w);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const uint32_t off = r_chunk(j, c4 >> 1) + (c4 & 1) * 8;
            sts64(rhi_row(j) + off, *reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
            sts64(rlo_row(j, j0) + off, h2_bits((x.x - f01.x) * 2048.f, (x.y - f01.y) * 2048.f),
                  h2_bits((x.z - f23.x) * 2048.f, (x.w - f23.y) * 2048.f));
        }
        __syncthreads();
    }
    DD_STAMP(10);
    if (dense) {
        for (int e = tid; e < heads_here * D; e += NT) qs[e] = __float2half_rn(load_as_f32(p.q, p.q_dtype, qbase + e) * f);
    } else if (warp < D / 16) {
        // q_rot[h][j] = sum_k q[h][k] R[j][k]  (rotation.py:81-110) on the tensor cores: warp w owns rows 16w..16w+15 of R
        // (A operand, ldmatrix), the query heads are the B operand.  A query that is not fp16 is split like R
        // (q = q_hi + 2^-11 q_lo); the product R_lo q_lo is below fp32 resolution.
        float ym[4] = {0.f, 0.f, 0.f, 0.f}, yc[4] = {0.f, 0.f, 0.f, 0.f};
        const int row = warp * 16 + (lane & 15);
        const uint32_t a_hi = rhi_row(row), a_lo = rlo_row(row, j0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = r_chunk(row, ks * 2 + (lane >> 4));
            uint32_t ah[4], al[4];
            ldsm_x4_at(ah, a_hi + off);
            ldsm_x4_at(al, a_lo + off);
            mma16816(ym, ah[0], ah[1], ah[2], ah[3], bh[ks][0], bh[ks][1]);
            mma16816(yc, al[0], al[1], al[2], al[3], bh[ks][0], bh[ks][1]);
            if (!q16) mma16816(yc, ah[0], ah[1], ah[2], ah[3], bl[ks][0], bl[ks][1]);
        }
        // accumulator layout: rows g, g+8 of the tile x heads 2t, 2t+1
        const int j = warp * 16 + g;
        qs[(2 * t) * D + j] = __float2half_rn((ym[0] + yc[0] * (1.f / 2048.f)) * f);
        qs[(2 * t + 1) * D + j] = __float2half_rn((ym[1] + yc[1] * (1.f / 2048.f)) * f);
        qs[(2 * t) * D + j + 8] = __float2half_rn((ym[2] + yc[2] * (1.f / 2048.f)) * f);
        qs[(2 * t + 1) * D + j + 8] = __float2half_rn((ym[3] + yc[3] * (1.f / 2048.f)) * f);
        DD_STAMP(11);
    }
    __syncthreads();       // rotated query visible; the split matrix is dead: its space joins the ring
    if (!dense && lane == 0) {
        fence_proxy_async();   // the matrix was read through the generic proxy; the copies write through the async one
#pragma unroll
        for (int i = 1; i < STAGES; ++i)
            if (i < n_my) issue(i, i);
    }
    DD_STAMP(3);

    WarpAcc<D> st;
    st.m[0] = st.m[1] = st.mt[0] = st.mt[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) st.o[mt][0] = st.o[mt][1] = st.o[mt][2] = st.o[mt][3] = 0.f;

    if (dense) {
        // ---------------- uncompressed tokens: sink then residual window, raw query ----------------
        uint32_t bq[D / 16][2];
        const __half* qh = qs + g * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
            bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
        }
        __half* Ks = reinterpret_cast<__half*>(gp(LUT_BASE)) + size_t(warp) * 2 * TILE * stage_ld<D>();
        __half* Vs = Ks + TILE * stage_ld<D>();
        const int64_t d_lo = int64_t(split - p.n_ps) * p.d_tps;
        dense_tiles<D, NW>(p, kvl, d_lo, d_lo + p.d_tps, Ks, Vs, bq, st, warp, lane);
    } else {
        // ---------------- packed tokens ------------------------------------------------------------------
        // Query fragments in the byte order of the 4-bit rows: thread t owns coordinates [t*32, t*32+32).
        uint32_t bq[D / 16][2];
        {
            const __half* qh = qs + g * D + t * (D / 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks) : 0u;
                bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks + 2) : 0u;
            }
        }
        // table addresses by byte-permute: {copy offset, byte value, 0x01, 0x00} = LUT_BASE + value * 256 + copy offset
        const uint32_t c4 = LUT_BASE | uint32_t(lane * 4);
        const uint32_t c2 = LUT_BASE | 128u | uint32_t((lane & 15) * 8);
        // value rows of a token pair are read in swapped order by the lanes with t >= 2 (bank conflicts); their
        // table copies pair the centroids the other way round
        const int sw = t >> 1;
        const uint32_t vo_a = KT + uint32_t(2 * t + sw) * (D / 4) + g * 4, vo_b = KT + uint32_t(2 * t + 1 - sw) * (D / 4) + g * 4;
        const int c_len = int(p.c_len);
        auto compute = [&](int stage, int i) {
            const uint32_t sb = stage_addr(stage), nb = nbuf0 + ((i / NCH) & 1) * NBUF + (i & (NCH - 1)) * (TILE * 4);
            const int tok0 = (first + i) * TILE;
            const uint4 q0 = ring128(sb + lane * 16);            // token g,   this thread's quarter row
            const uint4 q1 = ring128(sb + 512 + lane * 16);      // token g+8
            const float kn0 = __uint_as_float(ring32(nb + g * 4)), kn1 = __uint_as_float(ring32(nb + 32 + g * 4));
            const float vn0 = __uint_as_float(ring32(nb + NBUF / 2 + g * 4)), vn1 = __uint_as_float(ring32(nb + NBUF / 2 + 32 + g * 4));
            const uint32_t va = ring32(sb + vo_a), vb = ring32(sb + vo_b);
            const uint32_t vc = ring32(sb + vo_a + 8 * (D / 4)), vd = ring32(sb + vo_b + 8 * (D / 4));
            // two independent accumulators (even / odd k-steps) halve the dependent MMA chain
            float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                // bytes 2ks, 2ks+1 of the quarter row
                const int wi = ks >> 1;
                const uint32_t w0 = wi == 0 ? q0.x : wi == 1 ? q0.y : wi == 2 ? q0.z : q0.w;
                const uint32_t w1 = wi == 0 ? q1.x : wi == 1 ? q1.y : wi == 2 ? q1.z : q1.w;
                const int b0 = (ks & 1) * 2;
                const uint32_t a0 = lut32(__byte_perm(w0, c4, 0x7604 | (b0 << 4)));
                const uint32_t a1 = lut32(__byte_perm(w1, c4, 0x7604 | (b0 << 4)));
                const uint32_t a2 = lut32(__byte_perm(w0, c4, 0x7604 | ((b0 + 1) << 4)));
                const uint32_t a3 = lut32(__byte_perm(w1, c4, 0x7604 | ((b0 + 1) << 4)));
                if (ks & 1) mma16816(s2, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
                else mma16816(s, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += s2[i];
            uint32_t bp[2];
            softmax_direct(s, kn0, kn1, vn0, vn1, tok0 + TILE > c_len, tok0 + g < c_len, tok0 + g + 8 < c_len, st, bp);
            // pair the nibbles (two adjacent coordinates) of the two tokens: byte j of Z0 = (first word, nibble 2j) |
            // (second word, nibble 2j) << 4, Z1 the odd nibbles.  One 64-bit lookup then yields the two operand registers
            // that sit next to each other in the MMA (rows g and g+8 = the two coordinates, token pair in each).
            const uint32_t z0 = (va & 0x0F0F0F0Fu) | ((vb << 4) & 0xF0F0F0F0u), z1 = ((va >> 4) & 0x0F0F0F0Fu) | (vb & 0xF0F0F0F0u);
            const uint32_t w0 = (vc & 0x0F0F0F0Fu) | ((vd << 4) & 0xF0F0F0F0u), w1 = ((vc >> 4) & 0x0F0F0F0Fu) | (vd & 0xF0F0F0F0u);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint2 e01 = lut64(__byte_perm(z0, c2, 0x7604 | (k << 4)));   // m-tile 2k:   tokens 2t, 2t+1
                const uint2 e23 = lut64(__byte_perm(w0, c2, 0x7604 | (k << 4)));   //             tokens 2t+8, 2t+9
                const uint2 f01 = lut64(__byte_perm(z1, c2, 0x7604 | (k << 4)));   // m-tile 2k+1
                const uint2 f23 = lut64(__byte_perm(w1, c2, 0x7604 | (k << 4)));
                mma16816(st.o[2 * k], e01.x, e01.y, e23.x, e23.y, bp[0], bp[1]);
                mma16816(st.o[2 * k + 1], f01.x, f01.y, f23.x, f23.y, bp[0], bp[1]);
            }
        };
        // Up to five tiles per warp in flight; a stage is refilled (by one lane) as soon as the warp is done with it.
        int stage = 0, done = 0, nreq = n_my > 0 ? 1 : 0;     // nreq: chunks of norms requested so far
        uint32_t parity = 0;
        for (; done < n_my; ++done) {
            bool ok = !failed;
            if ((done & (NCH - 1)) == 0) {
                const int chunk = done / NCH;
                ok = ok && mbar_wait(my_nbars + (chunk & 1) * 8, uint32_t(chunk >> 1) & 1u);
                if (lane == 0 && (chunk + 1) * NCH < n_my) {      // the other buffer was last read a whole chunk ago
                    fence_proxy_async();
                    issue_norms(chunk + 1);
                }
                if ((chunk + 1) * NCH < n_my) nreq = chunk + 2;
            }
            ok = ok && mbar_wait(my_bars + stage * 8, parity);
            if (!__all_sync(0xffffffffu, ok)) {          // warp-uniform: the tile step below is full of warp collectives
                if (!failed) atomicCAS(&g_status, 0, ERR_RING);
                failed = true;
                break;
            }
            compute(stage, done);
            __syncwarp();       // every lane is done with this stage before it is refilled
            if (lane == 0 && done + STAGES < n_my) {
                fence_proxy_async();
                issue(stage, done + STAGES);
            }
            if (++stage == STAGES) { stage = 0; parity ^= 1u; }
        }
        if (failed) {
            // copies already requested may still land in the ring: give each a bounded chance to finish before the
            // ring is reused (tiles requested but not consumed: at most STAGES; at most two chunks of norms)
            const int requested = min(n_my, done + STAGES);
            for (int k = done; k < requested; ++k) {
                mbar_wait(my_bars + stage * 8, parity);
                if (++stage == STAGES) { stage = 0; parity ^= 1u; }
            }
            for (int c = max(nreq - 2, 0); c < nreq; ++c) mbar_wait(my_nbars + (c & 1) * 8, uint32_t(c >> 1) & 1u);
        }
    }

    // ---------------- CTA reduction over warps ----------------------------------------------------------------
    // Partials live in SLOT order: slot(c) = ((c & 15) >> 1) * 16 + (c >> 4) * 2 + (c & 1) for coordinate c, which is the
    // order the packed path's accumulator fragments come in (m-tile mt, row g, pair r -> slot mt * 16 + g * 2 + r);
    // the merging CTA returns to coordinate order.
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
    }
    __syncthreads();   // staging / tables / ring are dead from here on
    DD_STAMP(4);
    float* red = reinterpret_cast<float*>(gp(RING));
    {
        float* ro = red + size_t(warp) * RWF;               // [8][DS]: head-major
        float* rm = ro + HPG * DS;                          // [8] max, [8] sum
        if (2 * t < heads_here) {                           // lanes that hold only padding heads store nothing
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt) {
                if (!dense) {                                // rows g, g+8 of the m-tile are the pair of slot mt * 16 + g * 2
                    const int sl = mt * 16 + g * 2;
                    *reinterpret_cast<float2*>(ro + (2 * t) * DS + sl) = make_float2(st.o[mt][0], st.o[mt][2]);
                    *reinterpret_cast<float2*>(ro + (2 * t + 1) * DS + sl) = make_float2(st.o[mt][1], st.o[mt][3]);
                } else {                                     // rows are coordinates mt * 16 + g and + 8
                    const int sl = (g >> 1) * 16 + mt * 2 + (g & 1);
                    ro[(2 * t) * DS + sl] = st.o[mt][0]; ro[(2 * t + 1) * DS + sl] = st.o[mt][1];
                    ro[(2 * t) * DS + sl + 64] = st.o[mt][2]; ro[(2 * t + 1) * DS + sl + 64] = st.o[mt][3];
                }
            }
        }
        if (g == 0) {
            rm[2 * t] = st.m[0]; rm[2 * t + 1] = st.m[1];
            rm[HPG + 2 * t] = st.l[0]; rm[HPG + 2 * t + 1] = st.l[1];
        }
    }
    __syncthreads();
    DD_STAMP(12);
    const int64_t grp = (kvl * p.HG + hg);
    const int64_t pidx = grp * S + split;
    float* po = p.part_o + pidx * (int64_t(p.slots) * D);   // [slots][D] in slot order: packed splits in ROTATED space, dense splits unrotated
    float* pml = p.part_ml + pidx * (p.slots * 2);          // [slots][2]
    {
        // every thread recomputes the sixteen warp weights of its head: cheaper than a staged pass with two more barriers
        const float inv_vs = dense ? 1.f : 1.f / p.v_scale_hi;
        for (int e = tid; e < D * heads_here; e += NT) {     // e = h * D + slot: contiguous in the workspace
            const int h = e / D, sl = e - h * D;
            float mw[NW];
            float M = -INFINITY;
#pragma unroll
            for (int x = 0; x < NW; ++x) { mw[x] = red[size_t(x) * RWF + HPG * DS + h]; M = fmaxf(M, mw[x]); }
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int x = 0; x < NW; ++x) {
                const float w = (mw[x] == -INFINITY) ? 0.f : ex2(mw[x] - M);
                acc = fmaf(w, red[size_t(x) * RWF + h * DS + sl], acc);
                if (sl == 0) L = fmaf(w, red[size_t(x) * RWF + HPG * DS + HPG + h], L);
            }
            po[e] = acc * inv_vs;
            if (sl == 0) *reinterpret_cast<float2*>(pml + 2 * h) = make_float2(M, L);
        }
    }

    // ---------------- last arrival for this (sequence, KV head, head group) merges -----------------------
    __syncthreads();
    DD_STAMP(13);
    if (tid == 0) {
        __threadfence();       // cumulative: publishes the partial every thread of this CTA wrote before the barrier
        const int prev = atomicAdd(p.counters + grp, 1);
        s_misc[8] = (prev == S - 1) ? 1.f : 0.f;
        if (prev == S - 1) p.counters[grp] = 0;     // ready for the next launch
    }
    DD_STAMP(5);
    __syncthreads();
    if (s_misc[8] == 0.f) return;
    DD_STAMP(7);
    const int SL = p.slots;
    const int64_t base = grp * S;
    const int64_t stride = int64_t(SL) * D;
    float* s_acc = reinterpret_cast<float*>(gp(M_ACC));                         // [8][D] merged packed part, coordinate order
    float* s_ad = reinterpret_cast<float*>(gp(M_AD));                           // [8][D] merged unrotated part, coordinate order
    float* s_il = reinterpret_cast<float*>(gp(M_IL));                           // [8] 1 / sum
    float* s_pp = reinterpret_cast<float*>(gp(M_PP));                           // [NW][8][D]
    // One round of loads.  Thread = (head, slot) element: its partials of up to 24 splits; lane u of every warp:
    // the (max, sum) pair of split u for the warp's head (a warp's 32 elements share the head), passed on through the
    // warp's own staging row; thread = (slab of 8 rows of R, 4 columns): its 8 x 4 entries of R.
    constexpr int U = 24;
    constexpr int EPT = NH * D / NT;                                            // elements per thread: 1 or 2
    const int rs = tid >> 5, jq = tid & 31;                                     // rows 8 rs .. 8 rs + 7, columns 4 jq .. 4 jq + 3
    float v0[U];
    float4 rcol[8];
    float2* s_ml = reinterpret_cast<float2*>(gp(M_ML)) + warp * 32;             // [NW][32]
    {
        const bool live = tid < D * heads_here;
        const float* src = p.part_o + base * stride + tid;
#pragma unroll
        for (int u = 0; u < U; ++u) v0[u] = (live && u < S) ? __ldcg(src + u * stride) : 0.f;
        const float2* mls = reinterpret_cast<const float2*>(p.part_ml) + base * SL + (live ? tid / D : 0);
        s_ml[lane] = (live && lane < S) ? __ldcg(mls + lane * SL) : make_float2(-INFINITY, 0.f);
#pragma unroll
        for (int c = 0; c < 8; ++c) rcol[c] = __ldg(reinterpret_cast<const float4*>(p.rot + (rs * 8 + c) * D) + jq);
    }
    __syncwarp();
    DD_STAMP(8);
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int e = tid + i * NT;
        if (e < D * heads_here) {
            const int h = e / D, sl = e - h * D;
            const int c = ((sl >> 1) & 7) * 16 + (sl >> 4) * 2 + (sl & 1);      // coordinate of this slot
            const float* src = p.part_o + base * stride + e;
            const float2* mls = reinterpret_cast<const float2*>(p.part_ml) + base * SL + h;
            float M = -INFINITY;
            if (i == 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) M = fmaxf(M, s_ml[u].x);
                for (int sidx = U; sidx < S; ++sidx) M = fmaxf(M, __ldcg(mls + sidx * SL).x);
            } else {
                for (int sidx = 0; sidx < S; ++sidx) M = fmaxf(M, __ldcg(mls + sidx * SL).x);
            }
            float ap = 0.f, ad = 0.f, L = 0.f;
            if (i == 0) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float2 x = s_ml[u];
                    const float w = (x.x == -INFINITY) ? 0.f : ex2(x.x - M);               // splits past S carry -inf
                    L = fmaf(w, x.y, L);
                    if (u < p.n_ps) ap = fmaf(w, v0[u], ap); else ad = fmaf(w, v0[u], ad);
                }
            }
            for (int sidx = (i == 0 ? U : 0); sidx < S; ++sidx) {
                const float2 x = __ldcg(mls + sidx * SL);
                const float w = (x.x == -INFINITY) ? 0.f : ex2(x.x - M);
                L = fmaf(w, x.y, L);
                const float v = __ldcg(src + sidx * stride);
                if (sidx < p.n_ps) ap = fmaf(w, v, ap); else ad = fmaf(w, v, ad);
            }
            s_acc[h * D + c] = ap;
            s_ad[h * D + c] = ad;
            if (sl == 0) s_il[h] = 1.f / L;
        }
    }
    __syncthreads();
    DD_STAMP(14);
    // undo the rotation of the packed part once (y @ R, rotation.py:68-78): partial products over 8 rows of R
    {
        float acc[NH][4];
#pragma unroll
        for (int h = 0; h < NH; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            const float4 a0 = *reinterpret_cast<const float4*>(s_acc + h * D + rs * 8);
            const float4 a1 = *reinterpret_cast<const float4*>(s_acc + h * D + rs * 8 + 4);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                acc[h][0] = fmaf(a[c], rcol[c].x, acc[h][0]); acc[h][1] = fmaf(a[c], rcol[c].y, acc[h][1]);
                acc[h][2] = fmaf(a[c], rcol[c].z, acc[h][2]); acc[h][3] = fmaf(a[c], rcol[c].w, acc[h][3]);
            }
        }
#pragma unroll
        for (int h = 0; h < NH; ++h)
            *reinterpret_cast<float4*>(s_pp + (rs * HPG + h) * D + jq * 4) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
    }
    __syncthreads();
    DD_STAMP(15);
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int e = tid + i * NT;
        if (e < D * heads_here) {
            const int h = e / D, j = e - h * D;
            float v = s_ad[e];
#pragma unroll
            for (int x = 0; x < NW; ++x) v += s_pp[(x * HPG + h) * D + j];
            // fused gather: the group's first head in the peers' (batch, heads_total, d) buffers
            const int64_t gbase = (int64_t(blockIdx.z) * p.heads_total + p.head_offset + int64_t(blockIdx.y / p.HG) * p.G + (blockIdx.y % p.HG) * HPG) * D;
            store_result(p, qbase + e, gbase + e, v * s_il[h]);
        }
    }
    signal_peers(p);
    DD_STAMP(6);
}

// Consumer side of the fused gather: returns once the arrival counter (written by the peers' merge steps) has reached
// its target: `count` itself, or, with a `consumed` counter, *consumed + count, after which *consumed moves up by count
// (the launch parameters then never change, so the launch can sit in a CUDA graph).  Both counters live in this GPU's
// own memory; the poll is bounded (about two seconds), then a status is left.
__global__ void gather_wait_kernel(const unsigned long long* arrivals, unsigned long long* consumed, unsigned long long count, int max_polls) {
    if (threadIdx.x != 0) return;
    const unsigned long long target = consumed ? *consumed + count : count;
    if (consumed) *consumed = target;                       // also after a time-out: later waits keep their meaning
    for (int it = 0; it < max_polls; ++it) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(arrivals) : "memory");
        if (v >= target) return;
        __nanosleep(it < 64 ? 32 : 512);
    }
    atomicCAS(&g_status, 0, ERR_GATHER_WAIT);
}

static unsigned probe_smem_base() {
    // The kernel addresses its tables by absolute shared-window address; where the dynamic allocation starts is a
    // property of the device / driver, read once per device with a one-thread launch.
    static unsigned cache[64];
    static bool have[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ~0u;
    if (!have[dev]) {
        unsigned v = ~0u;
        smem_base_probe<<<1, 32, 1024>>>();
        if (cudaGetLastError() != cudaSuccess || cudaMemcpyFromSymbol(&v, g_probe_base, sizeof(v)) != cudaSuccess) return ~0u;
        cache[dev] = v;
        have[dev] = true;
    }
    return cache[dev];
}

}  // namespace dd

bool direct_supported() {
    const unsigned sb = dd::probe_smem_base();
    if (sb == ~0u || sb > dd::MAX_SBASE || (sb & 15u)) return false;
    int dev = 0, max_optin = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
    return size_t(dd::SMEM_END - sb) <= size_t(max_optin);
}

template <int NH> static int launch_nh(const DecodeParams& p, cudaStream_t s) {
    const unsigned sb = dd::probe_smem_base();
    const size_t smem = dd::SMEM_END - sb;
    static bool set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(dd::decode_direct_kernel<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev] = true;
    }
    // Programmatic stream serialisation: the grid may become resident before its predecessor on the stream
    // has finished; the kernel calls griddepcontrol.wait before it touches anything but constants.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(p.n_ps + p.n_ds), unsigned(p.Hkv * p.HG), unsigned(p.B));
    cfg.blockDim = dim3(dd::NT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = p.pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, dd::decode_direct_kernel<NH>, p);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: %s", cudaGetErrorString(e));
    return TQ_OK;
}

int launch_decode_direct(const DecodeParams& p, cudaStream_t s) {
    return p.slots <= 4 ? launch_nh<4>(p, s) : launch_nh<8>(p, s);
}

int launch_gather_wait(const unsigned long long* arrivals, unsigned long long* consumed, unsigned long long count, int max_polls, cudaStream_t s) {
    dd::gather_wait_kernel<<<1, 32, 0, s>>>(arrivals, consumed, count, max_polls);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_gather_wait: %s", cudaGetErrorString(e));
    return TQ_OK;
}

int decode_status_clear() {
    const int zero = 0;
    return cudaMemcpyToSymbol(dd::g_status, &zero, sizeof(int)) == cudaSuccess ? 0 : -1;
}

int decode_status_host() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, dd::g_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

}  // namespace tq

#ifdef TQ_TIMING
extern "C" int tq_debug_timing(unsigned long long* host_out, int n) {
    return int(cudaMemcpyFromSymbol(host_out, tq::dd::g_timing, sizeof(unsigned long long) * n));
}
#endif
