// Decode attention over a cache with 4-bit keys and 2-bit values at d = 128: the specialised kernel.
//
// Same decomposition as the general kernel of decode.cu (grid (splits, kv_heads * head_groups, batch); warps own
// 16-token tiles; S = K.Q^T, online softmax, O^T += V^T.P^T with mma.sync.m16n8k16; last-arrival merge), with the
// following differences, all aimed at the instruction count per tile and at the fixed cost per CTA:
//
//   * Raw packed tiles (1024 B of keys, 512 B of values, 2 x 64 B of norms) go from global memory straight into
//     registers, one tile ahead of the tile being computed; a warp owns a contiguous run of tiles and asks for them
//     in L2 several tiles earlier (prefetch.global.L2, one instruction per tile).  Nothing is staged through shared
//     memory: the shared-memory pipe is what bounds this kernel (64 wavefronts of table lookups per tile), and a
//     ring of bulk copies cost another 28 (12 to write a tile, 16 to read it back) plus their bank conflicts.
//   * Operand fragments come straight from lookup tables: byte of two 4-bit codes -> half2 of two key centroids;
//     byte of the 2-bit codes of a token pair -> two half2 value fragments.  The tables sit at shared-window
//     address 0x10000 with one 256-byte slot per byte value (32 conflict-free copies of the key entry, 16 of the
//     value entry), so the address of an entry is ONE byte-permute of (packed word, per-lane constant).
//   * Everything that depends only on the rotation matrix and the codebooks is built once per (rotation, codebooks)
//     by tq_decode_tables_build into a buffer in global memory (DirectTables): the 64 KB image of the lookup tables,
//     which a CTA fetches with one bulk copy, and R split into two fp16 matrices, R = R_hi + 2^-11 R_lo (both
//     products with an fp16 query are exact in the fp32 accumulators), laid out in mma A-fragment order so that
//     the eight rotating warps load their fragments straight into registers.
//   * All of that is requested BEFORE the kernel waits for its predecessor on the stream, and so is the warp's whole
//     run of packed tiles in L2 (L2 is the point of coherence, so a prefetch is harmless even while the cache is
//     still being written); after the wait only the query round trip and 16-24 MMAs stand between a CTA and its
//     tile loop, whose loads then hit L2.
//   * Partials stay in rotated space; the CTA that merges a (sequence, KV head) undoes the rotation once, in fp32,
//     reading R from global memory while the partials are in flight.
//
// The one mbarrier wait (arrival of the table image) is bounded; if it runs out the kernel records a status code
// (tq_device_status) and finishes with whatever it has.
#include <atomic>

#include "decode_dev.cuh"

// Development builds name a header that defines DD_STAMP(slot) (globaltimer stamps per CTA); product builds compile
// the hooks away.
#ifdef TQ_STAMP_HEADER
#include TQ_STAMP_HEADER
#else
#define DD_STAMP(slot)
#endif

namespace tq {

namespace dd {

constexpr int D = 128, NW = DIRECT_WARPS, NT = NW * 32;
constexpr uint32_t KT = TILE * (D / 2), VT = TILE * (D / 4);                                // bytes of a packed tile: 1024 + 512
constexpr int PF_AHEAD = 12;                                   // a tile is asked for in L2 this many tiles before it is loaded into registers

// Absolute shared-window addresses.  The dynamic allocation starts at `sbase` <= LO_BASE (reserved system bytes come
// first); the tables must start on a 64 KB boundary.
constexpr uint32_t HI_BYTES = 72u * 1024u;                     // above the tables: reduction scratch
constexpr uint32_t LUT_BAR = C_BASE + HI_BYTES;                // arrival of the table image
constexpr uint32_t QS = LUT_BAR + 64;                          // [8][D] half: scaled fp16 query (rotated or raw)
constexpr uint32_t MISC = QS + HPG * D * 2;                    // a few scalars
constexpr uint32_t SMEM_END = MISC + 64;
constexpr uint32_t MAX_SBASE = LO_BASE;
static_assert(SMEM_END <= 227u * 1024u, "shared-memory plan");
// phases after the main loop reuse the upper regions (CTA reduction, partial products) and the tables (merge)
constexpr int DS = D + 8, RWF = HPG * DS + 2 * HPG;            // floats per warp in the reduction buffer (2 DS = 16 mod 32: heads 2t, 2t+2 on different banks)
constexpr uint32_t RED = C_BASE;
static_assert(uint32_t(NW) * RWF * 4 <= HI_BYTES, "reduction scratch must fit above the tables");
constexpr uint32_t M_ACC = LUT_BASE;                           // float [8][D]: merged packed part, rotated space
constexpr uint32_t M_AD = M_ACC + HPG * D * 4;                 // float [8][D]: merged part of the uncompressed tokens
constexpr uint32_t M_IL = M_AD + HPG * D * 4;                  // float [8]: 1 / softmax denominator
constexpr uint32_t M_ML = M_IL + 64;                           // float2 [NW][32]: (max, sum) pairs, one staging row per warp
static_assert(M_ML + NW * 32 * 8 <= C_BASE, "merge scratch must fit in the table region");
constexpr uint32_t M_PP = C_BASE;                              // float [NW][8][D]: partial products with 8 rows of R each
static_assert(uint32_t(NW) * HPG * D * 4 <= HI_BYTES, "partial products must fit above the tables");
// CTAs that own uncompressed tokens use no tables: their warps stage fp16 tiles from LO_BASE on
constexpr uint32_t DSTAGE = 2u * TILE * stage_ld<D>() * 2u;    // keys + values of one tile
static_assert(LO_BASE + uint32_t(NW) * DSTAGE <= LUT_BAR, "dense staging must end before the barrier");

constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_TABLES = 102, ERR_LAYOUT = 103, ERR_GATHER_WAIT = 201;

constexpr int ROT_WARPS = D / 16;                              // warps that rotate the query: one 16-row slab of R each
static_assert(sizeof(DirectTables::rfrag) == sizeof(uint4) * ROT_WARPS * (D / 16) * 2 * 32, "rotation fragments");

__device__ int g_status = 0;
__device__ unsigned g_probe_base = 0;

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
// Streaming loads of the packed cache: read once, kept out of L1.
__device__ __forceinline__ uint4 ldg_stream128(const void* ptr) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream32(const void* ptr) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
    return v;
}
__device__ __forceinline__ void prefetch_l2(const void* ptr) { asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr)); }
__device__ __forceinline__ uint32_t h2_bits(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void smem_base_probe() {
    extern __shared__ __align__(16) unsigned char smem[];
    if (threadIdx.x == 0) g_probe_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
}

// One block builds the constants.  Table slot e at e * 256: +0 32 copies of half2(kc[e & 15], kc[e >> 4]); +128 16
// copies of the value entry (two half2: one per coordinate, each pairing the two tokens of a pair); copies r with
// (r & 2) serve lanes that read the token pair in swapped order.
__global__ void __launch_bounds__(1024) build_tables_kernel(const float* rot, const float* kc, const float* vc, float v_scale, int d, DirectTables* t) {
    __shared__ __half ctab[32];
    const int tid = threadIdx.x, nt = blockDim.x;
    if (tid < 32) {
        const int which = tid >> 4, k = tid & 15;
        float c = 0.f;
        if (k < (which ? 4 : 16)) c = (which ? vc : kc)[k];
        ctab[tid] = __float2half_rn(c * (which ? v_scale : 1.f));
    }
    if (tid == 0) { t->magic = TABLES_MAGIC; t->d = d; t->kb = 4; t->vb = 2; t->v_scale = v_scale; }
    __syncthreads();
    for (int idx = tid; idx < 256 * 16; idx += nt) {
        const int e = idx >> 4, q = idx & 15;
        uint4 v;
        if (q < 8) {
            const uint32_t u = h2_bits(__half2float(ctab[e & 15]), __half2float(ctab[e >> 4]));
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
        t->lut[idx] = v;
    }
    // A fragments (m16n8k16, row-major A) of the 16 x 16 blocks of R: a0 = (row g, cols 2t, 2t+1), a1 = (row g+8, same
    // cols), a2 = (row g, cols 2t+8, 2t+9), a3 = (row g+8, cols 2t+8, 2t+9); warp w owns rows 16 w .. 16 w + 15
    for (int idx = tid; d == D && idx < ROT_WARPS * (D / 16) * 32; idx += nt) {       // (other head dims: the streaming kernel's queries are rotated by a launch of their own)
        const int w = idx / ((D / 16) * 32), ks = (idx / 32) % (D / 16), lane = idx & 31, g = lane >> 2, tt = lane & 3;
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = w * 16 + g + (r & 1) * 8, col = ks * 16 + 2 * tt + (r >> 1) * 8;
            const float x0 = rot[row * D + col], x1 = rot[row * D + col + 1];
            const __half2 h = __floats2half2_rn(x0, x1);
            const float2 hf = __half22float2(h);
            hi[r] = *reinterpret_cast<const uint32_t*>(&h);
            lo[r] = h2_bits((x0 - hf.x) * 2048.f, (x1 - hf.y) * 2048.f);
        }
        t->rfrag[((w * (D / 16) + ks) * 2 + 0) * 32 + lane] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        t->rfrag[((w * (D / 16) + ks) * 2 + 1) * 32 + lane] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
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
    const float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]), vmax = fmaxf(vn0, vn1);
    if (__any_sync(0xffffffffu, mx0 > st.mt[0] || mx1 > st.mt[1] || vmax > st.vt)) softmax_refresh<D, 0>(mx0, mx1, vmax, st);
    const float p0 = ex2(s[0] - st.m[0]), p1 = ex2(s[1] - st.m[1]), p2 = ex2(s[2] - st.m[0]), p3 = ex2(s[3] - st.m[1]);
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    const float w0 = vn0 * st.vsc, w1 = vn1 * st.vsc;
    bp[0] = movm_t(pack_h2(p0 * w0, p1 * w0));
    bp[1] = movm_t(pack_h2(p2 * w1, p3 * w1));
}

// The registers one 16-token tile arrives in.
struct RawTile {
    uint4 q0, q1;              // token g, token g + 8: this thread's quarter of the 4-bit key row
    uint32_t va, vb, vc, vd;   // value words: rows 2t + sw, 2t + 1 - sw, and the same + 8
    float kn0, kn1, vn0, vn1;  // norms of tokens g, g + 8
};

// NH: query heads per group the rotations are compiled for (4 or 8); heads_here <= NH.
template <int NH>
__global__ void __launch_bounds__(NT, 1) decode_direct_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    auto gp = [&](uint32_t abs_addr) -> unsigned char* { return smem + (abs_addr - sbase); };   // generic pointer of a window address
    __half* qs = reinterpret_cast<__half*>(gp(QS));
    float* s_misc = reinterpret_cast<float*>(gp(MISC));
    const DirectTables* tb = static_cast<const DirectTables*>(p.tables);

    DD_STAMP(0);
    pdl_trigger();     // the next launch on the stream may become resident and run its own prologue
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;        // lane of the cache arrays
    const bool dense = split >= p.n_ps;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int64_t qbase = (int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG) * D;   // first query head of this group
    const int S = p.n_ps + p.n_ds;
    if (sbase > MAX_SBASE || (sbase & 15u)) {            // cannot happen after the host-side probe; never run on a bad plan
        if (tid == 0) atomicCAS(&g_status, 0, ERR_LAYOUT);
        return;
    }

    // ---------------- prologue on constants only (runs before the previous launch has finished) -----------
    uint4 rf[D / 16][2];                                 // this warp's A fragments of R_hi / R_lo, in flight across the wait
    bool failed = false;
    if (!dense) {
        if (tid == 0) {
            mbar_init(LUT_BAR, 1);
            fence_barrier_init();
            mbar_expect_tx(LUT_BAR, uint32_t(sizeof(tb->lut)));
            bulk_g2s(LUT_BASE, tb->lut, uint32_t(sizeof(tb->lut)), LUT_BAR);
        }
        if (warp < ROT_WARPS) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                rf[ks][0] = __ldg(tb->rfrag + ((warp * (D / 16) + ks) * 2 + 0) * 32 + lane);
                rf[ks][1] = __ldg(tb->rfrag + ((warp * (D / 16) + ks) * 2 + 1) * 32 + lane);
            }
        }
    }
    const float tb_scale = dense ? 1.f : __ldg(&tb->v_scale);
    const uint32_t tb_magic = dense ? TABLES_MAGIC : __ldg(&tb->magic);   // (used after the wait: no round trip here)

    // ---------------- this warp's run of packed tiles ----------------------------------------------------
    // warp w owns a contiguous run of the CTA's tiles: n_my tiles from tile `first`
    const int n_tiles = int((p.c_len + TILE - 1) / TILE);
    const int tile_lo = int(split * p.p_tps);
    const int tile_hi = dense ? 0 : min(tile_lo + int(p.p_tps), n_tiles);
#ifndef DD_ACTIVE_WARPS
#define DD_ACTIVE_WARPS NW
#endif
    constexpr int AW = DD_ACTIVE_WARPS;                  // (experiments: fewer warps share the CTA's tiles)
    const int n_cta = max(tile_hi - tile_lo, 0), t_base = n_cta / AW, t_extra = n_cta - t_base * AW;
    const int n_my = warp < AW ? t_base + (warp < t_extra ? 1 : 0) : 0;
    const int first = tile_lo + warp * t_base + min(warp, t_extra);
    const int64_t row0 = kvl * p.c_ls + int64_t(first) * TILE;
    const uint8_t* const k_run = p.k_hi + row0 * (D / 2);
    const uint8_t* const v_run = p.v_hi + row0 * (D / 4);
    const float* const kn_run = p.k_norms + row0;
    const float* const vn_run = p.v_norms + row0;
    // L2 prefetch, one instruction per tile: lanes 0-7 take the eight 128-byte lines of the key tile, lanes 8-11 the
    // four of the value tile, lanes 12 / 13 the line that holds the tile's key / value norms
    const uint8_t* pf_ptr = lane < 8 ? k_run + lane * 128
                          : lane < 12 ? v_run + (lane - 8) * 128
                          : reinterpret_cast<const uint8_t*>(lane == 12 ? kn_run : vn_run);
    const uint32_t pf_stride = lane < 8 ? KT : lane < 12 ? VT : TILE * 4;
    auto prefetch_tile = [&](int i) {
        if (lane < 14) prefetch_l2(pf_ptr + uint32_t(i) * pf_stride);
    };
    if (!dense) {
#pragma unroll 4
        for (int i = 0; i < min(n_my, PF_AHEAD); ++i) prefetch_tile(i);
    }
    DD_STAMP(1);
    pdl_wait();        // from here on: the query, the cache and the workspace of the previous launch are settled
    DD_STAMP(11);
    await_gather(p);   // (head-sharded decoding) ... and the peers' heads of an earlier call have arrived
    DD_STAMP(2);
    const float inv_vs = 1.f / tb_scale;
    if (tb_magic != TABLES_MAGIC) {                      // not a buffer tq_decode_tables_build filled
        if (tid == 0) atomicCAS(&g_status, 0, ERR_TABLES);
        failed = true;
    }

    // the first tile's registers: requested before the query round trip below
    // value rows of a token pair are read in swapped order by the lanes with t >= 2; their table copies pair the
    // centroids the other way round
    const int sw = t >> 1;
    const uint8_t* const kq_ptr = k_run + lane * 16;
    const uint8_t* const va_ptr = v_run + (2 * t + sw) * (D / 4) + g * 4;
    const uint8_t* const vb_ptr = v_run + (2 * t + 1 - sw) * (D / 4) + g * 4;
    auto load_tile = [&](RawTile& r, int i) {
        const uint8_t* kq = kq_ptr + uint32_t(i) * KT;
        r.q0 = ldg_stream128(kq);
        r.q1 = ldg_stream128(kq + KT / 2);
        r.va = ldg_stream32(va_ptr + uint32_t(i) * VT);
        r.vb = ldg_stream32(vb_ptr + uint32_t(i) * VT);
        r.vc = ldg_stream32(va_ptr + uint32_t(i) * VT + 8 * (D / 4));
        r.vd = ldg_stream32(vb_ptr + uint32_t(i) * VT + 8 * (D / 4));
        r.kn0 = __uint_as_float(ldg_stream32(kn_run + i * TILE + g));
        r.kn1 = __uint_as_float(ldg_stream32(kn_run + i * TILE + g + 8));
        r.vn0 = __uint_as_float(ldg_stream32(vn_run + i * TILE + g));
        r.vn1 = __uint_as_float(ldg_stream32(vn_run + i * TILE + g + 8));
    };
    RawTile ra, rb;
    if (!dense && !failed && n_my > 0) load_tile(ra, 0);

    // ---------------- the query heads of this group: (rotated) scaled fp16 ------------------------------------
    const float f = p.scale * LOG2E;
    if (dense) {
        for (int e = tid; e < heads_here * D; e += NT) qs[e] = __float2half_rn(load_as_f32(p.q, p.q_dtype, qbase + e) * f);
    } else if (warp < ROT_WARPS) {
        // q_rot[h][j] = sum_k q[h][k] R[j][k]  (rotation.py:81-110) on the tensor cores: warp w owns rows 16w..16w+15 of R
        // (A operand, fragments from the table buffer), the query heads are the B operand.  A query that is not fp16 is
        // split like R (q = q_hi + 2^-11 q_lo); the product R_lo q_lo is below fp32 resolution.
        const bool q16 = p.q_dtype == TQ_F16;
        uint32_t bh[D / 16][2], bl[D / 16][2];
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
        float ym[4] = {0.f, 0.f, 0.f, 0.f}, yc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            mma16816(ym, rf[ks][0].x, rf[ks][0].y, rf[ks][0].z, rf[ks][0].w, bh[ks][0], bh[ks][1]);
            mma16816(yc, rf[ks][1].x, rf[ks][1].y, rf[ks][1].z, rf[ks][1].w, bh[ks][0], bh[ks][1]);
            if (!q16) mma16816(yc, rf[ks][0].x, rf[ks][0].y, rf[ks][0].z, rf[ks][0].w, bl[ks][0], bl[ks][1]);
        }
        // accumulator layout: rows g, g+8 of the slab x heads 2t, 2t+1
        const int j = warp * 16 + g;
        qs[(2 * t) * D + j] = __float2half_rn((ym[0] + yc[0] * (1.f / 2048.f)) * f);
        qs[(2 * t + 1) * D + j] = __float2half_rn((ym[1] + yc[1] * (1.f / 2048.f)) * f);
        qs[(2 * t) * D + j + 8] = __float2half_rn((ym[2] + yc[2] * (1.f / 2048.f)) * f);
        qs[(2 * t + 1) * D + j + 8] = __float2half_rn((ym[3] + yc[3] * (1.f / 2048.f)) * f);
    }
    __syncthreads();       // (rotated) query visible
    DD_STAMP(3);

    WarpAcc<D> st;
    st.init();

    if (dense) {
        // ---------------- uncompressed tokens: sink then residual window, raw query ----------------
        uint32_t bq[D / 16][2];
        const __half* qh = qs + g * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
            bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
        }
        __half* Ks = reinterpret_cast<__half*>(gp(LO_BASE + uint32_t(warp) * DSTAGE));
        __half* Vs = Ks + TILE * stage_ld<D>();
        const int64_t d_lo = int64_t(split - p.n_ps) * p.d_tps;
        dense_tiles<D, NW, 0>(p, kvl, d_lo, d_lo + p.d_tps, Ks, Vs, bq, st, warp, lane);
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
        if (!failed && !mbar_wait(LUT_BAR, 0)) {         // the table image has landed (requested before the wait above)
            atomicCAS(&g_status, 0, ERR_TABLES);
            failed = true;
        }
        failed = __any_sync(0xffffffffu, failed);
        // table addresses by byte-permute: {copy offset, byte value, 0x01, 0x00} = LUT_BASE + value * 256 + copy offset
        const uint32_t c4 = LUT_BASE | uint32_t(lane * 4);
        const uint32_t c2 = LUT_BASE | 128u | uint32_t((lane & 15) * 8);
        const int c_len = int(p.c_len);
        const int tail_tile = (c_len & (TILE - 1)) ? n_tiles - 1 - first : -1;   // local index of the tile that is only partly inside the cache
        auto compute = [&](const RawTile& r, int i) {
            // two independent accumulators (even / odd k-steps) halve the dependent MMA chain
            float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                // bytes 2ks, 2ks+1 of the quarter row
                const int wi = ks >> 1;
                const uint32_t w0 = wi == 0 ? r.q0.x : wi == 1 ? r.q0.y : wi == 2 ? r.q0.z : r.q0.w;
                const uint32_t w1 = wi == 0 ? r.q1.x : wi == 1 ? r.q1.y : wi == 2 ? r.q1.z : r.q1.w;
                const int b0 = (ks & 1) * 2;
                const uint32_t a0 = lut32(__byte_perm(w0, c4, 0x7604 | (b0 << 4)));
                const uint32_t a1 = lut32(__byte_perm(w1, c4, 0x7604 | (b0 << 4)));
                const uint32_t a2 = lut32(__byte_perm(w0, c4, 0x7604 | ((b0 + 1) << 4)));
                const uint32_t a3 = lut32(__byte_perm(w1, c4, 0x7604 | ((b0 + 1) << 4)));
                if (ks & 1) mma16816(s2, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
                else mma16816(s, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) s[u] += s2[u];
            uint32_t bp[2];
            const int tok0 = (first + i) * TILE;
            softmax_direct(s, r.kn0, r.kn1, r.vn0, r.vn1, i == tail_tile, tok0 + g < c_len, tok0 + g + 8 < c_len, st, bp);
            // pair the nibbles (two adjacent coordinates) of the two tokens: byte j of Z0 = (first word, nibble 2j) |
            // (second word, nibble 2j) << 4, Z1 the odd nibbles.  One 64-bit lookup then yields the two operand registers
            // that sit next to each other in the MMA (rows g and g+8 = the two coordinates, token pair in each).
            const uint32_t z0 = (r.va & 0x0F0F0F0Fu) | ((r.vb << 4) & 0xF0F0F0F0u), z1 = ((r.va >> 4) & 0x0F0F0F0Fu) | (r.vb & 0xF0F0F0F0u);
            const uint32_t w0 = (r.vc & 0x0F0F0F0Fu) | ((r.vd << 4) & 0xF0F0F0F0u), w1 = ((r.vc >> 4) & 0x0F0F0F0Fu) | (r.vd & 0xF0F0F0F0u);
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
        // One tile in registers ahead of the tile being computed, PF_AHEAD further tiles on their way into L2; two tiles
        // per trip so that the register sets swap roles without copies.  Loads past the run's end are not issued.
        if (!failed) {
            for (int i = 0; i < n_my; i += 2) {
                if (i + 1 < n_my) load_tile(rb, i + 1);
                if (i + PF_AHEAD < n_my) prefetch_tile(i + PF_AHEAD);
                compute(ra, i);
                if (i + 1 < n_my) {
                    if (i + 2 < n_my) load_tile(ra, i + 2);
                    if (i + 1 + PF_AHEAD < n_my) prefetch_tile(i + 1 + PF_AHEAD);
                    compute(rb, i + 1);
                }
            }
        }
    }

    st.finish();       // accumulators back to true scale (the value scale is per warp)
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
    float* red = reinterpret_cast<float*>(gp(RED));
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
            // fused gather: staged in the result's element type (the rotated sums are no longer needed), sent below
            if (p.n_peers > 0) store_from_f32(s_acc, p.out_dtype, e, v * s_il[h]);
            else store_from_f32(p.out, p.out_dtype, qbase + e, v * s_il[h]);
        }
    }
    if (p.n_peers > 0) {
        const int grp = int((int64_t(blockIdx.z) * p.Hkv + blockIdx.y / p.HG) * p.HG + blockIdx.y % p.HG);
        const unsigned epoch = next_epoch(p, grp);
        __syncthreads();
        // the group's first head in the peers' (batch, heads_total, d) buffers
        const int64_t gbase = (int64_t(blockIdx.z) * p.heads_total + p.head_offset + int64_t(blockIdx.y / p.HG) * p.G + (blockIdx.y % p.HG) * HPG) * D;
        const int es = out_elem_bytes(p.out_dtype);
        DD_STAMP(9);
        publish_result(p, s_acc, heads_here * D * es, gbase * es, grp, epoch);
    }
    DD_STAMP(6);
}

// Consumer side of the fused gather as a launch of its own (for consumers that are not one of this library's kernels):
// returns once every word of this GPU's landing buffer carries the epoch of the latest call this GPU made into the slot
// (the producing launch is earlier on the stream, so the count is final) and writes the plain result.  The poll is bounded
// (about two seconds), then a status is left.
__global__ void __launch_bounds__(256) gather_wait_kernel(const unsigned long long* ll, const unsigned* epochs, int64_t n_words, uint32_t* out, int max_polls) {
    const unsigned epoch = *reinterpret_cast<const volatile unsigned*>(epochs);
    if (!collect_words(ll, int64_t(blockIdx.x) * blockDim.x + threadIdx.x, n_words, int64_t(gridDim.x) * blockDim.x, epoch, out, max_polls))
        atomicCAS(&g_status, 0, ERR_GATHER_WAIT);
}

unsigned probe_smem_base() {
    // The kernel addresses its tables by absolute shared-window address; where the dynamic allocation starts is a
    // property of the device / driver, read once per device with a one-thread launch (tq_decode_tables_build does it
    // at set-up; a decode call only if no tables were ever built on the device).
    static std::atomic<unsigned> cache[64];
    static std::atomic<bool> have[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return ~0u;
    if (!have[dev].load(std::memory_order_acquire)) {
        unsigned v = ~0u;
        smem_base_probe<<<1, 32, 1024>>>();
        if (cudaGetLastError() != cudaSuccess || cudaMemcpyFromSymbol(&v, g_probe_base, sizeof(v)) != cudaSuccess) return ~0u;
        cache[dev].store(v, std::memory_order_relaxed);
        have[dev].store(true, std::memory_order_release);
    }
    return cache[dev].load(std::memory_order_relaxed);
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

size_t direct_tables_bytes() { return sizeof(dd::DirectTables); }

int direct_tables_build(int d, const float* rot, const float* k_cent, const float* v_cent, float v_scale, void* tables, cudaStream_t s) {
    dd::build_tables_kernel<<<1, 1024, 0, s>>>(rot, k_cent, v_cent, v_scale > 0.f ? v_scale : 1.f, d, static_cast<dd::DirectTables*>(tables));
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_tables_build: %s", cudaGetErrorString(e));
    direct_supported();      // measures the shared-memory base of this device now, outside any capture
    return TQ_OK;
}

template <int NH> static int launch_nh(const DecodeParams& p, cudaStream_t s) {
    const unsigned sb = dd::probe_smem_base();
    const size_t smem = dd::SMEM_END - sb;
    static std::atomic<bool> set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(dd::decode_direct_kernel<NH>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev].store(true, std::memory_order_release);
    }
    // Programmatic stream serialisation: the grid may become resident before its predecessor on the stream
    // has finished; the kernel calls griddepcontrol.wait before it touches anything but constants (and, when the
    // caller vouches for them, the packed arrays).
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

int* decode_status_ptr() {
    static std::atomic<int*> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* v = cache[dev].load(std::memory_order_acquire);
    if (!v) {
        void* a = nullptr;
        if (cudaGetSymbolAddress(&a, dd::g_status) != cudaSuccess) return nullptr;
        v = static_cast<int*>(a);
        cache[dev].store(v, std::memory_order_release);
    }
    return v;
}

int launch_gather_wait(const unsigned long long* ll, const unsigned* epochs, int64_t n_words, void* out, int max_polls, cudaStream_t s) {
    const int64_t blocks = std::min<int64_t>((n_words + 255) / 256, 64);
    dd::gather_wait_kernel<<<unsigned(blocks), 256, 0, s>>>(ll, epochs, n_words, static_cast<uint32_t*>(out), max_polls);
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
