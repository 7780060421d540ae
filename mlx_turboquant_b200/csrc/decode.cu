// One decode step of attention computed directly on the compressed KV cache
// [fp16 sink | packed middle | fp16 residual window], split over the sequence (flash-decode), in ONE launch.
//
// decode_attn_kernel, grid (splits, kv_heads * head_groups, batch).  Every CTA
//   1. rotates the query heads of its GQA group once (q @ R^T, float32), folds scale*log2(e) in and keeps
//      fp16 copies in shared memory (CTAs that own uncompressed tokens keep the unrotated query instead);
//   2. runs the online-softmax attention over its token range of either the packed middle or the
//      uncompressed regions; values of the packed middle are accumulated in ROTATED space;
//   3. reduces its warps and writes one (max, sum, weighted-V) partial per query head to the workspace;
//   4. bumps a counter; the CTA that arrives last for a (sequence, KV head, head group) merges all partials
//      (log-sum-exp), undoes the rotation once (@ R), adds the unrotated part, normalises and writes the
//      output.  No CTA ever waits for another one: the last arrival is detected with one atomic add.
//
// Arithmetic: warps work on tiles of 16 tokens with mma.sync.m16n8k16 (fp16 operands, fp32 accumulation):
// S[16 tokens x 8 heads] = K_tile . Q^T, online softmax in registers, P transposed with movmatrix,
// O^T[d x 8 heads] += V_tile^T . P^T.  Tokens are the M dimension so a GQA group of up to 8 query heads
// shares every unpacked key/value.  The kernel is bound by HBM bytes (packed codes + norms), not by the
// tensor pipe; the contraction shape is tiny (N = 8), which is why the warp-level MMA is used here.
//
// Two ways to build the K / V^T operand fragments:
//   * general: a warp unpacks (or, for the fp16 regions, copies) its tile into shared memory as fp16 and reads
//     fragments back with ldmatrix - any bit width, fractional splits, d in {64, 96, 128, 256};
//   * direct (4-bit keys, 2-bit values, d = 128): raw packed tiles stream through a per-warp cp.async ring and
//     are turned into fragments through bank-conflict-free lookup tables in shared memory (byte -> half2),
//     never touching shared memory with unpacked data.  The coordinate order inside a fragment is permuted to
//     match the byte layout; the query fragments and the output mapping use the same permutation.
#include <algorithm>
#include <string_view>

#include "decode.cuh"

namespace tq {

// ---- small PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// Lookups in tables that are constant for the lifetime of the CTA: plain (non-volatile) asm so the compiler
// may hoist and batch them ahead of the MMAs that consume them.
__device__ __forceinline__ uint32_t lut32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lut64(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
// Reads of the cp.async ring: ordered after the wait / warp barrier that makes the data visible.
__device__ __forceinline__ uint32_t ring32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ring128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
// 16-byte asynchronous global -> shared copy; bytes past src_bytes are zero-filled (0 = read nothing).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Programmatic dependent launch: wait for the previous grid on the stream / let the next grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

#ifdef TQ_TIMING
// Phase timestamps (development builds only): [cta][8] globaltimer values.
__device__ unsigned long long g_tq_timing[4096 * 16];
__device__ __forceinline__ void stamp(int cta, int slot) {
    if (threadIdx.x == 0 && cta < 4096) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_tq_timing[cta * 16 + slot] = t;
    }
}
#define TQ_STAMP(slot) stamp(int(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z)), slot)
#else
#define TQ_STAMP(slot)
#endif

// ---- per-warp running softmax state ------------------------------------------------------------------
constexpr float MAX_SLACK = 6.f;   // scores may exceed the running reference by 2^6 before it is refreshed
template <int D> struct WarpAcc {
    float m[2], mt[2], l[2];   // heads 2t, 2t+1: reference max, refresh threshold, this lane's share of the sum
    float o[D / 16][4];        // O^T fragments: rows = coordinate slots, cols = heads
};

// s[0..1]: token g, heads 2t,2t+1;  s[2..3]: token g+8.  Returns the P^T operand for the PV mma.
// The softmax reference m is refreshed (with a cross-lane max and a rescale of the accumulators) only
// when some score exceeds it by more than MAX_SLACK; softmax is shift-invariant, so any reference that
// keeps exp2(s - m) inside the fp16 range is exact.
template <int D>
__device__ __forceinline__ void softmax_step(float (&s)[4], float kn0, float kn1, float vn0, float vn1, bool ok0,
                                             bool ok1, WarpAcc<D>& st, uint32_t (&bp)[2]) {
    s[0] = ok0 ? s[0] * kn0 : -INFINITY;
    s[1] = ok0 ? s[1] * kn0 : -INFINITY;
    s[2] = ok1 ? s[2] * kn1 : -INFINITY;
    s[3] = ok1 ? s[3] * kn1 : -INFINITY;
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
    // value norms ride on P (fp16, clamped below the fp16 maximum)
    const uint32_t h0 = pack_h2(fminf(p0 * vn0, 65504.f), fminf(p1 * vn0, 65504.f));
    const uint32_t h1 = pack_h2(fminf(p2 * vn1, 65504.f), fminf(p3 * vn1, 65504.f));
    bp[0] = movm_t(h0);   // tokens 2t,2t+1   x head g
    bp[1] = movm_t(h1);   // tokens 2t+8,2t+9 x head g
}

// ---- shared memory plan ----------------------------------------------------------------------------------
// BODY is reused by phases that never overlap in time:
//   general staging: per warp  Ks[16][D+8] + Vs[16][D+8] halves
//   direct:          T4 [256][32] u32 (32 KB) + T2 [256][16] uint2 (32 KB) + per-warp cp.async ring + R (64 KB)
//   CTA reduction:   per warp  o[D][8] floats + m[8] + l[8], then weights [NW][8]
//   merge (last CTA): split weights [8][MAX_SPLITS], rotated / raw sums [8][D] each, partial products
// After BODY: float query [8][D], fp16 query [8][D], four 16-entry fp16 centroid tables, a few scalars.
constexpr int MERGE_CPARTS = 4;       // thread slabs of the d x d product with R in the epilogue
template <int D> __host__ __device__ constexpr int stage_ld() { return D + 8; }
template <int D, int NW> __host__ __device__ constexpr size_t stage_bytes() { return size_t(NW) * 2 * TILE * stage_ld<D>() * sizeof(__half); }
template <int D, int NW> __host__ __device__ constexpr size_t reduce_bytes() {
    return size_t(NW) * (HPG * (D + 2) + 2 * HPG) * sizeof(float) + size_t(NW) * HPG * sizeof(float) + size_t(HPG) * D * sizeof(float) +
           size_t(MERGE_CPARTS) * HPG * D * sizeof(float);
}
constexpr size_t TABLE_BYTES = 65536;
constexpr int RING_STAGES = 3;
template <int D> __host__ __device__ constexpr int ring_stage_bytes() { return TILE * (D / 2 + D / 4 + 8); }
// direct path: the rotation matrix stays resident in shared memory behind the tables and the ring
template <int D, int NW> __host__ __device__ constexpr size_t rot_offset() { return TABLE_BYTES + size_t(NW) * RING_STAGES * ring_stage_bytes<D>(); }
// chunk (16 bytes) kc of row j of the resident matrix sits at chunk position rot_pos(j, kc) of that row: both a
// thread quartet reading along a row and a warp reading down a column hit distinct bank groups
__host__ __device__ constexpr int rot_pos(int j, int kc) { return (kc & ~7) | ((kc ^ j ^ ((kc >> 3) << 1)) & 7); }
template <int D> __host__ __device__ constexpr size_t merge_bytes() { return size_t(HPG) * MAX_SPLITS * sizeof(float2); }
template <int D, bool DIRECT> __host__ __device__ constexpr size_t body_bytes() {
    constexpr int NW = warps_per_cta(DIRECT);
    size_t s = stage_bytes<D, NW>();
    if (reduce_bytes<D, NW>() > s) s = reduce_bytes<D, NW>();
    if (merge_bytes<D>() > s) s = merge_bytes<D>();
    if (DIRECT && rot_offset<D, NW>() + size_t(D) * D * sizeof(float) > s) s = rot_offset<D, NW>() + size_t(D) * D * sizeof(float);
    return (s + 15) / 16 * 16;
}
template <int D> __host__ __device__ constexpr size_t tail_bytes() {
    return size_t(HPG) * D * sizeof(float) + size_t(HPG) * D * sizeof(__half) + 64 * sizeof(__half) + 16 * sizeof(float);
}
template <int D, bool DIRECT> __host__ __device__ constexpr size_t kernel_smem() { return body_bytes<D, DIRECT>() + tail_bytes<D>(); }

// One 16-token tile whose K and V sit in shared memory as fp16 [token][coordinate].
template <int D>
__device__ __forceinline__ void tile_from_smem(const __half* Ks, const __half* Vs, const uint32_t (&bq)[D / 16][2],
                                               float kn0, float kn1, float vn0, float vn1, bool ok0, bool ok1,
                                               WarpAcc<D>& st, int lane) {
    constexpr int LD = stage_ld<D>();
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
        const __half* base = Ks + (lane & 15) * LD + (lane >> 4) * 8;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, base + ks * 16);
            mma16816(s, a[0], a[1], a[2], a[3], bq[ks][0], bq[ks][1]);
        }
    }
    uint32_t bp[2];
    softmax_step<D>(s, kn0, kn1, vn0, vn1, ok0, ok1, st, bp);
    {
        const __half* base = Vs + ((lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
            uint32_t a[4];
            ldsm_x4_t(a, base + mt * 16);
            mma16816(st.o[mt], a[0], a[1], a[2], a[3], bp[0], bp[1]);
        }
    }
}

// Per-warp cp.async ring of raw packed tiles (direct path, d = 128): one tile = 1024 B of 4-bit keys, 512 B of
// 2-bit values, 2 x 64 B of norms.  Tokens past c_len are zero-filled without touching memory.
template <int D, int NW> struct RingCtx {
    static constexpr int KW = D / 2, VW = D / 4, KT = TILE * KW, VT = TILE * VW, STG = ring_stage_bytes<D>();
    uint32_t ring, v_dst;
    int tile_hi, first, c_len;
    const uint8_t *kbase, *vbase;
    const float* nbase;
    // Value rows are stored permuted inside each group of four (row r -> slot (r + r/4) mod 4) so that the four
    // rows {2t+c} a warp reads together fall into distinct banks.
    __device__ __forceinline__ static int vslot(int r) { return (r & ~3) | ((r + (r >> 2)) & 3); }
    __device__ __forceinline__ void init(const DecodeParams& p, unsigned char* smem, int64_t kvl, int split, int warp, int lane) {
        ring = static_cast<uint32_t>(__cvta_generic_to_shared(smem)) + uint32_t(TABLE_BYTES) + warp * (RING_STAGES * STG);
        v_dst = KT + vslot(lane >> 1) * VW + (lane & 1) * 16;
        const int n_tiles = int((p.c_len + TILE - 1) / TILE);
        const int tile_lo = int(split * p.p_tps);
        tile_hi = min(tile_lo + int(p.p_tps), n_tiles);
        first = tile_lo + warp;
        c_len = int(p.c_len);
        kbase = p.k_hi + kvl * p.c_ls * KW + lane * 16;
        vbase = p.v_hi + kvl * p.c_ls * VW + lane * 16;
        nbase = (lane < 4 ? p.k_norms : p.v_norms) + kvl * p.c_ls + (lane & 3) * 4;
    }
    __device__ __forceinline__ void issue(int stage, int tile, int lane) const {
        const uint32_t sb = ring + stage * STG;
        const int tok0 = tile * TILE;
        const int left = c_len - tok0;            // valid tokens from here on (>= 16 for all but the last tile)
        const uint8_t* ks = kbase + int64_t(tok0) * KW;
        cp_async16(sb + lane * 16, ks, (lane >> 2) < left ? 16 : 0);
        cp_async16(sb + 512 + lane * 16, ks + 512, (lane >> 2) + 8 < left ? 16 : 0);
        cp_async16(sb + v_dst, vbase + int64_t(tok0) * VW, (lane >> 1) < left ? 16 : 0);
        if (lane < 8) {
            const int ok = left - (lane & 3) * 4;
            cp_async16(sb + KT + VT + lane * 16, nbase + tok0, ok >= 4 ? 16 : ok > 0 ? ok * 4 : 0);
        }
    }
};

template <int D, bool DIRECT>
__global__ void __launch_bounds__(warps_per_cta(DIRECT) * 32, 1) decode_attn_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NW = warps_per_cta(DIRECT), NT = NW * 32;
    constexpr int LD = stage_ld<D>();
    constexpr size_t BODY = body_bytes<D, DIRECT>();
    float* qf = reinterpret_cast<float*>(smem + BODY);                       // [8][D] query, float32
    __half* qs = reinterpret_cast<__half*>(qf + HPG * D);                    // [8][D] scaled fp16 query (rotated or raw)
    __half* ctab = qs + HPG * D;                                             // kc_hi, kc_lo, vc_hi, vc_lo (16 each)
    float* s_misc = reinterpret_cast<float*>(ctab + 64);                     // [0..7] 1/L per head, [8] last-CTA flag

    TQ_STAMP(0);
    pdl_trigger();     // the next launch on the stream may become resident and run its own prologue
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;        // lane of the cache arrays
    const bool dense = split >= p.n_ps;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int64_t qbase = (int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG) * D;   // first query head of this group
    const int S = p.n_ps + p.n_ds;

    // ---------------- prologue on constants only (runs before the previous launch has finished) -----------
    if constexpr (DIRECT) {
        if (!dense) {
            uint32_t* T4 = reinterpret_cast<uint32_t*>(smem);               // [256][32]: byte -> half2(c[lo], c[hi])
            uint2* T2 = reinterpret_cast<uint2*>(smem + 32768);             // [256][16]: byte -> 2 x half2 (token pair)
            if (tid < 32) {
                const int which = tid >> 4, k = tid & 15;
                const float* src = which ? p.vc_hi : p.kc_hi;
                ctab[which * 32 + k] = __float2half_rn(k < (which ? 4 : 16) ? src[k] * (which ? p.v_scale_hi : 1.f) : 0.f);
            }
            __syncthreads();
            for (int e = tid; e < 256 * 8; e += NT) {     // 4 replicas per 128-bit store
                const int entry = e >> 3, q4 = e & 7;
                const __half2 h = __halves2half2(ctab[entry & 15], ctab[entry >> 4]);
                const uint32_t v = *reinterpret_cast<const uint32_t*>(&h);
                reinterpret_cast<uint4*>(T4)[entry * 8 + q4] = make_uint4(v, v, v, v);
            }
            for (int e = tid; e < 256 * 8; e += NT) {     // 2 replicas per 128-bit store
                const int entry = e >> 3, q2 = e & 7;
                const int n0 = entry & 15, n1 = entry >> 4;
                const __half2 h0 = __halves2half2(ctab[32 + (n0 & 3)], ctab[32 + (n0 >> 2)]);
                const __half2 h1 = __halves2half2(ctab[32 + (n1 & 3)], ctab[32 + (n1 >> 2)]);
                const uint32_t v0 = *reinterpret_cast<const uint32_t*>(&h0), v1 = *reinterpret_cast<const uint32_t*>(&h1);
                reinterpret_cast<uint4*>(T2)[entry * 8 + q2] = make_uint4(v0, v1, v0, v1);
            }
        }
    } else {
        if (!dense && tid < 64) {
            const int which = tid >> 4, k = tid & 15;
            const float* src = which == 0 ? p.kc_hi : which == 1 ? p.kc_lo : which == 2 ? p.vc_hi : p.vc_lo;
            const int bits = which == 0 ? p.kb_hi : which == 1 ? p.kb_lo : which == 2 ? p.vb_hi : p.vb_lo;
            const float sc = which == 2 ? p.v_scale_hi : which == 3 ? p.v_scale_lo : 1.f;
            ctab[tid] = __float2half_rn((src != nullptr && bits > 0 && k < (1 << bits)) ? src[k] * sc : 0.f);
        }
    }
    TQ_STAMP(1);
    pdl_wait();        // from here on: the query, the cache and the workspace of the previous launch are settled

    TQ_STAMP(2);
    RingCtx<D, NW> rc;
    // ---------------- the query heads of this group: float32, then (rotated) scaled fp16 --------------------
    // q_rot[h][j] = sum_k q[h][k] R[j][k]  (rotation.py:81-110)
    {
        const float f = p.scale * LOG2E;
        if constexpr (DIRECT) {
            // R (64 KB) is read ONCE per CTA with fully coalesced 128-bit loads and stays resident in shared
            // memory (the epilogue needs it again); chunk placement rot_pos() keeps both uses conflict-free.
            float4* rs = reinterpret_cast<float4*>(smem + rot_offset<D, NW>());
            float4 rr[(D * D / 4) / NT];
            if (!dense) {
#pragma unroll
                for (int i = 0; i < (D * D / 4) / NT; ++i) rr[i] = __ldg(reinterpret_cast<const float4*>(p.rot) + tid + i * NT);
            }
            // 16-byte chunk kc of a query row is stored at chunk kc ^ (kc >> 3): the four threads of a row
            // quartet read chunks 8 apart, which would otherwise share a bank group
            for (int e = tid; e < heads_here * D; e += NT) {
                const int kc = (e % D) >> 2;
                qf[(e - (e % D)) + ((kc ^ (kc >> 3)) << 2) + (e & 3)] = load_as_f32(p.q, p.q_dtype, qbase + e);
            }
            if (!dense) {
                // start streaming the first packed tiles: they land while the query is being rotated
                rc.init(p, smem, kvl, split, warp, lane);
#pragma unroll
                for (int i = 0; i < RING_STAGES - 1; ++i) {
                    if (rc.first + i * NW < rc.tile_hi) rc.issue(i, rc.first + i * NW, lane);
                    cp_async_commit();
                }
#pragma unroll
                for (int i = 0; i < (D * D / 4) / NT; ++i) {
                    const int idx = tid + i * NT, j = idx / (D / 4), k = idx - j * (D / 4);
                    rs[j * (D / 4) + rot_pos(j, k)] = rr[i];
                }
            }
            __syncthreads();
            if (dense) {
                for (int e = tid; e < heads_here * D; e += NT) {
                    const int kc = (e % D) >> 2;
                    qs[e] = __float2half_rn(qf[(e - (e % D)) + ((kc ^ (kc >> 3)) << 2) + (e & 3)] * f);
                }
            } else {
                // thread (j, part): columns [part*32, part*32+32) of row j; the four parts of a row are adjacent lanes
                constexpr int KP = NT / D, COLS = D / KP;
                static_assert(KP == 4, "direct path: four threads per row of R");
                const int j = tid >> 2, kp = tid & 3;
                float acc[HPG];
#pragma unroll
                for (int h = 0; h < HPG; ++h) acc[h] = 0.f;
#pragma unroll
                for (int k = 0; k < COLS / 4; ++k) {
                    const int kc = kp * (COLS / 4) + k;
                    const float4 r = rs[j * (D / 4) + rot_pos(j, kc)];
#pragma unroll
                    for (int h = 0; h < HPG; ++h) {
                        if (h < heads_here) {
                            const float4 x = *reinterpret_cast<const float4*>(qf + h * D + 4 * (kc ^ (kc >> 3)));
                            acc[h] = fmaf(x.x, r.x, fmaf(x.y, r.y, fmaf(x.z, r.z, fmaf(x.w, r.w, acc[h]))));
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < HPG; ++h) {
                    acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 1);
                    acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 2);
                    if (kp == 0 && h < heads_here) qs[h * D + j] = __float2half_rn(acc[h] * f);
                }
            }
        } else {
            // general path: thread (j, part) reads its slice of row j straight from global memory
            constexpr int KP = NT / D >= 4 ? 4 : NT / D >= 2 ? 2 : 1;     // slices per row (power of two)
            constexpr int COLS = D / KP;                                   // columns per slice
            const int j = tid / KP, kp = tid - j * KP;
            const bool rot_thread = !dense && j < D;
            constexpr int CH = COLS / 4 > 16 ? 16 : COLS / 4;             // float4 loads in flight per round
            const float4* row = reinterpret_cast<const float4*>(p.rot + int64_t(rot_thread ? j : 0) * D + kp * COLS);
            float4 rr[CH];
            if (rot_thread) {
#pragma unroll
                for (int k = 0; k < CH; ++k) rr[k] = __ldg(row + k);
            }
            for (int e = tid; e < heads_here * D; e += NT) qf[e] = load_as_f32(p.q, p.q_dtype, qbase + e);
            __syncthreads();
            if (dense) {
                for (int e = tid; e < heads_here * D; e += NT) qs[e] = __float2half_rn(qf[e] * f);
            } else {
                float acc[HPG];
#pragma unroll
                for (int h = 0; h < HPG; ++h) acc[h] = 0.f;
                if (rot_thread) {
#pragma unroll 1
                    for (int k0 = 0; k0 < COLS / 4; k0 += CH) {
                        if (k0 > 0) {
#pragma unroll
                            for (int k = 0; k < CH; ++k) rr[k] = __ldg(row + k0 + k);
                        }
#pragma unroll
                        for (int k = 0; k < CH; ++k) {
#pragma unroll
                            for (int h = 0; h < HPG; ++h) {
                                if (h < heads_here) {
                                    const float4 x = *reinterpret_cast<const float4*>(qf + h * D + kp * COLS + 4 * (k0 + k));
                                    acc[h] = fmaf(x.x, rr[k].x, fmaf(x.y, rr[k].y, fmaf(x.z, rr[k].z, fmaf(x.w, rr[k].w, acc[h]))));
                                }
                            }
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < HPG; ++h) {
#pragma unroll
                    for (int off = KP / 2; off; off >>= 1) acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], off);
                    if (rot_thread && kp == 0 && h < heads_here) qs[h * D + j] = __float2half_rn(acc[h] * f);
                }
            }
        }
    }
    __syncthreads();
    TQ_STAMP(3);

    WarpAcc<D> st;
    st.m[0] = st.m[1] = st.mt[0] = st.mt[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) st.o[mt][0] = st.o[mt][1] = st.o[mt][2] = st.o[mt][3] = 0.f;

    bool direct_order = false;   // which coordinate permutation the accumulators use

    if (dense) {
        // ---------------- uncompressed tokens: sink then residual window, raw query ----------------
        uint32_t bq[D / 16][2];
        {
            const __half* qh = qs + g * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
                bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
            }
        }
        __half* Ks = reinterpret_cast<__half*>(smem) + size_t(warp) * 2 * TILE * LD;
        __half* Vs = Ks + TILE * LD;
        const int64_t n_tok = p.sink_len + p.res_len;
        const int64_t tile_lo = int64_t(split - p.n_ps) * p.d_tps;
        const int64_t tile_hi = min(tile_lo + p.d_tps, (n_tok + TILE - 1) / TILE);
        for (int64_t tile = tile_lo + warp; tile < tile_hi; tile += NW) {
            const int64_t tok0 = tile * TILE;
            constexpr int NCH = TILE * (D / 8) / 32;          // 16-byte chunks per lane and tensor
            if (p.dense_dtype == TQ_F16) {
                uint4 kv[NCH], vv[NCH];                        // every load of the tile in flight before the first store
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const int c = lane + 32 * i, r = c / (D / 8), c8 = c - r * (D / 8);
                    const int64_t tok = tok0 + r;
                    kv[i] = make_uint4(0, 0, 0, 0); vv[i] = kv[i];
                    if (tok < n_tok) {
                        const bool in_sink = tok < p.sink_len;
                        const int64_t e = (in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len)) * D + c8 * 8;
                        kv[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(in_sink ? p.sink_k : p.res_k) + e));
                        vv[i] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(in_sink ? p.sink_v : p.res_v) + e));
                    }
                }
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const int c = lane + 32 * i, r = c / (D / 8), c8 = c - r * (D / 8);
                    *reinterpret_cast<uint4*>(Ks + r * LD + c8 * 8) = kv[i];
                    *reinterpret_cast<uint4*>(Vs + r * LD + c8 * 8) = vv[i];
                }
            } else {
                for (int c = lane; c < TILE * (D / 8); c += 32) {
                    const int r = c / (D / 8), c8 = c - r * (D / 8);
                    const int64_t tok = tok0 + r;
                    uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
                    if (tok < n_tok) {
                        const bool in_sink = tok < p.sink_len;
                        const int64_t e = (in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len)) * D + c8 * 8;
                        const void* kb = in_sink ? p.sink_k : p.res_k;
                        const void* vb = in_sink ? p.sink_v : p.res_v;
                        __half hk[8], hv[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            hk[i] = __float2half_rn(load_as_f32(kb, p.dense_dtype, e + i));
                            hv[i] = __float2half_rn(load_as_f32(vb, p.dense_dtype, e + i));
                        }
                        kv = *reinterpret_cast<uint4*>(hk);
                        vv = *reinterpret_cast<uint4*>(hv);
                    }
                    *reinterpret_cast<uint4*>(Ks + r * LD + c8 * 8) = kv;
                    *reinterpret_cast<uint4*>(Vs + r * LD + c8 * 8) = vv;
                }
            }
            __syncwarp();
            tile_from_smem<D>(Ks, Vs, bq, 1.f, 1.f, 1.f, 1.f, tok0 + g < n_tok, tok0 + g + 8 < n_tok, st, lane);
            __syncwarp();
        }
    } else if constexpr (!DIRECT) {
        // ---------------- packed tokens, general path: unpack into shared memory ---------------------
        uint32_t bq[D / 16][2];
        {
            const __half* qh = qs + g * D;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
                bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
            }
        }
        __half* Ks = reinterpret_cast<__half*>(smem) + size_t(warp) * 2 * TILE * LD;
        __half* Vs = Ks + TILE * LD;
        const int k_half = p.kb_lo ? D / 2 : D, v_half = p.vb_lo ? D / 2 : D;
        const int kw_hi = packed_bytes(k_half, p.kb_hi), kw_lo = p.kb_lo ? packed_bytes(D - k_half, p.kb_lo) : 0;
        const int vw_hi = packed_bytes(v_half, p.vb_hi), vw_lo = p.vb_lo ? packed_bytes(D - v_half, p.vb_lo) : 0;
        const int64_t tile_lo = int64_t(split) * p.p_tps;
        const int64_t tile_hi = min(tile_lo + p.p_tps, (p.c_len + TILE - 1) / TILE);
        for (int64_t tile = tile_lo + warp; tile < tile_hi; tile += NW) {
            const int64_t tok0 = tile * TILE;
            {
                const int r = lane >> 1, hr = lane & 1;
                const int64_t tok = tok0 + r;
                const bool live = tok < p.c_len;
                const int64_t row = kvl * p.c_ls + (live ? tok : 0);
                const uint8_t* kr_hi = p.k_hi + row * kw_hi;
                const uint8_t* kr_lo = p.kb_lo ? p.k_lo + row * kw_lo : nullptr;
                const uint8_t* vr_hi = p.v_hi + row * vw_hi;
                const uint8_t* vr_lo = p.vb_lo ? p.v_lo + row * vw_lo : nullptr;
                for (int jj = 0; jj < D / 2; jj += 2) {
                    const int j = hr * (D / 2) + jj;
                    __half2 kk = __float2half2_rn(0.f), vv = kk;
                    if (live) {
                        const __half k0 = j < k_half ? ctab[code_at(kr_hi, j, p.kb_hi)] : ctab[16 + code_at(kr_lo, j - k_half, p.kb_lo)];
                        const __half k1 = j + 1 < k_half ? ctab[code_at(kr_hi, j + 1, p.kb_hi)] : ctab[16 + code_at(kr_lo, j + 1 - k_half, p.kb_lo)];
                        const __half v0 = j < v_half ? ctab[32 + code_at(vr_hi, j, p.vb_hi)] : ctab[48 + code_at(vr_lo, j - v_half, p.vb_lo)];
                        const __half v1 = j + 1 < v_half ? ctab[32 + code_at(vr_hi, j + 1, p.vb_hi)] : ctab[48 + code_at(vr_lo, j + 1 - v_half, p.vb_lo)];
                        kk = __halves2half2(k0, k1);
                        vv = __halves2half2(v0, v1);
                    }
                    *reinterpret_cast<__half2*>(Ks + r * LD + j) = kk;
                    *reinterpret_cast<__half2*>(Vs + r * LD + j) = vv;
                }
            }
            const bool ok0 = tok0 + g < p.c_len, ok1 = tok0 + g + 8 < p.c_len;
            const int64_t n0 = kvl * p.c_ls + (ok0 ? tok0 + g : 0), n1 = kvl * p.c_ls + (ok1 ? tok0 + g + 8 : 0);
            const float kn0 = __ldg(p.k_norms + n0), kn1 = __ldg(p.k_norms + n1);
            const float vn0 = __ldg(p.v_norms + n0), vn1 = __ldg(p.v_norms + n1);
            __syncwarp();
            tile_from_smem<D>(Ks, Vs, bq, kn0, kn1, vn0, vn1, ok0, ok1, st, lane);
            __syncwarp();
        }
    } else {
        // ---------------- packed tokens, direct path: 4-bit keys, 2-bit values -------------------------
        direct_order = true;
        static_assert(!DIRECT || D == 128, "the direct path's shared-memory tile layout is written for d = 128");
        // Query fragments in the byte order of the 4-bit rows: thread t owns coordinates [t*D/4, (t+1)*D/4).
        uint32_t bq[D / 16][2];
        {
            const __half* qh = qs + g * D + t * (D / 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks) : 0u;
                bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks + 2) : 0u;
            }
        }
        using RC = RingCtx<D, NW>;
        constexpr int KT = RC::KT, VT = RC::VT, VW = RC::VW, STG = RC::STG;
        // 32-bit shared-window addresses of this lane's private table columns: entry e of T4 sits at
        // t4 + e*128, entry e of T2 at t2 + e*128 (one multiply-add each, no 64-bit address arithmetic).
        const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
        const uint32_t t4 = smem_base + lane * 4;
        const uint32_t t2 = smem_base + 32768 + (lane & 15) * 8;
        const uint32_t ring = rc.ring;
        const int c_len = rc.c_len, tile_hi = rc.tile_hi;
        const uint32_t vo0 = KT + RC::vslot(2 * t) * VW + g * 4, vo1 = KT + RC::vslot(2 * t + 1) * VW + g * 4;
        const uint32_t vo2 = KT + RC::vslot(2 * t + 8) * VW + g * 4, vo3 = KT + RC::vslot(2 * t + 9) * VW + g * 4;
        auto compute = [&](int stage, int tile) {
            const uint32_t sb = ring + stage * STG;
            const int tok0 = tile * TILE;
            const uint4 q0 = ring128(sb + lane * 16);            // token g,   this thread's quarter row
            const uint4 q1 = ring128(sb + 512 + lane * 16);      // token g+8
            const float kn0 = __uint_as_float(ring32(sb + KT + VT + g * 4)), kn1 = __uint_as_float(ring32(sb + KT + VT + 32 + g * 4));
            const float vn0 = __uint_as_float(ring32(sb + KT + VT + 64 + g * 4)), vn1 = __uint_as_float(ring32(sb + KT + VT + 96 + g * 4));
            const uint32_t va = ring32(sb + vo0), vb = ring32(sb + vo1), vc = ring32(sb + vo2), vd = ring32(sb + vo3);
            // two independent accumulators (even / odd k-steps) halve the dependent MMA chain
            float s[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                // bytes 2ks, 2ks+1 of the quarter row
                const int wi = ks >> 1;
                const uint32_t w0 = wi == 0 ? q0.x : wi == 1 ? q0.y : wi == 2 ? q0.z : q0.w;
                const uint32_t w1 = wi == 0 ? q1.x : wi == 1 ? q1.y : wi == 2 ? q1.z : q1.w;
                const int b0 = (ks & 1) * 2;
                const uint32_t a0 = lut32(__byte_perm(w0, 0, 0x4440 | b0) * 128u + t4);
                const uint32_t a1 = lut32(__byte_perm(w1, 0, 0x4440 | b0) * 128u + t4);
                const uint32_t a2 = lut32(__byte_perm(w0, 0, 0x4440 | (b0 + 1)) * 128u + t4);
                const uint32_t a3 = lut32(__byte_perm(w1, 0, 0x4440 | (b0 + 1)) * 128u + t4);
                if (ks & 1) mma16816(s2, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
                else mma16816(s, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] += s2[i];
            uint32_t bp[2];
            softmax_step<D>(s, kn0, kn1, vn0, vn1, tok0 + g < c_len, tok0 + g + 8 < c_len, st, bp);
            // interleave the 2-bit codes of a token pair: nibble k of X = (A code 2k) | (B code 2k) << 2
            const uint32_t x0 = (va & 0x33333333u) | ((vb << 2) & 0xCCCCCCCCu);
            const uint32_t y0 = ((va >> 2) & 0x33333333u) | (vb & 0xCCCCCCCCu);
            const uint32_t x1 = (vc & 0x33333333u) | ((vd << 2) & 0xCCCCCCCCu);
            const uint32_t y1 = ((vc >> 2) & 0x33333333u) | (vd & 0xCCCCCCCCu);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint2 fa = lut64(__byte_perm(x0, 0, 0x4440 | k) * 128u + t2);   // rows g,   tokens 2t,2t+1   -> m-tiles 2k, 2k+1
                const uint2 fb = lut64(__byte_perm(y0, 0, 0x4440 | k) * 128u + t2);   // rows g+8
                const uint2 fc = lut64(__byte_perm(x1, 0, 0x4440 | k) * 128u + t2);   // rows g,   tokens 2t+8,2t+9
                const uint2 fd = lut64(__byte_perm(y1, 0, 0x4440 | k) * 128u + t2);
                mma16816(st.o[2 * k], fa.x, fb.x, fc.x, fd.x, bp[0], bp[1]);
                mma16816(st.o[2 * k + 1], fa.y, fb.y, fc.y, fd.y, bp[0], bp[1]);
            }
        };
        // Software pipeline: RING_STAGES - 1 tiles in flight per warp (the first ones were issued before the query
        // was rotated).  One commit group per slot, issued or not, keeps the group count uniform; cp.async
        // completion is tracked by hardware (no spin waits).
        const int first = rc.first;
        int stage = 0;
        for (int tile = first; tile < tile_hi; tile += NW) {
            const int ahead = tile + (RING_STAGES - 1) * NW;
            const int st_in = stage == 0 ? RING_STAGES - 1 : stage - 1;
            if (ahead < tile_hi) rc.issue(st_in, ahead, lane);
            cp_async_commit();
            cp_async_wait<RING_STAGES - 1>();
            __syncwarp();
            compute(stage, tile);
            __syncwarp();       // every lane is done with this stage before it is refilled
            stage = stage == RING_STAGES - 1 ? 0 : stage + 1;
        }
        cp_async_wait<0>();
    }

    // ---------------- CTA reduction over warps ----------------------------------------------------------------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
    }
    __syncthreads();   // staging / tables / ring are dead from here on
    TQ_STAMP(4);
    constexpr int DS = D + 2;                               // row stride (floats): keeps the 64-bit stores below 2-way conflicts
    constexpr int RW = HPG * DS + 2 * HPG;                  // floats per warp in the reduction buffer
    float* red = reinterpret_cast<float*>(smem);
    float* wts = red + size_t(NW) * RW;                     // [NW][8] per-warp weights exp2(m_w - M)
    float* s_acc = wts + NW * HPG;                          // [8][D] reduced accumulator of this CTA
    float* s_pp = s_acc + HPG * D;                          // [MERGE_CPARTS][8][D] partial products with R
    {
        float* ro = red + size_t(warp) * RW;                // [8][DS]: head-major
        float* rm = ro + HPG * DS;                          // [8] max, [8] sum
        if (2 * t < heads_here) {                           // lanes that hold only padding heads store nothing
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt) {
                if (direct_order) {                          // rows g, g+8 of the tile are coordinates c0, c0+1
                    const int c0 = g * (D / 8) + 2 * mt;
                    *reinterpret_cast<float2*>(ro + (2 * t) * DS + c0) = make_float2(st.o[mt][0], st.o[mt][2]);
                    *reinterpret_cast<float2*>(ro + (2 * t + 1) * DS + c0) = make_float2(st.o[mt][1], st.o[mt][3]);
                } else {
                    const int c0 = mt * 16 + g;
                    ro[(2 * t) * DS + c0] = st.o[mt][0]; ro[(2 * t + 1) * DS + c0] = st.o[mt][1];
                    ro[(2 * t) * DS + c0 + 8] = st.o[mt][2]; ro[(2 * t + 1) * DS + c0 + 8] = st.o[mt][3];
                }
            }
        }
        if (g == 0) {
            rm[2 * t] = st.m[0]; rm[2 * t + 1] = st.m[1];
            rm[HPG + 2 * t] = st.l[0]; rm[HPG + 2 * t + 1] = st.l[1];
        }
    }
    __syncthreads();
    const int64_t grp = (kvl * p.HG + hg);
    const int64_t pidx = grp * S + split;
    float* po = p.part_o + pidx * (int64_t(p.slots) * D);   // [slots][D], always in UNROTATED space
    float* pml = p.part_ml + pidx * (p.slots * 2);          // [slots][2]
    if (tid < NW * HPG) {
        const int w = tid / HPG, h = tid - w * HPG;
        float M = -INFINITY;
#pragma unroll
        for (int x = 0; x < NW; ++x) M = fmaxf(M, red[size_t(x) * RW + HPG * DS + h]);
        const float mw = red[size_t(w) * RW + HPG * DS + h];
        const float f = (mw == -INFINITY) ? 0.f : ex2(mw - M);
        wts[w * HPG + h] = f;
        if (w == 0 && h < heads_here) pml[2 * h] = M;
    }
    __syncthreads();
    if (tid < heads_here) {
        float L = 0.f;
#pragma unroll
        for (int x = 0; x < NW; ++x) L = fmaf(wts[x * HPG + tid], red[size_t(x) * RW + HPG * DS + HPG + tid], L);
        pml[2 * tid + 1] = L;
    }
    const int v_half = p.vb_lo ? D / 2 : D;
    for (int e = tid; e < D * heads_here; e += NT) {         // e = h * D + c: contiguous in the workspace
        const int h = e / D, c = e - h * D;
        float acc = 0.f;
#pragma unroll
        for (int x = 0; x < NW; ++x) acc = fmaf(wts[x * HPG + h], red[size_t(x) * RW + h * DS + c], acc);
        if (dense) po[e] = acc;                              // uncompressed tokens were never rotated
        else s_acc[e] = acc / (c < v_half ? p.v_scale_hi : p.v_scale_lo);
    }
    if (!dense) {
        // Packed tokens were accumulated in rotated space: undo the rotation here, once per CTA
        // (y @ R, rotation.py:68-78), so that the merge only has to add partials.  Thread (slab, j).
        __syncthreads();
        constexpr int JT = NT / MERGE_CPARTS, ROWS = D / MERGE_CPARTS;
        const int slab = tid / JT, jt = tid - slab * JT;
        for (int j = jt; j < D; j += JT) {
            float acc[HPG];
#pragma unroll
            for (int h = 0; h < HPG; ++h) acc[h] = 0.f;
#pragma unroll 4
            for (int c4 = 0; c4 < ROWS / 4; ++c4) {
                float r[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = slab * ROWS + c4 * 4 + u;
                    if constexpr (DIRECT) r[u] = reinterpret_cast<const float*>(smem + rot_offset<D, NW>())[(c * (D / 4) + rot_pos(c, j >> 2)) * 4 + (j & 3)];
                    else r[u] = __ldg(p.rot + int64_t(c) * D + j);
                }
#pragma unroll
                for (int h = 0; h < HPG; ++h) {
                    if (h < heads_here) {
                        const float4 a = *reinterpret_cast<const float4*>(s_acc + h * D + slab * ROWS + c4 * 4);
                        acc[h] = fmaf(a.x, r[0], fmaf(a.y, r[1], fmaf(a.z, r[2], fmaf(a.w, r[3], acc[h]))));
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < HPG; ++h)
                if (h < heads_here) s_pp[(slab * HPG + h) * D + j] = acc[h];
        }
        __syncthreads();
        for (int e = tid; e < D * heads_here; e += NT) {
            const int h = e / D, j = e - h * D;
            float v = 0.f;
#pragma unroll
            for (int x = 0; x < MERGE_CPARTS; ++x) v += s_pp[(x * HPG + h) * D + j];
            po[e] = v;
        }
    }

    // ---------------- last arrival for this (sequence, KV head, head group) merges -----------------------
    __syncthreads();
    if (tid == 0) {
        __threadfence();       // cumulative: publishes the partial every thread of this CTA wrote before the barrier
        const int prev = atomicAdd(p.counters + grp, 1);
        s_misc[8] = (prev == S - 1) ? 1.f : 0.f;
        if (prev == S - 1) {
            __threadfence();
            p.counters[grp] = 0;     // ready for the next launch
        }
    }
    TQ_STAMP(5);
    __syncthreads();
    if (s_misc[8] == 0.f) return;
    TQ_STAMP(7);
    const int SL = p.slots;
    const int64_t base = grp * S;
    // thread (h, c) loads its partial accumulators of up to 24 splits while other threads fetch the (max, sum)
    // pairs into shared memory: one round of loads; the log-sum-exp weights are then recomputed per thread
    float2* s_ml = reinterpret_cast<float2*>(smem);                             // [8][MAX_SPLITS]
    constexpr int U = 24;
    const int e0 = tid;                                                         // first (h, c) element of this thread
    float v0[U];
    {
        const int h = e0 / D, c = e0 - h * D;
        const float* src = p.part_o + (base * SL + h) * D + c;
        const int64_t stride = int64_t(SL) * D;
#pragma unroll
        for (int u = 0; u < U; ++u) v0[u] = (e0 < D * heads_here && u < S) ? __ldcg(src + u * stride) : 0.f;
    }
    for (int idx = tid; idx < heads_here * S; idx += NT) {
        const int h = idx / S, sidx = idx - h * S;
        s_ml[h * MAX_SPLITS + sidx] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + ((base + sidx) * SL + h) * 2));
    }
    __syncthreads();
    TQ_STAMP(8);
    for (int e = tid; e < D * heads_here; e += NT) {
        const int h = e / D, c = e - h * D;
        const float* src = p.part_o + (base * SL + h) * D + c;
        const int64_t stride = int64_t(SL) * D;
        const float2* ml = s_ml + h * MAX_SPLITS;
        float M = -INFINITY;
        for (int sidx = 0; sidx < S; ++sidx) M = fmaxf(M, ml[sidx].x);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (u < S) {
                const float2 x = ml[u];
                const float w = (x.x == -INFINITY) ? 0.f : ex2(x.x - M);
                L = fmaf(w, x.y, L);
                acc = fmaf(w, (e == e0) ? v0[u] : __ldcg(src + u * stride), acc);
            }
        }
        for (int sidx = U; sidx < S; ++sidx) {
            const float2 x = ml[sidx];
            const float w = (x.x == -INFINITY) ? 0.f : ex2(x.x - M);
            L = fmaf(w, x.y, L);
            acc = fmaf(w, __ldcg(src + sidx * stride), acc);
        }
        store_from_f32(p.out, p.out_dtype, qbase + e, acc / L);
    }
    TQ_STAMP(6);
}

// ---- host side ------------------------------------------------------------------------------------
static int g_tune_ctas_per_sm = 1;     // CTAs of the general path resident per SM (split heuristic)
static int g_tune_force_general = 0;   // 1: never take the direct path (testing)
static int g_tune_splits = 0;          // > 0: fixed number of packed splits
static int g_tune_pdl = 1;             // programmatic dependent launch between consecutive calls

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

struct SplitPlan { int n_ps, n_ds, hg; int64_t p_tps, d_tps; };

static SplitPlan plan_splits(int batch, int n_q_heads, int n_kv_heads, int64_t c_len, int64_t dense_len, int sms, bool direct) {
    const int NW = warps_per_cta(direct);
    SplitPlan s{};
    const int G = n_q_heads / n_kv_heads;
    s.hg = (G + HPG - 1) / HPG;
    const int64_t lanes = int64_t(batch) * n_kv_heads * s.hg;
    const int64_t p_tiles = (c_len + TILE - 1) / TILE, d_tiles = (dense_len + TILE - 1) / TILE;
    if (d_tiles > 0) {
        s.d_tps = direct ? NW : 2 * NW;   // tiles per dense CTA: one (16 warps) or two (8 warps) per warp
        s.n_ds = int((d_tiles + s.d_tps - 1) / s.d_tps);
        if (s.n_ds > 64) { s.d_tps = (d_tiles + 63) / 64; s.n_ds = int((d_tiles + s.d_tps - 1) / s.d_tps); }
    }
    if (p_tiles > 0) {
        // all CTAs of the grid resident at once: (packed + dense splits) * lanes <= SMs * CTAs per SM
        const int64_t slots = int64_t(sms) * (direct ? 1 : g_tune_ctas_per_sm);
        int64_t want = g_tune_splits > 0 ? g_tune_splits : slots / lanes - s.n_ds;
        const int64_t max_useful = (p_tiles + 2 * NW - 1) / (2 * NW);   // at least two tiles per warp
        if (want > max_useful) want = max_useful;
        if (want < 1) want = 1;
        if (want > MAX_SPLITS - 64) want = MAX_SPLITS - 64;
        s.p_tps = (p_tiles + want - 1) / want;
        s.n_ps = int((p_tiles + s.p_tps - 1) / s.p_tps);
    }
    return s;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The arrival counters sit at the start of the workspace so that their position does not depend on the plan.
struct WsLayout { size_t counters, part_o, part_ml, total; };

static WsLayout ws_layout(int batch, int n_q_heads, int n_kv_heads, int d, const SplitPlan& s) {
    WsLayout w{};
    const size_t groups = size_t(batch) * n_kv_heads * s.hg;
    const size_t parts = groups * size_t(s.n_ps + s.n_ds);
    const size_t slots = size_t(std::min(n_q_heads / n_kv_heads, HPG));
    w.counters = 0;
    w.part_o = align_up(groups * sizeof(int), 256);
    w.part_ml = align_up(w.part_o + parts * slots * d * sizeof(float), 256);
    w.total = align_up(w.part_ml + parts * slots * 2 * sizeof(float), 256);
    return w;
}

template <int D, bool DIRECT> static int launch_decode(const DecodeParams& p, cudaStream_t s) {
    constexpr size_t smem = kernel_smem<D, DIRECT>();
    static bool set[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel<D, DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev] = true;
    }
    // Programmatic stream serialisation: the grid may become resident before its predecessor on the stream
    // has finished; the kernel calls griddepcontrol.wait before it touches anything but constants.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(p.n_ps + p.n_ds), unsigned(p.Hkv * p.HG), unsigned(p.B));
    cfg.blockDim = dim3(warps_per_cta(DIRECT) * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_tune_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attn_kernel<D, DIRECT>, p);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: %s", cudaGetErrorString(e));
    return TQ_OK;
}

// Validates the arguments, picks the path and the split plan and fills the kernel parameters.
int decode_prepare(const tq_decode_args* a, void* workspace, size_t workspace_bytes, DecodeParams* out, bool* direct_out) {
    if (!a) return fail(TQ_ERR_INVALID, "tq_decode_attn: null args");
    const int d = a->d;
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: batch=%d q_heads=%d kv_heads=%d", a->batch, a->n_q_heads, a->n_kv_heads);
    if (d != 64 && d != 96 && d != 128 && d != 256) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: d=%d (64, 96, 128 or 256)", d);
    if (a->c_len < 0 || a->sink_len < 0 || a->res_len < 0 || a->c_len + a->sink_len + a->res_len == 0)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: the cache holds no tokens");
    if (a->c_len >= (int64_t(1) << 30)) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: c_len too large");
    if (!a->q || !a->rot || !a->out || !workspace) return fail(TQ_ERR_INVALID, "tq_decode_attn: null pointer");
    if (a->q_dtype < 0 || a->q_dtype > 2 || a->out_dtype < 0 || a->out_dtype > 2 || a->dense_dtype < 0 || a->dense_dtype > 2)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: bad dtype");
    if (!aligned(a->rot, 16)) return fail(TQ_ERR_INVALID, "tq_decode_attn: rot must be 16-byte aligned");
    if (a->c_len > 0) {
        if (!bits_ok(a->k_bits_hi) || !bits_ok(a->v_bits_hi) || (a->k_bits_lo && !bits_ok(a->k_bits_lo)) || (a->v_bits_lo && !bits_ok(a->v_bits_lo)))
            return fail(TQ_ERR_INVALID, "Unsupported bit-width. Use 1, 2, 3, or 4.");
        if (!a->k_hi || !a->v_hi || !a->k_norms || !a->v_norms || !a->k_cent_hi || !a->v_cent_hi || (a->k_bits_lo && (!a->k_lo || !a->k_cent_lo)) ||
            (a->v_bits_lo && (!a->v_lo || !a->v_cent_lo)))
            return fail(TQ_ERR_INVALID, "tq_decode_attn: null packed-cache pointer");
        if (a->c_lane_stride < a->c_len) return fail(TQ_ERR_INVALID, "tq_decode_attn: c_lane_stride < c_len");
        if (a->k_qjl_bits || a->v_qjl_bits) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: QJL sketches are not supported by this build");
    }
    if ((a->sink_len > 0 && (!a->sink_k || !a->sink_v || a->sink_lane_stride < a->sink_len)) ||
        (a->res_len > 0 && (!a->res_k || !a->res_v || a->res_lane_stride < a->res_len)))
        return fail(TQ_ERR_INVALID, "tq_decode_attn: bad sink / residual buffers");
    if (a->dense_dtype == TQ_F16 && ((a->sink_len > 0 && (!aligned(a->sink_k, 16) || !aligned(a->sink_v, 16))) ||
                                     (a->res_len > 0 && (!aligned(a->res_k, 16) || !aligned(a->res_v, 16)))))
        return fail(TQ_ERR_INVALID, "tq_decode_attn: fp16 sink / residual buffers must be 16-byte aligned");
    if (!aligned(workspace, 256)) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace must be 256-byte aligned");

    const int64_t dense_len = a->sink_len + a->res_len;
    // direct path: 4-bit keys / 2-bit values, d = 128, rows and norms addressable in aligned 16-byte chunks
    const bool direct = !g_tune_force_general && d == 128 && a->c_len > 0 && a->k_bits_hi == 4 && a->k_bits_lo == 0 &&
                        a->v_bits_hi == 2 && a->v_bits_lo == 0 && aligned(a->k_hi, 16) && aligned(a->v_hi, 16) &&
                        aligned(a->k_norms, 16) && aligned(a->v_norms, 16) && a->c_lane_stride % 16 == 0;
    const SplitPlan sp = plan_splits(a->batch, a->n_q_heads, a->n_kv_heads, a->c_len, dense_len, sm_count(), direct);
    const WsLayout wl = ws_layout(a->batch, a->n_q_heads, a->n_kv_heads, d, sp);
    if (wl.total > workspace_bytes) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace %zu B < %zu B", workspace_bytes, wl.total);
    if (sp.n_ps + sp.n_ds > MAX_SPLITS) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: too many splits");

    DecodeParams p{};
    p.B = a->batch; p.Hq = a->n_q_heads; p.Hkv = a->n_kv_heads; p.G = p.Hq / p.Hkv; p.HG = sp.hg; p.D = d; p.slots = std::min(p.G, HPG);
    p.c_len = a->c_len; p.c_ls = a->c_lane_stride;
    p.kb_hi = a->k_bits_hi; p.kb_lo = a->k_bits_lo; p.vb_hi = a->v_bits_hi; p.vb_lo = a->v_bits_lo;
    p.k_hi = a->k_hi; p.k_lo = a->k_lo; p.v_hi = a->v_hi; p.v_lo = a->v_lo;
    p.k_norms = a->k_norms; p.v_norms = a->v_norms;
    p.kc_hi = a->k_cent_hi; p.kc_lo = a->k_cent_lo; p.vc_hi = a->v_cent_hi; p.vc_lo = a->v_cent_lo;
    p.dense_dtype = a->dense_dtype;
    p.sink_k = a->sink_k; p.sink_v = a->sink_v; p.res_k = a->res_k; p.res_v = a->res_v;
    p.sink_len = a->sink_len; p.sink_ls = a->sink_lane_stride; p.res_len = a->res_len; p.res_ls = a->res_lane_stride;
    p.n_ps = sp.n_ps; p.n_ds = sp.n_ds; p.p_tps = sp.p_tps; p.d_tps = sp.d_tps;
    p.q = a->q; p.q_dtype = a->q_dtype; p.scale = a->scale; p.rot = a->rot;
    p.v_scale_hi = a->v_cent_scale_hi > 0.f ? a->v_cent_scale_hi : 1.f;
    p.v_scale_lo = a->v_cent_scale_lo > 0.f ? a->v_cent_scale_lo : 1.f;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    p.counters = reinterpret_cast<int*>(ws + wl.counters);
    p.part_o = reinterpret_cast<float*>(ws + wl.part_o); p.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
    p.out = a->out; p.out_dtype = a->out_dtype;
    *out = p;
    *direct_out = direct;
    return TQ_OK;
}

int decode_launch(const DecodeParams& p, bool direct, cudaStream_t s) {
    if (direct) return launch_decode<128, true>(p, s);
    if (p.D == 64) return launch_decode<64, false>(p, s);
    if (p.D == 96) return launch_decode<96, false>(p, s);
    if (p.D == 128) return launch_decode<128, false>(p, s);
    return launch_decode<256, false>(p, s);
}

}  // namespace tq

using namespace tq;

#ifdef TQ_TIMING
extern "C" int tq_debug_timing(unsigned long long* host_out, int n) {
    return int(cudaMemcpyFromSymbol(host_out, g_tq_timing, sizeof(unsigned long long) * n));
}
#endif

extern "C" int tq_set_tuning(const char* key, int value) {
    if (!key) return fail(TQ_ERR_INVALID, "tq_set_tuning: null key");
    const std::string_view k(key);
    if (k == "decode_ctas_per_sm" && value >= 1 && value <= 8) g_tune_ctas_per_sm = value;
    else if (k == "decode_force_general" && (value == 0 || value == 1)) g_tune_force_general = value;
    else if (k == "decode_pdl" && (value == 0 || value == 1)) g_tune_pdl = value;
    else if (k == "decode_splits" && value >= 0 && value <= MAX_SPLITS - 64) g_tune_splits = value;
    else return fail(TQ_ERR_INVALID, "tq_set_tuning: unknown key or bad value: %s=%d", key, value);
    return TQ_OK;
}

extern "C" float tq_fp16_table_scale(const float* centroids_host, int n) {
    // Scale s in [1, 2) that minimises the worst relative error of fp16(s * c_i): the decode kernel keeps
    // value centroids in fp16, and with only 2^bits distinct levels their rounding error is systematic.
    if (!centroids_host || n <= 0) return 1.f;
    float best = 1.f;
    double best_err = 1e30;
    for (int i = 0; i < (1 << 16); ++i) {
        const float sc = 1.f + float(i) / float(1 << 16);
        double worst = 0.0;
        for (int k = 0; k < n; ++k) {
            const float v = centroids_host[k] * sc;
            if (v == 0.f) continue;
            const float r = __half2float(__float2half_rn(v));
            const double e = fabs(double(r) - double(v)) / fabs(double(v));
            if (e > worst) worst = e;
        }
        if (worst < best_err) { best_err = worst; best = sc; }
    }
    return best;
}

extern "C" size_t tq_decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len,
                                            int64_t dense_len) {
    if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || d <= 0 || n_q_heads % n_kv_heads || c_len < 0 || dense_len < 0) return 0;
    // The larger of the two split plans tq_decode_attn can choose for these sizes (current tuning values).
    const size_t a = ws_layout(batch, n_q_heads, n_kv_heads, d, plan_splits(batch, n_q_heads, n_kv_heads, c_len, dense_len, sm_count(), false)).total;
    const size_t b = ws_layout(batch, n_q_heads, n_kv_heads, d, plan_splits(batch, n_q_heads, n_kv_heads, c_len, dense_len, sm_count(), true)).total;
    return a > b ? a : b;
}

extern "C" int tq_decode_attn(const tq_decode_args* a, void* stream) {
    DecodeParams p;
    bool direct = false;
    int rc = decode_prepare(a, a ? a->workspace : nullptr, a ? a->workspace_bytes : 0, &p, &direct);
    if (rc) return rc;
    return decode_launch(p, direct, static_cast<cudaStream_t>(stream));
}
