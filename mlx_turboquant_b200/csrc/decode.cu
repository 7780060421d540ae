// One decode step of attention computed directly on the compressed KV cache
// [fp16 sink | packed middle | fp16 residual window], split over the sequence (flash-decode).
//
// Three launches per call:
//   decode_prep_kernel     rotates the query once (q @ R^T), folds scale*log2(e) in, stores fp16 copies
//   decode_partial_kernel  grid (splits, kv_heads * head_groups, batch); every CTA owns a token range of
//                          either the packed middle or the uncompressed regions and produces one
//                          (max, sum, weighted-V) partial per query head
//   decode_merge_kernel    log-sum-exp merge of the partials, one inverse rotation (@ R) of the part that
//                          was accumulated in rotated space, normalisation, output
//
// Arithmetic: warps work on tiles of 16 tokens with mma.sync.m16n8k16 (fp16 operands, fp32
// accumulation): S[16 tokens x 8 heads] = K_tile . Q^T, online softmax in registers, P transposed with
// movmatrix, O^T[d x 8 heads] += V_tile^T . P^T.  Tokens are the M dimension so a GQA group of up to 8
// query heads shares every unpacked key/value.  The kernel is bound by HBM bytes (packed codes + norms),
// not by the tensor pipe; the contraction shape is tiny (N = 8).
//
// Two ways to build the K / V^T operand fragments:
//   * general: a warp unpacks (or, for the fp16 regions, copies) its tile into shared memory as fp16 and
//     reads fragments back with ldmatrix - any bit width, fractional splits, any d multiple of 16;
//   * direct (4-bit keys, 2-bit values, d = 128): packed words go from global memory to registers and
//     are turned into fragments through bank-conflict-free lookup tables in shared memory
//     (byte -> half2), never touching shared memory with unpacked data.  The coordinate order inside a
//     fragment is permuted to match the byte layout; the query fragments and the output mapping use the
//     same permutation, so results are unchanged.
#include <algorithm>
#include <string_view>

#include "common.cuh"

namespace tq {

constexpr int NW = 8;                 // warps per CTA
constexpr int TILE = 16;              // tokens per warp tile
constexpr int HPG = 8;                // query heads per head group (the mma N dimension)
constexpr float LOG2E = 1.4426950408889634f;

struct DecodeParams {
    int B, Hq, Hkv, G, HG, D;
    int slots;                         // head slots per partial = min(G, 8)
    int64_t c_len, c_ls;
    int kb_hi, kb_lo, vb_hi, vb_lo;
    const uint8_t *k_hi, *k_lo, *v_hi, *v_lo;
    const float *k_norms, *v_norms;
    const float *kc_hi, *kc_lo, *vc_hi, *vc_lo;
    int dense_dtype;
    const void *sink_k, *sink_v, *res_k, *res_v;
    int64_t sink_len, sink_ls, res_len, res_ls;
    int n_ps, n_ds;                    // packed / dense splits
    int64_t p_tps, d_tps;              // tiles per split
    const void* q; int q_dtype; float scale; const float* rot;
    float v_scale_hi, v_scale_lo;      // value centroids are multiplied by this before the fp16 cast (undone in the merge)
    __half *q_rot, *q_raw;             // workspace: (B, Hq, D) each, pre-scaled
    float *part_o, *part_ml;           // workspace: (B, Hkv, HG, S, slots, D) and (.., slots, 2)
    void* out; int out_dtype;
};

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
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
// Programmatic dependent launch: wait for the producer grid / let the consumer grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- query preparation ----------------------------------------------------------------------------
// grid (B*Hq), D threads.  q_rot[j] = sum_k q[k] R[j][k]  (rotation.py:81-110); both copies are scaled by
// scale*log2(e) so the softmax can use exp2.  Thread j streams row j of R with independent 128-bit loads.
__global__ void __launch_bounds__(256) decode_prep_kernel(DecodeParams p) {
    __shared__ __align__(16) float sq[256];
    pdl_trigger();     // the partial kernel may start building its tables right away
    pdl_wait();        // the query (and the workspace) may come from the launch just before this one
    const int bh = blockIdx.x, d = p.D, j = threadIdx.x;
    const float f = p.scale * LOG2E;
    const float v = load_as_f32(p.q, p.q_dtype, int64_t(bh) * d + j);
    sq[j] = v;
    __syncthreads();
    const float4* row = reinterpret_cast<const float4*>(p.rot + int64_t(j) * d);
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
    for (int k = 0; k < d / 4; ++k) {
        const float4 r = __ldg(row + k);
        const float4 x = *reinterpret_cast<const float4*>(sq + 4 * k);
        a0 = fmaf(x.x, r.x, a0); a1 = fmaf(x.y, r.y, a1); a2 = fmaf(x.z, r.z, a2); a3 = fmaf(x.w, r.w, a3);
    }
    p.q_raw[int64_t(bh) * d + j] = __float2half_rn(v * f);
    p.q_rot[int64_t(bh) * d + j] = __float2half_rn(((a0 + a1) + (a2 + a3)) * f);
}

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

// Shared-memory layout of one CTA (a CTA is either "packed" or "dense", so the regions overlap):
//   general staging: per warp  Ks[16][D+8] + Vs[16][D+8] halves
//   direct tables:   T4 [256][32] u32 (32 KB) + T2 [256][16] uint2 (32 KB)
//   final reduction: per warp  o[D][8] floats + m[8] + l[8]
template <int D> __host__ __device__ constexpr int stage_ld() { return D + 8; }
template <int D> __host__ __device__ constexpr size_t stage_bytes() { return size_t(NW) * 2 * TILE * stage_ld<D>() * sizeof(__half); }
template <int D> __host__ __device__ constexpr size_t reduce_bytes() { return size_t(NW) * (D * HPG + 2 * HPG) * sizeof(float); }
constexpr size_t TABLE_BYTES = 65536;
template <int D, bool DIRECT> __host__ __device__ constexpr size_t partial_smem() {
    size_t s = stage_bytes<D>();
    if (reduce_bytes<D>() > s) s = reduce_bytes<D>();
    if (DIRECT && TABLE_BYTES > s) s = TABLE_BYTES;
    return s + 4 * 16 * sizeof(__half);   // + the four 16-entry centroid tables
}

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

// grid (n_ps + n_ds, Hkv * HG, B), NW*32 threads.
template <int D, bool DIRECT>
__global__ void __launch_bounds__(NW * 32, DIRECT ? 2 : 1) decode_partial_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int LD = stage_ld<D>();
    constexpr size_t BODY = partial_smem<D, DIRECT>() - 4 * 16 * sizeof(__half);
    __half* ctab = reinterpret_cast<__half*>(smem + BODY);   // kc_hi, kc_lo, vc_hi, vc_lo (16 each)

    pdl_trigger();     // lets the merge launch get resident early; it waits for this grid to finish
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;        // lane of the cache arrays
    const bool dense = split >= p.n_ps;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int64_t qbase = (int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG) * D;   // first query head of this group

    WarpAcc<D> st;
    st.m[0] = st.m[1] = st.mt[0] = st.mt[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) st.o[mt][0] = st.o[mt][1] = st.o[mt][2] = st.o[mt][3] = 0.f;

    bool direct_order = false;   // which coordinate permutation the accumulators use

    if (dense) {
        // ---------------- uncompressed tokens: sink then residual window, raw query ----------------
        pdl_wait();        // the scaled query copies come from the prep launch
        uint32_t bq[D / 16][2];
        {
            const __half* qh = p.q_raw + qbase + int64_t(g) * D;
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
            for (int c = lane; c < TILE * (D / 8); c += 32) {
                const int r = c / (D / 8), c8 = c - r * (D / 8);
                const int64_t tok = tok0 + r;
                uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
                if (tok < n_tok) {
                    const bool in_sink = tok < p.sink_len;
                    const int64_t row = in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len);
                    const void* kb = in_sink ? p.sink_k : p.res_k;
                    const void* vb = in_sink ? p.sink_v : p.res_v;
                    const int64_t e = row * D + c8 * 8;
                    if (p.dense_dtype == TQ_F16) {
                        kv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(kb) + e));
                        vv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(vb) + e));
                    } else {
                        __half hk[8], hv[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            hk[i] = __float2half_rn(load_as_f32(kb, p.dense_dtype, e + i));
                            hv[i] = __float2half_rn(load_as_f32(vb, p.dense_dtype, e + i));
                        }
                        kv = *reinterpret_cast<uint4*>(hk);
                        vv = *reinterpret_cast<uint4*>(hv);
                    }
                }
                *reinterpret_cast<uint4*>(Ks + r * LD + c8 * 8) = kv;
                *reinterpret_cast<uint4*>(Vs + r * LD + c8 * 8) = vv;
            }
            __syncwarp();
            tile_from_smem<D>(Ks, Vs, bq, 1.f, 1.f, 1.f, 1.f, tok0 + g < n_tok, tok0 + g + 8 < n_tok, st, lane);
            __syncwarp();
        }
    } else if constexpr (!DIRECT) {
        // ---------------- packed tokens, general path: unpack into shared memory ---------------------
        if (tid < 64) {
            const int which = tid >> 4, k = tid & 15;
            const float* src = which == 0 ? p.kc_hi : which == 1 ? p.kc_lo : which == 2 ? p.vc_hi : p.vc_lo;
            const int bits = which == 0 ? p.kb_hi : which == 1 ? p.kb_lo : which == 2 ? p.vb_hi : p.vb_lo;
            const float sc = which == 2 ? p.v_scale_hi : which == 3 ? p.v_scale_lo : 1.f;
            ctab[tid] = __float2half_rn((src != nullptr && bits > 0 && k < (1 << bits)) ? src[k] * sc : 0.f);
        }
        pdl_wait();        // the rotated query comes from the prep launch
        __syncthreads();
        uint32_t bq[D / 16][2];
        {
            const __half* qh = p.q_rot + qbase + int64_t(g) * D;
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
        uint32_t* T4 = reinterpret_cast<uint32_t*>(smem);               // [256][32]: byte -> half2(c[lo], c[hi])
        uint2* T2 = reinterpret_cast<uint2*>(smem + 32768);             // [256][16]: byte -> 2 x half2 (token pair)
        if (tid < 32) {
            const int which = tid >> 4, k = tid & 15;
            const float* src = which ? p.vc_hi : p.kc_hi;
            ctab[which * 32 + k] = __float2half_rn(k < (which ? 4 : 16) ? src[k] * (which ? p.v_scale_hi : 1.f) : 0.f);
        }
        __syncthreads();
        for (int e = tid; e < 256 * 8; e += NW * 32) {     // 4 replicas per 128-bit store
            const int entry = e >> 3, q4 = e & 7;
            const __half2 h = __halves2half2(ctab[entry & 15], ctab[entry >> 4]);
            const uint32_t v = *reinterpret_cast<const uint32_t*>(&h);
            reinterpret_cast<uint4*>(T4)[entry * 8 + q4] = make_uint4(v, v, v, v);
        }
        for (int e = tid; e < 256 * 8; e += NW * 32) {     // 2 replicas per 128-bit store
            const int entry = e >> 3, q2 = e & 7;
            const int n0 = entry & 15, n1 = entry >> 4;
            const __half2 h0 = __halves2half2(ctab[32 + (n0 & 3)], ctab[32 + (n0 >> 2)]);
            const __half2 h1 = __halves2half2(ctab[32 + (n1 & 3)], ctab[32 + (n1 >> 2)]);
            const uint32_t v0 = *reinterpret_cast<const uint32_t*>(&h0), v1 = *reinterpret_cast<const uint32_t*>(&h1);
            reinterpret_cast<uint4*>(T2)[entry * 8 + q2] = make_uint4(v0, v1, v0, v1);
        }
        pdl_wait();        // the rotated query comes from the prep launch
        __syncthreads();
        // Query fragments in the byte order of the 4-bit rows: thread t owns coordinates [t*D/4, (t+1)*D/4).
        uint32_t bq[D / 16][2];
        {
            const __half* qh = p.q_rot + qbase + int64_t(g) * D + t * (D / 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks) : 0u;
                bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + 4 * ks + 2) : 0u;
            }
        }
        constexpr int KW = D / 2, VW = D / 4;            // bytes per token
        constexpr int KQ = KW / 4 / 4;                   // 32-bit words in a thread's quarter of a key row
        constexpr int VQ = VW / 8 / 4;                   // 32-bit words in a thread's eighth of a value row
        static_assert(KQ >= 1 && VQ >= 1 && KQ % 4 == 0, "direct path needs d a multiple of 128");
        // 32-bit shared-window addresses of this lane's private table columns: entry e of T4 sits at
        // t4 + e*128, entry e of T2 at t2 + e*128 (one IMAD each, no 64-bit address arithmetic).
        const uint32_t t4 = static_cast<uint32_t>(__cvta_generic_to_shared(T4)) + lane * 4;
        const uint32_t t2 = static_cast<uint32_t>(__cvta_generic_to_shared(T2)) + (lane & 15) * 8;
        const int64_t tile_lo = int64_t(split) * p.p_tps;
        const int64_t tile_hi = min(tile_lo + p.p_tps, (p.c_len + TILE - 1) / TILE);
        const int64_t last = p.c_len - 1;
        const uint8_t* kbase = p.k_hi + kvl * p.c_ls * KW + t * (KQ * 4);
        const uint8_t* vbase = p.v_hi + kvl * p.c_ls * VW + g * (VQ * 4);
        const float* knb = p.k_norms + kvl * p.c_ls;
        const float* vnb = p.v_norms + kvl * p.c_ls;

        struct Raw { uint4 k[2][KQ / 4]; uint32_t v[4][VQ]; float n[4]; };
        auto issue_loads = [&](Raw& r, int64_t tok0) {
            if (tok0 + TILE <= p.c_len) {      // whole tile in range: constant offsets from three bases
                const uint8_t* kp = kbase + (tok0 + g) * KW;
                const uint8_t* vp = vbase + (tok0 + 2 * t) * VW;
#pragma unroll
                for (int i = 0; i < KQ / 4; ++i) {
                    r.k[0][i] = __ldg(reinterpret_cast<const uint4*>(kp) + i);
                    r.k[1][i] = __ldg(reinterpret_cast<const uint4*>(kp + 8 * KW) + i);
                }
#pragma unroll
                for (int i = 0; i < VQ; ++i) {
                    r.v[0][i] = __ldg(reinterpret_cast<const uint32_t*>(vp) + i);
                    r.v[1][i] = __ldg(reinterpret_cast<const uint32_t*>(vp + VW) + i);
                    r.v[2][i] = __ldg(reinterpret_cast<const uint32_t*>(vp + 8 * VW) + i);
                    r.v[3][i] = __ldg(reinterpret_cast<const uint32_t*>(vp + 9 * VW) + i);
                }
                r.n[0] = __ldg(knb + tok0 + g); r.n[1] = __ldg(knb + tok0 + g + 8);
                r.n[2] = __ldg(vnb + tok0 + g); r.n[3] = __ldg(vnb + tok0 + g + 8);
            } else {                            // the one ragged tile at the very end: clamp every token index
                const int64_t ta = min(tok0 + g, last), tb = min(tok0 + g + 8, last);
#pragma unroll
                for (int i = 0; i < KQ / 4; ++i) {
                    r.k[0][i] = __ldg(reinterpret_cast<const uint4*>(kbase + ta * KW) + i);
                    r.k[1][i] = __ldg(reinterpret_cast<const uint4*>(kbase + tb * KW) + i);
                }
                const int64_t v0 = min(tok0 + 2 * t, last), v1 = min(tok0 + 2 * t + 1, last);
                const int64_t v2 = min(tok0 + 2 * t + 8, last), v3 = min(tok0 + 2 * t + 9, last);
#pragma unroll
                for (int i = 0; i < VQ; ++i) {
                    r.v[0][i] = __ldg(reinterpret_cast<const uint32_t*>(vbase + v0 * VW) + i);
                    r.v[1][i] = __ldg(reinterpret_cast<const uint32_t*>(vbase + v1 * VW) + i);
                    r.v[2][i] = __ldg(reinterpret_cast<const uint32_t*>(vbase + v2 * VW) + i);
                    r.v[3][i] = __ldg(reinterpret_cast<const uint32_t*>(vbase + v3 * VW) + i);
                }
                r.n[0] = __ldg(knb + ta); r.n[1] = __ldg(knb + tb); r.n[2] = __ldg(vnb + ta); r.n[3] = __ldg(vnb + tb);
            }
        };
        auto compute = [&](const Raw& r, int64_t tok0) {
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                // bytes 2ks, 2ks+1 of this thread's quarter row, for tokens g and g+8
                const uint4& q0 = r.k[0][ks >> 3];
                const uint4& q1 = r.k[1][ks >> 3];
                const int wi = (ks >> 1) & 3;
                const uint32_t w0 = wi == 0 ? q0.x : wi == 1 ? q0.y : wi == 2 ? q0.z : q0.w;
                const uint32_t w1 = wi == 0 ? q1.x : wi == 1 ? q1.y : wi == 2 ? q1.z : q1.w;
                const int b0 = (ks & 1) * 2;
                const uint32_t a0 = lds32(__byte_perm(w0, 0, 0x4440 | b0) * 128u + t4);
                const uint32_t a1 = lds32(__byte_perm(w1, 0, 0x4440 | b0) * 128u + t4);
                const uint32_t a2 = lds32(__byte_perm(w0, 0, 0x4440 | (b0 + 1)) * 128u + t4);
                const uint32_t a3 = lds32(__byte_perm(w1, 0, 0x4440 | (b0 + 1)) * 128u + t4);
                mma16816(s, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
            }
            uint32_t bp[2];
            softmax_step<D>(s, r.n[0], r.n[1], r.n[2], r.n[3], tok0 + g < p.c_len, tok0 + g + 8 < p.c_len, st, bp);
#pragma unroll
            for (int i = 0; i < VQ; ++i) {
                // interleave the 2-bit codes of a token pair: nibble k of X = (A code 2k) | (B code 2k) << 2
                const uint32_t x0 = (r.v[0][i] & 0x33333333u) | ((r.v[1][i] << 2) & 0xCCCCCCCCu);
                const uint32_t y0 = ((r.v[0][i] >> 2) & 0x33333333u) | (r.v[1][i] & 0xCCCCCCCCu);
                const uint32_t x1 = (r.v[2][i] & 0x33333333u) | ((r.v[3][i] << 2) & 0xCCCCCCCCu);
                const uint32_t y1 = ((r.v[2][i] >> 2) & 0x33333333u) | (r.v[3][i] & 0xCCCCCCCCu);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint2 fa = lds64(__byte_perm(x0, 0, 0x4440 | k) * 128u + t2);   // rows g,   tokens 2t,2t+1   -> m-tiles 2k, 2k+1
                    const uint2 fb = lds64(__byte_perm(y0, 0, 0x4440 | k) * 128u + t2);   // rows g+8
                    const uint2 fc = lds64(__byte_perm(x1, 0, 0x4440 | k) * 128u + t2);   // rows g,   tokens 2t+8,2t+9
                    const uint2 fd = lds64(__byte_perm(y1, 0, 0x4440 | k) * 128u + t2);
                    const int mt = i * 8 + 2 * k;
                    mma16816(st.o[mt], fa.x, fb.x, fc.x, fd.x, bp[0], bp[1]);
                    mma16816(st.o[mt + 1], fa.y, fb.y, fc.y, fd.y, bp[0], bp[1]);
                }
            }
        };
        // two register buffers, loads for the next tile in flight while the current one is computed
        Raw ra, rb;
        int64_t tile = tile_lo + warp;
        if (tile < tile_hi) issue_loads(ra, tile * TILE);
        while (tile < tile_hi) {
            if (tile + NW < tile_hi) issue_loads(rb, (tile + NW) * TILE);
            compute(ra, tile * TILE);
            tile += NW;
            if (tile >= tile_hi) break;
            if (tile + NW < tile_hi) issue_loads(ra, (tile + NW) * TILE);
            compute(rb, tile * TILE);
            tile += NW;
        }
    }

    // ---------------- CTA reduction over warps, then one partial per head to the workspace ---------------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
    }
    __syncthreads();   // staging / tables are dead from here on
    float* red = reinterpret_cast<float*>(smem);
    float* ro = red + size_t(warp) * (D * HPG + 2 * HPG);   // [D][8]
    float* rm = ro + D * HPG;                               // [8] max, [8] sum
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) {
        int c0, c1;
        if (direct_order) { c0 = g * (D / 8) + 2 * mt; c1 = c0 + 1; }
        else { c0 = mt * 16 + g; c1 = c0 + 8; }
        *reinterpret_cast<float2*>(ro + c0 * HPG + 2 * t) = make_float2(st.o[mt][0], st.o[mt][1]);
        *reinterpret_cast<float2*>(ro + c1 * HPG + 2 * t) = make_float2(st.o[mt][2], st.o[mt][3]);
    }
    if (g == 0) {
        rm[2 * t] = st.m[0]; rm[2 * t + 1] = st.m[1];
        rm[HPG + 2 * t] = st.l[0]; rm[HPG + 2 * t + 1] = st.l[1];
    }
    __syncthreads();
    const int64_t pidx = ((kvl * p.HG + hg) * (p.n_ps + p.n_ds) + split);
    float* po = p.part_o + pidx * (int64_t(p.slots) * D);
    float* pml = p.part_ml + pidx * (p.slots * 2);
    for (int e = tid; e < D * HPG; e += NW * 32) {
        const int h = e / D, c = e - h * D;           // output layout [head][coordinate]
        if (h >= heads_here) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, red[size_t(w) * (D * HPG + 2 * HPG) + D * HPG + h]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float* rw = red + size_t(w) * (D * HPG + 2 * HPG);
            const float mw = rw[D * HPG + h];
            const float f = (mw == -INFINITY) ? 0.f : ex2(mw - M);
            acc = fmaf(f, rw[c * HPG + h], acc);
            L = fmaf(f, rw[D * HPG + HPG + h], L);
        }
        po[h * D + c] = acc;
        if (c == 0) { pml[2 * h] = M; pml[2 * h + 1] = L; }
    }
}

// grid (Hq, B), 256 threads: merge the splits of one query head and undo the rotation once.
// Three short phases, each a single round of independent loads: (1) split weights from the per-split
// (max, sum) pairs, (2) weighted sum of the partial accumulators over splits, (3) the d x d product with R.
constexpr int MERGE_T = 256, MAX_SPLITS = 512;
__global__ void __launch_bounds__(MERGE_T) decode_merge_kernel(DecodeParams p) {
    __shared__ float s_w[MAX_SPLITS];
    __shared__ float s_part[4][256];   // partial sums per thread group
    __shared__ float s_rot[256], s_raw[256];
    __shared__ float s_inv;
    pdl_wait();        // partial accumulators come from the launch just before this one
    pdl_trigger();
    const int h = blockIdx.x, b = blockIdx.y, d = p.D, tid = threadIdx.x;
    const int hkv = h / p.G, hl = h - hkv * p.G, hg = hl / HPG, hs = hl - hg * HPG;
    const int S = p.n_ps + p.n_ds, SL = p.slots;
    const int64_t base = ((int64_t(b) * p.Hkv + hkv) * p.HG + hg) * S;
    // (1) warp 0: weights exp2(m_s - M) and the normaliser
    if (tid < 32) {
        float mloc[MAX_SPLITS / 32], lloc[MAX_SPLITS / 32];
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            const int sidx = tid + 32 * i;
            mloc[i] = -INFINITY; lloc[i] = 0.f;
            if (sidx < S) {
                const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + ((base + sidx) * SL + hs) * 2);
                mloc[i] = ml.x; lloc[i] = ml.y;
            }
            M = fmaxf(M, mloc[i]);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_SPLITS / 32; ++i) {
            const int sidx = tid + 32 * i;
            const float w = (mloc[i] == -INFINITY) ? 0.f : ex2(mloc[i] - M);
            if (sidx < S) s_w[sidx] = w;
            L = fmaf(w, lloc[i], L);
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        if (tid == 0) s_inv = 1.f / L;
    }
    __syncthreads();
    // (2) thread (c, part): sum over the splits congruent to `part`
    const int JW = d >= 128 ? 128 : d, parts = MERGE_T / JW;
    const int part = tid / JW, cj = tid - part * JW;
    for (int c = cj; c < d; c += JW) {
        float rot = 0.f, raw = 0.f;
        if (part < parts) {
#pragma unroll 4
            for (int sidx = part; sidx < p.n_ps; sidx += parts) rot = fmaf(s_w[sidx], p.part_o[((base + sidx) * SL + hs) * d + c], rot);
            for (int sidx = p.n_ps + part; sidx < S; sidx += parts) raw = fmaf(s_w[sidx], p.part_o[((base + sidx) * SL + hs) * d + c], raw);
        }
        __syncthreads();
        if (part < parts) { s_part[part][c] = rot; }
        __syncthreads();
        if (part == 0) {
            float v = 0.f;
            for (int q = 0; q < parts; ++q) v += s_part[q][c];
            const int v_half = p.vb_lo ? d / 2 : d;
            s_rot[c] = v / (c < v_half ? p.v_scale_hi : p.v_scale_lo);
        }
        __syncthreads();
        if (part < parts) { s_part[part][c] = raw; }
        __syncthreads();
        if (part == 0) {
            float v = 0.f;
            for (int q = 0; q < parts; ++q) v += s_part[q][c];
            s_raw[c] = v;
        }
    }
    __syncthreads();
    // (3) thread (j, part): rows [part*d/parts, (part+1)*d/parts) of R, column j  (y @ R, rotation.py:68-78)
    for (int j = cj; j < d; j += JW) {
        float r = 0.f;
        if (part < parts) {
            const int c0 = part * (d / parts), c1 = c0 + d / parts;
#pragma unroll 8
            for (int c = c0; c < c1; ++c) r = fmaf(s_rot[c], __ldg(p.rot + int64_t(c) * d + j), r);
        }
        __syncthreads();
        if (part < parts) s_part[part][j] = r;
        __syncthreads();
        if (part == 0) {
            float v = s_raw[j];
            for (int q = 0; q < parts; ++q) v += s_part[q][j];
            store_from_f32(p.out, p.out_dtype, (int64_t(b) * p.Hq + h) * d + j, v * s_inv);
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------
static int g_tune_ctas_per_sm = 2;     // CTAs the partial kernel keeps resident per SM (split heuristic)
static int g_tune_force_general = 0;   // 1: never take the direct path (testing)
static int g_tune_splits = 0;          // > 0: fixed number of packed splits
static int g_tune_pdl = 1;             // programmatic dependent launch between the three kernels

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

static SplitPlan plan_splits(int batch, int n_q_heads, int n_kv_heads, int64_t c_len, int64_t dense_len, int sms) {
    SplitPlan s{};
    const int G = n_q_heads / n_kv_heads;
    s.hg = (G + HPG - 1) / HPG;
    const int64_t lanes = int64_t(batch) * n_kv_heads * s.hg;
    const int64_t p_tiles = (c_len + TILE - 1) / TILE, d_tiles = (dense_len + TILE - 1) / TILE;
    if (d_tiles > 0) {
        s.d_tps = 2 * NW;   // two tiles per warp
        s.n_ds = int((d_tiles + s.d_tps - 1) / s.d_tps);
        if (s.n_ds > 64) { s.d_tps = (d_tiles + 63) / 64; s.n_ds = int((d_tiles + s.d_tps - 1) / s.d_tps); }
    }
    if (p_tiles > 0) {
        // all CTAs of the grid resident at once: (packed + dense splits) * lanes <= SMs * CTAs per SM
        const int64_t slots = int64_t(sms) * g_tune_ctas_per_sm;
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

struct WsLayout { size_t q_rot, q_raw, part_o, part_ml, total; };

static WsLayout ws_layout(int batch, int n_q_heads, int n_kv_heads, int d, const SplitPlan& s) {
    WsLayout w{};
    const size_t qn = size_t(batch) * n_q_heads * d * sizeof(__half);
    const size_t parts = size_t(batch) * n_kv_heads * s.hg * size_t(s.n_ps + s.n_ds);
    const size_t slots = size_t(std::min(n_q_heads / n_kv_heads, HPG));
    w.q_rot = 0;
    w.q_raw = align_up(w.q_rot + qn, 256);
    w.part_o = align_up(w.q_raw + qn, 256);
    w.part_ml = align_up(w.part_o + parts * slots * d * sizeof(float), 256);
    w.total = align_up(w.part_ml + parts * slots * 2 * sizeof(float), 256);
    return w;
}

// Launch with programmatic stream serialisation: the kernel may become resident before its predecessor
// on the stream has finished; every kernel here calls griddepcontrol.wait before touching dependent data.
template <typename K> static int launch_pdl(K kernel, dim3 grid, unsigned block, size_t smem, cudaStream_t s,
                                            const DecodeParams& p, const char* what) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_tune_pdl ? 1 : 0;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return TQ_OK;
}

template <int D, bool DIRECT> static int launch_partial(const DecodeParams& p, cudaStream_t s) {
    constexpr size_t smem = partial_smem<D, DIRECT>();
    static bool set[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_partial_kernel<D, DIRECT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev] = true;
    }
    dim3 grid(unsigned(p.n_ps + p.n_ds), unsigned(p.Hkv * p.HG), unsigned(p.B));
    return launch_pdl(decode_partial_kernel<D, DIRECT>, grid, NW * 32, smem, s, p, "tq_decode_attn (partial)");
}

}  // namespace tq

using namespace tq;

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
    // Same split plan tq_decode_attn will use for these sizes (and the current tuning values).
    const SplitPlan s = plan_splits(batch, n_q_heads, n_kv_heads, c_len, dense_len, sm_count());
    return ws_layout(batch, n_q_heads, n_kv_heads, d, s).total;
}

extern "C" int tq_decode_attn(const tq_decode_args* a, void* stream) {
    if (!a) return fail(TQ_ERR_INVALID, "tq_decode_attn: null args");
    const int d = a->d;
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: batch=%d q_heads=%d kv_heads=%d", a->batch, a->n_q_heads, a->n_kv_heads);
    if (d != 64 && d != 96 && d != 128 && d != 256) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: d=%d (64, 96, 128 or 256)", d);
    if (a->c_len < 0 || a->sink_len < 0 || a->res_len < 0 || a->c_len + a->sink_len + a->res_len == 0)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: the cache holds no tokens");
    if (!a->q || !a->rot || !a->out || !a->workspace) return fail(TQ_ERR_INVALID, "tq_decode_attn: null pointer");
    if (a->q_dtype < 0 || a->q_dtype > 2 || a->out_dtype < 0 || a->out_dtype > 2 || a->dense_dtype < 0 || a->dense_dtype > 2)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: bad dtype");
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
    if (!aligned(a->workspace, 256)) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace must be 256-byte aligned");

    const int64_t dense_len = a->sink_len + a->res_len;
    const SplitPlan sp = plan_splits(a->batch, a->n_q_heads, a->n_kv_heads, a->c_len, dense_len, sm_count());
    const WsLayout wl = ws_layout(a->batch, a->n_q_heads, a->n_kv_heads, d, sp);
    if (wl.total > a->workspace_bytes) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace %zu B < %zu B", a->workspace_bytes, wl.total);
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
    unsigned char* ws = static_cast<unsigned char*>(a->workspace);
    p.q_rot = reinterpret_cast<__half*>(ws + wl.q_rot); p.q_raw = reinterpret_cast<__half*>(ws + wl.q_raw);
    p.part_o = reinterpret_cast<float*>(ws + wl.part_o); p.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
    p.out = a->out; p.out_dtype = a->out_dtype;

    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int rc = launch_pdl(decode_prep_kernel, dim3(unsigned(p.B * p.Hq)), unsigned(d), 0, s, p, "tq_decode_attn (prep)");
    if (rc) return rc;

    const bool direct = !g_tune_force_general && d == 128 && a->c_len > 0 && a->k_bits_hi == 4 && a->k_bits_lo == 0 &&
                        a->v_bits_hi == 2 && a->v_bits_lo == 0 && aligned(a->k_hi, 16) && aligned(a->v_hi, 16);
    if (direct) rc = launch_partial<128, true>(p, s);
    else if (d == 64) rc = launch_partial<64, false>(p, s);
    else if (d == 96) rc = launch_partial<96, false>(p, s);
    else if (d == 128) rc = launch_partial<128, false>(p, s);
    else rc = launch_partial<256, false>(p, s);
    if (rc) return rc;

    return launch_pdl(decode_merge_kernel, dim3(unsigned(p.Hq), unsigned(p.B)), MERGE_T, 0, s, p, "tq_decode_attn (merge)");
}
