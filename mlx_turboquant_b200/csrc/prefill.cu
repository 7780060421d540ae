// Causal attention for SEVERAL query tokens per sequence (prefill chunks, multi-token steps) computed directly on the
// compressed KV cache [fp16 sink | packed middle | fp16 recent tokens]: what the reference does as dense reassembly
// (cache.py:674-706) followed by the consumer's masked scaled-dot-product attention, and only sketched for packed keys
// (kernels.py:558-590: T_q up to 32; docs/FUSED_ATTENTION_DESIGN.md:281-283).
//
// The query tokens are the LAST t_q tokens of the cache (the caller appended them first): query i sits at absolute
// position total - t_q + i and sees every cached token up to and including itself.
//
// Grid (query blocks, kv_heads * head_groups, batch), 8 warps per CTA.  A CTA owns 64 "columns": query tokens x the
// query heads of one GQA group (G padded to 1, 2, 4 or 8 columns per token).  It walks the cache in stages of 64 tokens;
// a stage is unpacked (codes -> centroids, fp16) into shared memory ONCE by all warps together and then used by every
// warp for its own 8 columns with the decode kernels' tile step: S[16 tokens x 8 columns] = K_tile . Q^T
// (mma.sync.m16n8k16, fp16 operands, fp32 accumulation), online softmax with per-element causal masks, O^T += V^T . P^T.
// Compared with the decode kernels the unpacking is amortised over 64 columns instead of 8.  Packed tokens are scored
// with the rotated query and accumulated in rotated space; the uncompressed tokens use the raw query and a second
// accumulator; both share the softmax state, and the rotation is undone once at the end.
#include <algorithm>

#include "decode_dev.cuh"

namespace tq {

namespace pf {

constexpr int NW = 8, NT = NW * 32, COLS = NW * 8, STG = 64;      // warps, threads, query columns per CTA, tokens per stage

struct Params {
    DecodeParams c;            // the cache (lengths, packed arrays, norms, centroid tables, uncompressed regions, rotation, scale)
    const void* q; int q_dtype;            // (B, Hq, Tq, D)
    void* out; int out_dtype;              // (B, Hq, Tq, D)
    int Tq;
    int64_t q_pos0;            // absolute position of query token 0
    int GP, QT;                // columns per query token (G padded: 1, 2, 4, 8), query tokens per CTA (COLS / GP)
};

template <int D> __host__ __device__ constexpr size_t smem_bytes() {
    return size_t(COLS) * D * 4 + size_t(COLS) * D * 2 + 2 * size_t(STG) * stage_ld<D>() * 2 + 64 * 2 + 256 * 4 + 256 * 8 + 64;
}

// Softmax step with a mask per element: ok[i] says whether s[i] (token row g / g + 8, column 2t / 2t + 1) takes part.
template <int D, int NZ>
__device__ __forceinline__ void softmax_masked(float (&s)[4], float kn0, float kn1, float vn0, float vn1, const bool (&ok)[4], WarpAcc<D, NZ>& st,
                                               uint32_t (&bp)[2]) {
    s[0] = ok[0] ? s[0] * kn0 : -INFINITY;
    s[1] = ok[1] ? s[1] * kn0 : -INFINITY;
    s[2] = ok[2] ? s[2] * kn1 : -INFINITY;
    s[3] = ok[3] ? s[3] * kn1 : -INFINITY;
    vn0 = (ok[0] || ok[1]) ? vn0 : 0.f;
    vn1 = (ok[2] || ok[3]) ? vn1 : 0.f;
    const float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]), vmax = fmaxf(vn0, vn1);
    if (__any_sync(0xffffffffu, mx0 > st.mt[0] || mx1 > st.mt[1] || vmax > st.vt)) softmax_refresh<D, NZ>(mx0, mx1, vmax, st);
    const float p0 = ex2(s[0] - st.m[0]), p1 = ex2(s[1] - st.m[1]), p2 = ex2(s[2] - st.m[0]), p3 = ex2(s[3] - st.m[1]);
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    const float w0 = vn0 * st.vsc, w1 = vn1 * st.vsc;
    bp[0] = movm_t(pack_h2(p0 * w0, p1 * w0));
    bp[1] = movm_t(pack_h2(p2 * w1, p3 * w1));
}

template <int D>
__global__ void __launch_bounds__(NT, 1) prefill_attn_kernel(Params P) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int LD = stage_ld<D>();
    const DecodeParams& p = P.c;
    float* qf = reinterpret_cast<float*>(smem);                                  // [COLS][D] raw query, float32
    __half* qs = reinterpret_cast<__half*>(qf + COLS * D);                       // [COLS][D] scaled fp16 query (rotated, later raw)
    __half* Ks = qs + COLS * D;                                                  // [STG][LD]
    __half* Vs = Ks + STG * LD;                                                  // [STG][LD]
    __half* ctab = Vs + STG * LD;                                                // kc_hi, kc_lo, vc_hi, vc_lo (16 each)
    uint32_t* t4 = reinterpret_cast<uint32_t*>(ctab + 64);                       // byte of two 4-bit codes -> half2 of key centroids
    uint2* t2 = reinterpret_cast<uint2*>(t4 + 256);                              // byte of four 2-bit codes -> 4 value centroids
    float* scratch = reinterpret_cast<float*>(Ks);                               // the stage doubles as scratch outside the loops

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int tq0 = blockIdx.x * P.QT;                                           // first query token of this CTA
    const int GP = P.GP;
    // column c of the CTA: query token tq0 + c / GP, head (within the group) c % GP
    auto col_valid = [&](int c) { return (c % GP) < heads_here && tq0 + c / GP < P.Tq; };
    auto col_q_index = [&](int c) -> int64_t {                                   // element offset of the column's query / output row
        const int h = hkv * p.G + hg * HPG + (c % GP);
        return ((int64_t(b) * p.Hq + h) * P.Tq + (tq0 + c / GP)) * D;
    };

    // ---------------- constants, query block ------------------------------------------------------------------
    if (tid < 64) {
        const int which = tid >> 4, k = tid & 15;
        const float* src = which == 0 ? p.kc_hi : which == 1 ? p.kc_lo : which == 2 ? p.vc_hi : p.vc_lo;
        const int bits = which == 0 ? p.kb_hi : which == 1 ? p.kb_lo : which == 2 ? p.vb_hi : p.vb_lo;
        const float sc = which == 2 ? p.v_scale_hi : which == 3 ? p.v_scale_lo : 1.f;     // value tables: fp16 under a table-wide scale, divided out at the end
        ctab[tid] = __float2half_rn((src != nullptr && bits > 0 && k < (1 << bits)) ? src[k] * sc : 0.f);
    }
    for (int e = tid; e < COLS * D; e += NT) {
        const int c = e / D, k = e - c * D;
        qf[e] = col_valid(c) ? load_as_f32(P.q, P.q_dtype, col_q_index(c) + k) : 0.f;
    }
    __syncthreads();
    const bool fast_k = p.kb_hi == 4 && p.kb_lo == 0 && p.words_ok, fast_v = p.vb_hi == 2 && p.vb_lo == 0 && p.words_ok;
    if (fast_k || fast_v) {
        for (int e = tid; e < 256; e += NT) {
            const __half2 hk = __halves2half2(ctab[e & 15], ctab[e >> 4]);
            t4[e] = *reinterpret_cast<const uint32_t*>(&hk);
            const __half2 v01 = __halves2half2(ctab[32 + (e & 3)], ctab[32 + ((e >> 2) & 3)]);
            const __half2 v23 = __halves2half2(ctab[32 + ((e >> 4) & 3)], ctab[32 + (e >> 6)]);
            t2[e] = make_uint2(*reinterpret_cast<const uint32_t*>(&v01), *reinterpret_cast<const uint32_t*>(&v23));
        }
    }
    const float f = p.scale * LOG2E;
    // q_rot[c][j] = sum_k q[c][k] R[j][k] (rotation.py:81-110): 32 rows of R at a time through shared memory; thread = (row j
    // of the slab, 8 columns)
    {
        constexpr int RS = D + 1;
        const int jl = tid & 31, cg = tid >> 5;
        for (int j0 = 0; j0 < D; j0 += 32) {
            __syncthreads();
            for (int e = tid; e < 32 * D; e += NT) {
                const int r = e / D, k = e - r * D;
                scratch[r * RS + k] = __ldg(p.rot + int64_t(j0 + r) * D + k);
            }
            __syncthreads();
            float acc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] = 0.f;
            for (int k = 0; k < D; ++k) {
                const float r = scratch[jl * RS + k];
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[u] = fmaf(qf[(cg * 8 + u) * D + k], r, acc[u]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) qs[(cg * 8 + u) * D + j0 + jl] = __float2half_rn(acc[u] * f);
        }
    }
    __syncthreads();

    // this warp's columns: 8 warp + (0..7); this lane's two: 8 warp + 2t, + 1
    const int c0 = warp * 8 + 2 * t;
    // absolute positions this lane's columns may look at (everything at or before the query token); -1: not a column
    const int64_t qp0 = col_valid(c0) ? P.q_pos0 + tq0 + c0 / GP : -1, qp1 = col_valid(c0 + 1) ? P.q_pos0 + tq0 + (c0 + 1) / GP : -1;
    int64_t wq_max = max(qp0, qp1);                                              // the latest position any column of this warp sees
#pragma unroll
    for (int off = 1; off < 4; off <<= 1) wq_max = max(wq_max, __shfl_xor_sync(0xffffffffu, wq_max, off));
    const int64_t cta_q_max = P.q_pos0 + min(tq0 + P.QT, P.Tq) - 1;              // the latest position any column of the CTA sees

    constexpr int NZ = D / 16;
    WarpAcc<D, NZ> st;          // o: packed tokens (rotated space), z: uncompressed tokens
    st.init();
    uint32_t bq[D / 16][2];
    auto load_bq = [&]() {
        const __half* qh = qs + (warp * 8 + g) * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            bq[ks][0] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t);
            bq[ks][1] = *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8);
        }
    };
    load_bq();

    // One 16-token sub-tile of the stage for this warp: scores, masked softmax, values into acc (o or z).
    // pos0: absolute position of the sub-tile's first token; n_ok: tokens of the sub-tile inside the region.
    auto sub_tile = [&](int mt, int64_t pos0, int n_ok, float kn0, float kn1, float vn0, float vn1, float (&acc)[D / 16][4]) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const __half* base = Ks + (mt * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4];
                ldsm_x4(a, base + ks * 16);
                mma16816(s, a[0], a[1], a[2], a[3], bq[ks][0], bq[ks][1]);
            }
        }
        const bool r0 = g < n_ok, r1 = g + 8 < n_ok;
        const bool ok[4] = {r0 && pos0 + g <= qp0, r0 && pos0 + g <= qp1, r1 && pos0 + g + 8 <= qp0, r1 && pos0 + g + 8 <= qp1};
        uint32_t bp[2];
        softmax_masked<D, NZ>(s, kn0, kn1, vn0, vn1, ok, st, bp);
        {
            const __half* base = Vs + (mt * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
            for (int m = 0; m < D / 16; ++m) {
                uint32_t a[4];
                ldsm_x4_t(a, base + m * 16);
                mma16816(acc[m], a[0], a[1], a[2], a[3], bp[0], bp[1]);
            }
        }
    };

    // ---------------- packed tokens: absolute positions sink_len .. sink_len + c_len - 1 ----------------------------
    {
        const int64_t vis = min(p.c_len, cta_q_max - p.sink_len + 1);   // packed tokens some column of the CTA sees
        const int k_half = p.kb_lo ? D / 2 : D, v_half = p.vb_lo ? D / 2 : D;
        const int kw_hi = packed_bytes(k_half, p.kb_hi), kw_lo = p.kb_lo ? packed_bytes(D - k_half, p.kb_lo) : 0;
        const int vw_hi = packed_bytes(v_half, p.vb_hi), vw_lo = p.vb_lo ? packed_bytes(D - v_half, p.vb_lo) : 0;
        for (int64_t tok0 = 0; tok0 < vis; tok0 += STG) {
            __syncthreads();                                                     // the previous stage has been read
            const int rows = int(min(int64_t(STG), p.c_len - tok0));
            // ---- unpack the stage: whole 32-bit words through byte tables for 4-bit keys / 2-bit values, code by code otherwise
            if (fast_k) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.k_hi + (kvl * p.c_ls + tok0) * (D / 2));
                for (int i = tid; i < STG * (D / 2) / 4; i += NT) {
                    const int r = (4 * i) / (D / 2), cb = 4 * i - r * (D / 2);
                    const uint32_t w = r < rows ? __ldg(src + i) : 0u;
                    uint4 o;
                    o.x = t4[w & 255u]; o.y = t4[(w >> 8) & 255u]; o.z = t4[(w >> 16) & 255u]; o.w = t4[w >> 24];
                    *reinterpret_cast<uint4*>(Ks + r * LD + 2 * cb) = o;
                }
            }
            if (fast_v) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.v_hi + (kvl * p.c_ls + tok0) * (D / 4));
                for (int i = tid; i < STG * (D / 4) / 4; i += NT) {
                    const int r = (4 * i) / (D / 4), cb = 4 * i - r * (D / 4);
                    const uint32_t w = r < rows ? __ldg(src + i) : 0u;
                    const uint2 a = t2[w & 255u], bb = t2[(w >> 8) & 255u], cc = t2[(w >> 16) & 255u], ee = t2[w >> 24];
                    *reinterpret_cast<uint4*>(Vs + r * LD + 4 * cb) = make_uint4(a.x, a.y, bb.x, bb.y);
                    *reinterpret_cast<uint4*>(Vs + r * LD + 4 * cb + 8) = make_uint4(cc.x, cc.y, ee.x, ee.y);
                }
            }
            if (!fast_k || !fast_v) {
                for (int e = tid; e < STG * (D / 2); e += NT) {
                    const int r = e / (D / 2), j = 2 * (e - r * (D / 2));
                    const bool live = r < rows;
                    const int64_t row = kvl * p.c_ls + (live ? tok0 + r : 0);
                    __half2 kk = __float2half2_rn(0.f), vv = kk;
                    if (live) {
                        if (!fast_k) {
                            const uint8_t* kr_hi = p.k_hi + row * kw_hi;
                            const uint8_t* kr_lo = p.kb_lo ? p.k_lo + row * kw_lo : nullptr;
                            const __half k0 = j < k_half ? ctab[code_at(kr_hi, j, p.kb_hi)] : ctab[16 + code_at(kr_lo, j - k_half, p.kb_lo)];
                            const __half k1 = j + 1 < k_half ? ctab[code_at(kr_hi, j + 1, p.kb_hi)] : ctab[16 + code_at(kr_lo, j + 1 - k_half, p.kb_lo)];
                            kk = __halves2half2(k0, k1);
                        }
                        if (!fast_v) {
                            const uint8_t* vr_hi = p.v_hi + row * vw_hi;
                            const uint8_t* vr_lo = p.vb_lo ? p.v_lo + row * vw_lo : nullptr;
                            const __half v0 = j < v_half ? ctab[32 + code_at(vr_hi, j, p.vb_hi)] : ctab[48 + code_at(vr_lo, j - v_half, p.vb_lo)];
                            const __half v1 = j + 1 < v_half ? ctab[32 + code_at(vr_hi, j + 1, p.vb_hi)] : ctab[48 + code_at(vr_lo, j + 1 - v_half, p.vb_lo)];
                            vv = __halves2half2(v0, v1);
                        }
                    }
                    if (!fast_k) *reinterpret_cast<__half2*>(Ks + r * LD + j) = kk;
                    if (!fast_v) *reinterpret_cast<__half2*>(Vs + r * LD + j) = vv;
                }
            }
            __syncthreads();
#pragma unroll 1
            for (int mt = 0; mt < STG / 16; ++mt) {
                const int64_t t0 = tok0 + mt * 16, pos0 = p.sink_len + t0;
                if (t0 >= p.c_len || pos0 > wq_max) break;                       // past the cache, or nothing this warp's columns see
                const int n_ok = int(min(int64_t(16), p.c_len - t0));
                const int64_t n0 = kvl * p.c_ls + t0 + (g < n_ok ? g : 0), n1 = kvl * p.c_ls + t0 + (g + 8 < n_ok ? g + 8 : 0);
                sub_tile(mt, pos0, n_ok, __ldg(p.k_norms + n0), __ldg(p.k_norms + n1), __ldg(p.v_norms + n0), __ldg(p.v_norms + n1), st.o);
            }
        }
    }

    // ---------------- uncompressed tokens: sink (positions 0 ..), recent (positions sink_len + c_len ..), raw query ----------------
    __syncthreads();
    for (int e = tid; e < COLS * D; e += NT) qs[e] = __float2half_rn(qf[e] * f);
    __syncthreads();
    load_bq();
    {
        const int64_t n_dense = p.sink_len + p.res_len;
        for (int64_t tok0 = 0; tok0 < n_dense; tok0 += STG) {
            __syncthreads();
            // stage 64 tokens as fp16; float32 / bfloat16 tokens under a per-token power-of-two scale (largest magnitude into
            // [2^7, 2^8)) whose inverse goes where the packed tokens have their norms
            float* sck = reinterpret_cast<float*>(t2);                           // [STG] key scales, [STG] value scales (the tables are dead)
            float* scv = sck + STG;
            // lanes (r, quarter): 4 lanes per token row
            {
                const int r = tid >> 2, qd = tid & 3;
                const int64_t tok = tok0 + r;
                float mk = 0.f, mv = 0.f;
                const bool live = tok < n_dense;
                const bool in_sink = tok < p.sink_len;
                const int64_t e0 = live ? (in_sink ? kvl * p.sink_ls + tok : kvl * p.res_ls + (tok - p.sink_len)) * D + qd * (D / 4) : 0;
                const void* kb = in_sink ? p.sink_k : p.res_k;
                const void* vb = in_sink ? p.sink_v : p.res_v;
                if (live && p.dense_dtype != TQ_F16) {
                    for (int i = 0; i < D / 4; ++i) {
                        mk = fmaxf(mk, fabsf(load_as_f32(kb, p.dense_dtype, e0 + i)));
                        mv = fmaxf(mv, fabsf(load_as_f32(vb, p.dense_dtype, e0 + i)));
                    }
                }
                mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, 1)); mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, 2));
                mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, 1)); mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, 2));
                const int ek = (__float_as_int(mk) >> 23) & 0xff, ev = (__float_as_int(mv) >> 23) & 0xff;
                const float fk = (ek >= 16 && ek <= 240) ? __int_as_float((261 - ek) << 23) : 1.f;
                const float fv = (ev >= 16 && ev <= 240) ? __int_as_float((261 - ev) << 23) : 1.f;
                if (qd == 0) { sck[r] = 1.f / fk; scv[r] = 1.f / fv; }
                for (int i = 0; i < D / 4; i += 2) {
                    __half2 kk = __float2half2_rn(0.f), vv = kk;
                    if (live) {
                        kk = __floats2half2_rn(load_as_f32(kb, p.dense_dtype, e0 + i) * fk, load_as_f32(kb, p.dense_dtype, e0 + i + 1) * fk);
                        vv = __floats2half2_rn(load_as_f32(vb, p.dense_dtype, e0 + i) * fv, load_as_f32(vb, p.dense_dtype, e0 + i + 1) * fv);
                    }
                    *reinterpret_cast<__half2*>(Ks + r * LD + qd * (D / 4) + i) = kk;
                    *reinterpret_cast<__half2*>(Vs + r * LD + qd * (D / 4) + i) = vv;
                }
            }
            __syncthreads();
#pragma unroll 1
            for (int mt = 0; mt < STG / 16; ++mt) {
                const int64_t t0 = tok0 + mt * 16;
                if (t0 >= n_dense) break;
                const int n_ok = int(min(int64_t(16), n_dense - t0));
                // a sub-tile may straddle the sink / recent boundary: positions are per token
                const int64_t ta = t0 + g, tb = t0 + g + 8;
                const int64_t pa = ta < p.sink_len ? ta : p.c_len + ta, pb = tb < p.sink_len ? tb : p.c_len + tb;
                if ((t0 < p.sink_len ? t0 : p.c_len + t0) > wq_max) break;       // positions only grow from here on: nothing left this warp's columns see
                float s[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const __half* base = Ks + (mt * 16 + (lane & 15)) * LD + (lane >> 4) * 8;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        uint32_t a[4];
                        ldsm_x4(a, base + ks * 16);
                        mma16816(s, a[0], a[1], a[2], a[3], bq[ks][0], bq[ks][1]);
                    }
                }
                const bool r0 = g < n_ok, r1 = g + 8 < n_ok;
                const bool ok[4] = {r0 && pa <= qp0, r0 && pa <= qp1, r1 && pb <= qp0, r1 && pb <= qp1};
                uint32_t bp[2];
                softmax_masked<D, NZ>(s, sck[mt * 16 + g], sck[mt * 16 + g + 8], scv[mt * 16 + g], scv[mt * 16 + g + 8], ok, st, bp);
                {
                    const __half* base = Vs + (mt * 16 + (lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int m = 0; m < D / 16; ++m) {
                        uint32_t a[4];
                        ldsm_x4_t(a, base + m * 16);
                        mma16816(st.z[m], a[0], a[1], a[2], a[3], bp[0], bp[1]);
                    }
                }
            }
        }
    }

    // ---------------- finish: undo the value scale and the rotation of the packed part, normalise, store ----------------
    st.finish();
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
    }
    __syncthreads();                                                             // the stage is dead: it becomes [COLS][D] floats
    {
        // rotated-space sums of the packed part, column-major into scratch (rows mt * 16 + g, + 8; columns 2t, 2t + 1)
        float* so = qf;                                                          // the raw query is dead too: [COLS][D] result of the dense part
        const int cA = warp * 8 + 2 * t;
#pragma unroll
        for (int m = 0; m < D / 16; ++m) {
            const int j = m * 16 + g;
            const int v_half = p.vb_lo ? D / 2 : D;
            const float i0 = 1.f / (j < v_half ? p.v_scale_hi : p.v_scale_lo), i1 = 1.f / (j + 8 < v_half ? p.v_scale_hi : p.v_scale_lo);
            scratch[cA * D + j] = st.o[m][0] * i0; scratch[(cA + 1) * D + j] = st.o[m][1] * i0;
            scratch[cA * D + j + 8] = st.o[m][2] * i1; scratch[(cA + 1) * D + j + 8] = st.o[m][3] * i1;
            so[cA * D + j] = st.z[m][0]; so[(cA + 1) * D + j] = st.z[m][1];
            so[cA * D + j + 8] = st.z[m][2]; so[(cA + 1) * D + j + 8] = st.z[m][3];
        }
        float* sl = reinterpret_cast<float*>(t4);                                // [COLS] softmax denominators
        if (g == 0) { sl[cA] = st.l[0]; sl[cA + 1] = st.l[1]; }
    }
    __syncthreads();
    {
        // out[c][j] = (sum_k acc_p[c][k] R[k][j] + acc_d[c][j]) / l[c]  (y @ R, rotation.py:68-78): the warp's 8 columns, lane -> j = lane + 32 i
        const float* so = qf;
        const float* sl = reinterpret_cast<const float*>(t4);
        float acc[8][D / 32];
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int i = 0; i < D / 32; ++i) acc[u][i] = 0.f;
        if (p.c_len > 0) {
            for (int k = 0; k < D; ++k) {
                float r[D / 32];
#pragma unroll
                for (int i = 0; i < D / 32; ++i) r[i] = __ldg(p.rot + int64_t(k) * D + lane + 32 * i);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const float a = scratch[(warp * 8 + u) * D + k];
#pragma unroll
                    for (int i = 0; i < D / 32; ++i) acc[u][i] = fmaf(a, r[i], acc[u][i]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int c = warp * 8 + u;
            if (!col_valid(c)) continue;
            const float il = 1.f / sl[c];
            const int64_t o = col_q_index(c);
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                const int j = lane + 32 * i;
                store_from_f32(P.out, P.out_dtype, o + j, (acc[u][i] + so[c * D + j]) * il);
            }
        }
    }
}

template <int D> static int launch(const Params& P, cudaStream_t s) {
    constexpr size_t smem = smem_bytes<D>();
    static bool set[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_prefill_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev] = true;
    }
    const dim3 grid(unsigned((P.Tq + P.QT - 1) / P.QT), unsigned(P.c.Hkv * P.c.HG), unsigned(P.c.B));
    prefill_attn_kernel<D><<<grid, NT, smem, s>>>(P);
    return check_launch("tq_prefill_attn");
}

}  // namespace pf

}  // namespace tq

namespace tq {
// prefill_tc.cu: the tensor-core kernel for head_dim 128 with 4-bit keys and 2-bit values
bool prefill_tc_applicable(const tq_decode_args* a, int t_q);
int launch_prefill_tc(const DecodeParams& c, const void* q, int q_dtype, void* out, int out_dtype, int t_q, int64_t q_pos0, cudaStream_t s);
int g_tune_prefill_tc = 1;     // 0: always the mma.sync kernel (testing)
}  // namespace tq

using namespace tq;

extern "C" int tq_prefill_attn(const tq_decode_args* a, int t_q, void* stream) {
    if (!a) return fail(TQ_ERR_INVALID, "tq_prefill_attn: null args");
    const int d = a->d;
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads || t_q <= 0)
        return fail(TQ_ERR_INVALID, "tq_prefill_attn: batch=%d q_heads=%d kv_heads=%d t_q=%d", a->batch, a->n_q_heads, a->n_kv_heads, t_q);
    if (d != 64 && d != 96 && d != 128 && d != 256) return fail(TQ_ERR_UNSUPPORTED, "tq_prefill_attn: d=%d (64, 96, 128 or 256)", d);
    const int64_t total = a->c_len + a->sink_len + a->res_len;
    if (a->c_len < 0 || a->sink_len < 0 || a->res_len < 0 || total < t_q)
        return fail(TQ_ERR_INVALID, "tq_prefill_attn: the cache holds %lld tokens, fewer than the %d query tokens", (long long)total, t_q);
    if (!a->q || !a->rot || !a->out) return fail(TQ_ERR_INVALID, "tq_prefill_attn: null pointer");
    if (a->gather) return fail(TQ_ERR_UNSUPPORTED, "tq_prefill_attn: no fused gather");
    if (a->k_qjl_bits) return fail(TQ_ERR_UNSUPPORTED, "tq_prefill_attn: caches with a QJL sketch take the dense route");
    if (a->q_dtype < 0 || a->q_dtype > 2 || a->out_dtype < 0 || a->out_dtype > 2 || a->dense_dtype < 0 || a->dense_dtype > 2)
        return fail(TQ_ERR_INVALID, "tq_prefill_attn: bad dtype");
    if (a->c_len > 0) {
        if (!bits_ok(a->k_bits_hi) || !bits_ok(a->v_bits_hi) || (a->k_bits_lo && !bits_ok(a->k_bits_lo)) || (a->v_bits_lo && !bits_ok(a->v_bits_lo)))
            return fail(TQ_ERR_INVALID, "Unsupported bit-width. Use 1, 2, 3, or 4.");
        if (!a->k_hi || !a->v_hi || !a->k_norms || !a->v_norms || !a->k_cent_hi || !a->v_cent_hi || (a->k_bits_lo && (!a->k_lo || !a->k_cent_lo)) ||
            (a->v_bits_lo && (!a->v_lo || !a->v_cent_lo)))
            return fail(TQ_ERR_INVALID, "tq_prefill_attn: null packed-cache pointer");
        if (a->c_lane_stride < a->c_len) return fail(TQ_ERR_INVALID, "tq_prefill_attn: c_lane_stride < c_len");
    }
    if ((a->sink_len > 0 && (!a->sink_k || !a->sink_v || a->sink_lane_stride < a->sink_len)) ||
        (a->res_len > 0 && (!a->res_k || !a->res_v || a->res_lane_stride < a->res_len)))
        return fail(TQ_ERR_INVALID, "tq_prefill_attn: bad sink / residual buffers");
    pf::Params P{};
    DecodeParams& p = P.c;
    p.B = a->batch; p.Hq = a->n_q_heads; p.Hkv = a->n_kv_heads; p.G = p.Hq / p.Hkv; p.HG = (p.G + HPG - 1) / HPG; p.D = d;
    p.c_len = a->c_len; p.c_ls = a->c_lane_stride;
    p.kb_hi = a->k_bits_hi; p.kb_lo = a->k_bits_lo; p.vb_hi = a->v_bits_hi; p.vb_lo = a->v_bits_lo;
    p.k_hi = a->k_hi; p.k_lo = a->k_lo; p.v_hi = a->v_hi; p.v_lo = a->v_lo;
    p.k_norms = a->k_norms; p.v_norms = a->v_norms;
    p.kc_hi = a->k_cent_hi; p.kc_lo = a->k_cent_lo; p.vc_hi = a->v_cent_hi; p.vc_lo = a->v_cent_lo;
    p.dense_dtype = a->dense_dtype;
    p.sink_k = a->sink_k; p.sink_v = a->sink_v; p.res_k = a->res_k; p.res_v = a->res_v;
    p.sink_len = a->sink_len; p.sink_ls = a->sink_lane_stride; p.res_len = a->res_len; p.res_ls = a->res_lane_stride;
    p.scale = a->scale; p.rot = a->rot;
    p.v_scale_hi = a->v_cent_scale_hi > 0.f ? a->v_cent_scale_hi : 1.f;
    p.v_scale_lo = a->v_cent_scale_lo > 0.f ? a->v_cent_scale_lo : 1.f;
    p.words_ok = (a->c_len > 0 && aligned(a->k_hi, 4) && aligned(a->v_hi, 4)) ? 1 : 0;
    P.q = a->q; P.q_dtype = a->q_dtype; P.out = a->out; P.out_dtype = a->out_dtype; P.Tq = t_q;
    P.q_pos0 = total - t_q;
    const int gmin = std::min(p.G, HPG);
    P.GP = gmin <= 1 ? 1 : gmin <= 2 ? 2 : gmin <= 4 ? 4 : 8;
    P.QT = pf::COLS / P.GP;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (g_tune_prefill_tc && prefill_tc_applicable(a, t_q)) return launch_prefill_tc(p, a->q, a->q_dtype, a->out, a->out_dtype, t_q, P.q_pos0, s);
    if (d == 64) return pf::launch<64>(P, s);
    if (d == 96) return pf::launch<96>(P, s);
    if (d == 128) return pf::launch<128>(P, s);
    return pf::launch<256>(P, s);
}
