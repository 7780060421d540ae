// One decode step of attention computed directly on the compressed KV cache
// [fp16 sink | packed middle | fp16 residual window], split over the sequence (flash-decode), in ONE launch.
//
// This file: the host side (argument checks, split plan, workspace layout, launch) and the GENERAL kernel, which
// handles every bit width (1-4, fractional splits) and d in {64, 96, 128, 256}.  4-bit keys with 2-bit values at
// d = 128 take the table-lookup kernel of decode_direct.cu instead, and the same widths at d = 96 / 128 (sign sketches
// allowed) the persistent streaming kernel of decode_stream.cu once every warp of its grid gets a long run of tiles.
//
// decode_attn_kernel, grid (splits, kv_heads * head_groups, batch).  Every CTA
//   1. rotates the query heads of its GQA group once (q @ R^T, float32), folds scale*log2(e) in and keeps
//      fp16 copies in shared memory (CTAs that own uncompressed tokens keep the unrotated query instead);
//   2. runs the online-softmax attention over its token range of either the packed middle or the
//      uncompressed regions; values of the packed middle are accumulated in ROTATED space;
//   3. reduces its warps, undoes the rotation of its partial (@ R) and writes one (max, sum, weighted-V)
//      partial per query head to the workspace;
//   4. bumps a counter; the CTA that arrives last for a (sequence, KV head, head group) merges all partials
//      (log-sum-exp), normalises and writes the output.  No CTA ever waits for another one: the last arrival
//      is detected with one atomic add.
//
// Arithmetic: warps work on tiles of 16 tokens with mma.sync.m16n8k16 (fp16 operands, fp32 accumulation):
// S[16 tokens x 8 heads] = K_tile . Q^T, online softmax in registers, P transposed with movmatrix,
// O^T[d x 8 heads] += V_tile^T . P^T.  Tokens are the M dimension so a GQA group of up to 8 query heads
// shares every unpacked key/value.  A warp unpacks (or, for the fp16 regions, copies) its tile into shared
// memory as fp16 and reads the operand fragments back with ldmatrix.
#include <algorithm>
#include <string_view>

#include <cstring>

#include "decode_dev.cuh"

namespace tq {

constexpr int GNW = 8;                 // warps per CTA of the general kernel

// ---- shared memory plan ----------------------------------------------------------------------------------
// BODY is reused by phases that never overlap in time:
//   staging:         per warp  Ks[16][D+8] + Vs[16][D+8] halves
//   CTA reduction:   per warp  o[D][8] floats + m[8] + l[8], then weights [NW][8]
//   merge (last CTA): split weights [8][MAX_SPLITS]
// After BODY: float query [8][D], fp16 query [8][D], four 16-entry fp16 centroid tables, a few scalars.
constexpr int MERGE_CPARTS = 4;       // thread slabs of the d x d product with R in the epilogue
template <int D, int NW> __host__ __device__ constexpr size_t stage_bytes() { return size_t(NW) * 2 * TILE * stage_ld<D>() * sizeof(__half); }
constexpr int QM = 32;                // QJL projections per sketch (one 32-bit sign word per token)
constexpr float QJL_C = 1.2533141373155003f;   // sqrt(pi / 2), qjl.py:91-92
template <int D, int NW> __host__ __device__ constexpr size_t reduce_bytes() {
    return size_t(NW) * (HPG * (D + 2) + 2 * HPG + HPG * QM) * sizeof(float) + size_t(HPG) * QM * sizeof(float) + size_t(NW) * HPG * sizeof(float) + size_t(HPG) * D * sizeof(float) +
           size_t(MERGE_CPARTS) * HPG * D * sizeof(float);
}
template <int D> __host__ __device__ constexpr size_t merge_bytes() { return size_t(HPG) * MAX_SPLITS * sizeof(float2); }
template <int D> __host__ __device__ constexpr size_t body_bytes() {
    size_t s = stage_bytes<D, GNW>();
    if (reduce_bytes<D, GNW>() > s) s = reduce_bytes<D, GNW>();
    if (merge_bytes<D>() > s) s = merge_bytes<D>();
    return (s + 15) / 16 * 16;
}
// Copies of each entry of the whole-byte tables (lane l reads copy l mod TREP): random entries then spread over the
// banks instead of piling up; as many as fit beside two resident CTAs.
template <int D> __host__ __device__ constexpr int table_rep() { return D == 128 ? 8 : 16; }
template <int D> __host__ __device__ constexpr size_t tail_bytes() {
    return size_t(HPG) * D * sizeof(float) + size_t(HPG) * D * sizeof(__half) + 64 * sizeof(__half) + 16 * sizeof(float) +
           size_t(HPG) * QM * sizeof(__half) + size_t(table_rep<D>()) * (256 * sizeof(uint32_t) + 256 * sizeof(uint2));
}
template <int D> __host__ __device__ constexpr size_t kernel_smem() { return body_bytes<D>() + tail_bytes<D>(); }

// half2 of two signs (+1 for a set bit, -1 otherwise) from bit 0 of a and bit 0 of b
__device__ __forceinline__ uint32_t sign_pair(uint32_t a, uint32_t b) { return 0xBC00BC00u ^ ((a & 1u) << 15) ^ ((b & 1u) << 31); }
// the same from one word that holds the two sign bits at positions 15 and 31
__device__ __forceinline__ uint32_t sign_pair16(uint32_t x) { return 0xBC00BC00u ^ (x & 0x80008000u); }

// QJL: the cache also keeps, per packed token, the signs of 32 random projections S r of the quantization residual r
// and its norm gamma; the reference adds  (sqrt(pi/2) / d) * gamma * (signs @ S)  to the dequantized vector
// (cache.py:396-427, qjl.py:70-94).  In attention that is
//   scores:  += (c/d) gamma_k[t] * sum_p sign_p(t) (S q)[p]            -> one more small MMA on +-1 operands
//   output:  += (c/d) (sum_t p_t gamma_v[t] signs(t)) @ S               -> 32 more accumulator rows, applied at the end
template <int D, bool QJL>
__global__ void __launch_bounds__(GNW * 32, D <= 128 ? 2 : 1) decode_attn_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NW = GNW, NT = NW * 32;
    constexpr int LD = stage_ld<D>();
    constexpr size_t BODY = body_bytes<D>();
    float* qf = reinterpret_cast<float*>(smem + BODY);                       // [8][D] query, float32
    __half* qs = reinterpret_cast<__half*>(qf + HPG * D);                    // [8][D] scaled fp16 query (rotated or raw)
    __half* ctab = qs + HPG * D;                                             // kc_hi, kc_lo, vc_hi, vc_lo (16 each)
    float* s_misc = reinterpret_cast<float*>(ctab + 64);                     // [0..7] 1/L per head, [8] last-CTA flag
    __half* us = reinterpret_cast<__half*>(s_misc + 16);                     // [8][32] fp16 (S q) * scale * log2(e)  (QJL)
    constexpr int TREP = table_rep<D>();
    uint2* t2 = reinterpret_cast<uint2*>(us + HPG * QM);                     // [256][TREP] byte of four 2-bit codes -> 4 value centroids
    uint32_t* t4 = reinterpret_cast<uint32_t*>(t2 + 256 * TREP);             // [256][TREP] byte of two 4-bit codes -> half2 of key centroids

    pdl_trigger();     // the next launch on the stream may become resident and run its own prologue
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, hkv = blockIdx.y / p.HG, hg = blockIdx.y % p.HG, b = blockIdx.z;
    const int64_t kvl = int64_t(b) * p.Hkv + hkv;        // lane of the cache arrays
    const bool dense = split >= p.n_ps;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const int64_t qbase = (int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG) * D;   // first query head of this group
    const int S = p.n_ps + p.n_ds;

    // ---------------- prologue on constants only (runs before the previous launch has finished) -----------
    if (!dense && tid < 64) {
        const int which = tid >> 4, k = tid & 15;
        const float* src = which == 0 ? p.kc_hi : which == 1 ? p.kc_lo : which == 2 ? p.vc_hi : p.vc_lo;
        const int bits = which == 0 ? p.kb_hi : which == 1 ? p.kb_lo : which == 2 ? p.vb_hi : p.vb_lo;
        const float sc = which == 2 ? p.v_scale_hi : which == 3 ? p.v_scale_lo : 1.f;
        ctab[tid] = __float2half_rn((src != nullptr && bits > 0 && k < (1 << bits)) ? src[k] * sc : 0.f);
    }
    // whole-byte tables for the two commonest widths (4-bit keys, 2-bit values, not fractional): a tile is then
    // unpacked a 32-bit word at a time instead of a code at a time
    const bool fast_k = !dense && p.kb_hi == 4 && p.kb_lo == 0 && p.words_ok, fast_v = !dense && p.vb_hi == 2 && p.vb_lo == 0 && p.words_ok;
    if (fast_k || fast_v) {
        __syncthreads();
        for (int idx = tid; idx < 256 * TREP; idx += NT) {
            const int e = idx / TREP;
            const __half2 hk = __halves2half2(ctab[e & 15], ctab[e >> 4]);
            t4[idx] = *reinterpret_cast<const uint32_t*>(&hk);
            const __half2 v01 = __halves2half2(ctab[32 + (e & 3)], ctab[32 + ((e >> 2) & 3)]);
            const __half2 v23 = __halves2half2(ctab[32 + ((e >> 4) & 3)], ctab[32 + (e >> 6)]);
            t2[idx] = make_uint2(*reinterpret_cast<const uint32_t*>(&v01), *reinterpret_cast<const uint32_t*>(&v23));
        }
    }
    pdl_wait();        // from here on: the query, the cache and the workspace of the previous launch are settled
    await_gather(p);   // (head-sharded decoding) ... and the peers' heads of an earlier call have arrived

    // ---------------- the query heads of this group: float32, then (rotated) scaled fp16 --------------------
    // q_rot[h][j] = sum_k q[h][k] R[j][k]  (rotation.py:81-110)
    {
        const float f = p.scale * LOG2E;
        {
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
        if (QJL && !dense) {
            // (S q)[h][p] for the unrotated query, already in the log2 domain; thread (h, p)
            const int h = tid >> 5, pp = tid & 31;
            float acc = 0.f;
            if (h < heads_here) {
                for (int k = 0; k < D; ++k) acc = fmaf(qf[h * D + k], __ldg(p.qjl_proj + pp * D + k), acc);
            }
            us[h * QM + pp] = __float2half_rn(acc * f);
        }
    }
    __syncthreads();

    constexpr int NZ = QJL ? QM / 16 : 0;
    WarpAcc<D, NZ> st;
    st.init();

    uint32_t bq[D / 16][2];
    {
        const __half* qh = qs + g * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            bq[ks][0] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t) : 0u;
            bq[ks][1] = g < heads_here ? *reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8) : 0u;
        }
    }
    uint32_t bu[QM / 16][2];          // (S q) fragments, B operand: k = sketch index, n = head
    auto& zacc = st.z;                // sketch rows of the output, this warp's share (rescaled with the other accumulators)
#pragma unroll
    for (int ks = 0; ks < QM / 16; ++ks) {
        // k-slot (ks, register hh, half e) of lane t stands for sketch index 4 t + 2 ks + hh + 16 e: the two halves of an
        // operand register are then bits 16 apart in a token's sign word, and one shift + one logic op builds the register
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int pidx = 4 * t + 2 * ks + hh;
            bu[ks][hh] = 0u;
            if (QJL && g < heads_here) {
                const __half2 u2 = __halves2half2(us[g * QM + pidx], us[g * QM + pidx + 16]);
                bu[ks][hh] = *reinterpret_cast<const uint32_t*>(&u2);
            }
        }
    }
    __half* Ks = reinterpret_cast<__half*>(smem) + size_t(warp) * 2 * TILE * LD;
    __half* Vs = Ks + TILE * LD;
    if (dense) {
        // ---------------- uncompressed tokens: sink then residual window, raw query ----------------
        const int64_t tile_lo = int64_t(split - p.n_ps) * p.d_tps;
        dense_tiles<D, NW, NZ>(p, kvl, tile_lo, tile_lo + p.d_tps, Ks, Vs, bq, st, warp, lane);
    } else {
        // ---------------- packed tokens: unpack into shared memory ---------------------
        const int k_half = p.kb_lo ? D / 2 : D, v_half = p.vb_lo ? D / 2 : D;
        const int kw_hi = packed_bytes(k_half, p.kb_hi), kw_lo = p.kb_lo ? packed_bytes(D - k_half, p.kb_lo) : 0;
        const int vw_hi = packed_bytes(v_half, p.vb_hi), vw_lo = p.vb_lo ? packed_bytes(D - v_half, p.vb_lo) : 0;
        const int64_t tile_lo = int64_t(split) * p.p_tps;
        const int64_t tile_hi = min(tile_lo + p.p_tps, (p.c_len + TILE - 1) / TILE);
        // Word-at-a-time path: the packed words of tile i+1 are loaded (into registers) before tile i is unpacked, and a
        // tile's norms / sketches are requested before its unpacking starts, so global latency overlaps shared-memory work.
        constexpr int TSH = TREP == 16 ? 4 : 3;                                                 // log2(TREP)
        const uint32_t my_copy = lane & (TREP - 1);
        auto tix = [&](uint32_t w, int byte) -> uint32_t {      // index of this lane's copy of the entry for byte `byte` of w
            const uint32_t field = byte * 8 >= TSH ? (w >> (byte * 8 - TSH)) : (w << (TSH - byte * 8));
            return (field & (255u << TSH)) | my_copy;
        };
        constexpr int KWPL = (TILE * D / 2 / 4) / 32, VWPL = (TILE * D / 4 / 4 + 31) / 32;     // words per lane: keys, values
        constexpr bool PREFETCH = D <= 128;                                                     // (register budget)
        uint32_t kw[KWPL], vw[VWPL];
        auto load_words = [&](int64_t tile, uint32_t (&kd)[KWPL], uint32_t (&vd)[VWPL]) {
            const int64_t tok0 = tile * TILE;
            const int rows = tile < tile_hi ? int(min(int64_t(TILE), p.c_len - tok0)) : 0;     // rows of this tile inside the cache
            if (fast_k) {
                // 16 rows of D/2 bytes are contiguous: word i of the tile = row (4 i) / (D/2), bytes (4 i) % (D/2) ...
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.k_hi + (kvl * p.c_ls + tok0) * (D / 2));
#pragma unroll
                for (int j = 0; j < KWPL; ++j) {
                    const int i = lane + 32 * j, r = (4 * i) / (D / 2);
                    kd[j] = r < rows ? __ldg(src + i) : 0u;
                }
            }
            if (fast_v) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(p.v_hi + (kvl * p.c_ls + tok0) * (D / 4));
#pragma unroll
                for (int j = 0; j < VWPL; ++j) {
                    const int i = lane + 32 * j, r = (4 * i) / (D / 4);
                    vd[j] = (i < TILE * D / 4 / 4 && r < rows) ? __ldg(src + i) : 0u;
                }
            }
        };
        if (PREFETCH) load_words(tile_lo + warp, kw, vw);
        for (int64_t tile = tile_lo + warp; tile < tile_hi; tile += NW) {
            const int64_t tok0 = tile * TILE;
            const bool ok0 = tok0 + g < p.c_len, ok1 = tok0 + g + 8 < p.c_len;
            const int64_t n0 = kvl * p.c_ls + (ok0 ? tok0 + g : 0), n1 = kvl * p.c_ls + (ok1 ? tok0 + g + 8 : 0);
            const float kn0 = __ldg(p.k_norms + n0), kn1 = __ldg(p.k_norms + n1);
            const float vn0 = __ldg(p.v_norms + n0), vn1 = __ldg(p.v_norms + n1);
            uint32_t zk0 = 0, zk1 = 0, zv[4] = {0, 0, 0, 0};
            float gk0 = 0.f, gk1 = 0.f, gv0 = 0.f, gv1 = 0.f;
            if (QJL) {
                zk0 = ok0 ? __ldg(p.k_qbits + n0) : 0u; zk1 = ok1 ? __ldg(p.k_qbits + n1) : 0u;
                gk0 = ok0 ? __ldg(p.k_qgamma + n0) * (QJL_C / D) : 0.f; gk1 = ok1 ? __ldg(p.k_qgamma + n1) * (QJL_C / D) : 0.f;
                gv0 = ok0 ? __ldg(p.v_qgamma + n0) : 0.f; gv1 = ok1 ? __ldg(p.v_qgamma + n1) : 0.f;
                const int64_t nb = kvl * p.c_ls + tok0;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int tk = 2 * t + (u & 1) + (u >> 1) * 8;                    // tokens 2t, 2t+1, 2t+8, 2t+9
                    zv[u] = tok0 + tk < p.c_len ? __ldg(p.v_qbits + nb + tk) : 0u;
                }
            }
            uint32_t kc[KWPL], vc[VWPL];
            if (PREFETCH) {
#pragma unroll
                for (int j = 0; j < KWPL; ++j) kc[j] = kw[j];
#pragma unroll
                for (int j = 0; j < VWPL; ++j) vc[j] = vw[j];
                load_words(tile + NW, kw, vw);          // next tile of this warp (zeros past the end)
            } else {
                load_words(tile, kc, vc);
            }
            if (fast_k) {
#pragma unroll
                for (int j = 0; j < KWPL; ++j) {
                    const int i = lane + 32 * j, r = (4 * i) / (D / 2), cb = 4 * i - r * (D / 2);
                    const uint32_t w = kc[j];
                    uint4 o;
                    // rows past the end of the cache were loaded as zero words: they unpack to centroid 0, a finite value
                    // that the softmax's mask (ok0 / ok1) keeps out of every sum
                    o.x = t4[tix(w, 0)]; o.y = t4[tix(w, 1)]; o.z = t4[tix(w, 2)]; o.w = t4[tix(w, 3)];
                    *reinterpret_cast<uint4*>(Ks + r * LD + 2 * cb) = o;
                }
            }
            if (fast_v) {
#pragma unroll
                for (int j = 0; j < VWPL; ++j) {
                    const int i = lane + 32 * j, r = (4 * i) / (D / 4), cb = 4 * i - r * (D / 4);
                    if (i < TILE * D / 4 / 4) {
                        const uint32_t w = vc[j];
                        const uint2 a = t2[tix(w, 0)], b = t2[tix(w, 1)], c = t2[tix(w, 2)], e = t2[tix(w, 3)];
                        const uint4 o0 = make_uint4(a.x, a.y, b.x, b.y), o1 = make_uint4(c.x, c.y, e.x, e.y);
                        *reinterpret_cast<uint4*>(Vs + r * LD + 4 * cb) = o0;
                        *reinterpret_cast<uint4*>(Vs + r * LD + 4 * cb + 8) = o1;
                    }
                }
            }
            if (!fast_k || !fast_v) {
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
                    if (!fast_k) *reinterpret_cast<__half2*>(Ks + r * LD + j) = kk;
                    if (!fast_v) *reinterpret_cast<__half2*>(Vs + r * LD + j) = vv;
                }
            }
            __syncwarp();
            if (!QJL) {
                tile_from_smem<D, NZ>(Ks, Vs, bq, kn0, kn1, vn0, vn1, ok0, ok1, st, lane);
            } else {
                // scores: MSE part scaled by the key norm plus the sketch part scaled by (c/d) gamma
                float s[4] = {0.f, 0.f, 0.f, 0.f}, sq[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const __half* base = Ks + (lane & 15) * LD + (lane >> 4) * 8;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        uint32_t a[4];
                        ldsm_x4(a, base + ks * 16);
                        mma16816(s, a[0], a[1], a[2], a[3], bq[ks][0], bq[ks][1]);
                    }
                }
                {
                    // signs of sketch indices 4 t + q (+ 16) of tokens g and g + 8: bits 12 + q and 28 + q after one shift
                    const uint32_t zs0 = zk0 << (12 - 4 * t), zs1 = zk1 << (12 - 4 * t);
#pragma unroll
                    for (int ks = 0; ks < QM / 16; ++ks)
                        mma16816(sq, sign_pair16(zs0 << (3 - 2 * ks)), sign_pair16(zs1 << (3 - 2 * ks)), sign_pair16(zs0 << (2 - 2 * ks)),
                                 sign_pair16(zs1 << (2 - 2 * ks)), bu[ks][0], bu[ks][1]);
                }
                s[0] = fmaf(s[0], kn0, sq[0] * gk0); s[1] = fmaf(s[1], kn0, sq[1] * gk0);
                s[2] = fmaf(s[2], kn1, sq[2] * gk1); s[3] = fmaf(s[3], kn1, sq[3] * gk1);
                uint32_t bp[2];
                float pr[4];
                softmax_step<D, NZ>(s, 1.f, 1.f, vn0, vn1, ok0, ok1, st, bp, pr, fmaxf(gv0, gv1));
                {
                    const __half* base = Vs + ((lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
                    for (int mt = 0; mt < D / 16; ++mt) {
                        uint32_t a[4];
                        ldsm_x4_t(a, base + mt * 16);
                        mma16816(st.o[mt], a[0], a[1], a[2], a[3], bp[0], bp[1]);
                    }
                }
                // sketch rows of the output: z[p][h] += sum_t sign_p(t) * (p_t * gamma_v[t]); P^T operand as for the values
                // pr carries the value scale, which was chosen with the residual norms in view
                const uint32_t bz0 = movm_t(pack_h2(pr[0] * gv0, pr[1] * gv0));
                const uint32_t bz1 = movm_t(pack_h2(pr[2] * gv1, pr[3] * gv1));
                {
                    // operand registers pair two tokens' signs of one sketch row: put the tokens' half-words side by side
                    // (row r of token A at bit r, of token B at bit r + 16), then one shift + one logic op per register
                    const uint32_t x01 = __byte_perm(zv[0], zv[1], 0x5410) << (7 - g), y01 = __byte_perm(zv[0], zv[1], 0x7632) << (7 - g);
                    const uint32_t x23 = __byte_perm(zv[2], zv[3], 0x5410) << (7 - g), y23 = __byte_perm(zv[2], zv[3], 0x7632) << (7 - g);
                    // rows g, g + 8 (from x) and 16 + g, 24 + g (from y); bit 15 - 8 = row g + 8 now, row g after 8 more
                    mma16816(zacc[0], sign_pair16(x01 << 8), sign_pair16(x01), sign_pair16(x23 << 8), sign_pair16(x23), bz0, bz1);
                    mma16816(zacc[1], sign_pair16(y01 << 8), sign_pair16(y01), sign_pair16(y23 << 8), sign_pair16(y23), bz0, bz1);
                }
            }
            __syncwarp();
        }
    }

    st.finish();       // accumulators back to true scale (the value scale is per warp)
    // ---------------- CTA reduction over warps ----------------------------------------------------------------
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
    }
    __syncthreads();   // staging / tables / ring are dead from here on
    constexpr int DS = D + 2;                               // row stride (floats): keeps the 64-bit stores below 2-way conflicts
    constexpr int RW = HPG * DS + 2 * HPG + HPG * QM;       // floats per warp in the reduction buffer: o, (m, l), sketch rows
    float* red = reinterpret_cast<float*>(smem);
    float* wts = red + size_t(NW) * RW;                     // [NW][8] per-warp weights exp2(m_w - M)
    float* s_z = wts + NW * HPG;                            // [8][32] reduced sketch rows of this CTA
    float* s_acc = s_z + HPG * QM;                          // [8][D] reduced accumulator of this CTA
    float* s_pp = s_acc + HPG * D;                          // [MERGE_CPARTS][8][D] partial products with R
    {
        float* ro = red + size_t(warp) * RW;                // [8][DS]: head-major
        float* rm = ro + HPG * DS;                          // [8] max, [8] sum
        if (2 * t < heads_here) {                           // lanes that hold only padding heads store nothing
#pragma unroll
            for (int mt = 0; mt < D / 16; ++mt) {
                const int c0 = mt * 16 + g;
                ro[(2 * t) * DS + c0] = st.o[mt][0]; ro[(2 * t + 1) * DS + c0] = st.o[mt][1];
                ro[(2 * t) * DS + c0 + 8] = st.o[mt][2]; ro[(2 * t + 1) * DS + c0 + 8] = st.o[mt][3];
            }
        }
        if (g == 0) {
            rm[2 * t] = st.m[0]; rm[2 * t + 1] = st.m[1];
            rm[HPG + 2 * t] = st.l[0]; rm[HPG + 2 * t + 1] = st.l[1];
        }
        if (QJL) {
            float* rz = rm + 2 * HPG;                        // [8 heads][32 sketch rows]
#pragma unroll
            for (int mt = 0; mt < QM / 16; ++mt) {
                rz[(2 * t) * QM + mt * 16 + g] = zacc[mt][0]; rz[(2 * t + 1) * QM + mt * 16 + g] = zacc[mt][1];
                rz[(2 * t) * QM + mt * 16 + g + 8] = zacc[mt][2]; rz[(2 * t + 1) * QM + mt * 16 + g + 8] = zacc[mt][3];
            }
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
    if (QJL && !dense && tid < HPG * QM) {
        const int h = tid / QM, pp = tid - h * QM;
        float acc = 0.f;
#pragma unroll
        for (int x = 0; x < NW; ++x) acc = fmaf(wts[x * HPG + h], red[size_t(x) * RW + HPG * DS + 2 * HPG + h * QM + pp], acc);
        s_z[tid] = acc * (QJL_C / D);
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
                    r[u] = __ldg(p.rot + int64_t(c) * D + j);
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
            if (QJL) {                                       // (c/d) * z @ S, in unrotated space (qjl.py:89-92)
#pragma unroll 8
                for (int pp = 0; pp < QM; ++pp) v = fmaf(s_z[h * QM + pp], __ldg(p.qjl_proj + pp * D + j), v);
            }
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
    __syncthreads();
    if (s_misc[8] == 0.f) return;
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
        // fused gather: staged in the result's element type where the float32 query sat, sent below
        if (p.n_peers > 0) store_from_f32(qf, p.out_dtype, e, acc / L);
        else store_from_f32(p.out, p.out_dtype, qbase + e, acc / L);
    }
    if (p.n_peers > 0) {
        const unsigned epoch = next_epoch(p, int(grp));
        __syncthreads();
        // the group's first head in the peers' (batch, heads_total, d) buffers
        const int64_t gbase = (int64_t(blockIdx.z) * p.heads_total + p.head_offset + int64_t(blockIdx.y / p.HG) * p.G + (blockIdx.y % p.HG) * HPG) * D;
        const int es = out_elem_bytes(p.out_dtype);
        publish_result(p, qf, heads_here * D * es, gbase * es, int(grp), epoch);
    }
}

// ---- host side ------------------------------------------------------------------------------------
static int g_tune_ctas_per_sm = 2;     // CTAs of the general path resident per SM at d <= 128 (split heuristic)
static int g_tune_wait_polls = 2000000;  // polls of a word of a gather before the wait gives up (about a microsecond each: some two seconds)
constexpr int64_t MAX_AWAIT_WORDS_IN_KERNEL = 8192;
static int g_tune_force_general = 0;   // 1: never take the direct path (testing)
static int g_tune_splits = 0;          // > 0: fixed number of packed splits
extern int g_tune_dequantize_tc;       // rowops.cu: 0 = dequantize always on the CUDA-core row kernel
extern int g_tune_prefill_tc;          // prefill.cu: 0 = several-query-token attention always on the mma.sync kernel
static int g_tune_pdl = 1;             // programmatic dependent launch between consecutive calls
static int g_tune_stream = 1;          // 0: never take the streaming kernel
static int g_tune_stream_min_run = 24; // fewest packed tiles per warp for which the streaming kernel is chosen over the table-lookup kernel (a third of it over the general kernel)
static int g_tune_stream_max_parts = 40;  // most partials per lane with which it is chosen over the table-lookup kernel (64 over the general kernel)

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
    const int NW = direct ? DIRECT_WARPS : GNW;
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
        // Splits per lane.  While the whole grid fits on the device at once ((packed + dense splits) * lanes <= SMs * CTAs
        // per SM) more splits are better.  Past that point CTAs queue: the estimate is total work over the slots plus half
        // of one packed CTA for the ragged end, in units of one tile, with a CTA's fixed cost (tables, query rotation,
        // reduction, merge) counted as so many tiles.  No CTA waits for another, so residency is not required.
        const int64_t slots = int64_t(sms) * (direct ? 1 : g_tune_ctas_per_sm);
        const double fixed_p = direct ? 146.0 : 80.0, fixed_d = direct ? 100.0 : 40.0;
        int64_t max_useful = (p_tiles + 2 * NW - 1) / (2 * NW);   // at least two tiles per warp
        if (max_useful > MAX_SPLITS - 64) max_useful = MAX_SPLITS - 64;
        if (max_useful < 1) max_useful = 1;
        int64_t want = 1;
        if (g_tune_splits > 0) {
            want = std::min<int64_t>(g_tune_splits, max_useful);
        } else {
            double best = 0.0;
            for (int64_t w = 1; w <= max_useful; ++w) {
                const double cta = fixed_p + double(p_tiles) / double(w);
                double t = cta;
                if (lanes * (w + s.n_ds) > slots)
                    t = (double(lanes * w) * cta + double(lanes * s.n_ds) * fixed_d) / double(slots) + 0.5 * cta;
                if (w == 1 || t < best) { best = t; want = w; }
            }
        }
        s.p_tps = (p_tiles + want - 1) / want;
        s.n_ps = int((p_tiles + s.p_tps - 1) / s.p_tps);
    }
    return s;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The arrival counters sit at the start of the workspace, in an area of fixed size: calls of different shapes that
// share a workspace must never see one another's partials where they expect counters left at zero.
constexpr size_t COUNTER_AREA = 65536;      // 16384 (sequence, KV head, head group) triples; beyond that the area grows
struct WsLayout { size_t counters, part_o, part_ml, total; };

static WsLayout ws_layout(int batch, int n_q_heads, int n_kv_heads, int d, const SplitPlan& s) {
    WsLayout w{};
    const size_t groups = size_t(batch) * n_kv_heads * s.hg;
    const size_t parts = groups * size_t(s.n_ps + s.n_ds);
    const size_t slots = size_t(std::min(n_q_heads / n_kv_heads, HPG));
    w.counters = 0;
    w.part_o = align_up(std::max(groups * sizeof(int), COUNTER_AREA), 256);
    w.part_ml = align_up(w.part_o + parts * slots * d * sizeof(float), 256);
    w.total = align_up(w.part_ml + parts * slots * 2 * sizeof(float), 256);
    return w;
}

template <int D, bool QJL> static int launch_decode(const DecodeParams& p, cudaStream_t s) {
    constexpr size_t smem = kernel_smem<D>();
    static bool set[16] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel<D, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev] = true;
    }
    // Programmatic stream serialisation: the grid may become resident before its predecessor on the stream
    // has finished; the kernel calls griddepcontrol.wait before it touches anything but constants.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(p.n_ps + p.n_ds), unsigned(p.Hkv * p.HG), unsigned(p.B));
    cfg.blockDim = dim3(GNW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_tune_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attn_kernel<D, QJL>, p);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: %s", cudaGetErrorString(e));
    return TQ_OK;
}

// Validates the arguments, picks the path and the split plan and fills the kernel parameters.
int decode_prepare(const tq_decode_args* a, void* workspace, size_t workspace_bytes, DecodeParams* out, bool* direct_out,
                   const void* k_new, const void* v_new) {
    if (!a) return fail(TQ_ERR_INVALID, "tq_decode_attn: null args");
    const int n_new = k_new ? 1 : 0;
    if (n_new) {
        if (!v_new || !a->res_k || !a->res_v || a->res_lane_stride <= a->res_len)
            return fail(TQ_ERR_INVALID, "tq_decode_step: the recent-token buffers have no room for the new token (%lld of %lld rows used)",
                        (long long)a->res_len, (long long)a->res_lane_stride);
        if (!aligned(k_new, 16) || !aligned(v_new, 16) || !aligned(a->res_k, 16) || !aligned(a->res_v, 16) || (a->d * (a->dense_dtype == TQ_F32 ? 4 : 2)) % 16)
            return fail(TQ_ERR_INVALID, "tq_decode_step: new rows and recent-token buffers must be 16-byte aligned");
    }
    const int d = a->d;
    if (a->batch <= 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->n_q_heads % a->n_kv_heads)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: batch=%d q_heads=%d kv_heads=%d", a->batch, a->n_q_heads, a->n_kv_heads);
    if (d != 64 && d != 96 && d != 128 && d != 256) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: d=%d (64, 96, 128 or 256)", d);
    if (a->c_len < 0 || a->sink_len < 0 || a->res_len < 0 || a->c_len + a->sink_len + a->res_len + n_new == 0)
        return fail(TQ_ERR_INVALID, "tq_decode_attn: the cache holds no tokens");
    if (a->c_len >= (int64_t(1) << 30)) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: c_len too large");
    if (!a->q || !a->rot || (!a->out && !a->gather) || !workspace) return fail(TQ_ERR_INVALID, "tq_decode_attn: null pointer");
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
        if (a->k_qjl_bits || a->v_qjl_bits || a->k_qjl_gamma || a->v_qjl_gamma) {
            if (!a->k_qjl_bits || !a->v_qjl_bits || !a->k_qjl_gamma || !a->v_qjl_gamma || !a->qjl_proj)
                return fail(TQ_ERR_INVALID, "tq_decode_attn: QJL needs the projection matrix and both sides' sign words and residual norms");
        }
    }
    if ((a->sink_len > 0 && (!a->sink_k || !a->sink_v || a->sink_lane_stride < a->sink_len)) ||
        (a->res_len > 0 && (!a->res_k || !a->res_v || a->res_lane_stride < a->res_len + n_new)))
        return fail(TQ_ERR_INVALID, "tq_decode_attn: bad sink / residual buffers");
    if (a->dense_dtype == TQ_F16 && ((a->sink_len > 0 && (!aligned(a->sink_k, 16) || !aligned(a->sink_v, 16))) ||
                                     (a->res_len > 0 && (!aligned(a->res_k, 16) || !aligned(a->res_v, 16)))))
        return fail(TQ_ERR_INVALID, "tq_decode_attn: fp16 sink / residual buffers must be 16-byte aligned");
    if (!aligned(workspace, 256)) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace must be 256-byte aligned");

    const int64_t dense_len = a->sink_len + a->res_len + n_new;
    // direct path: 4-bit keys / 2-bit values, d = 128, rows and norms addressable in aligned 16-byte chunks
    if (a->tables && !aligned(a->tables, 256)) return fail(TQ_ERR_INVALID, "tq_decode_attn: tables must be 256-byte aligned");
    const bool direct = !g_tune_force_general && a->tables && d == 128 && a->c_len > 0 && a->k_bits_hi == 4 && a->k_bits_lo == 0 &&
                        a->v_bits_hi == 2 && a->v_bits_lo == 0 && !a->k_qjl_bits && aligned(a->k_hi, 16) && aligned(a->v_hi, 16) &&
                        aligned(a->k_norms, 16) && aligned(a->v_norms, 16) && a->c_lane_stride % 16 == 0 && direct_supported();
    // streaming path: the same widths at d = 96 / 128, sign sketches allowed, when every warp of a persistent grid gets a long run of tiles
    const bool qjl = a->c_len > 0 && a->k_qjl_bits != nullptr;
    bool stream = g_tune_stream && !g_tune_force_general && a->tables && (d == 96 || d == 128) && a->c_len > 0 && a->k_bits_hi == 4 && a->k_bits_lo == 0 &&
                  a->v_bits_hi == 2 && a->v_bits_lo == 0 && aligned(a->k_hi, 16) && aligned(a->v_hi, 16) && aligned(a->k_norms, 16) &&
                  aligned(a->v_norms, 16) && a->c_lane_stride % 16 == 0 && !a->gather && !a->await_ll &&
                  (!qjl || (aligned(a->k_qjl_bits, 16) && aligned(a->v_qjl_bits, 16) && aligned(a->k_qjl_gamma, 16) && aligned(a->v_qjl_gamma, 16) && aligned(a->qjl_proj, 16)));
    StreamPlan stp{};
    if (stream) {
        stp = stream_plan(a->batch, a->n_q_heads, a->n_kv_heads, d, a->c_len, dense_len, sm_count());
        // against the table-lookup kernel it pays once runs are long and the merge has few partials per lane; against the
        // general kernel (sign sketches, d = 96) almost always
        const int min_run = direct ? g_tune_stream_min_run : std::max(1, g_tune_stream_min_run / 3);
        const int max_parts = direct ? std::min(g_tune_stream_max_parts, 64) : 64;
        stream = stp.range >= min_run && stp.npp + stp.nd <= max_parts && stream_supported(d, qjl);
    }
    const SplitPlan sp = plan_splits(a->batch, a->n_q_heads, a->n_kv_heads, a->c_len, dense_len, sm_count(), direct);
    const WsLayout wl = ws_layout(a->batch, a->n_q_heads, a->n_kv_heads, d, sp);
    const size_t st_base = align_up(std::max(size_t(a->batch) * a->n_kv_heads * sp.hg * sizeof(int), COUNTER_AREA), 256);
    if (stream && st_base + stp.q16_bytes + stp.part_bytes > workspace_bytes) stream = false;   // (a workspace sized for the other kernels only)
    if (!stream && wl.total > workspace_bytes) return fail(TQ_ERR_INVALID, "tq_decode_attn: workspace %zu B < %zu B", workspace_bytes, wl.total);
    if (sp.n_ps + sp.n_ds > MAX_SPLITS) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn: too many splits");

    DecodeParams p{};
    p.B = a->batch; p.Hq = a->n_q_heads; p.Hkv = a->n_kv_heads; p.G = p.Hq / p.Hkv; p.HG = sp.hg; p.D = d; p.slots = std::min(p.G, HPG);
    p.c_len = a->c_len; p.c_ls = a->c_lane_stride;
    p.kb_hi = a->k_bits_hi; p.kb_lo = a->k_bits_lo; p.vb_hi = a->v_bits_hi; p.vb_lo = a->v_bits_lo;
    p.k_hi = a->k_hi; p.k_lo = a->k_lo; p.v_hi = a->v_hi; p.v_lo = a->v_lo;
    p.k_norms = a->k_norms; p.v_norms = a->v_norms;
    p.kc_hi = a->k_cent_hi; p.kc_lo = a->k_cent_lo; p.vc_hi = a->v_cent_hi; p.vc_lo = a->v_cent_lo;
    p.dense_dtype = a->dense_dtype;
    if (a->c_len > 0 && a->k_qjl_bits) {
        p.qjl_proj = a->qjl_proj; p.k_qbits = a->k_qjl_bits; p.v_qbits = a->v_qjl_bits; p.k_qgamma = a->k_qjl_gamma; p.v_qgamma = a->v_qjl_gamma;
    }
    p.sink_k = a->sink_k; p.sink_v = a->sink_v; p.res_k = a->res_k; p.res_v = a->res_v;
    p.sink_len = a->sink_len; p.sink_ls = a->sink_lane_stride; p.res_len = a->res_len; p.res_ls = a->res_lane_stride;
    p.k_new = k_new; p.v_new = v_new; p.res_k_w = const_cast<void*>(a->res_k); p.res_v_w = const_cast<void*>(a->res_v);
    p.n_ps = sp.n_ps; p.n_ds = sp.n_ds; p.p_tps = sp.p_tps; p.d_tps = sp.d_tps;
    p.q = a->q; p.q_dtype = a->q_dtype; p.scale = a->scale; p.rot = a->rot;
    p.v_scale_hi = a->v_cent_scale_hi > 0.f ? a->v_cent_scale_hi : 1.f;
    p.v_scale_lo = a->v_cent_scale_lo > 0.f ? a->v_cent_scale_lo : 1.f;
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    p.counters = reinterpret_cast<int*>(ws + wl.counters);
    p.part_o = reinterpret_cast<float*>(ws + wl.part_o); p.part_ml = reinterpret_cast<float*>(ws + wl.part_ml);
    p.out = a->out; p.out_dtype = a->out_dtype;
    p.n_peers = 0; p.heads_total = a->n_q_heads; p.head_offset = 0;
    if (a->gather) {
        const tq_peer_gather* gth = a->gather;
        if (gth->n_peers < 1 || gth->n_peers > TQ_MAX_PEERS || gth->head_offset < 0 || gth->heads_total < gth->head_offset + a->n_q_heads)
            return fail(TQ_ERR_INVALID, "tq_decode_attn: gather: n_peers %d, heads %d + %d of %d", gth->n_peers, gth->head_offset, a->n_q_heads,
                        gth->heads_total);
        for (int r = 0; r < gth->n_peers; ++r)
            if (!gth->ll[r] || !aligned(gth->ll[r], 8)) return fail(TQ_ERR_INVALID, "tq_decode_attn: gather: null or misaligned landing buffer of peer %d", r);
        if (!gth->epochs || !aligned(gth->epochs, 4)) return fail(TQ_ERR_INVALID, "tq_decode_attn: gather: null or misaligned epoch array");
        p.n_peers = gth->n_peers; p.heads_total = gth->heads_total; p.head_offset = gth->head_offset;
        for (int r = 0; r < gth->n_peers; ++r) p.peer_ll[r] = gth->ll[r];
        p.epochs = gth->epochs;
    }
    if (a->await_ll) {
        if (!a->await_epochs || !aligned(a->await_ll, 8) || !aligned(a->await_epochs, 4) || !aligned(a->await_out, 4) || a->await_words < 1)
            return fail(TQ_ERR_INVALID, "tq_decode_attn: await: null or misaligned buffers, or no words");
        p.await_ll = a->await_ll; p.await_epochs = a->await_epochs; p.await_words = a->await_words; p.await_out = a->await_out;
        p.await_polls = g_tune_wait_polls;
        if (!(p.status = decode_status_ptr())) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: cannot locate the status word");
    }
    p.pdl = g_tune_pdl;
    p.words_ok = (a->c_len > 0 && aligned(a->k_hi, 4) && aligned(a->v_hi, 4)) ? 1 : 0;   // packed rows readable as 32-bit words
    p.tables = (direct || stream) ? a->tables : nullptr;
    if (stream) {
        p.st_grid = stp.grid; p.st_npp = stp.npp; p.st_nd = stp.nd; p.st_dt = stp.dt; p.st_range = stp.range;
        p.st_q16 = reinterpret_cast<__half*>(ws + st_base);
        p.st_part = reinterpret_cast<float*>(ws + st_base + stp.q16_bytes);
        if (!(p.status = decode_status_ptr())) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: cannot locate the status word");
    }
    *out = p;
    *direct_out = direct && !stream;
    return TQ_OK;
}

int decode_launch(const DecodeParams& p0, bool direct, cudaStream_t s) {
    DecodeParams p = p0;
    if (p.await_ll && p.await_words > MAX_AWAIT_WORDS_IN_KERNEL) {      // too many words for every CTA to poll: a wait launch first
        if (int rc = launch_gather_wait(p.await_ll, p.await_epochs, p.await_words, p.await_out, p.await_polls, s)) return rc;
        p.await_ll = nullptr;
    }
    if (p.st_grid > 0) return launch_decode_stream(p, s);
    if (direct) return launch_decode_direct(p, s);
    const bool qjl = p.qjl_proj != nullptr;
    if (p.D == 64) return qjl ? launch_decode<64, true>(p, s) : launch_decode<64, false>(p, s);
    if (p.D == 96) return qjl ? launch_decode<96, true>(p, s) : launch_decode<96, false>(p, s);
    if (p.D == 128) return qjl ? launch_decode<128, true>(p, s) : launch_decode<128, false>(p, s);
    return qjl ? launch_decode<256, true>(p, s) : launch_decode<256, false>(p, s);
}

}  // namespace tq

using namespace tq;

extern "C" int tq_set_tuning(const char* key, int value) {
    if (!key) return fail(TQ_ERR_INVALID, "tq_set_tuning: null key");
    const std::string_view k(key);
    if (k == "decode_ctas_per_sm" && value >= 1 && value <= 8) g_tune_ctas_per_sm = value;
    else if (k == "decode_force_general" && (value == 0 || value == 1)) g_tune_force_general = value;
    else if (k == "decode_pdl" && (value == 0 || value == 1)) g_tune_pdl = value;
    else if (k == "decode_stream" && (value == 0 || value == 1)) g_tune_stream = value;
    else if (k == "decode_stream_min_run" && value >= 1 && value <= (1 << 20)) g_tune_stream_min_run = value;
    else if (k == "decode_stream_max_parts" && value >= 1 && value <= 64) g_tune_stream_max_parts = value;
    else if (k == "decode_splits" && value >= 0 && value <= MAX_SPLITS - 64) g_tune_splits = value;
    else if (k == "gather_wait_polls" && value >= 1000 && value <= 4000000) g_tune_wait_polls = value;
    else if (k == "prefill_tc" && (value == 0 || value == 1)) g_tune_prefill_tc = value;
    else if (k == "dequantize_tc" && (value == 0 || value == 1)) g_tune_dequantize_tc = value;
    else return fail(TQ_ERR_INVALID, "tq_set_tuning: unknown key or bad value: %s=%d", key, value);
    return TQ_OK;
}

extern "C" int tq_decode_kernel_choice(const tq_decode_args* a) {
    DecodeParams p;
    bool direct = false;
    if (decode_prepare(a, a ? a->workspace : nullptr, a ? a->workspace_bytes : 0, &p, &direct)) return -1;
    return p.st_grid > 0 ? 2 : direct ? 1 : 0;
}

extern "C" int tq_gather_wait(const unsigned long long* ll, const unsigned* epochs, int64_t n_words, void* out, void* stream) {
    if (!ll || !epochs || !aligned(ll, 8) || !aligned(epochs, 4) || !aligned(out, 4) || n_words < 1)
        return fail(TQ_ERR_INVALID, "tq_gather_wait: null or misaligned buffers, or no words");
    return launch_gather_wait(ll, epochs, n_words, out, g_tune_wait_polls, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t tq_gather_groups(int batch, int n_q_heads, int n_kv_heads) {
    if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return 0;
    const int G = n_q_heads / n_kv_heads;
    return int64_t(batch) * n_kv_heads * ((G + HPG - 1) / HPG);     // one merging CTA per (sequence, KV head, head group)
}

// ---- peer-visible buffers (CUDA IPC) -----------------------------------------------------------------
extern "C" int tq_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle || bytes == 0) return fail(TQ_ERR_INVALID, "tq_peer_buffer_create: bad arguments");
    void* d = nullptr;
    cudaError_t e = cudaMalloc(&d, bytes);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_peer_buffer_create: cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
    cudaIpcMemHandle_t h;
    if ((e = cudaMemset(d, 0, bytes)) != cudaSuccess || (e = cudaIpcGetMemHandle(&h, d)) != cudaSuccess) {
        cudaFree(d);
        return fail(TQ_ERR_LAUNCH, "tq_peer_buffer_create: %s", cudaGetErrorString(e));
    }
    std::memcpy(handle, &h, 64);
    *ptr = d;
    return TQ_OK;
}

extern "C" int tq_peer_buffer_open(const unsigned char handle[64], int peer_device, void** ptr) {
    if (!ptr || !handle) return fail(TQ_ERR_INVALID, "tq_peer_buffer_open: bad arguments");
    int dev = 0, can = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && dev != peer_device) e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_peer_buffer_open: %s", cudaGetErrorString(e));
    if (dev != peer_device && !can) return fail(TQ_ERR_UNSUPPORTED, "tq_peer_buffer_open: device %d cannot address device %d", dev, peer_device);
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    void* d = nullptr;
    e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_peer_buffer_open: %s", cudaGetErrorString(e));
    *ptr = d;
    return TQ_OK;
}

extern "C" int tq_peer_buffer_close(void* ptr) {
    cudaError_t e = ptr ? cudaIpcCloseMemHandle(ptr) : cudaSuccess;
    return e == cudaSuccess ? TQ_OK : fail(TQ_ERR_LAUNCH, "tq_peer_buffer_close: %s", cudaGetErrorString(e));
}

extern "C" int tq_peer_buffer_destroy(void* ptr) {
    cudaError_t e = ptr ? cudaFree(ptr) : cudaSuccess;
    return e == cudaSuccess ? TQ_OK : fail(TQ_ERR_LAUNCH, "tq_peer_buffer_destroy: %s", cudaGetErrorString(e));
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

extern "C" size_t tq_decode_tables_bytes(int d, int k_bits, int v_bits) {
    return ((d == 128 || d == 96) && k_bits == 4 && v_bits == 2) ? direct_tables_bytes() : 0;
}

extern "C" int tq_decode_tables_build(int d, const float* rot, const float* k_cent, int k_bits, const float* v_cent, int v_bits,
                                      float v_cent_scale, void* tables, size_t bytes, void* stream) {
    const size_t need = tq_decode_tables_bytes(d, k_bits, v_bits);
    if (need == 0) return fail(TQ_ERR_UNSUPPORTED, "tq_decode_tables_build: no kernel uses prebuilt constants for d=%d at %d-bit keys / %d-bit values", d, k_bits, v_bits);
    if (!rot || !k_cent || !v_cent || !tables) return fail(TQ_ERR_INVALID, "tq_decode_tables_build: null pointer");
    if (!aligned(tables, 256) || bytes < need) return fail(TQ_ERR_INVALID, "tq_decode_tables_build: the buffer must be 256-byte aligned and hold %zu bytes", need);
    return direct_tables_build(d, rot, k_cent, v_cent, v_cent_scale, tables, static_cast<cudaStream_t>(stream));
}

namespace tq {
size_t decode_workspace_bytes_split_kernels(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len, int64_t dense_len) {
    if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || d <= 0 || n_q_heads % n_kv_heads || c_len < 0 || dense_len < 0) return 0;
    // The larger of the two split plans tq_decode_attn can choose for these sizes (current tuning values).
    const size_t a = ws_layout(batch, n_q_heads, n_kv_heads, d, plan_splits(batch, n_q_heads, n_kv_heads, c_len, dense_len, sm_count(), false)).total;
    const size_t b = ws_layout(batch, n_q_heads, n_kv_heads, d, plan_splits(batch, n_q_heads, n_kv_heads, c_len, dense_len, sm_count(), true)).total;
    return std::max(a, b);
}
}  // namespace tq

extern "C" size_t tq_decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len,
                                            int64_t dense_len) {
    const size_t a = decode_workspace_bytes_split_kernels(batch, n_q_heads, n_kv_heads, d, c_len, dense_len);
    if (a == 0) return 0;
    size_t c = 0;
    if ((d == 96 || d == 128) && c_len > 0) {      // the streaming kernel's layout: counters' area, prepared queries, partials
        const StreamPlan sp = stream_plan(batch, n_q_heads, n_kv_heads, d, c_len, dense_len, sm_count());
        const int hg = (n_q_heads / n_kv_heads + HPG - 1) / HPG;
        if (sp.npp + sp.nd <= 64)
            c = align_up(std::max(size_t(batch) * n_kv_heads * hg * sizeof(int), COUNTER_AREA), 256) + sp.q16_bytes + sp.part_bytes;
    }
    return std::max(a, c);
}

extern "C" int tq_decode_step(const tq_decode_args* a, const void* k_new, const void* v_new, void* stream) {
    if (!k_new || !v_new) return fail(TQ_ERR_INVALID, "tq_decode_step: null new rows");
    DecodeParams p;
    bool direct = false;
    int rc = decode_prepare(a, a ? a->workspace : nullptr, a ? a->workspace_bytes : 0, &p, &direct, k_new, v_new);
    if (rc) return rc;
    const size_t counter_bytes = size_t(p.B) * p.Hkv * p.HG * sizeof(int);
    if (counter_bytes > COUNTER_AREA) {
        cudaError_t e = cudaMemsetAsync(p.counters, 0, counter_bytes, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_step: clearing counters: %s", cudaGetErrorString(e));
    }
    return decode_launch(p, direct, static_cast<cudaStream_t>(stream));
}

extern "C" int tq_decode_attn(const tq_decode_args* a, void* stream) {
    DecodeParams p;
    bool direct = false;
    int rc = decode_prepare(a, a ? a->workspace : nullptr, a ? a->workspace_bytes : 0, &p, &direct);
    if (rc) return rc;
    const size_t counter_bytes = size_t(p.B) * p.Hkv * p.HG * sizeof(int);
    if (counter_bytes > COUNTER_AREA) {        // more triples than the fixed area holds: clear them for this call
        cudaError_t e = cudaMemsetAsync(p.counters, 0, counter_bytes, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: clearing counters: %s", cudaGetErrorString(e));
    }
    return decode_launch(p, direct, static_cast<cudaStream_t>(stream));
}