// Row-wise kernels that contain the d x d rotation as an exact float32 contraction on CUDA cores:
//   tq_rotate         y = x @ R^T   or  x = y @ R
//   tq_quantize_pack  norm -> normalise -> rotate -> boundary count -> pack (+ QJL sketch)   [any dtype, any d]
//   tq_dequantize     unpack -> centroid -> inverse rotation -> scale (+ QJL correction)
//
// One CTA owns BM = 64 rows.  The (normalised / looked-up) rows sit transposed in shared memory for
// the whole CTA lifetime; R streams through a small shared tile.  256 threads hold 4x4 accumulators.
// This is the general-purpose path; fp16 rows with d = 128 take the tensor-core kernel in
// quantize_tc.cu instead.
#include "common.cuh"

namespace tq {

constexpr int BM = 64, BN = 64, BK = 16, XS_LD = BM + 4, WS_LD = BN + 4, NT = 256;
enum { MODE_ROTATE = 0, MODE_QUANT = 1, MODE_DEQUANT = 2 };

struct RowArgs {
    int mode, d, inverse;
    int64_t n_lanes, n_rows;
    // input rows
    const void* x; int x_dtype; int64_t x_lane_stride, x_row_stride;
    const float* rot;
    // quantize
    const float* bnd_hi; const float* bnd_lo; int bits_hi, bits_lo;
    uint8_t* p_hi; uint8_t* p_lo; float* norms_out; int64_t q_lane_stride; float* y_out;
    const float* qjl_proj_rot; uint32_t* qjl_bits_out; float* qjl_gamma_out;
    // dequantize
    const uint8_t* in_hi; const uint8_t* in_lo; const float* norms_in; int64_t in_lane_stride;
    const float* cent_hi; const float* cent_lo;
    const float* qjl_proj; const uint32_t* qjl_bits_in; const float* qjl_gamma_in;
    void* out; int out_dtype; int64_t out_lane_stride, out_row_stride;
};

__global__ void __launch_bounds__(NT) rowops_kernel(RowArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int d = a.d;
    float* xs = reinterpret_cast<float*>(smem_raw);                       // [d][XS_LD]
    float* ws = xs + size_t(d) * XS_LD;                                   // [BK][WS_LD]
    float* tab = ws + BK * WS_LD;                                         // 64 floats: bnd/cent hi [0,16) lo [16,32); norm [.. per row below]
    float* rown = tab + 32;                                               // [BM] row norms
    float* es = rown + BM;                                                // [BM][d+1] residuals (quantize + QJL only)
    const bool want_qjl_q = a.mode == MODE_QUANT && a.qjl_bits_out != nullptr;
    uint8_t* cs = reinterpret_cast<uint8_t*>(es + (want_qjl_q ? size_t(BM) * (d + 1) : 0));  // [BM][d] codes

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t total_rows = a.n_lanes * a.n_rows;
    const int64_t row0 = int64_t(blockIdx.x) * BM;
    const int half = a.bits_lo ? d / 2 : d;

    if (tid < 32) {
        const int s = tid >> 4, k = tid & 15;
        float v = 0.f;
        if (a.mode == MODE_QUANT) {
            const float* src = s ? a.bnd_lo : a.bnd_hi;
            const int nb = (1 << (s ? a.bits_lo : a.bits_hi)) - 1;
            if (src && k < nb) v = src[k];
        } else if (a.mode == MODE_DEQUANT) {
            const float* src = s ? a.cent_lo : a.cent_hi;
            const int nc = 1 << (s ? a.bits_lo : a.bits_hi);
            if (src && k < nc) v = src[k];
        }
        tab[tid] = v;
    }
    __syncthreads();

    // ---- prologue: fill xs[k][m] ------------------------------------------------------------------
    if (a.mode == MODE_DEQUANT) {
        const int w_hi = packed_bytes(half, a.bits_hi), w_lo = a.bits_lo ? packed_bytes(d - half, a.bits_lo) : 0;
        for (int e = tid; e < BM * d; e += NT) {
            const int m = e / d, k = e - m * d;
            const int64_t row = row0 + m;
            float v = 0.f;
            if (row < total_rows) {
                const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
                const int64_t pr = o * a.in_lane_stride + r;
                v = (k < half) ? tab[code_at(a.in_hi + pr * w_hi, k, a.bits_hi)]
                               : tab[16 + code_at(a.in_lo + pr * w_lo, k - half, a.bits_lo)];
            }
            xs[k * XS_LD + m] = v;
        }
        if (tid < BM) {
            const int64_t row = row0 + tid;
            float nv = 0.f;
            if (row < total_rows) {
                const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
                nv = a.norms_in[o * a.in_lane_stride + r];
            }
            rown[tid] = nv;
        }
    } else {
        // each warp owns 8 rows; lanes stride the row so global reads coalesce
        for (int mi = 0; mi < BM / 8; ++mi) {
            const int m = warp * (BM / 8) + mi;
            const int64_t row = row0 + m;
            const bool live = row < total_rows;
            int64_t base = 0;
            if (live) {
                const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
                base = o * a.x_lane_stride + r * a.x_row_stride;
            }
            float v[8];
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int k = lane + 32 * i;
                v[i] = (live && k < d) ? load_as_f32(a.x, a.x_dtype, base + k) : 0.f;
                ss = fmaf(v[i], v[i], ss);
            }
            float inv_den = 1.f;
            if (a.mode == MODE_QUANT) {
#pragma unroll
                for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                const float nrm = sqrtf(ss);
                inv_den = fmaxf(nrm, 1e-10f);   // divide (not multiply by a reciprocal): cache.py:237-238
                if (lane == 0) {
                    rown[m] = nrm;
                    if (live) {
                        const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
                        a.norms_out[o * a.q_lane_stride + r] = nrm;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int k = lane + 32 * i;
                if (k < d) xs[k * XS_LD + m] = (a.mode == MODE_QUANT) ? v[i] / inv_den : v[i];
            }
        }
    }
    __syncthreads();

    // ---- contraction: acc[m][j] = sum_k xs[k][m] * W[k][j] -----------------------------------------
    const int ty = tid >> 4, tx = tid & 15;
    const bool w_is_rt = (a.mode == MODE_QUANT) || (a.mode == MODE_ROTATE && !a.inverse);  // W = R^T
    for (int j0 = 0; j0 < d; j0 += BN) {
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        for (int k0 = 0; k0 < d; k0 += BK) {
#pragma unroll
            for (int i = 0; i < (BK * BN) / NT; ++i) {
                const int e = tid + NT * i;
                int kk, j;
                if (w_is_rt) { kk = e & (BK - 1); j = e / BK; } else { j = e & (BN - 1); kk = e / BN; }
                float wv = 0.f;
                if (j0 + j < d) wv = w_is_rt ? __ldg(a.rot + int64_t(j0 + j) * d + k0 + kk) : __ldg(a.rot + int64_t(k0 + kk) * d + j0 + j);
                ws[kk * WS_LD + j] = wv;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                const float4 xa = *reinterpret_cast<const float4*>(xs + (k0 + kk) * XS_LD + ty * 4);
                const float4 wb = *reinterpret_cast<const float4*>(ws + kk * WS_LD + tx * 4);
                const float xv[4] = {xa.x, xa.y, xa.z, xa.w}, wv[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
            }
            __syncthreads();
        }
        // ---- epilogue for this column tile ---------------------------------------------------------
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int m = ty * 4 + i;
            const int64_t row = row0 + m;
            if (row >= total_rows) continue;
            const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = j0 + tx * 4 + j;
                if (col >= d) continue;
                const float y = acc[i][j];
                if (a.mode == MODE_ROTATE) {
                    reinterpret_cast<float*>(a.out)[row * d + col] = y;
                } else if (a.mode == MODE_QUANT) {
                    const int side = col >= half ? 1 : 0;
                    // how many boundaries y strictly exceeds (codebook.py:220-223): for a non-decreasing list a binary
                    // search gives the counting loop's answer with one compare per bit, NaN included (0)
                    uint32_t c = 0;
                    for (uint32_t st = 1u << ((side ? a.bits_lo : a.bits_hi) - 1); st; st >>= 1)
                        if (y > tab[side * 16 + c + st - 1]) c += st;
                    cs[m * d + col] = uint8_t(c);
                    if (a.y_out) a.y_out[row * d + col] = y;
                    if (want_qjl_q) es[m * (d + 1) + col] = y - (side ? a.cent_lo : a.cent_hi)[c];
                } else {
                    float v = y * rown[m];
                    if (a.qjl_bits_in) {
                        const int64_t pr = o * a.in_lane_stride + r;
                        const uint32_t zb = a.qjl_bits_in[pr];
                        float s = 0.f;
#pragma unroll 8
                        for (int p = 0; p < 32; ++p) {
                            const float sp = __ldg(a.qjl_proj + p * d + col);
                            s += ((zb >> p) & 1u) ? sp : -sp;
                        }
                        v += (1.2533141373155003f / float(d)) * a.qjl_gamma_in[pr] * s;   // sqrt(pi/2)/d, qjl.py:91-92
                    }
                    store_from_f32(a.out, a.out_dtype, o * a.out_lane_stride + r * a.out_row_stride + col, v);
                }
            }
        }
    }
    if (a.mode != MODE_QUANT) return;
    __syncthreads();

    // ---- pack: one thread per output byte -----------------------------------------------------------
    {
        const int w_hi = packed_bytes(half, a.bits_hi), w_lo = a.bits_lo ? packed_bytes(d - half, a.bits_lo) : 0;
        const int w_all = w_hi + w_lo;
        for (int e = tid; e < BM * w_all; e += NT) {
            const int m = e / w_all, b = e - m * w_all;
            const int64_t row = row0 + m;
            if (row >= total_rows) continue;
            const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
            const int64_t pr = o * a.q_lane_stride + r;
            if (b < w_hi) a.p_hi[pr * w_hi + b] = packed_byte_from_codes(cs + m * d, b, a.bits_hi);
            else a.p_lo[pr * w_lo + (b - w_hi)] = packed_byte_from_codes(cs + m * d + half, b - w_hi, a.bits_lo);
        }
    }
    // ---- QJL sketch of the residual, in rotated space: (x - xhat) @ S^T = |x| * (y - yhat) @ (S R^T)^T ----
    if (want_qjl_q) {
        // S R^T (32 x d) moves into the dead operand tile, rows padded to d + 1 floats so that lane p reading column k
        // of its own row hits bank (p + k) mod 32; each warp then sketches its eight rows with one pass over k
        float* sp = xs;                                      // [32][d + 1]: fits, 32 (d + 1) <= d * XS_LD for every d
        for (int e = tid; e < 32 * d; e += NT) {
            const int pp = e / d, k = e - pp * d;
            sp[pp * (d + 1) + k] = __ldg(a.qjl_proj_rot + e);
        }
        __syncthreads();
        constexpr int RPW = BM / (NT / 32);                  // rows per warp: 8
        float dot[RPW], ee[RPW];
#pragma unroll
        for (int mi = 0; mi < RPW; ++mi) dot[mi] = ee[mi] = 0.f;
        const float* srow = sp + lane * (d + 1);
        const float* e0 = es + size_t(warp) * RPW * (d + 1);
        for (int k = 0; k < d; ++k) {
            const float sv = srow[k];
#pragma unroll
            for (int mi = 0; mi < RPW; ++mi) dot[mi] = fmaf(e0[mi * (d + 1) + k], sv, dot[mi]);     // e: broadcast read
        }
        for (int k = lane; k < d; k += 32) {
#pragma unroll
            for (int mi = 0; mi < RPW; ++mi) { const float v = e0[mi * (d + 1) + k]; ee[mi] = fmaf(v, v, ee[mi]); }
        }
#pragma unroll
        for (int mi = 0; mi < RPW; ++mi) {
            const int m = warp * RPW + mi;
            const int64_t row = row0 + m;
            float en = ee[mi];
#pragma unroll
            for (int off = 16; off; off >>= 1) en += __shfl_xor_sync(0xffffffffu, en, off);
            const float nrm = rown[m];
            uint32_t bits = __ballot_sync(0xffffffffu, dot[mi] >= 0.f);
            if (nrm == 0.f) bits = 0xffffffffu;   // zero row: the reference's residual is exactly 0, and 0 >= 0
            if (lane == 0 && row < total_rows) {
                const int64_t o = row / a.n_rows, r = row - o * a.n_rows;
                a.qjl_bits_out[o * a.q_lane_stride + r] = bits;
                a.qjl_gamma_out[o * a.q_lane_stride + r] = nrm * sqrtf(en);
            }
        }
    }
}

static size_t rowops_smem(int d, int mode, bool qjl_q) {
    size_t f = size_t(d) * XS_LD + BK * WS_LD + 32 + BM;
    if (qjl_q) f += size_t(BM) * (d + 1);
    size_t b = f * sizeof(float);
    if (mode == MODE_QUANT) b += size_t(BM) * d;
    return b;
}

static int launch_rowops(const RowArgs& a, cudaStream_t s, const char* what) {
    const int64_t total = a.n_lanes * a.n_rows;
    if (total == 0) return TQ_OK;
    const size_t smem = rowops_smem(a.d, a.mode, a.mode == MODE_QUANT && a.qjl_bits_out);
    static thread_local size_t cur_max[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && smem > cur_max[dev]) {
        cudaError_t e = cudaFuncSetAttribute(rowops_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "%s: shared memory %zu B: %s", what, smem, cudaGetErrorString(e));
        cur_max[dev] = smem;
    }
    const int64_t blocks = (total + BM - 1) / BM;
    if (blocks > 0x7fffffff) return fail(TQ_ERR_INVALID, "%s: too many rows", what);
    rowops_kernel<<<unsigned(blocks), NT, smem, s>>>(a);
    return check_launch(what);
}

static bool d_ok(int d) { return d >= 16 && d <= 256 && d % 16 == 0; }
static bool dtype_ok(int t) { return t == TQ_F16 || t == TQ_BF16 || t == TQ_F32; }

}  // namespace tq

using namespace tq;

extern "C" int tq_rotate(const void* x, int x_dtype, const float* rot, float* out, int64_t n, int d, int inverse,
                         void* stream) {
    if (!d_ok(d)) return fail(TQ_ERR_UNSUPPORTED, "tq_rotate: d=%d (need a multiple of 16 in 16..256)", d);
    if (!dtype_ok(x_dtype) || n < 0) return fail(TQ_ERR_INVALID, "tq_rotate: bad dtype or n");
    if (n == 0) return TQ_OK;
    if (!x || !rot || !out) return fail(TQ_ERR_INVALID, "tq_rotate: null pointer");
    RowArgs a{};
    a.mode = MODE_ROTATE; a.d = d; a.inverse = inverse; a.n_lanes = 1; a.n_rows = n;
    a.x = x; a.x_dtype = x_dtype; a.x_lane_stride = 0; a.x_row_stride = d; a.rot = rot; a.out = out;
    return launch_rowops(a, static_cast<cudaStream_t>(stream), "tq_rotate");
}

int tq_quantize_pack_tc(const tq_quantize_args* q, cudaStream_t s, bool* handled);

extern "C" int tq_quantize_pack(const tq_quantize_args* q, void* stream) {
    if (!q) return fail(TQ_ERR_INVALID, "tq_quantize_pack: null args");
    if (!d_ok(q->d)) return fail(TQ_ERR_UNSUPPORTED, "tq_quantize_pack: d=%d (need a multiple of 16 in 16..256)", q->d);
    if (!bits_ok(q->bits_hi) || (q->bits_lo && !bits_ok(q->bits_lo))) return fail(TQ_ERR_INVALID, "Unsupported bit-width: %d/%d. Use 1, 2, 3, or 4.", q->bits_hi, q->bits_lo);
    if (!dtype_ok(q->x_dtype) || q->n_lanes < 0 || q->n_rows < 0) return fail(TQ_ERR_INVALID, "tq_quantize_pack: bad dtype or sizes");
    if (q->n_lanes == 0 || q->n_rows == 0) return TQ_OK;
    if (!q->x || !q->rot || !q->bnd_hi || !q->packed_hi || !q->norms) return fail(TQ_ERR_INVALID, "tq_quantize_pack: null pointer");
    if (q->bits_lo && (!q->bnd_lo || !q->packed_lo)) return fail(TQ_ERR_INVALID, "tq_quantize_pack: fractional mode needs bnd_lo and packed_lo");
    const int half = q->bits_lo ? q->d / 2 : q->d;
    if ((half * q->bits_hi) % 8 || (q->bits_lo && ((q->d - half) * q->bits_lo) % 8) || (q->bits_hi == 3 && half % 8) || (q->bits_lo == 3 && (q->d - half) % 8))
        return fail(TQ_ERR_INVALID, "tq_quantize_pack: d=%d does not pack at %d/%d bits", q->d, q->bits_hi, q->bits_lo);
    if (q->qjl_bits && (!q->qjl_proj_rot || !q->qjl_gamma || !q->cent_hi || (q->bits_lo && !q->cent_lo))) return fail(TQ_ERR_INVALID, "tq_quantize_pack: QJL needs proj, gamma and centroids");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    bool handled = false;
    int rc = tq_quantize_pack_tc(q, s, &handled);
    if (handled) return rc;
    RowArgs a{};
    a.mode = MODE_QUANT; a.d = q->d; a.n_lanes = q->n_lanes; a.n_rows = q->n_rows;
    a.x = q->x; a.x_dtype = q->x_dtype; a.x_lane_stride = q->x_lane_stride; a.x_row_stride = q->x_row_stride;
    a.rot = q->rot; a.bnd_hi = q->bnd_hi; a.bnd_lo = q->bnd_lo; a.bits_hi = q->bits_hi; a.bits_lo = q->bits_lo;
    a.p_hi = q->packed_hi; a.p_lo = q->packed_lo; a.norms_out = q->norms; a.q_lane_stride = q->out_lane_stride;
    a.y_out = q->y_out; a.qjl_proj_rot = q->qjl_proj_rot; a.qjl_bits_out = q->qjl_bits; a.qjl_gamma_out = q->qjl_gamma;
    a.cent_hi = q->cent_hi; a.cent_lo = q->cent_lo;
    return launch_rowops(a, s, "tq_quantize_pack");
}

namespace tq {
int tq_dequantize_tc(const tq_dequantize_args* q, cudaStream_t s, bool* handled);      // dequantize_tc.cu
int g_tune_dequantize_tc = 1;      // 0: always the row kernel (testing)
}  // namespace tq

extern "C" int tq_dequantize(const tq_dequantize_args* q, void* stream) {
    if (!q) return fail(TQ_ERR_INVALID, "tq_dequantize: null args");
    if (!d_ok(q->d)) return fail(TQ_ERR_UNSUPPORTED, "tq_dequantize: d=%d (need a multiple of 16 in 16..256)", q->d);
    if (!bits_ok(q->bits_hi) || (q->bits_lo && !bits_ok(q->bits_lo))) return fail(TQ_ERR_INVALID, "Unsupported bit-width: %d/%d. Use 1, 2, 3, or 4.", q->bits_hi, q->bits_lo);
    if (!dtype_ok(q->out_dtype) || q->n_lanes < 0 || q->n_rows < 0) return fail(TQ_ERR_INVALID, "tq_dequantize: bad dtype or sizes");
    if (q->n_lanes == 0 || q->n_rows == 0) return TQ_OK;
    if (!q->packed_hi || !q->norms || !q->cent_hi || !q->rot || !q->out) return fail(TQ_ERR_INVALID, "tq_dequantize: null pointer");
    if (q->bits_lo && (!q->packed_lo || !q->cent_lo)) return fail(TQ_ERR_INVALID, "tq_dequantize: fractional mode needs packed_lo and cent_lo");
    if (q->qjl_bits && (!q->qjl_proj || !q->qjl_gamma)) return fail(TQ_ERR_INVALID, "tq_dequantize: QJL needs proj and gamma");
    if (g_tune_dequantize_tc) {
        bool handled = false;
        const int rc = tq_dequantize_tc(q, static_cast<cudaStream_t>(stream), &handled);
        if (handled) return rc;
    }
    RowArgs a{};
    a.mode = MODE_DEQUANT; a.d = q->d; a.inverse = 1; a.n_lanes = q->n_lanes; a.n_rows = q->n_rows;
    a.rot = q->rot; a.in_hi = q->packed_hi; a.in_lo = q->packed_lo; a.norms_in = q->norms; a.in_lane_stride = q->in_lane_stride;
    a.bits_hi = q->bits_hi; a.bits_lo = q->bits_lo; a.cent_hi = q->cent_hi; a.cent_lo = q->cent_lo;
    a.qjl_proj = q->qjl_proj; a.qjl_bits_in = q->qjl_bits; a.qjl_gamma_in = q->qjl_gamma;
    a.out = q->out; a.out_dtype = q->out_dtype; a.out_lane_stride = q->out_lane_stride; a.out_row_stride = q->out_row_stride;
    return launch_rowops(a, static_cast<cudaStream_t>(stream), "tq_dequantize");
}
