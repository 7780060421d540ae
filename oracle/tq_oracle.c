/*
 * C restatement of the reference's device kernel bodies, for the CPU.  TEST INFRASTRUCTURE, NOT PRODUCT
 * CODE: only the tests, the smoke check and the benchmark's CPU-baseline leg load this library.
 *
 * The reference (alex-rentel/mlx-turboquant v1.0.4) writes these loops in Metal Shading Language inside
 * mlx_turboquant/kernels.py; each function below follows the cited kernel body statement by statement
 * (one CPU loop iteration per Metal thread), in float32.  Parity status: pinned - checked against the
 * fixtures generated from the reference's Python path (tests/test_oracle_golden.py) at the reference's
 * own tolerance for kernel-vs-Python agreement.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC -o libtq_oracle.so tq_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int tqo_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* code j of a packed row: 4-bit kernels.py:106-115, 2-bit :149-153, 3-bit :183-200 */
static inline unsigned code_at(const uint8_t* row, int j, int bits) {
    if (bits == 4) { unsigned b = row[j / 2]; return (j % 2 == 0) ? (b & 0x0Fu) : ((b >> 4) & 0x0Fu); }
    if (bits == 2) { return (row[j / 4] >> ((j % 4) * 2)) & 0x03u; }
    if (bits == 1) { return (row[j / 8] >> (j % 8)) & 1u; }
    const uint8_t* g = row + (j / 8) * 3;
    unsigned b0 = g[0], b1 = g[1], b2 = g[2];
    switch (j % 8) {
        case 0: return b0 & 7u;
        case 1: return (b0 >> 3) & 7u;
        case 2: return ((b0 >> 6) | (b1 << 2)) & 7u;
        case 3: return (b1 >> 1) & 7u;
        case 4: return (b1 >> 4) & 7u;
        case 5: return ((b1 >> 7) | (b2 << 1)) & 7u;
        case 6: return (b2 >> 2) & 7u;
        default: return (b2 >> 5) & 7u;
    }
}

/* turboquant_dequant_{2,3,4}bit (kernels.py:89-125, 139-160, 173-208):
 * out[row, col] = norm[row] * sum_j centroid[idx(row, j)] * rotation[j, col] */
void tqo_dequantize_rows(const uint8_t* packed, const float* norms, int64_t n, int d, int bits, const float* cent,
                         const float* rot, float* out) {
    const int w = d * bits / 8;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < n; ++row) {
        float* acc = out + row * d;
        for (int c = 0; c < d; ++c) acc[c] = 0.0f;
        const uint8_t* pr = packed + row * w;
        for (int j = 0; j < d; ++j) {            /* same j order per output element as the kernel's serial loop */
            const float cv = cent[code_at(pr, j, bits)];
            const float* rr = rot + (int64_t)j * d;
            for (int c = 0; c < d; ++c) acc[c] += cv * rr[c];
        }
        const float nv = norms[row];
        for (int c = 0; c < d; ++c) acc[c] = nv * acc[c];
    }
}

/* Quantize rows.  Norm as in turboquant_quant_4bit_norms (kernels.py:230-240: serial sum of squares, sqrt);
 * normalisation by DIVISION by max(norm, 1e-10) as on the supported path (cache.py:237-238), not the
 * unwired kernel's reciprocal multiply (kernels.py:265-266); rotation, boundary count and packing as in
 * turboquant_quant_4bit_pack (kernels.py:276-298) generalised to 1-4 bits (packing.py:9-208). */
void tqo_quantize_rows(const float* x, int64_t n, int d, const float* rot, const float* bnd, int bits, uint8_t* packed,
                       float* norms, float* y_out) {
    const int w = d * bits / 8, nb = (1 << bits) - 1;
#pragma omp parallel
    {
        float* xn = (float*)malloc(sizeof(float) * (size_t)d);
        uint8_t* codes = (uint8_t*)malloc((size_t)d);
#pragma omp for schedule(static)
        for (int64_t row = 0; row < n; ++row) {
            const float* xr = x + row * d;
            float ss = 0.0f;
            for (int j = 0; j < d; ++j) ss += xr[j] * xr[j];
            const float nrm = sqrtf(ss);
            norms[row] = nrm;
            const float den = nrm > 1e-10f ? nrm : 1e-10f;
            for (int j = 0; j < d; ++j) xn[j] = xr[j] / den;
            for (int j = 0; j < d; ++j) {
                const float* rr = rot + (int64_t)j * d;
                float y = 0.0f;
                for (int k = 0; k < d; ++k) y += rr[k] * xn[k];
                if (y_out) y_out[row * d + j] = y;
                unsigned idx = 0;
                for (int b = 0; b < nb; ++b) idx += (y > bnd[b]) ? 1u : 0u;
                codes[j] = (uint8_t)idx;
            }
            uint8_t* pr = packed + row * w;
            memset(pr, 0, (size_t)w);
            if (bits == 3) {
                for (int g = 0; g < d / 8; ++g) {
                    unsigned v = 0;
                    for (int i = 0; i < 8; ++i) v |= (unsigned)codes[g * 8 + i] << (3 * i);
                    pr[g * 3] = (uint8_t)v; pr[g * 3 + 1] = (uint8_t)(v >> 8); pr[g * 3 + 2] = (uint8_t)(v >> 16);
                }
            } else {
                const int per = 8 / bits;
                for (int j = 0; j < d; ++j) pr[j / per] |= (uint8_t)(codes[j] << (bits * (j % per)));
            }
        }
        free(xn);
        free(codes);
    }
}

/* turboquant_fused_qk_{2,3,4}bit (kernels.py:439-479, 488-506, 517-548):
 * out[q, k] = norms[k] * sum_j q_rot[q, j] * centroid[idx(k, j)] */
void tqo_qk_scores(const float* q_rot, const uint8_t* packed, const float* norms, const float* cent, int bits, int d,
                   int64_t t_q, int64_t t_kv, float* out) {
    const int w = d * bits / 8;
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < t_kv; ++k) {
        for (int64_t q = 0; q < t_q; ++q) {
            float acc = 0.0f;
            for (int j = 0; j < d; ++j) acc += q_rot[q * d + j] * cent[code_at(packed + k * w, j, bits)];
            out[q * t_kv + k] = norms[k] * acc;
        }
    }
}

/* float32 softmax(scale * q k^T) v with GQA head sharing, one query token per head; stands in for the
 * third-party attention call the reference's consumer makes on the dense cache output.
 * q (B, Hq, D); k, v (B, Hkv, T, D); out (B, Hq, D). */
void tqo_attention(const float* q, const float* k, const float* v, int B, int Hq, int Hkv, int64_t T, int D, float scale,
                   float* out) {
    const int rep = Hq / Hkv;
#pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)T);
#pragma omp for schedule(dynamic, 1)
        for (int bh = 0; bh < B * Hq; ++bh) {
            const int b = bh / Hq, h = bh % Hq;
            const float* qv = q + (int64_t)bh * D;
            const float* kk = k + ((int64_t)b * Hkv + h / rep) * T * D;
            const float* vv = v + ((int64_t)b * Hkv + h / rep) * T * D;
            float mx = -INFINITY;
            for (int64_t t = 0; t < T; ++t) {
                float acc = 0.0f;
                for (int j = 0; j < D; ++j) acc += qv[j] * kk[t * D + j];
                s[t] = acc * scale;
                if (s[t] > mx) mx = s[t];
            }
            float den = 0.0f;
            float* o = out + (int64_t)bh * D;
            for (int j = 0; j < D; ++j) o[j] = 0.0f;
            for (int64_t t = 0; t < T; ++t) {
                const float p = expf(s[t] - mx);
                den += p;
                for (int j = 0; j < D; ++j) o[j] += p * vv[t * D + j];
            }
            for (int j = 0; j < D; ++j) o[j] /= den;
        }
        free(s);
    }
}
