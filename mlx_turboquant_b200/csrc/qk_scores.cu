// Raw QK scores straight from packed keys, single head:
//   out[q, k] = norms[k] * sum_j q_rot[q, j] * centroids[code(k, j)]
// One thread per key token, eight queries per pass held in registers; the query block and the
// centroid table sit in shared memory.
#include "common.cuh"

namespace tq {

constexpr int QK_Q = 8, QK_T = 128;

__global__ void __launch_bounds__(QK_T) qk_scores_kernel(const float* __restrict__ q_rot,
                                                         const uint8_t* __restrict__ packed,
                                                         const float* __restrict__ norms,
                                                         const float* __restrict__ cent, int bits, int d, int64_t t_q,
                                                         int64_t t_kv, float* __restrict__ out) {
    extern __shared__ float sm[];
    float* sq = sm;               // [QK_Q][d]
    float* sc = sm + QK_Q * d;    // [16]
    const int64_t q0 = int64_t(blockIdx.y) * QK_Q;
    const int nq = (t_q - q0) < QK_Q ? int(t_q - q0) : QK_Q;
    for (int e = threadIdx.x; e < QK_Q * d; e += QK_T) {
        const int qi = e / d;
        sq[e] = qi < nq ? q_rot[(q0 + qi) * d + (e - qi * d)] : 0.f;
    }
    if (threadIdx.x < 16) sc[threadIdx.x] = threadIdx.x < (1 << bits) ? cent[threadIdx.x] : 0.f;
    __syncthreads();
    const int64_t k = int64_t(blockIdx.x) * QK_T + threadIdx.x;
    if (k >= t_kv) return;
    const uint8_t* row = packed + k * packed_bytes(d, bits);
    float acc[QK_Q];
#pragma unroll
    for (int i = 0; i < QK_Q; ++i) acc[i] = 0.f;
    for (int j = 0; j < d; ++j) {
        const float c = sc[code_at(row, j, bits)];
#pragma unroll
        for (int i = 0; i < QK_Q; ++i) acc[i] = fmaf(sq[i * d + j], c, acc[i]);
    }
    const float nk = norms[k];
    for (int i = 0; i < nq; ++i) out[(q0 + i) * t_kv + k] = nk * acc[i];
}

}  // namespace tq

using namespace tq;

extern "C" int tq_qk_scores(const float* q_rot, const uint8_t* packed, const float* norms, const float* centroids,
                            int bits, int d, int64_t t_q, int64_t t_kv, float* out, void* stream) {
    if (bits != 2 && bits != 3 && bits != 4) return fail(TQ_ERR_INVALID, "tq_qk_scores: bits=%d (2, 3 or 4)", bits);
    if (d <= 0 || d % 8 || d > 1024 || t_q < 0 || t_kv < 0) return fail(TQ_ERR_INVALID, "tq_qk_scores: bad sizes");
    if (t_q == 0 || t_kv == 0) return TQ_OK;   // empty result, as kernels.py:569-570
    if (!q_rot || !packed || !norms || !centroids || !out) return fail(TQ_ERR_INVALID, "tq_qk_scores: null pointer");
    dim3 grid(unsigned((t_kv + QK_T - 1) / QK_T), unsigned((t_q + QK_Q - 1) / QK_Q));
    const size_t smem = (size_t(QK_Q) * d + 16) * sizeof(float);
    qk_scores_kernel<<<grid, QK_T, smem, static_cast<cudaStream_t>(stream)>>>(q_rot, packed, norms, centroids, bits, d, t_q, t_kv, out);
    return check_launch("tq_qk_scores");
}
