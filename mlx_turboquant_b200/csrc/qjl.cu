// Stand-alone 1-bit quantized Johnson-Lindenstrauss sketch (qjl.py:47-94), float32 on CUDA cores:
//   tq_qjl_quantize    signs[r][p] = (sum_k x[r][k] S[p][k] >= 0),  gamma[r] = |x[r]|
//   tq_qjl_dequantize  out[r][j] = (sqrt(pi/2) / d) * gamma[r] * sum_p (signs[r][p] ? +S[p][j] : -S[p][j])
// S is (m, d) row-major with any m (TurboQuantProd uses m = d, the cache m = 32).  The sketch the cache keeps per token
// is produced inside the fused quantize kernels instead; these two serve the reference's free functions and
// TurboQuantProd (quantizer.py:142-195).
//
// Both kernels: a CTA of 256 threads owns 64 rows; S streams through shared memory 32 projections at a time.
#include "common.cuh"

namespace tq {

namespace qjl {

constexpr int ROWS = 64, NT = 256, PCH = 32, RPW = ROWS / (NT / 32);   // rows per CTA, threads, projections per chunk, rows per warp

// quantize: warp w owns rows 8 w .. 8 w + 7; lane p computes projection p of the chunk for those rows
__global__ void __launch_bounds__(NT) qjl_quantize_kernel(const float* __restrict__ x, const float* __restrict__ proj, uint8_t* __restrict__ signs,
                                                          float* __restrict__ gamma, int64_t n, int d, int m) {
    extern __shared__ __align__(16) float sm[];
    float* xs = sm;                         // [ROWS][d + 1]
    float* ps = xs + ROWS * (d + 1);        // [PCH][d + 1]: lane p reading column k hits bank (p + k) mod 32
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row0 = int64_t(blockIdx.x) * ROWS;
    for (int e = tid; e < ROWS * d; e += NT) {
        const int r = e / d, k = e - r * d;
        xs[r * (d + 1) + k] = row0 + r < n ? x[(row0 + r) * d + k] : 0.f;
    }
    __syncthreads();
    {   // norms: lanes stride the row
        for (int mi = 0; mi < RPW; ++mi) {
            const int r = warp * RPW + mi;
            float ss = 0.f;
            for (int k = lane; k < d; k += 32) { const float v = xs[r * (d + 1) + k]; ss = fmaf(v, v, ss); }
#pragma unroll
            for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            if (lane == 0 && row0 + r < n) gamma[row0 + r] = sqrtf(ss);
        }
    }
    for (int p0 = 0; p0 < m; p0 += PCH) {
        __syncthreads();                    // the previous chunk has been read
        for (int e = tid; e < PCH * d; e += NT) {
            const int pp = e / d, k = e - pp * d;
            ps[pp * (d + 1) + k] = p0 + pp < m ? __ldg(proj + int64_t(p0 + pp) * d + k) : 0.f;
        }
        __syncthreads();
        float dot[RPW];
#pragma unroll
        for (int mi = 0; mi < RPW; ++mi) dot[mi] = 0.f;
        const float* srow = ps + lane * (d + 1);
        const float* x0 = xs + warp * RPW * (d + 1);
        for (int k = 0; k < d; ++k) {
            const float sv = srow[k];
#pragma unroll
            for (int mi = 0; mi < RPW; ++mi) dot[mi] = fmaf(x0[mi * (d + 1) + k], sv, dot[mi]);      // x: broadcast read
        }
        if (p0 + lane < m) {
#pragma unroll
            for (int mi = 0; mi < RPW; ++mi) {
                const int64_t row = row0 + warp * RPW + mi;
                if (row < n) signs[row * m + p0 + lane] = dot[mi] >= 0.f ? 1 : 0;
            }
        }
    }
}

// dequantize: thread j-group owns output columns; the signs of the CTA's rows sit in shared memory as +-1 floats
__global__ void __launch_bounds__(NT) qjl_dequantize_kernel(const uint8_t* __restrict__ signs, const float* __restrict__ gamma, const float* __restrict__ proj,
                                                            float* __restrict__ out, int64_t n, int d, int m, float c) {
    extern __shared__ __align__(16) float sm[];
    float* zs = sm;                         // [ROWS][PCH]: +-1
    float* ps = zs + ROWS * PCH;            // [PCH][d]
    const int tid = threadIdx.x;
    const int64_t row0 = int64_t(blockIdx.x) * ROWS;
    // thread -> column j = tid % d' and a slab of rows; d <= 256 = NT, so threads beyond d idle in the product (d < NT: several row slabs)
    const int slabs = max(NT / d, 1), j = tid % d, slab = tid / d;
    const int rows_per_slab = (ROWS + slabs - 1) / slabs;
    const bool active = slab < slabs;
    float acc[ROWS];                        // only rows_per_slab of them are used (ROWS when d = 256)
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    for (int p0 = 0; p0 < m; p0 += PCH) {
        __syncthreads();
        for (int e = tid; e < ROWS * PCH; e += NT) {
            const int r = e / PCH, pp = e - r * PCH;
            float z = 0.f;
            if (row0 + r < n && p0 + pp < m) z = signs[(row0 + r) * m + p0 + pp] ? 1.f : -1.f;
            zs[e] = z;
        }
        for (int e = tid; e < PCH * d; e += NT) {
            const int pp = e / d, k = e - pp * d;
            ps[e] = p0 + pp < m ? __ldg(proj + int64_t(p0 + pp) * d + k) : 0.f;
        }
        __syncthreads();
        if (active) {
            for (int pp = 0; pp < PCH; ++pp) {
                const float sv = ps[pp * d + j];
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (r < rows_per_slab) acc[r] = fmaf(zs[(slab * rows_per_slab + r) * PCH + pp], sv, acc[r]);     // z: broadcast read
            }
        }
    }
    if (active) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int rr = slab * rows_per_slab + r;
            const int64_t row = row0 + rr;
            if (r < rows_per_slab && rr < ROWS && row < n) out[row * d + j] = c * gamma[row] * acc[r];
        }
    }
}

}  // namespace qjl

}  // namespace tq

using namespace tq;

extern "C" int tq_qjl_quantize(const float* x, const float* proj, uint8_t* signs, float* gamma, int64_t n, int d, int m, void* stream) {
    if (n < 0 || d < 1 || d > 256 || m < 1) return fail(TQ_ERR_INVALID, "tq_qjl_quantize: n=%lld d=%d m=%d (d <= 256)", (long long)n, d, m);
    if (n == 0) return TQ_OK;
    if (!x || !proj || !signs || !gamma) return fail(TQ_ERR_INVALID, "tq_qjl_quantize: null pointer");
    const size_t smem = size_t(qjl::ROWS + qjl::PCH) * (d + 1) * sizeof(float);
    static thread_local size_t cur[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && smem > cur[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qjl::qjl_quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_qjl_quantize: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        cur[dev] = smem;
    }
    const int64_t blocks = (n + qjl::ROWS - 1) / qjl::ROWS;
    if (blocks > 0x7fffffff) return fail(TQ_ERR_INVALID, "tq_qjl_quantize: too many rows");
    qjl::qjl_quantize_kernel<<<unsigned(blocks), qjl::NT, smem, static_cast<cudaStream_t>(stream)>>>(x, proj, signs, gamma, n, d, m);
    return check_launch("tq_qjl_quantize");
}

extern "C" int tq_qjl_dequantize(const uint8_t* signs, const float* gamma, const float* proj, float* out, int64_t n, int d, int m, void* stream) {
    if (n < 0 || d < 1 || d > 256 || m < 1) return fail(TQ_ERR_INVALID, "tq_qjl_dequantize: n=%lld d=%d m=%d (d <= 256)", (long long)n, d, m);
    if (n == 0) return TQ_OK;
    if (!signs || !gamma || !proj || !out) return fail(TQ_ERR_INVALID, "tq_qjl_dequantize: null pointer");
    const size_t smem = (size_t(qjl::ROWS) * qjl::PCH + size_t(qjl::PCH) * d) * sizeof(float);
    static thread_local size_t cur[16] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && smem > cur[dev]) {
        cudaError_t e = cudaFuncSetAttribute(qjl::qjl_dequantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_qjl_dequantize: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        cur[dev] = smem;
    }
    const int64_t blocks = (n + qjl::ROWS - 1) / qjl::ROWS;
    if (blocks > 0x7fffffff) return fail(TQ_ERR_INVALID, "tq_qjl_dequantize: too many rows");
    const float c = 1.2533141373155003f / float(d);      // sqrt(pi / 2) / d, qjl.py:91-92
    qjl::qjl_dequantize_kernel<<<unsigned(blocks), qjl::NT, smem, static_cast<cudaStream_t>(stream)>>>(signs, gamma, proj, out, n, d, m, c);
    return check_launch("tq_qjl_dequantize");
}
