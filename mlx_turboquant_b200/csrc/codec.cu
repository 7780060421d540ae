// Bit-packing codec and scalar quantizer kernels (HBM-bound byte work, no tensor cores).
//
// pack / unpack move 32 codes per thread with 128-bit loads or stores when the buffers allow
// it, and fall back to a one-group-per-thread kernel for ragged sizes or unaligned pointers.
#include <algorithm>

#include "common.cuh"

namespace tq {

static thread_local char g_err[512];
char* err_buf() { return g_err; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return TQ_OK;
}

// ---- 32 codes <-> bits*4 bytes -----------------------------------------------------------------

// Squeeze the four byte-wide codes of `w` into 4*BITS contiguous bits.
template <int BITS> __device__ __forceinline__ uint32_t squeeze4(uint32_t w) {
    constexpr uint32_t m = (1u << BITS) - 1u;
    return (w & m) | ((w >> (8 - BITS)) & (m << BITS)) | ((w >> (16 - 2 * BITS)) & (m << (2 * BITS))) |
           ((w >> (24 - 3 * BITS)) & (m << (3 * BITS)));
}
// Inverse: spread 4*BITS bits into four byte-wide codes.
template <int BITS> __device__ __forceinline__ uint32_t spread4(uint32_t v) {
    constexpr uint32_t m = (1u << BITS) - 1u;
    return (v & m) | (((v >> BITS) & m) << 8) | (((v >> (2 * BITS)) & m) << 16) | (((v >> (3 * BITS)) & m) << 24);
}

template <int BITS>
__global__ void __launch_bounds__(256) pack32_kernel(const uint4* __restrict__ idx, uint32_t* __restrict__ out,
                                                     int64_t n_groups) {
    int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (g >= n_groups) return;
    uint4 a = __ldg(idx + 2 * g), b = __ldg(idx + 2 * g + 1);
    uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t* o = out + g * BITS;
    if (BITS == 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = squeeze4<4>(w[2 * k]) | (squeeze4<4>(w[2 * k + 1]) << 16);
    } else if (BITS == 2) {
#pragma unroll
        for (int k = 0; k < 2; ++k)
            o[k] = squeeze4<2>(w[4 * k]) | (squeeze4<2>(w[4 * k + 1]) << 8) | (squeeze4<2>(w[4 * k + 2]) << 16) |
                   (squeeze4<2>(w[4 * k + 3]) << 24);
    } else if (BITS == 1) {
        uint32_t v = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) v |= squeeze4<1>(w[k]) << (4 * k);
        o[0] = v;
    } else {  // 3-bit: four 24-bit groups -> three words
        uint32_t q[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = squeeze4<3>(w[2 * k]) | (squeeze4<3>(w[2 * k + 1]) << 12);
        o[0] = q[0] | (q[1] << 24);
        o[1] = (q[1] >> 8) | (q[2] << 16);
        o[2] = (q[2] >> 16) | (q[3] << 8);
    }
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack32_kernel(const uint32_t* __restrict__ in, uint4* __restrict__ idx,
                                                       int64_t n_groups) {
    int64_t g = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (g >= n_groups) return;
    const uint32_t* p = in + g * BITS;
    uint32_t w[8];
    if (BITS == 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint32_t v = __ldg(p + k);
            w[2 * k] = spread4<4>(v & 0xFFFFu);
            w[2 * k + 1] = spread4<4>(v >> 16);
        }
    } else if (BITS == 2) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            uint32_t v = __ldg(p + k);
#pragma unroll
            for (int j = 0; j < 4; ++j) w[4 * k + j] = spread4<2>((v >> (8 * j)) & 0xFFu);
        }
    } else if (BITS == 1) {
        uint32_t v = __ldg(p);
#pragma unroll
        for (int k = 0; k < 8; ++k) w[k] = spread4<1>((v >> (4 * k)) & 0xFu);
    } else {
        uint32_t a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
        uint32_t q[4] = {a & 0xFFFFFFu, (a >> 24) | ((b & 0xFFFFu) << 8), (b >> 16) | ((c & 0xFFu) << 16), c >> 8};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            w[2 * k] = spread4<3>(q[k] & 0xFFFu);
            w[2 * k + 1] = spread4<3>(q[k] >> 12);
        }
    }
    idx[2 * g] = make_uint4(w[0], w[1], w[2], w[3]);
    idx[2 * g + 1] = make_uint4(w[4], w[5], w[6], w[7]);
}

// Ragged / unaligned fallback: one thread per output byte (pack) or per code (unpack).
__global__ void pack_bytes_kernel(const uint8_t* __restrict__ idx, uint8_t* __restrict__ out, int64_t n, int d,
                                  int bits) {
    const int w = packed_bytes(d, bits);
    int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (i >= n * w) return;
    int64_t row = i / w;
    out[i] = packed_byte_from_codes(idx + row * d, int(i - row * w), bits);
}

__global__ void unpack_codes_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ idx, int64_t n, int d,
                                    int bits) {
    const int w = packed_bytes(d, bits);
    int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (i >= n * d) return;
    int64_t row = i / d;
    idx[i] = uint8_t(code_at(in + row * w, int(i - row * d), bits));
}

// ---- scalar quantizer --------------------------------------------------------------------------

__global__ void __launch_bounds__(256) quantize_scalar_kernel(const float* __restrict__ y,
                                                              const float* __restrict__ bnd, int n_bnd,
                                                              uint8_t* __restrict__ idx, int64_t count, int vec) {
    __shared__ float sb[256];
    for (int i = threadIdx.x; i < n_bnd; i += blockDim.x) sb[i] = bnd[i];
    __syncthreads();
    int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (vec) {  // 8 values per thread, 2x128-bit loads, one 64-bit store
        if (t * 8 >= count) return;
        float4 a = __ldg(reinterpret_cast<const float4*>(y) + 2 * t);
        float4 b = __ldg(reinterpret_cast<const float4*>(y) + 2 * t + 1);
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t c[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int k = 0; k < n_bnd; ++k) {
            float bk = sb[k];
#pragma unroll
            for (int j = 0; j < 8; ++j) c[j] += (v[j] > bk) ? 1u : 0u;
        }
        uint2 o;
        o.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
        o.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
        reinterpret_cast<uint2*>(idx)[t] = o;
    } else {
        if (t >= count) return;
        float v = y[t];
        uint32_t c = 0;
        for (int k = 0; k < n_bnd; ++k) c += (v > sb[k]) ? 1u : 0u;
        idx[t] = uint8_t(c);
    }
}

__global__ void __launch_bounds__(256) dequantize_scalar_kernel(const uint8_t* __restrict__ idx,
                                                                const float* __restrict__ cent, int n_cent,
                                                                float* __restrict__ out, int64_t count, int vec) {
    __shared__ float sc[256];
    for (int i = threadIdx.x; i < 256; i += blockDim.x) sc[i] = (i < n_cent) ? cent[i] : 0.f;
    __syncthreads();
    int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (vec) {
        if (t * 4 >= count) return;
        uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(idx) + t);
        reinterpret_cast<float4*>(out)[t] =
            make_float4(sc[w & 255u], sc[(w >> 8) & 255u], sc[(w >> 16) & 255u], sc[w >> 24]);
    } else {
        if (t >= count) return;
        out[t] = sc[idx[t]];
    }
}

// Boundary count + pack for eight consecutive coordinates of one row; one thread per group of 8.
__global__ void __launch_bounds__(256) quantize_rotated_kernel(const float* __restrict__ y, int64_t n, int d,
                                                               const float* __restrict__ bnd_hi, int bits_hi,
                                                               const float* __restrict__ bnd_lo, int bits_lo,
                                                               uint8_t* __restrict__ p_hi, uint8_t* __restrict__ p_lo) {
    __shared__ float sb[2][16];
    if (threadIdx.x < 32) {
        int s = threadIdx.x >> 4, k = threadIdx.x & 15;
        const float* src = s ? bnd_lo : bnd_hi;
        int nb = (1 << (s ? bits_lo : bits_hi)) - 1;
        sb[s][k] = (src != nullptr && k < nb) ? src[k] : 0.f;
    }
    __syncthreads();
    const int gpr = d / 8;  // groups per row
    int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
    if (t >= n * gpr) return;
    int64_t row = t / gpr;
    int g = int(t - row * gpr);
    const int half = bits_lo ? d / 2 : d;
    const int side = (g * 8 >= half) ? 1 : 0;
    const int bits = side ? bits_lo : bits_hi;
    const int nb = (1 << bits) - 1;
    const float* yr = y + row * d + g * 8;
    uint8_t c[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float v = yr[j];
        uint32_t k = 0;
        for (int b = 0; b < nb; ++b) k += (v > sb[side][b]) ? 1u : 0u;
        c[j] = uint8_t(k);
    }
    const int cols = side ? d - half : half;
    const int gl = side ? g - half / 8 : g;  // group index inside this packed array
    uint8_t* dst = (side ? p_lo : p_hi) + row * packed_bytes(cols, bits) + gl * bits;
    for (int b = 0; b < bits; ++b) dst[b] = packed_byte_from_codes(c, b, bits);
}

static inline unsigned blocks_for(int64_t work, int per_block) { return unsigned((work + per_block - 1) / per_block); }

}  // namespace tq

using namespace tq;

extern "C" int tq_version(void) { return TQ_ABI_VERSION; }
extern "C" const char* tq_last_error(void) { return err_buf(); }

extern "C" int tq_pack(const uint8_t* idx, uint8_t* packed, int64_t n, int d, int bits, void* stream) {
    if (!bits_ok(bits)) return fail(TQ_ERR_INVALID, "Unsupported bit-width: %d. Use 1, 2, 3, or 4.", bits);
    const int per = bits == 4 ? 2 : bits == 2 ? 4 : 8;
    if (n < 0 || d <= 0 || d % per) return fail(TQ_ERR_INVALID, "Last dimension %d must be divisible by %d for %d-bit packing", d, per, bits);
    if (n == 0) return TQ_OK;
    if (!idx || !packed) return fail(TQ_ERR_INVALID, "tq_pack: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t total = n * int64_t(d);
    if (total % 32 == 0 && aligned(idx, 16) && aligned(packed, 4)) {
        const int64_t g = total / 32;
        const unsigned nb = blocks_for(g, 256);
        if (bits == 4) pack32_kernel<4><<<nb, 256, 0, s>>>(reinterpret_cast<const uint4*>(idx), reinterpret_cast<uint32_t*>(packed), g);
        else if (bits == 3) pack32_kernel<3><<<nb, 256, 0, s>>>(reinterpret_cast<const uint4*>(idx), reinterpret_cast<uint32_t*>(packed), g);
        else if (bits == 2) pack32_kernel<2><<<nb, 256, 0, s>>>(reinterpret_cast<const uint4*>(idx), reinterpret_cast<uint32_t*>(packed), g);
        else pack32_kernel<1><<<nb, 256, 0, s>>>(reinterpret_cast<const uint4*>(idx), reinterpret_cast<uint32_t*>(packed), g);
    } else {
        pack_bytes_kernel<<<blocks_for(n * packed_bytes(d, bits), 256), 256, 0, s>>>(idx, packed, n, d, bits);
    }
    return check_launch("tq_pack");
}

extern "C" int tq_unpack(const uint8_t* packed, uint8_t* idx, int64_t n, int d, int bits, void* stream) {
    if (!bits_ok(bits)) return fail(TQ_ERR_INVALID, "Unsupported bit-width: %d. Use 1, 2, 3, or 4.", bits);
    const int per = bits == 4 ? 2 : bits == 2 ? 4 : 8;
    if (n < 0 || d <= 0 || d % per) return fail(TQ_ERR_INVALID, "Last dimension %d must be divisible by %d for %d-bit packing", d, per, bits);
    if (n == 0) return TQ_OK;
    if (!idx || !packed) return fail(TQ_ERR_INVALID, "tq_unpack: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t total = n * int64_t(d);
    if (total % 32 == 0 && aligned(idx, 16) && aligned(packed, 4)) {
        const int64_t g = total / 32;
        const unsigned nb = blocks_for(g, 256);
        if (bits == 4) unpack32_kernel<4><<<nb, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint4*>(idx), g);
        else if (bits == 3) unpack32_kernel<3><<<nb, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint4*>(idx), g);
        else if (bits == 2) unpack32_kernel<2><<<nb, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint4*>(idx), g);
        else unpack32_kernel<1><<<nb, 256, 0, s>>>(reinterpret_cast<const uint32_t*>(packed), reinterpret_cast<uint4*>(idx), g);
    } else {
        unpack_codes_kernel<<<blocks_for(total, 256), 256, 0, s>>>(packed, idx, n, d, bits);
    }
    return check_launch("tq_unpack");
}

extern "C" int tq_quantize_scalar(const float* y, const float* boundaries, int n_bnd, uint8_t* idx, int64_t count,
                                  void* stream) {
    if (n_bnd < 0 || n_bnd > 255 || count < 0) return fail(TQ_ERR_INVALID, "tq_quantize_scalar: n_bnd=%d count=%lld", n_bnd, (long long)count);
    if (count == 0) return TQ_OK;
    if (!y || !idx || (n_bnd && !boundaries)) return fail(TQ_ERR_INVALID, "tq_quantize_scalar: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec = (count % 8 == 0 && aligned(y, 16) && aligned(idx, 8)) ? 1 : 0;
    quantize_scalar_kernel<<<blocks_for(vec ? count / 8 : count, 256), 256, 0, s>>>(y, boundaries, n_bnd, idx, count, vec);
    return check_launch("tq_quantize_scalar");
}

extern "C" int tq_dequantize_scalar(const uint8_t* idx, const float* centroids, int n_cent, float* out, int64_t count,
                                    void* stream) {
    if (n_cent <= 0 || n_cent > 256 || count < 0) return fail(TQ_ERR_INVALID, "tq_dequantize_scalar: n_cent=%d", n_cent);
    if (count == 0) return TQ_OK;
    if (!idx || !centroids || !out) return fail(TQ_ERR_INVALID, "tq_dequantize_scalar: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vec = (count % 4 == 0 && aligned(idx, 4) && aligned(out, 16)) ? 1 : 0;
    dequantize_scalar_kernel<<<blocks_for(vec ? count / 4 : count, 256), 256, 0, s>>>(idx, centroids, n_cent, out, count, vec);
    return check_launch("tq_dequantize_scalar");
}

extern "C" int tq_quantize_from_rotated(const float* y, int64_t n, int d, const float* bnd_hi, int bits_hi,
                                        const float* bnd_lo, int bits_lo, uint8_t* packed_hi, uint8_t* packed_lo,
                                        void* stream) {
    if (!bits_ok(bits_hi) || (bits_lo && !bits_ok(bits_lo))) return fail(TQ_ERR_INVALID, "Unsupported bit-width: %d/%d. Use 1, 2, 3, or 4.", bits_hi, bits_lo);
    if (n < 0 || d <= 0 || d % (bits_lo ? 16 : 8)) return fail(TQ_ERR_INVALID, "tq_quantize_from_rotated: d=%d must be a multiple of %d", d, bits_lo ? 16 : 8);
    if (n == 0) return TQ_OK;
    if (!y || !bnd_hi || !packed_hi || (bits_lo && (!bnd_lo || !packed_lo))) return fail(TQ_ERR_INVALID, "tq_quantize_from_rotated: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    quantize_rotated_kernel<<<blocks_for(n * (d / 8), 256), 256, 0, s>>>(y, n, d, bnd_hi, bits_hi, bnd_lo, bits_lo, packed_hi, packed_lo);
    return check_launch("tq_quantize_from_rotated");
}

// ---- append rows to the uncompressed token buffers ------------------------------------------------------
namespace tq {
// One launch copies the new rows of keys AND values: thread -> (tensor, lane, row, 16-byte chunk).
__global__ void append_rows_kernel(const uint4* __restrict__ k_new, const uint4* __restrict__ v_new, uint4* __restrict__ k_buf,
                                   uint4* __restrict__ v_buf, int64_t lanes, int64_t t_new, int chunks, int64_t src_ls, int64_t dst_ls,
                                   int64_t dst_row0) {
    const int64_t total = 2 * lanes * t_new * chunks;
    for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const int c = int(i % chunks);
        int64_t r = i / chunks;
        const int64_t row = r % t_new; r /= t_new;
        const int64_t lane = r % lanes;
        const bool is_v = r >= lanes;
        const uint4* src = (is_v ? v_new : k_new) + (lane * src_ls + row) * chunks + c;
        uint4* dst = (is_v ? v_buf : k_buf) + (lane * dst_ls + dst_row0 + row) * chunks + c;
        *dst = __ldg(src);
    }
}
}  // namespace tq

extern "C" int tq_append_tokens(const void* k_new, const void* v_new, void* k_buf, void* v_buf, int64_t lanes, int64_t t_new,
                                int64_t row_bytes, int64_t src_lane_stride, int64_t dst_lane_stride, int64_t dst_row0, void* stream) {
    using namespace tq;
    if (lanes < 0 || t_new < 0 || row_bytes <= 0 || dst_row0 < 0 || src_lane_stride < t_new || dst_lane_stride < dst_row0 + t_new)
        return fail(TQ_ERR_INVALID, "tq_append_tokens: bad sizes");
    if (lanes == 0 || t_new == 0) return TQ_OK;
    if (!k_new || !v_new || !k_buf || !v_buf) return fail(TQ_ERR_INVALID, "tq_append_tokens: null pointer");
    if (row_bytes % 16 || !aligned(k_new, 16) || !aligned(v_new, 16) || !aligned(k_buf, 16) || !aligned(v_buf, 16))
        return fail(TQ_ERR_UNSUPPORTED, "tq_append_tokens: rows must be multiples of 16 bytes at 16-byte aligned addresses");
    const int chunks = int(row_bytes / 16);
    const int64_t total = 2 * lanes * t_new * chunks;
    const int threads = 256;
    const unsigned blocks = unsigned(std::min<int64_t>((total + threads - 1) / threads, 148 * 8));
    append_rows_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(k_new), static_cast<const uint4*>(v_new), static_cast<uint4*>(k_buf), static_cast<uint4*>(v_buf),
        lanes, t_new, chunks, src_lane_stride, dst_lane_stride, dst_row0);
    return check_launch("tq_append_tokens");
}
