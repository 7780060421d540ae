// Shared host/device helpers for libtq_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/tq_abi.h"

namespace tq {

// ---- thread-local error text -----------------------------------------------------------------
char* err_buf();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline bool bits_ok(int b) { return b >= 1 && b <= 4; }
// bytes per packed row of n codes
__host__ __device__ inline int packed_bytes(int n_codes, int bits) { return n_codes * bits / 8; }

// ---- device helpers --------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float load_as_f32(const void* p, int dtype, int64_t i) {
    if (dtype == TQ_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    if (dtype == TQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_from_f32(void* p, int dtype, int64_t i, float v) {
    if (dtype == TQ_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
    else if (dtype == TQ_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[i] = v;
}

// Code j (0-based) of a packed row, reference layouts (packing.py:37-59, 102-131, 159-173, 197-208).
__device__ __forceinline__ uint32_t code_at(const uint8_t* row, int j, int bits) {
    if (bits == 4) return (row[j >> 1] >> ((j & 1) * 4)) & 15u;
    if (bits == 2) return (row[j >> 2] >> ((j & 3) * 2)) & 3u;
    if (bits == 1) return (row[j >> 3] >> (j & 7)) & 1u;
    const uint8_t* g = row + (j >> 3) * 3;
    uint32_t w = g[0] | (uint32_t(g[1]) << 8) | (uint32_t(g[2]) << 16);
    return (w >> ((j & 7) * 3)) & 7u;
}

// Output byte `b` of a packed row built from unpacked codes c[0..n) (packing.py:9-34, 62-99, 134-194).
__device__ __forceinline__ uint8_t packed_byte_from_codes(const uint8_t* c, int b, int bits) {
    if (bits == 4) return uint8_t(c[2 * b] | (c[2 * b + 1] << 4));
    if (bits == 2) return uint8_t(c[4 * b] | (c[4 * b + 1] << 2) | (c[4 * b + 2] << 4) | (c[4 * b + 3] << 6));
    if (bits == 1) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) v |= uint32_t(c[8 * b + i] & 1u) << i;
        return uint8_t(v);
    }
    const uint8_t* g = c + (b / 3) * 8;
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= uint32_t(g[i] & 7u) << (3 * i);
    return uint8_t(w >> (8 * (b % 3)));
}

}  // namespace tq
