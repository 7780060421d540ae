// Declarations shared by the decode-attention translation units.
#pragma once

#include "common.cuh"

namespace tq {

__host__ __device__ constexpr int warps_per_cta(bool direct) { return direct ? 16 : 8; }   // warps per CTA
constexpr int TILE = 16;              // tokens per warp tile
constexpr int HPG = 8;                // query heads per head group (the mma N dimension)
constexpr int MAX_SPLITS = 512;
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
    float *part_o, *part_ml;           // workspace: (B, Hkv, HG, S, slots, D) and (B, Hkv, HG, S, slots, 2)
    int* counters;                     // workspace: (B, Hkv, HG) arrival counters, zero between launches
    void* out; int out_dtype;
};

// Validates the arguments, picks the path and the split plan and fills the kernel parameters for the given
// scratch buffer (which must be zero-filled before its first use; the kernel leaves its counters at zero).
int decode_prepare(const tq_decode_args* a, void* workspace, size_t workspace_bytes, DecodeParams* out, bool* direct_out);
int decode_launch(const DecodeParams& p, bool direct, cudaStream_t s);

}  // namespace tq
