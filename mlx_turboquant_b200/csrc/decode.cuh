// Declarations shared by the decode-attention translation units.
#pragma once

#include "common.cuh"

namespace tq {

constexpr int DIRECT_WARPS = 16;     // warps per CTA of the 4-bit-key / 2-bit-value kernel
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
    const float* qjl_proj;             // S (32, D), or null: no QJL sketches
    const uint32_t *k_qbits, *v_qbits; // sign words of the residual sketches, one per packed token
    const float *k_qgamma, *v_qgamma;  // residual norms
    int dense_dtype;
    const void *sink_k, *sink_v, *res_k, *res_v;
    int64_t sink_len, sink_ls, res_len, res_ls;
    const void *k_new, *v_new;         // one new row per cache lane to append at row res_len and attend to (or null)
    void *res_k_w, *res_v_w;           // the recent-token buffers, writable (append)
    int n_ps, n_ds;                    // packed / dense splits
    int64_t p_tps, d_tps;              // tiles per split
    const void* q; int q_dtype; float scale; const float* rot;
    float v_scale_hi, v_scale_lo;      // value centroids are multiplied by this before the fp16 cast (undone in the merge)
    float *part_o, *part_ml;           // workspace: (B, Hkv, HG, S, slots, D) and (B, Hkv, HG, S, slots, 2)
    int* counters;                     // workspace: (B, Hkv, HG) arrival counters, zero between launches
    void* out; int out_dtype;
    int pdl;                           // launch with programmatic stream serialisation
    int words_ok;                      // packed key / value rows start on 4-byte boundaries
    const void* tables;                // prebuilt constants of the direct kernel (decode_direct.cu: DirectTables), or null
    // fused gather (n_peers > 0): the merging CTAs send their heads, as {payload, epoch} words, into every peer's landing
    // buffer at the place of head index head_offset + local head
    int n_peers, heads_total, head_offset;
    unsigned long long* peer_ll[TQ_MAX_PEERS];
    unsigned* epochs;                  // this GPU's call counts per (sequence, KV head, head group) of the slot
    // wait for an earlier call's gather before the query is read (or null): every word of the landing buffer carries
    // the epoch of that call; the first CTA also unpacks it into await_out
    const unsigned long long* await_ll;
    const unsigned* await_epochs;
    int64_t await_words;
    void* await_out;
    int await_polls;
    int* status;                       // the device's status word (first bounded wait that ran out)
};

// Validates the arguments, picks the path and the split plan and fills the kernel parameters for the given
// scratch buffer (which must be zero-filled before its first use; the kernel leaves its counters at zero).
int decode_prepare(const tq_decode_args* a, void* workspace, size_t workspace_bytes, DecodeParams* out, bool* direct_out,
                   const void* k_new = nullptr, const void* v_new = nullptr);
int decode_launch(const DecodeParams& p, bool direct, cudaStream_t s);

// decode_direct.cu: the kernel for 4-bit keys / 2-bit values at d = 128.  direct_supported() checks once per
// device (one tiny synchronous probe launch on first use) that the kernel's shared-memory plan fits the device.
bool direct_supported();
size_t direct_tables_bytes();
int direct_tables_build(const float* rot, const float* k_cent, const float* v_cent, float v_scale, void* tables, cudaStream_t s);
int launch_decode_direct(const DecodeParams& p, cudaStream_t s);
int launch_gather_wait(const unsigned long long* ll, const unsigned* epochs, int64_t n_words, void* out, int max_polls, cudaStream_t s);
int* decode_status_ptr();          // device address of the status word on the current device (null on error)
int decode_status_host();          // code of the first bounded wait that ran out on this device (0 = none), -1 on error

}  // namespace tq
