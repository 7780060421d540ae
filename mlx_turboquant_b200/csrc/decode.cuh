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
    // streaming kernel (decode_stream.cu): every warp of a persistent grid walks its own contiguous run of the packed
    // tiles of all cache lanes; partials per (lane, slot) and the prepared queries live in the workspace
    int st_grid;                       // CTAs of the persistent grid (0: another kernel runs)
    int st_npp, st_nd, st_dt;          // packed-partial slots per lane; dense items per lane and tiles per dense item
    int64_t st_range;                  // packed tiles per warp
    __half* st_q16;                    // workspace: per query head [rotated | raw | sketch] scaled fp16 query
    float* st_part;                    // workspace: partials (lane, slot, head, D + 36)
};

// Constants of the 4-bit-key / 2-bit-value kernels in global memory, built once per (rotation, codebooks) by
// tq_decode_tables_build: the 64 KB image of the shared-memory lookup tables (slot e at e * 256: 32 copies of
// half2(kc[e & 15], kc[e >> 4]), then 16 copies of the value entry) and, for d = 128, R split into two fp16 matrices in
// mma A-fragment order.
namespace dd {
constexpr uint32_t TABLES_MAGIC = 0x54513432u;
struct DirectTables {
    uint32_t magic; int d, kb, vb; float v_scale; uint32_t pad[59];          // 256 B
    uint4 lut[256 * 16];                                       // image of the shared-memory tables (64 KB)
    uint4 rfrag[8 * 8 * 2 * 32];                               // d = 128: [warp][k-step][hi | lo][lane] mma A fragments of R_hi, R_lo (64 KB)
};
static_assert(sizeof(DirectTables) == 256 + 65536 + 65536, "table buffer layout");
constexpr uint32_t LO_BASE = 2048u;                            // lowest shared-window address the kernels use
constexpr uint32_t LUT_BASE = 0x10000u;                        // 256 slots of 256 B, addressed by one byte-permute
constexpr uint32_t C_BASE = 0x20000u;                          // first byte above the tables
unsigned probe_smem_base();                                    // shared-window address where dynamic shared memory starts (~0u on error)
}  // namespace dd

// Validates the arguments, picks the path and the split plan and fills the kernel parameters for the given
// scratch buffer (which must be zero-filled before its first use; the kernel leaves its counters at zero).
int decode_prepare(const tq_decode_args* a, void* workspace, size_t workspace_bytes, DecodeParams* out, bool* direct_out,
                   const void* k_new = nullptr, const void* v_new = nullptr);
int decode_launch(const DecodeParams& p, bool direct, cudaStream_t s);
// Scratch the general and the table-lookup kernel need for these sizes (the streaming kernel may need more; a call whose
// workspace is too small for it takes one of the other two).
size_t decode_workspace_bytes_split_kernels(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len, int64_t dense_len);

// decode_direct.cu: the kernel for 4-bit keys / 2-bit values at d = 128.  direct_supported() checks once per
// device (one tiny synchronous probe launch on first use) that the kernel's shared-memory plan fits the device.
bool direct_supported();
size_t direct_tables_bytes();
int direct_tables_build(int d, const float* rot, const float* k_cent, const float* v_cent, float v_scale, void* tables, cudaStream_t s);
int launch_decode_direct(const DecodeParams& p, cudaStream_t s);
// decode_stream.cu: persistent kernel for 4-bit keys / 2-bit values at d = 96 / 128 (sign sketches optional) when the
// packed tokens of all lanes amount to many tiles per warp.
struct StreamPlan { int grid, npp, nd, dt; int64_t range; size_t q16_bytes, part_bytes; };
bool stream_supported(int d, bool qjl);
StreamPlan stream_plan(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len, int64_t dense_len, int sms);
int launch_decode_stream(const DecodeParams& p, cudaStream_t s);
int launch_gather_wait(const unsigned long long* ll, const unsigned* epochs, int64_t n_words, void* out, int max_polls, cudaStream_t s);
int* decode_status_ptr();          // device address of the status word on the current device (null on error)
int decode_status_host();          // code of the first bounded wait that ran out on this device (0 = none), -1 on error

}  // namespace tq
