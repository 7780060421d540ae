/*
 * tq_abi.h - C ABI of libtq_b200.so: TurboQuant KV-cache compression and attention over the
 * compressed cache, as hand-written sm_100a CUDA kernels.
 *
 * The reference (alex-rentel/mlx-turboquant v1.0.4) is pure Python on MLX and has no FFI; each
 * entry point below names the reference function whose device-side work it replaces
 * (file:line inside that project).
 *
 * Conventions
 *   - Every pointer is a caller-owned DEVICE pointer unless it is marked "host".
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = legacy
 *     default stream) and allocates nothing.  Exceptions, both once per device and both to be
 *     made outside stream capture: tq_decode_tables_build synchronises (it also measures where
 *     the device places dynamic shared memory), and so does the first tq_decode_attn on a device
 *     when no tables were ever built there.
 *   - Calls act on the device that is current when they are made; pointers must belong to it.
 *   - Return value: TQ_OK or a negative TQ_ERR_*; tq_last_error() gives the thread-local text.
 *     Nothing throws, aborts or traps.
 *   - "rows" are vectors of length d.  Row r of lane o lives at
 *     base + o*lane_stride + r*row_stride (strides in ELEMENTS of that array; packed arrays
 *     count strides in rows of their own byte width).
 *   - Packed byte layouts are the reference's (packing.py:9-208): 4-bit v0|v1<<4; 2-bit
 *     v0|v1<<2|v2<<4|v3<<6; 1-bit bit i = v_i; 3-bit 8 codes -> 3 bytes little-endian.
 *   - bits_lo == 0 means integer bit-width (one packed array, bits_hi for all d coordinates).
 *     bits_lo > 0 is the reference's fractional mode (cache.py:253-274): coordinates
 *     [0, d/2) at bits_hi into packed_hi, [d/2, d) at bits_lo into packed_lo.
 */
#ifndef TQ_ABI_H
#define TQ_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TQ_ABI_VERSION 2

enum { TQ_OK = 0, TQ_ERR_INVALID = -1, TQ_ERR_UNSUPPORTED = -2, TQ_ERR_LAUNCH = -3, TQ_ERR_TIMEOUT = -4 };
enum { TQ_F16 = 0, TQ_BF16 = 1, TQ_F32 = 2 };

/* Library / ABI version (TQ_ABI_VERSION). */
int tq_version(void);
/* Text of the last error on the calling thread ("" if none). Host pointer, owned by the library. */
const char* tq_last_error(void);

/* ---- codec ------------------------------------------------------------------------------ */

/* pack_indices (packing.py:211-222): idx (n, d) u8 -> packed (n, d*bits/8) u8, bits in 1..4. */
int tq_pack(const uint8_t* idx, uint8_t* packed, int64_t n, int d, int bits, void* stream);
/* unpack_indices (packing.py:225-236). */
int tq_unpack(const uint8_t* packed, uint8_t* idx, int64_t n, int d, int bits, void* stream);
/* quantize_scalar (codebook.py:203-225): idx = #{b : y > boundary_b}; n_bnd <= 255. */
int tq_quantize_scalar(const float* y, const float* boundaries, int n_bnd, uint8_t* idx, int64_t count,
                       void* stream);
/* dequantize_scalar (codebook.py:228-238): out = centroids[idx]. */
int tq_dequantize_scalar(const uint8_t* idx, const float* centroids, int n_cent, float* out, int64_t count,
                         void* stream);
/* quantize_scalar + pack_indices on already-rotated float32 rows (cache.py:249-250, 269-273).
 * Bit-exact with the reference given the same y. */
int tq_quantize_from_rotated(const float* y, int64_t n, int d, const float* bnd_hi, int bits_hi,
                             const float* bnd_lo, int bits_lo, uint8_t* packed_hi, uint8_t* packed_lo,
                             void* stream);

/* ---- rotation --------------------------------------------------------------------------- */

/* rotate / pre_rotate_query (rotation.py:55-65, 81-110): out = x @ R^T; inverse != 0 gives
 * inverse_rotate (rotation.py:68-78): out = x @ R.  x (n, d) of x_dtype, rot (d, d) f32, out f32. */
int tq_rotate(const void* x, int x_dtype, const float* rot, float* out, int64_t n, int d, int inverse,
              void* stream);

/* ---- quantize: norm -> normalise -> rotate -> boundary count -> pack ---------------------- */

typedef struct {
    const void* x;            /* (n_lanes, n_rows, d) of x_dtype */
    int x_dtype;              /* TQ_F16 / TQ_BF16 / TQ_F32 */
    int d;                    /* 64, 96, 128 or 256 (any multiple of 16 up to 256) */
    int64_t n_lanes, n_rows;  /* lanes = batch*kv_heads, rows = tokens of this chunk */
    int64_t x_lane_stride, x_row_stride; /* elements */
    const float* rot;         /* (d, d) float32, row-major */
    const float* bnd_hi; int bits_hi;    /* 2^bits_hi - 1 boundaries, non-decreasing (a codebook's are; the kernels search them) */
    const float* bnd_lo; int bits_lo;    /* 0 = integer mode */
    uint8_t* packed_hi;       /* row (o, r) at packed_hi + (o*out_lane_stride + r)*width_hi */
    uint8_t* packed_lo;       /* fractional mode only */
    float* norms;             /* (o*out_lane_stride + r) */
    int64_t out_lane_stride;  /* rows */
    /* optional 1-bit QJL sketch of the residual (cache.py:396-427, qjl.py:47-67); NULL = off.
     * qjl_proj_rot is S @ R^T (m, d) float32 with m == 32; centroids are needed for the residual. */
    const float* qjl_proj_rot; const float* cent_hi; const float* cent_lo;
    uint32_t* qjl_bits;       /* bit i = sign of projection i (1 = non-negative) */
    float* qjl_gamma;         /* ||x - dequant(x)|| */
    float* y_out;             /* optional (n_lanes*n_rows, d) float32 rotated rows, or NULL */
} tq_quantize_args;

/* TurboQuantMSE.quantize / cache._quantize_kv(_fractional) (quantizer.py:54-85, cache.py:232-274);
 * metal_quantize_4bit (kernels.py:363-409). */
int tq_quantize_pack(const tq_quantize_args* a, void* stream);

/* The tensor-core quantize kernel (fp16 rows, d = 128) and the 4-bit-key / 2-bit-value decode kernel wait on
 * mbarriers with an iteration limit; if a wait ever runs out the kernel drains and finishes, and this returns the
 * code of the first such wait on the current device (quantize 1-9, decode 101-103 and 106-108, several-query-token attention 104, dequantize 105, gather wait 201; 0 = none).  Synchronises the
 * device; no reference counterpart. */
int tq_device_status(void);
/* Back to 0 (after the caller has dealt with a reported time-out). */
int tq_device_status_clear(void);

/* ---- dequantize: unpack -> centroid -> inverse rotation -> scale ------------------------- */

typedef struct {
    const uint8_t* packed_hi; const uint8_t* packed_lo; const float* norms;
    int64_t n_lanes, n_rows, in_lane_stride;  /* rows */
    int d; int bits_hi, bits_lo;
    const float* cent_hi; const float* cent_lo; const float* rot;
    /* optional QJL correction added to the output (qjl.py:70-94): S (m, d), m == 32 */
    const float* qjl_proj; const uint32_t* qjl_bits; const float* qjl_gamma;
    void* out; int out_dtype; int64_t out_lane_stride, out_row_stride; /* elements */
} tq_dequantize_args;

/* TurboQuantMSE.dequantize / cache._dequantize_kv(_fractional) / metal_dequantize
 * (quantizer.py:87-109, cache.py:276-343, kernels.py:313-360). */
int tq_dequantize(const tq_dequantize_args* a, void* stream);

/* ---- QJL sketch ---------------------------------------------------------------------------- */

/* qjl_quantize (qjl.py:47-67): signs[r][p] = (x[r] . S[p] >= 0) as one byte (0 / 1) each, gamma[r] = |x[r]|.
 * x (n, d) float32, proj S (m, d) float32, d <= 256, any m. */
int tq_qjl_quantize(const float* x, const float* proj, uint8_t* signs, float* gamma, int64_t n, int d, int m, void* stream);
/* qjl_dequantize (qjl.py:70-94): out[r] = (sqrt(pi/2) / d) * gamma[r] * (z[r] @ S), z = +1 where signs != 0, else -1. */
int tq_qjl_dequantize(const uint8_t* signs, const float* gamma, const float* proj, float* out, int64_t n, int d, int m,
                      void* stream);

/* ---- fused QK scores --------------------------------------------------------------------- */

/* fused_qk_scores_{2,3,4}bit (kernels.py:558-629): out[q,k] = norms[k] * sum_j q_rot[q,j]*c[idx(k,j)];
 * raw scores, single head. q_rot (t_q, d) f32, packed (t_kv, d*bits/8), out (t_q, t_kv) f32. */
int tq_qk_scores(const float* q_rot, const uint8_t* packed, const float* norms, const float* centroids,
                 int bits, int d, int64_t t_q, int64_t t_kv, float* out, void* stream);

/* ---- uncompressed token buffers ------------------------------------------------------------ */

/* Appends t_new rows per lane to the key AND value buffers of the residual window (or the sink) in one launch:
 * dst[(lane * dst_lane_stride + dst_row0 + r)] = src[(lane * src_lane_stride + r)], rows of row_bytes bytes
 * (a multiple of 16; all pointers 16-byte aligned).  The slice assignments of update_and_fetch
 * (cache.py:632-672, 577-618). */
int tq_append_tokens(const void* k_new, const void* v_new, void* k_buf, void* v_buf, int64_t lanes, int64_t t_new,
                     int64_t row_bytes, int64_t src_lane_stride, int64_t dst_lane_stride, int64_t dst_row0, void* stream);

/* ---- decode attention over [fp16 sink | packed middle | fp16 residual] ------------------- */

struct tq_peer_gather;

typedef struct {
    int batch, n_q_heads, n_kv_heads, d;
    const void* q; int q_dtype;              /* (batch, n_q_heads, d): one query token */
    float scale;                             /* softmax scale, normally d^-0.5 */
    const float* rot;                        /* (d, d) */
    /* packed middle: lane = b*n_kv_heads + h, token t at row lane*c_lane_stride + t */
    int64_t c_len, c_lane_stride;
    int k_bits_hi, k_bits_lo, v_bits_hi, v_bits_lo;
    const uint8_t *k_hi, *k_lo, *v_hi, *v_lo;
    const float *k_norms, *v_norms;
    const float *k_cent_hi, *k_cent_lo, *v_cent_hi, *v_cent_lo;
    /* The kernel holds value centroids in fp16; a table-wide scale from tq_fp16_table_scale() applied
     * before the cast (and divided out of the result) keeps that rounding below 1e-4. 0 = no scaling. */
    float v_cent_scale_hi, v_cent_scale_lo;
    /* optional QJL sketches of the K and V residuals (m == 32); qjl_proj is S (m, d).  All five or none: the
     * scores gain (sqrt(pi/2)/d) gamma_k sign_k.(S q), the output (sqrt(pi/2)/d) (sum_t p_t gamma_v sign_v) @ S,
     * which is attention over the reference's corrected dense K / V (cache.py:396-427, qjl.py:70-94). */
    const float* qjl_proj;
    const uint32_t *k_qjl_bits, *v_qjl_bits; const float *k_qjl_gamma, *v_qjl_gamma;
    /* uncompressed regions, (lanes, cap, d) of dense_dtype; *_len valid tokens */
    int dense_dtype;
    const void *sink_k, *sink_v; int64_t sink_len, sink_lane_stride;   /* stride in tokens */
    const void *res_k, *res_v;   int64_t res_len,  res_lane_stride;
    void* out; int out_dtype;                /* (batch, n_q_heads, d) */
    /* >= tq_decode_workspace_bytes(...), 256-byte aligned, ZERO-FILLED before its first use (it holds
     * arrival counters that every launch leaves at zero again); one buffer per stream in flight. */
    void* workspace; size_t workspace_bytes;
    /* Optional fused gather of the result for head-sharded decoding (see tq_peer_gather below), or NULL: `out` then
     * is not written; every peer's buffer is. */
    const struct tq_peer_gather* gather;
    /* Optional constants from tq_decode_tables_build for this (rot, k_cent_hi, v_cent_hi, v_cent_scale_hi), or NULL.
     * With them the 4-bit-key / 2-bit-value kernel at d = 128 copies its lookup tables and the split rotation matrix
     * instead of rebuilding them in every CTA of every launch; without them those shapes take the general kernel. */
    const void* tables;
    /* Optional (head-sharded decoding, see tq_peer_gather): before it reads q the kernel waits, bounded like
     * tq_gather_wait and with the same status on expiry, until the gather of an EARLIER call on this stream (a
     * different slot than this call's own `gather`) is complete on this GPU: every one of the await_words words of
     * the landing buffer await_ll carries the epoch await_epochs[0].  It also writes the plain result to await_out
     * (may be NULL).  This is the consumer side of the exchange folded into the next kernel's prologue: no wait
     * launch between two decode calls (beyond 8192 words the library enqueues the wait launch itself).  NULL await_ll:
     * no wait. */
    const unsigned long long* await_ll;
    const unsigned int* await_epochs;
    int64_t await_words;
    void* await_out;
} tq_decode_args;

/* Ordering on the stream.  tq_decode_attn is launched with programmatic stream serialisation (unless the "decode_pdl"
 * tuning knob is 0): its CTAs may become resident while the preceding kernel on the stream is still finishing.  Before
 * that kernel has completed they read only rot, the centroid tables and `tables` (which the preceding kernel must not
 * write) and ask for lines of the packed arrays in L2 (harmless whoever is writing them); q, the cache contents, the
 * workspace and the output are touched only after the preceding kernel has completed and its writes are visible. */

/* Bytes of the constants buffer for tq_decode_args.tables (host arithmetic); 0 when no kernel uses prebuilt constants
 * for this shape (today: d = 128 with 4-bit keys and 2-bit values has one). */
size_t tq_decode_tables_bytes(int d, int k_bits, int v_bits);
/* Fills `tables` (device, 256-byte aligned, tq_decode_tables_bytes(...) bytes) from the rotation matrix (d, d), the key
 * centroids (2^k_bits) and the value centroids (2^v_bits), all device float32, and the fp16 table scale the calls will
 * use as v_cent_scale_hi (0 = 1).  Call once per (device, rotation, codebooks) at set-up, outside stream capture:
 * it synchronises the stream.  No reference counterpart (the reference keeps rotation and codebooks as process-wide
 * cached arrays, rotation.py:12, codebook.py:32; this is the same cache in the layout the kernel consumes). */
int tq_decode_tables_build(int d, const float* rot, const float* k_cent, int k_bits, const float* v_cent, int v_bits,
                           float v_cent_scale, void* tables, size_t bytes, void* stream);

/* Fused output gather (no reference counterpart; the reference is single-device).  When one sequence's KV heads are
 * dealt to several GPUs of a node (one process per GPU), the consumer usually needs all heads' outputs on every GPU.
 * Instead of a collective after the kernel, the kernel's merge step sends the heads it produced into EVERY peer's
 * landing buffer through peer-mapped addresses, as 64-bit words {4 bytes of the result, 32-bit epoch} written with one
 * store each: a word is complete when its epoch is, so no fence, flag or acknowledgement follows the data.  The epoch
 * is the number of calls made into the slot so far; `epochs` (this GPU's own memory, zero at the start) holds it per
 * (sequence, KV head, head group) of the call - tq_gather_groups(...) entries.  Every rank makes the same calls with
 * the same sizes, so a gather is complete on a GPU once every word of its landing buffer carries that GPU's own
 * epochs[0].  The consumer waits for that either inside the next decode call (await_* in tq_decode_args) or with
 * tq_gather_wait on its stream; both also unpack the words into a plain (batch, heads_total, d) result.  Nothing reads
 * peer memory.  ll[r] is rank r's landing buffer, batch * heads_total * d * sizeof(out element) / 4 words, 8-byte
 * aligned, zero at the start, as an address valid on THIS device (the caller's own buffer at its own rank); the call's
 * heads land at the place of head index head_offset ... + n_q_heads - 1.  A slot may take its next call only after
 * every rank has consumed the previous one (use at least two slots in turn). */
#define TQ_MAX_PEERS 8
typedef struct tq_peer_gather {
    int n_peers;                                   /* 1 ... TQ_MAX_PEERS */
    int heads_total, head_offset;
    unsigned long long* ll[TQ_MAX_PEERS];
    unsigned int* epochs;
} tq_peer_gather;

/* Scratch bytes tq_decode_attn needs for these sizes (host-side arithmetic only). */
size_t tq_decode_workspace_bytes(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len,
                                 int64_t dense_len);

/* One decode step of attention computed directly on the compressed cache.  Replaces what the
 * reference does as dense reassembly (cache.py:674-706) followed by the consumer's
 * scaled-dot-product attention; the math on packed keys is that of kernels.py:439-479
 * (pre-rotated query, rotation.py:81-110) extended with softmax and values. */
int tq_decode_attn(const tq_decode_args* a, void* stream);

/* One decode step in one launch: the new token's key and value rows (k_new, v_new: (batch, n_kv_heads, d) of dense_dtype,
 * contiguous, 16-byte aligned) are stored at row res_len of res_k / res_v - which must be writable and have room,
 * res_lane_stride > res_len - and attention runs over [sink | packed | res_len recent tokens | the new token].  a->res_len
 * is the length BEFORE the call; the caller counts the token afterwards.  The append of update_and_fetch
 * (cache.py:632-672) folded into the attention that follows it; the caller still decides when tokens leave the buffer
 * for compression (tq_quantize_pack) and when a token belongs to the sink instead. */
int tq_decode_step(const tq_decode_args* a, const void* k_new, const void* v_new, void* stream);

/* Causal attention for t_q query tokens per sequence - the LAST t_q tokens of the cache, appended by the caller
 * beforehand: query i sits at position c_len + sink_len + res_len - t_q + i and sees every cached token up to and
 * including itself.  a->q and a->out are (batch, n_q_heads, t_q, d); workspace, tables and gather are not used.  Caches
 * with a QJL sketch are refused with TQ_ERR_UNSUPPORTED (their callers take the dense route).  Replaces dense
 * reassembly (cache.py:674-706) + the consumer's masked attention for prefill chunks and multi-token steps; the
 * reference only sketched it for packed keys (kernels.py:558-590, docs/FUSED_ATTENTION_DESIGN.md:281-283). */
int tq_prefill_attn(const tq_decode_args* a, int t_q, void* stream);

/* Same computation as tq_decode_attn for callers that can neither lend a workspace nor allocate one at call
 * time (a process that gave the whole device to its own memory pool at start-up; a step loop that cannot afford
 * a driver allocation).  It has no counterpart in the reference.  `workspace` / `workspace_bytes` in the
 * arguments are ignored: scratch comes from a TQ_DECODE_STATIC_SCRATCH_BYTES array inside the library, present
 * on every GPU that loads it.  Sizes that need more are refused with TQ_ERR_UNSUPPORTED.  The first call on a
 * device looks the array's address up (do it outside stream capture); under CUDA's default lazy module loading that
 * is also when the driver reserves the array's bytes on the device, so a process that is about to give all remaining
 * memory to its own pool makes the first call before it does (or runs with CUDA_MODULE_LOADING=EAGER); if the
 * reservation fails the call says so (TQ_ERR_LAUNCH).  All calls on a device share the array: order them on one
 * stream, calls that overlap on the GPU race.  Allocates nothing itself. */
#define TQ_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
int tq_decode_attn_static(const tq_decode_args* a, void* stream);

/* Number of (sequence, KV head, head group) blocks one tq_decode_attn call with these sizes merges = entries of
 * tq_peer_gather.epochs (host arithmetic). */
int64_t tq_gather_groups(int batch, int n_q_heads, int n_kv_heads);

/* Enqueues a small kernel that returns once every one of the n_words words of the landing buffer `ll` carries the
 * epoch epochs[0] - `epochs` being the tq_peer_gather array of this GPU, final by then because the producing call is
 * earlier on the stream - and writes the 4-byte payloads to `out` (the plain result; may be NULL).  Relaxed loads at
 * system scope in a loop with a back-off, about two seconds at most per word; if the limit is reached the kernel
 * records status 201 for tq_device_status() and returns; the stream continues and the result is not to be trusted.
 * The arguments are the same for every step, so the launch can be captured in a CUDA graph.  For consumers that are
 * not this library's kernels; between two decode calls the await_* fields of tq_decode_args do the same without a
 * launch. */
int tq_gather_wait(const unsigned long long* ll, const unsigned int* epochs, int64_t n_words, void* out, void* stream);

/* Device buffers that other processes on the node can map (CUDA IPC), for the outputs and counters above.
 * create: cudaMalloc + zero fill on the current device, returns the address and a 64-byte handle to pass to the peers
 * by any host channel; open: maps a peer's buffer into this process for kernels on the CURRENT device (refused with
 * TQ_ERR_UNSUPPORTED when the current device cannot address peer_device's memory); close / destroy undo them.  These
 * four are the only calls of the library that allocate, and only when asked. */
int tq_peer_buffer_create(size_t bytes, void** ptr, unsigned char handle[64]);
int tq_peer_buffer_open(const unsigned char handle[64], int peer_device, void** ptr);
int tq_peer_buffer_close(void* ptr);
int tq_peer_buffer_destroy(void* ptr);

/* Scale s in [1, 2) minimising max_i |fp16(s*c_i) - s*c_i| / |s*c_i| for a HOST array of n centroids
 * (no reference counterpart; pure host arithmetic). */
float tq_fp16_table_scale(const float* centroids_host, int n);

/* Host-side tuning knobs of the split heuristic (process-wide; no reference counterpart):
 *   "decode_ctas_per_sm" 1..8, "decode_splits" 0 (auto)..448, "decode_force_general" 0/1,
 *   "dequantize_tc" 0/1 (tq_dequantize at d = 64 / 96 / 128 without QJL correction: the tcgen05 kernel, default, or always the
 *   CUDA-core row kernel),
 *   "prefill_tc" 0/1 (tq_prefill_attn at d = 128 with at least 64 query rows: the tcgen05 kernel, default, or always
 *   the mma.sync kernel),
 *   "decode_pdl" 0/1 (programmatic dependent launch: a call's prologue overlaps the previous kernel's tail),
 *   "gather_wait_polls" 1000..4000000 (polls of one word of a gather before the wait gives up; default 2000000, some two seconds),
 *   "decode_stream" 0/1 (the persistent streaming kernel for 4-bit keys / 2-bit values at d = 96 / 128 may be chosen, default, or never),
 *   "decode_stream_min_run" 1.. (fewest packed 16-token tiles per warp of the persistent grid for which it is chosen over the
 *   table-lookup kernel, default 24; over the general kernel a third of that),
 *   "decode_stream_max_parts" 1..64 (most partial results per lane with which it is chosen over the table-lookup kernel; default 40).
 * Changing them changes tq_decode_workspace_bytes for the same sizes. */
int tq_set_tuning(const char* key, int value);

/* Which kernel tq_decode_attn would run for these arguments under the current tuning (no launch; no reference counterpart):
 * 0 = general kernel (any width, d = 64 / 96 / 128 / 256), 1 = table-lookup kernel (4-bit keys / 2-bit values, d = 128: one CTA
 * per (sequence, KV head, split)), 2 = streaming kernel (the same widths at d = 96 / 128, sign sketches allowed: persistent
 * grid, chosen when the packed tokens of all lanes give every warp a long run).  Negative: the arguments are invalid
 * (tq_last_error has the text). */
int tq_decode_kernel_choice(const tq_decode_args* a);

#ifdef __cplusplus
}
#endif
#endif /* TQ_ABI_H */
