// Device-side building blocks shared by the decode-attention kernels: PTX wrappers, the per-warp online-softmax
// state, and the 16-token tile step on fp16 operands staged in shared memory.
#pragma once

#include "decode.cuh"

namespace tq {

// ---- small PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_ptr));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movm_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// Lookups in tables that are constant for the lifetime of the CTA: plain (non-volatile) asm so the compiler
// may hoist and batch them ahead of the MMAs that consume them.
__device__ __forceinline__ uint32_t lut32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lut64(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
// Reads of the cp.async ring: ordered after the wait / warp barrier that makes the data visible.
__device__ __forceinline__ uint32_t ring32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ring128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
// 16-byte asynchronous global -> shared copy; bytes past src_bytes are zero-filled (0 = read nothing).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Programmatic dependent launch: wait for the previous grid on the stream / let the next grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- per-warp running softmax state ------------------------------------------------------------------
constexpr float MAX_SLACK = 6.f;   // scores may exceed the running reference by 2^6 before it is refreshed
// ---- result stores ---------------------------------------------------------------------------------
// Fused gather, producer side.  The merging CTA first stages its heads in shared memory in the result's element type
// (`stage`, 4-byte aligned, `bytes` = heads * D * element size) and passes a barrier; then every thread calls this.
// Each 4 bytes of the block travel as one 64-bit word {payload, epoch} written with a single store into every peer's
// landing buffer: a word is complete when its epoch is, so no fence and no separate flag follow the data and nothing
// waits for the stores to be acknowledged.  `byte_off` is where the group's first head sits in a (batch, heads_total, d)
// result; `epoch` is this (slot, group)'s call count including this call (the caller read epochs[grp] + 1 before the
// barrier), stored back for the next call.
__device__ __forceinline__ void publish_result(const DecodeParams& p, const void* stage, int bytes, int64_t byte_off, int grp, unsigned epoch) {
    const int n_words = bytes >> 2;
    const uint32_t* src = static_cast<const uint32_t*>(stage);
    const int64_t w0 = byte_off >> 2;
    for (int i = threadIdx.x; i < n_words * p.n_peers; i += blockDim.x) {
        const int r = i / n_words, w = i - r * n_words;
        const unsigned long long v = static_cast<unsigned long long>(src[w]) | (static_cast<unsigned long long>(epoch) << 32);
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.peer_ll[r] + w0 + w), "l"(v) : "memory");
    }
    if (threadIdx.x == 0) p.epochs[grp] = epoch;
}
__device__ __forceinline__ int out_elem_bytes(int dtype) { return dtype == TQ_F32 ? 4 : 2; }
__device__ __forceinline__ unsigned next_epoch(const DecodeParams& p, int grp) {
    return p.n_peers > 0 ? *reinterpret_cast<const volatile unsigned*>(p.epochs + grp) + 1u : 0u;
}

// Fused gather, consumer side: polls the words of this GPU's landing buffer until each carries `epoch` (bounded: a
// thread that runs out of polls gives up on its remaining words too) and, if `out` is given, writes the payloads there
// as the plain (batch, heads_total, d) result.  Returns false if a word never arrived.
__device__ __forceinline__ bool collect_words(const unsigned long long* ll, int64_t first, int64_t n_words, int64_t stride, unsigned epoch,
                                              uint32_t* out, int max_polls) {
    for (int64_t w = first; w < n_words; w += stride) {
        unsigned long long v;
        int it = 0;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(ll + w) : "memory");
            if (static_cast<unsigned>(v >> 32) == epoch) break;
            if (++it >= max_polls) return false;
            if (it > 64) __nanosleep(500);
        }
        if (out) out[w] = static_cast<uint32_t>(v);
    }
    return true;
}
// ... inside the kernel that follows on the stream: every thread calls it after griddepcontrol.wait (the producing call
// of this GPU is complete by then, so its epoch is final; every rank makes the same calls, so it is the peers' epoch
// too).  Every CTA checks every word - the whole result has to be in before any of the query may be believed - and
// the first CTA also writes the plain copy.
__device__ __forceinline__ void await_gather(const DecodeParams& p) {
    if (p.await_ll == nullptr) return;
    const unsigned epoch = *reinterpret_cast<const volatile unsigned*>(p.await_epochs);
    const bool first_cta = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
    if (!collect_words(p.await_ll, threadIdx.x, p.await_words, blockDim.x, epoch, first_cta ? static_cast<uint32_t*>(p.await_out) : nullptr, p.await_polls))
        atomicCAS(p.status, 0, 201);
    __syncthreads();
}

// NZ: extra accumulator tiles that share the softmax weights (the QJL sketch rows of the output).
template <int D, int NZ = 0> struct WarpAcc {
    float m[2], mt[2], l[2];   // heads 2t, 2t+1: reference max, refresh threshold, this lane's share of the sum
    float vsc, vt;             // power-of-two scale applied to (weight * value norm) before the fp16 cast; norms above vt force a new one
    float o[D / 16][4];        // O^T fragments: rows = coordinate slots, cols = heads; hold vsc * (true sums)
    float z[NZ ? NZ : 1][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = mt[0] = mt[1] = -INFINITY;
        l[0] = l[1] = 0.f;
        vsc = 1.f; vt = 0.f;   // the first tile with a non-zero value norm picks the scale
#pragma unroll
        for (int i = 0; i < D / 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
        for (int i = 0; i < (NZ ? NZ : 1); ++i) z[i][0] = z[i][1] = z[i][2] = z[i][3] = 0.f;
    }
    // undo the value scale: afterwards o / z hold the true weighted sums
    __device__ __forceinline__ void finish() {
        const float r = 1.f / vsc;     // exact: vsc is a power of two
#pragma unroll
        for (int i = 0; i < D / 16; ++i) { o[i][0] *= r; o[i][1] *= r; o[i][2] *= r; o[i][3] *= r; }
#pragma unroll
        for (int i = 0; i < NZ; ++i) { z[i][0] *= r; z[i][1] *= r; z[i][2] *= r; z[i][3] *= r; }
    }
};

// The softmax weights p = exp2(s - m) reach the value MMAs as fp16 operands p * |v| * vsc.  m is refreshed lazily, so
// p <= 2^MAX_SLACK; vsc is a power of two chosen so that the largest value norm seen so far lands in [128, 256), which
// keeps every operand below 2^14 whatever the norms' magnitude (the reference works in float32, cache.py:276-343) and
// keeps small norms clear of the fp16 subnormals.  A norm above vt = 1023 / vsc forces a new scale; the accumulators are
// rescaled like they are for a new maximum.
constexpr float VSC_CAP = 1023.f;

// The rare branch of the softmax step: new reference maxima and / or a new value scale.  vmax: the largest value norm of
// the tile in this lane (lanes with the same g hold the same norms).
template <int D, int NZ>
__device__ __forceinline__ void softmax_refresh(float mx0, float mx1, float vmax, WarpAcc<D, NZ>& st) {
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    }
    const float mn0 = fmaxf(fmaxf(st.m[0], mx0), -1e30f), mn1 = fmaxf(fmaxf(st.m[1], mx1), -1e30f);
    float a0 = ex2(st.m[0] - mn0), a1 = ex2(st.m[1] - mn1);
    st.m[0] = mn0; st.m[1] = mn1;
    st.mt[0] = mn0 + MAX_SLACK; st.mt[1] = mn1 + MAX_SLACK;
    st.l[0] *= a0; st.l[1] *= a1;
    if (vmax > st.vt) {                                              // warp-uniform
        int eb = (__float_as_int(vmax) >> 23) & 0xff;                // biased exponent of the largest norm
        eb = min(max(eb, 16), 240);                                  // (subnormal, infinite and NaN norms: any finite scale)
        const float nsc = __int_as_float((261 - eb) << 23);          // 2^(7 - floor(log2 vmax)): vmax * nsc in [128, 256)
        const float r = nsc / st.vsc;
        a0 *= r; a1 *= r;
        st.vsc = nsc;
        st.vt = VSC_CAP / nsc;
    }
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) {
        st.o[mt][0] *= a0; st.o[mt][1] *= a1; st.o[mt][2] *= a0; st.o[mt][3] *= a1;
    }
#pragma unroll
    for (int i = 0; i < NZ; ++i) {
        st.z[i][0] *= a0; st.z[i][1] *= a1; st.z[i][2] *= a0; st.z[i][3] *= a1;
    }
}

// s[0..1]: token g, heads 2t,2t+1;  s[2..3]: token g+8.  Returns the P^T operand for the PV mma.
// The softmax reference m is refreshed (with a cross-lane max and a rescale of the accumulators) only
// when some score exceeds it by more than MAX_SLACK; softmax is shift-invariant, so any reference that
// keeps exp2(s - m) inside the fp16 range is exact.  p_out (optional) receives the four weights times vsc.
template <int D, int NZ>
__device__ __forceinline__ void softmax_step(float (&s)[4], float kn0, float kn1, float vn0, float vn1, bool ok0,
                                             bool ok1, WarpAcc<D, NZ>& st, uint32_t (&bp)[2], float* p_out = nullptr, float vx = 0.f) {
    s[0] = ok0 ? s[0] * kn0 : -INFINITY;
    s[1] = ok0 ? s[1] * kn0 : -INFINITY;
    s[2] = ok1 ? s[2] * kn1 : -INFINITY;
    s[3] = ok1 ? s[3] * kn1 : -INFINITY;
    vn0 = ok0 ? vn0 : 0.f; vn1 = ok1 ? vn1 : 0.f;
    // vx: any other magnitude that will multiply the weights p_out (the QJL residual norms of the tile)
    const float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]), vmax = fmaxf(fmaxf(vn0, vn1), vx);
    if (__any_sync(0xffffffffu, mx0 > st.mt[0] || mx1 > st.mt[1] || vmax > st.vt)) softmax_refresh<D, NZ>(mx0, mx1, vmax, st);
    const float p0 = ex2(s[0] - st.m[0]), p1 = ex2(s[1] - st.m[1]), p2 = ex2(s[2] - st.m[0]), p3 = ex2(s[3] - st.m[1]);
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    if (p_out) { p_out[0] = p0 * st.vsc; p_out[1] = p1 * st.vsc; p_out[2] = p2 * st.vsc; p_out[3] = p3 * st.vsc; }
    // value norms ride on P (fp16)
    const float w0 = vn0 * st.vsc, w1 = vn1 * st.vsc;
    const uint32_t h0 = pack_h2(p0 * w0, p1 * w0);
    const uint32_t h1 = pack_h2(p2 * w1, p3 * w1);
    bp[0] = movm_t(h0);   // tokens 2t,2t+1   x head g
    bp[1] = movm_t(h1);   // tokens 2t+8,2t+9 x head g
}

template <int D> __host__ __device__ constexpr int stage_ld() { return D + 8; }

// One 16-token tile whose K and V sit in shared memory as fp16 [token][coordinate].
template <int D, int NZ>
__device__ __forceinline__ void tile_from_smem(const __half* Ks, const __half* Vs, const uint32_t (&bq)[D / 16][2],
                                               float kn0, float kn1, float vn0, float vn1, bool ok0, bool ok1,
                                               WarpAcc<D, NZ>& st, int lane) {
    constexpr int LD = stage_ld<D>();
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
        const __half* base = Ks + (lane & 15) * LD + (lane >> 4) * 8;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, base + ks * 16);
            mma16816(s, a[0], a[1], a[2], a[3], bq[ks][0], bq[ks][1]);
        }
    }
    uint32_t bp[2];
    softmax_step<D, NZ>(s, kn0, kn1, vn0, vn1, ok0, ok1, st, bp);
    {
        const __half* base = Vs + ((lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
            uint32_t a[4];
            ldsm_x4_t(a, base + mt * 16);
            mma16816(st.o[mt], a[0], a[1], a[2], a[3], bp[0], bp[1]);
        }
    }
}

// Staging scale of a token row from the float bits of its largest magnitude: 2^(7 - floor(log2 max)); rows of zeros
// (and non-finite rows) keep scale 1.
__device__ __forceinline__ float stage_scale(uint32_t max_bits) {
    const int e = int(max_bits >> 23) & 0xff;
    return (e >= 16 && e <= 240) ? __int_as_float((261 - e) << 23) : 1.f;
}

// Attention over the uncompressed tokens [sink | residual window] of cache lane kvl with the unrotated query:
// this warp takes tiles tile_lo + warp, + NW, ... below tile_hi; Ks / Vs are its fp16 staging buffers.
template <int D, int NW, int NZ>
__device__ __forceinline__ void dense_tiles(const DecodeParams& p, int64_t kvl, int64_t tile_lo, int64_t tile_hi_in, __half* Ks, __half* Vs,
                                            const uint32_t (&bq)[D / 16][2], WarpAcc<D, NZ>& st, int warp, int lane) {
    constexpr int LD = stage_ld<D>();
    const int g = lane >> 2;
    // tokens [0, sink_len) sit in the sink, the next res_len in the recent-token buffer; a token that this very call appends
    // (k_new / v_new: one row per lane) comes last and is read from where the caller left it
    const int64_t n_tok = p.sink_len + p.res_len + (p.k_new ? 1 : 0);
    const int64_t tile_hi = min(tile_hi_in, (n_tok + TILE - 1) / TILE);
    auto row_of = [&](int64_t tok, bool keys, int64_t& e) -> const void* {     // base pointer and element offset of a token's row
        if (tok < p.sink_len) { e = (kvl * p.sink_ls + tok) * D; return keys ? p.sink_k : p.sink_v; }
        const int64_t r = tok - p.sink_len;
        if (r < p.res_len) { e = (kvl * p.res_ls + r) * D; return keys ? p.res_k : p.res_v; }
        e = kvl * D;
        return keys ? p.k_new : p.v_new;
    };
    if (p.k_new) {
        // the warp that owns the new token's tile also stores the row at the end of the recent-token buffer (the caller's
        // slice assignment, cache.py:632-672); CTAs of different head groups write the same bytes
        const int64_t new_tile = (n_tok - 1) / TILE;
        if (new_tile >= tile_lo && new_tile < tile_hi && (new_tile - tile_lo) % NW == warp) {
            const int es = p.dense_dtype == TQ_F32 ? 4 : 2;
            const int64_t dst = (kvl * p.res_ls + p.res_len) * D * es, src = kvl * D * es;
            for (int c = lane; c < D * es / 16; c += 32) {
                *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.res_k_w) + dst + c * 16) = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.k_new) + src) + c);
                *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.res_v_w) + dst + c * 16) = __ldg(reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(p.v_new) + src) + c);
            }
        }
    }
    for (int64_t tile = tile_lo + warp; tile < tile_hi; tile += NW) {
        const int64_t tok0 = tile * TILE;
        float sck = 1.f, scv = 1.f;                       // staging scales of row lane >> 1 (keys, values)
        constexpr int NCH = TILE * (D / 8) / 32;          // 16-byte chunks per lane and tensor
        if (p.dense_dtype == TQ_F16) {
            uint4 kv[NCH], vv[NCH];                        // every load of the tile in flight before the first store
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int c = lane + 32 * i, r = c / (D / 8), c8 = c - r * (D / 8);
                const int64_t tok = tok0 + r;
                kv[i] = make_uint4(0, 0, 0, 0); vv[i] = kv[i];
                if (tok < n_tok) {
                    int64_t e;
                    const __half* kb = static_cast<const __half*>(row_of(tok, true, e));
                    const __half* vb = static_cast<const __half*>(row_of(tok, false, e));
                    kv[i] = __ldg(reinterpret_cast<const uint4*>(kb + e + c8 * 8));
                    vv[i] = __ldg(reinterpret_cast<const uint4*>(vb + e + c8 * 8));
                }
            }
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int c = lane + 32 * i, r = c / (D / 8), c8 = c - r * (D / 8);
                *reinterpret_cast<uint4*>(Ks + r * LD + c8 * 8) = kv[i];
                *reinterpret_cast<uint4*>(Vs + r * LD + c8 * 8) = vv[i];
            }
        } else {
            // float32 / bfloat16 tokens can lie outside the fp16 range: every token row is staged as fp16 under its own
            // power-of-two scale (largest magnitude into [2^7, 2^8)); the scores and the softmax weights take the inverse
            // scales where the packed tokens take their norms.  Each lane folds the largest magnitude of its 16-byte chunks
            // into the row's slot (the 16 bytes of padding at the end of the row's staging line: keys' maximum in word 0,
            // values' in word 1; non-negative floats order like integers).
            if (lane < TILE) *reinterpret_cast<uint2*>(Ks + lane * LD + D) = make_uint2(0u, 0u);
            __syncwarp();
            // Two passes over the tile's 16-byte chunks, four chunks of one tensor in flight at a time (few registers: this code sits
            // inside kernels whose main loops need them): first the row maxima, then - the chunks come from L1 / L2 now - the scaled
            // conversion.  ES: bytes per element.
            const int es = p.dense_dtype == TQ_BF16 ? 2 : 4;
            const int cpr = D * es / 16;                      // chunks per row
            const int n_chunks = TILE * cpr;
            auto chunk_ptr = [&](int c, bool keys) -> const uint4* {
                const int r = c / cpr, cc = c - r * cpr;
                const int64_t tok = tok0 + r;
                if (tok >= n_tok) return nullptr;
                int64_t e;
                const unsigned char* base = static_cast<const unsigned char*>(row_of(tok, keys, e));
                return reinterpret_cast<const uint4*>(base + e * es) + cc;
            };
#pragma unroll 1
            for (int side = 0; side < 2; ++side) {
#pragma unroll 1
                for (int c0 = lane; c0 < n_chunks; c0 += 128) {
                    uint4 x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint4* src = c0 + 32 * u < n_chunks ? chunk_ptr(c0 + 32 * u, side == 0) : nullptr;
                        x[u] = src ? __ldg(src) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (c0 + 32 * u >= n_chunks) continue;
                        uint32_t mb;
                        if (es == 2) {
                            const uint32_t m = 0x7fff7fffu;
                            const uint32_t a = __vmaxu2(__vmaxu2(x[u].x & m, x[u].y & m), __vmaxu2(x[u].z & m, x[u].w & m));
                            mb = max(a & 0xffffu, a >> 16) << 16;
                        } else {
                            const uint32_t m = 0x7fffffffu;
                            mb = max(max(x[u].x & m, x[u].y & m), max(x[u].z & m, x[u].w & m));
                        }
                        atomicMax(reinterpret_cast<uint32_t*>(Ks + ((c0 + 32 * u) / cpr) * LD + D) + side, mb);
                    }
                }
            }
            __syncwarp();
#pragma unroll 1
            for (int side = 0; side < 2; ++side) {
                __half* dst = side == 0 ? Ks : Vs;
#pragma unroll 1
                for (int c0 = lane; c0 < n_chunks; c0 += 128) {
                    uint4 x[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint4* src = c0 + 32 * u < n_chunks ? chunk_ptr(c0 + 32 * u, side == 0) : nullptr;
                        x[u] = src ? __ldg(src) : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int c = c0 + 32 * u;
                        if (c >= n_chunks) continue;
                        const int r = c / cpr, cc = c - r * cpr;
                        const float f = stage_scale(reinterpret_cast<const uint32_t*>(Ks + r * LD + D)[side]);
                        if (es == 2) {
                            auto two = [&](uint32_t w) -> uint32_t { return pack_h2(__uint_as_float(w << 16) * f, __uint_as_float(w & 0xffff0000u) * f); };
                            *reinterpret_cast<uint4*>(dst + r * LD + cc * 8) = make_uint4(two(x[u].x), two(x[u].y), two(x[u].z), two(x[u].w));
                        } else {
                            *reinterpret_cast<uint2*>(dst + r * LD + cc * 4) =
                                make_uint2(pack_h2(__uint_as_float(x[u].x) * f, __uint_as_float(x[u].y) * f), pack_h2(__uint_as_float(x[u].z) * f, __uint_as_float(x[u].w) * f));
                        }
                    }
                }
            }
            __syncwarp();
            {
                const uint2 mx = *reinterpret_cast<const uint2*>(Ks + (lane >> 1) * LD + D);
                sck = stage_scale(mx.x);
                scv = stage_scale(mx.y);
            }
        }
        __syncwarp();
        // inverse scales of rows g and g + 8 (1 for fp16 tokens)
        const float ik0 = 1.f / __shfl_sync(0xffffffffu, sck, 2 * g), ik1 = 1.f / __shfl_sync(0xffffffffu, sck, 2 * g + 16);
        const float iv0 = 1.f / __shfl_sync(0xffffffffu, scv, 2 * g), iv1 = 1.f / __shfl_sync(0xffffffffu, scv, 2 * g + 16);
        tile_from_smem<D, NZ>(Ks, Vs, bq, ik0, ik1, iv0, iv1, tok0 + g < n_tok, tok0 + g + 8 < n_tok, st, lane);
        __syncwarp();
    }
}

}  // namespace tq
