// Decode attention over a cache with 4-bit keys and 2-bit values at d = 96 or 128, with or without the QJL sign
// sketches: the streaming kernel, for calls whose packed tokens amount to many 16-token tiles per warp (many sequences
// and / or many KV heads: the batched-serving shapes).
//
// Where the other two kernels give every (sequence, KV head, split) a CTA of its own - whose fixed cost (tables, query
// rotation, reduction over warps, merge) is paid per CTA and whose count rarely divides the SMs evenly - this one runs
// ONE persistent CTA of 16 warps per SM and deals the packed tiles of ALL cache lanes out as one flat sequence, an equal
// contiguous run per warp.  A run touches one or two lanes (more when lanes are short); per lane it touches a warp
// writes one partial (max, sum, weighted values in rotated space, sketch rows) straight from its registers.  Nothing in
// the main loop is shared between warps: no barrier, no reduction, no atomics.
//
// Three launches, chained with programmatic dependent launch:
//   1. stream_query_kernel   rotates every query head once (q R^T, and S q for the sketches) into the workspace as
//                            scaled fp16 - 16 heads per block, R and S staged in shared memory;
//   2. decode_stream_kernel  the persistent grid.  Raw packed tiles (keys, values, norms, sign words, residual norms:
//                            4 to 8 arrays) reach a warp through its own ring of NS stages in shared memory: a stage is
//                            the tile's arrays back to back, every lane copies three or four 16-byte chunks of it with
//                            asynchronous copies and arrives on the stage's mbarrier when they have landed (whole
//                            sectors whatever the row length, no registers held across the global-memory latency,
//                            NS - 1 tiles in flight per warp).  Operand fragments come from the byte tables of
//                            decode_direct.cu (one byte-permute forms the address); at d = 96 a row group owns three
//                            bytes of the 24-byte value row, read as the two aligned words around them.  The
//                            uncompressed tokens (sink, recent window, the token a step appends) are dealt out too, a
//                            few tiles per warp, before the packed runs start; their staging buffer is the warp's ring.
//   3. stream_merge_kernel   a thread per (lane, head, coordinate): log-sum-exp merge of the lane's partials, rotation of
//                            the packed part back (y R, float32, R staged in shared memory), sketch rows times S,
//                            normalisation, store.
//
// The loop is bound by the integer pipe (byte-permutes, logic ops and shifts that turn packed codes and sign bits into
// operands): measured 375 warp-instructions per 16-token tile at d = 96 with sketches, 288 at d = 128 without.
//
// Every mbarrier wait is bounded; a wait that runs out records a status (tq_device_status), the warp drains the copies
// it still has in flight (bounded again) and stops.
#include <algorithm>
#include <atomic>

#include "decode_dev.cuh"

namespace tq {
namespace ds {

using dd::C_BASE;
using dd::DirectTables;
using dd::LO_BASE;
using dd::LUT_BASE;
using dd::TABLES_MAGIC;

#ifndef TQ_STREAM_WARPS
#define TQ_STREAM_WARPS 16
#endif
constexpr int NW = TQ_STREAM_WARPS, NT = NW * 32;
// Ring stages per warp and copies of the tile loop's body.  The depth of the ring makes no difference to the time (2, 3, 4,
// 6 measured: the wait finds its stage complete); with as many copies of the body as stages the stage offsets fold into the
// instructions, which pays at d = 128 (3 %) and not at d = 96.
template <int D> struct Ring { static constexpr int NS = D == 128 ? 2 : 4, UNROLL = D == 128 ? 2 : 1; };
constexpr int QM = 32;                         // sketch rows (one 32-bit sign word per token)
constexpr float QJL_C = 1.2533141373155003f;   // sqrt(pi / 2), qjl.py:91-92
constexpr uint32_t WAIT_LIMIT = 4u << 20;
constexpr int ERR_TABLES = 106, ERR_RING = 107, ERR_LAYOUT = 108;
constexpr int MAX_PARTS = 64;                  // partial slots per lane the merge handles

template <int D, bool QJL> struct Plan {
    static constexpr uint32_t KT = TILE * D / 2, VT = TILE * D / 4, SC = TILE * 4;   // bytes per tile: keys, values, one scalar array
    static constexpr int NSC = QJL ? 6 : 2;
    static constexpr uint32_t O_V = KT, O_KN = KT + VT, O_VN = O_KN + SC, O_KB = O_VN + SC, O_KG = O_KB + SC, O_VB = O_KG + SC, O_VG = O_VB + SC;
    static constexpr int NS = Ring<D>::NS;
    static constexpr uint32_t STAGE = KT + VT + NSC * SC;
    static constexpr uint32_t RING = NS * STAGE;
    static constexpr uint32_t DSTAGE = 2u * TILE * stage_ld<D>() * 2u;               // fp16 keys + values of one uncompressed tile
    static constexpr uint32_t AREA = ((RING > DSTAGE ? RING : DSTAGE) + 127u) / 128u * 128u;
    static constexpr int LOW = int((LUT_BASE - LO_BASE) / AREA) < NW ? int((LUT_BASE - LO_BASE) / AREA) : NW;   // warps whose area lies below the tables
    static constexpr uint32_t BARS = C_BASE + uint32_t(NW - LOW) * AREA;             // the tables' barrier, then NW * NS ring barriers
    static constexpr uint32_t SMEM_END = BARS + 8u * (1 + NW * NS) + 56u;
    static_assert(SMEM_END <= 227u * 1024u, "shared-memory plan");
    static_assert(STAGE % 16 == 0 && AREA % 128 == 0, "bulk copies need 16-byte alignment");
    __host__ __device__ static constexpr uint32_t area(int w) { return w < LOW ? LO_BASE + uint32_t(w) * AREA : C_BASE + uint32_t(w - LOW) * AREA; }
};

__host__ __device__ constexpr int q_stride(int d) { return 2 * d + QM; }       // halves per query head in the workspace: rotated | raw | sketch
__host__ __device__ constexpr int part_stride(int d) { return d + QM + 4; }    // floats per head of a partial: values | sketch rows | max, sum, pad

// ---- PTX wrappers ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Bulk copy global -> this CTA's shared memory; bytes a multiple of 16, both addresses 16-byte aligned.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Reads of a ring stage at base + a compile-time offset (the offset travels in the instruction): ordered after the wait
// that made the stage visible.
template <uint32_t OFF> __device__ __forceinline__ uint32_t ring32o(uint32_t base) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1 + %2];" : "=r"(v) : "r"(base), "n"(OFF) : "memory");
    return v;
}
template <uint32_t OFF> __device__ __forceinline__ float ring_f32o(uint32_t base) { return __uint_as_float(ring32o<OFF>(base)); }
template <uint32_t OFF> __device__ __forceinline__ uint4 ring128o(uint32_t base) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(base), "n"(OFF) : "memory");
    return v;
}

// Token of the tile that sits in MMA row / k slot s.  Slots 2a + e (a = 0..3, e = 0, 1) of the lower half hold tokens
// a + 4 (e ^ (a >> 1)), the upper half the same + 8: the four lanes of a thread group then read value words of four
// consecutive tokens (lanes t >= 2 read their pair in swapped order), the eight row groups key rows of eight consecutive
// tokens - both free of bank conflicts at 24- and 48-byte rows.
__device__ __forceinline__ int tok_of_slot(int s) {
    const int a = (s & 7) >> 1, e = s & 1;
    return a + 4 * (e ^ (a >> 1)) + (s & 8);
}

// ---- launch 1: the queries ------------------------------------------------------------------------------
// q_rot[h][j] = sum_k q[h][k] R[j][k] (rotation.py:81-110), u[h][p] = sum_k q[h][k] S[p][k] (qjl.py:70-94), both times
// scale * log2(e), as fp16; the raw query likewise (for the uncompressed tokens).  Block = QPB query heads; R and S are
// staged in shared memory with coalesced loads (rows padded by 4 floats: the 128-bit row reads of 8 consecutive threads
// then cover all 32 banks); thread = (row of R or S, half of the block's heads).
constexpr int QPB = 16, QNT = 256;
template <int D> __host__ __device__ constexpr size_t query_smem() { return (size_t(D + QM) * (D + 4) + size_t(QPB) * D) * sizeof(float); }
template <int D>
__global__ void __launch_bounds__(QNT) stream_query_kernel(DecodeParams p) {
    extern __shared__ __align__(16) unsigned char smem_q[];
    constexpr int LDR = D + 4, QS = q_stride(D);
    float* rs = reinterpret_cast<float*>(smem_q);                // [D + 32][LDR]: R, then S
    float* qf = rs + (D + QM) * LDR;                             // [QPB][D]
    const int tid = threadIdx.x;
    const int64_t n_q = int64_t(p.B) * p.Hq, q0 = int64_t(blockIdx.x) * QPB;
    const int rows = D + (p.qjl_proj ? QM : 0);
    pdl_trigger();
    for (int i = tid; i < rows * (D / 4); i += QNT) {            // constants: before the wait
        const int r = i / (D / 4), k4 = i - r * (D / 4);
        const float4 x = __ldg(reinterpret_cast<const float4*>(r < D ? p.rot + int64_t(r) * D : p.qjl_proj + int64_t(r - D) * D) + k4);
        *reinterpret_cast<float4*>(rs + r * LDR + 4 * k4) = x;
    }
    pdl_wait();
    const float f = p.scale * LOG2E;
    for (int e = tid; e < QPB * D; e += QNT) {
        const int v = e / D, c = e - v * D;
        const float x = q0 + v < n_q ? load_as_f32(p.q, p.q_dtype, (q0 + v) * D + c) : 0.f;
        qf[e] = x;
        if (q0 + v < n_q) p.st_q16[(q0 + v) * QS + D + c] = __float2half_rn(x * f);
    }
    __syncthreads();
    const int vh = tid / 128, r0 = tid - vh * 128;               // heads vh * 8 .. vh * 8 + 7 of the block
    for (int r = r0; r < rows; r += 128) {
        const float4* row = reinterpret_cast<const float4*>(rs + r * LDR);
        float acc[8];
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] = 0.f;
#pragma unroll 4
        for (int k = 0; k < D / 4; ++k) {
            const float4 x = row[k];
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const float4 y = *reinterpret_cast<const float4*>(qf + (vh * 8 + v) * D + 4 * k);
                acc[v] = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, acc[v]))));
            }
        }
        const int dst = r < D ? r : 2 * D + (r - D);
#pragma unroll
        for (int v = 0; v < 8; ++v)
            if (q0 + vh * 8 + v < n_q) p.st_q16[(q0 + vh * 8 + v) * QS + dst] = __float2half_rn(acc[v] * f);
    }
}

// Three-input logic in ONE instruction with both constants in registers (written as two C operators with two literal
// constants the compiler emits two instructions: an instruction takes one immediate only).  The integer pipe is what
// bounds this kernel.
template <int LUT> __device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
    return d;
}
// loop-invariant constants kept in registers (the asm hides their values from constant propagation)
__device__ __forceinline__ uint32_t reg_const(uint32_t v) {
    uint32_t r;
    asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}
struct BitConsts { uint32_t sign_mask, minus_ones, lo_nibbles; };
// half2 of two signs (+1 for a set bit) from a word that holds the two sign bits at positions 15 and 31: (x & 0x80008000) ^ 0xBC00BC00
__device__ __forceinline__ uint32_t sign_pair16(uint32_t x, const BitConsts& k) { return lop3<0x6A>(x, k.sign_mask, k.minus_ones); }
// (a & 0x0F0F0F0F) | (b & 0xF0F0F0F0)
__device__ __forceinline__ uint32_t nibble_mix(uint32_t a, uint32_t b, const BitConsts& k) { return lop3<0xE4>(a, b, k.lo_nibbles); }

// Softmax step on scores that already carry the key norms (and the sketch term); tokens past the end of the cache come
// in with score -inf and norm 0.  pr: the four weights times the value scale.
template <int D, int NZ>
__device__ __forceinline__ void softmax_stream(float (&s)[4], float vn0, float vn1, float vx, WarpAcc<D, NZ>& st, uint32_t (&bp)[2], float (&pr)[4]) {
    const float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]), vmax = fmaxf(fmaxf(vn0, vn1), vx);
    if (__any_sync(0xffffffffu, mx0 > st.mt[0] || mx1 > st.mt[1] || vmax > st.vt)) softmax_refresh<D, NZ>(mx0, mx1, vmax, st);
    const float p0 = ex2(s[0] - st.m[0]), p1 = ex2(s[1] - st.m[1]), p2 = ex2(s[2] - st.m[0]), p3 = ex2(s[3] - st.m[1]);
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    pr[0] = p0 * st.vsc; pr[1] = p1 * st.vsc; pr[2] = p2 * st.vsc; pr[3] = p3 * st.vsc;
    bp[0] = movm_t(pack_h2(pr[0] * vn0, pr[1] * vn0));
    bp[1] = movm_t(pack_h2(pr[2] * vn1, pr[3] * vn1));
}

// ---- launch 2: the persistent grid ----------------------------------------------------------------------
template <int D, bool QJL>
__global__ void __launch_bounds__(NT, 1) decode_stream_kernel(DecodeParams p) {
    using P = Plan<D, QJL>;
    constexpr int NZ = QJL ? QM / 16 : 0, NS = P::NS;
    constexpr int QS = q_stride(D), PS = part_stride(D);
    constexpr int KW = D / 32;                 // 32-bit words of a quarter key row
    extern __shared__ __align__(16) unsigned char smem[];
    const uint32_t sbase = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    if (sbase > LO_BASE || (sbase & 15u)) {            // cannot happen after the host-side probe; never run on a bad plan
        if (tid == 0) atomicCAS(p.status, 0, ERR_LAYOUT);
        return;
    }
    const DirectTables* tb = static_cast<const DirectTables*>(p.tables);
    pdl_trigger();
    const uint32_t lut_bar = P::BARS, bar0 = P::BARS + 8u + uint32_t(warp) * NS * 8u, my_area = P::area(warp);
    if (tid == 0) mbar_init(lut_bar, 1);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bar0 + 8u * s, 32);      // every lane arrives when its copies into the stage have completed
        fence_barrier_init();
    }
    __syncthreads();
    if (tid == 0) {
        mbar_expect_tx(lut_bar, uint32_t(sizeof(tb->lut)));
        bulk_g2s(LUT_BASE, tb->lut, uint32_t(sizeof(tb->lut)), lut_bar);
    }
    const uint32_t tb_magic = __ldg(&tb->magic);
    pdl_wait();        // the prepared queries, the cache and the workspace are settled from here on
    bool failed = false;
    if (tb_magic != TABLES_MAGIC) {
        if (tid == 0) atomicCAS(p.status, 0, ERR_TABLES);
        failed = true;
    }

    const int L = p.B * p.Hkv * p.HG;                          // cache lanes x head groups
    const int n_tiles = int((p.c_len + TILE - 1) / TILE);      // packed tiles per lane
    const int n_slots = p.st_npp + p.st_nd;                    // partial slots per lane
    const int wg = blockIdx.x * NW + warp, n_warps = gridDim.x * NW;
    const int c_len = int(p.c_len);
    auto heads_of = [&](int a) { return min(HPG, p.G - (a % p.HG) * HPG); };
    auto qhead_of = [&](int a) -> int64_t {                    // first query head of lane a
        const int kvl = a / p.HG, hg = a - kvl * p.HG, b = kvl / p.Hkv, hkv = kvl - b * p.Hkv;
        return int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG;
    };

    // ---------------- uncompressed tokens: items i in [i0, i1) of the L * nd (lane, run of dt tiles) pairs ----------------
    if (p.st_nd > 0 && !failed) {
        const int64_t n_items = int64_t(L) * p.st_nd;
        const int i0 = int((int64_t(wg) * n_items + n_warps - 1) / n_warps), i1 = int((int64_t(wg + 1) * n_items + n_warps - 1) / n_warps);
        __half* Ks = reinterpret_cast<__half*>(smem + (my_area - sbase));
        __half* Vs = Ks + TILE * stage_ld<D>();
        for (int i = i0; i < i1; ++i) {
            const int a = i / p.st_nd, part = i - a * p.st_nd, heads_here = heads_of(a);
            const __half* qh = p.st_q16 + (qhead_of(a) + g) * QS + D;        // raw query of head g
            uint32_t bq[D / 16][2];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                bq[ks][0] = g < heads_here ? __ldcg(reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t)) : 0u;
                bq[ks][1] = g < heads_here ? __ldcg(reinterpret_cast<const uint32_t*>(qh + ks * 16 + 2 * t + 8)) : 0u;
            }
            WarpAcc<D, 0> sd;
            sd.init();
            dense_tiles<D, 1, 0>(p, a / p.HG, int64_t(part) * p.st_dt, int64_t(part + 1) * p.st_dt, Ks, Vs, bq, sd, 0, lane);
            sd.finish();
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                sd.l[0] += __shfl_xor_sync(0xffffffffu, sd.l[0], off);
                sd.l[1] += __shfl_xor_sync(0xffffffffu, sd.l[1], off);
            }
            float* pp = p.st_part + (int64_t(a) * n_slots + p.st_npp + part) * p.slots * PS;
            if (2 * t < heads_here) {
                const bool two = 2 * t + 1 < heads_here;
                float* h0 = pp + (2 * t) * PS;
                float* h1 = h0 + PS;
#pragma unroll
                for (int mt = 0; mt < D / 16; ++mt) {           // rows are coordinates mt * 16 + g and + 8
                    const int c = mt * 16 + g;
                    h0[c] = sd.o[mt][0]; h0[c + 8] = sd.o[mt][2];
                    if (two) { h1[c] = sd.o[mt][1]; h1[c + 8] = sd.o[mt][3]; }
                }
                if (g == 0) {
                    h0[D + QM] = sd.m[0]; h0[D + QM + 1] = sd.l[0];
                    if (two) { h1[D + QM] = sd.m[1]; h1[D + QM + 1] = sd.l[1]; }
                }
            }
            __syncwarp();
        }
    }

    // ---------------- packed tokens: flat tiles [T0, T1) of the L * n_tiles ----------------------------------
    const int64_t total = int64_t(L) * n_tiles;
    const int64_t T0 = min(int64_t(wg) * p.st_range, total), T1 = min(T0 + p.st_range, total);
    const int n_my = failed ? 0 : int(T1 - T0);
    if (n_my > 0) {
        if (!mbar_wait(lut_bar, 0)) {                  // the table image has landed (requested before the wait above)
            atomicCAS(p.status, 0, ERR_TABLES);
            failed = true;
        }
        failed = __any_sync(0xffffffffu, failed);
    }
    if (n_my > 0 && !failed) {
        // A stage is the tile's arrays back to back (keys, values, norms, sign words, residual norms) = NCH 16-byte chunks;
        // lane l copies chunks l, l + 32, ... with one asynchronous 16-byte copy each (no bulk copies in the loop: a bulk
        // copy is issued by one elected lane at a time and costs a dozen instructions).  Every lane's arrival on the
        // stage's barrier is tied to the completion of its own copies.  Sources advance by 16 rows per tile.
        constexpr int NCH = int(P::STAGE / 16), NC = (NCH + 31) / 32;
        const unsigned char* cp_ptr[NC];
        uint32_t cp_step[NC];
        int ia = int(T0 / n_tiles), iti = int(T0 - int64_t(ia) * n_tiles);    // lane and tile of the next copy
        {
            const int64_t row = int64_t(ia / p.HG) * p.c_ls + int64_t(iti) * TILE;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                const int c = lane + 32 * j;
                const unsigned char* base = p.k_hi;
                uint32_t rb = D / 2, off = 16u * c;
                if (c >= int((P::KT + P::VT) / 16)) {
                    const int sidx = c - int((P::KT + P::VT) / 16), arr = sidx >> 2;
                    base = reinterpret_cast<const unsigned char*>(arr == 0 ? static_cast<const void*>(p.k_norms) : arr == 1 ? static_cast<const void*>(p.v_norms)
                                                                  : arr == 2 ? static_cast<const void*>(p.k_qbits) : arr == 3 ? static_cast<const void*>(p.k_qgamma)
                                                                  : arr == 4 ? static_cast<const void*>(p.v_qbits) : static_cast<const void*>(p.v_qgamma));
                    rb = 4; off = 16u * (sidx & 3);
                } else if (c >= int(P::KT / 16)) {
                    base = p.v_hi; rb = D / 4; off = 16u * (c - int(P::KT / 16));
                }
                cp_ptr[j] = base + row * rb + off;
                cp_step[j] = TILE * rb;
            }
        }
        auto issue = [&](int stage) {
            const uint32_t bar = bar0 + 8u * stage, dst = my_area + uint32_t(stage) * P::STAGE + 16u * lane;
#pragma unroll
            for (int j = 0; j < NC; ++j) {
                if (32 * (j + 1) <= NCH || lane + 32 * j < NCH) cp_async16(dst + 512u * j, cp_ptr[j], 16);
                cp_ptr[j] += cp_step[j];
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
            if (++iti == n_tiles) {          // the next copy starts the next lane: same rows again (next head group) or the next lane's storage
                const int64_t jump = ((ia + 1) / p.HG != ia / p.HG ? p.c_ls : 0) - int64_t(n_tiles) * TILE;
#pragma unroll
                for (int j = 0; j < NC; ++j) cp_ptr[j] += jump * int64_t(cp_step[j] / TILE);
                iti = 0; ++ia;
            }
        };
        __syncwarp();
#pragma unroll 1
        for (int n = 0; n < min(n_my, NS); ++n) issue(n);

        // table addresses by byte-permute: {copy offset, byte value, 0x01, 0x00} = LUT_BASE + value * 256 + copy offset
        const uint32_t c4 = LUT_BASE | uint32_t(lane * 4);
        const uint32_t c2 = LUT_BASE | 128u | uint32_t((lane & 15) * 8);
        const int tokA = tok_of_slot(g);                            // tokens of MMA rows g and g + 8: tokA, tokA + 8
        const int sw = t >> 1;                                      // lanes t >= 2 read their token pair in swapped order (so do their table copies)
        const int tokP = tok_of_slot(2 * t), tokQ = tok_of_slot(2 * t + 1);   // tokens of k slots 2t, 2t+1 (and + 8)
        const int tokV0 = sw ? tokQ : tokP, tokV1 = sw ? tokP : tokQ;
        // per-lane offsets into a stage; everything else is an immediate
        const uint32_t k_off = uint32_t(tokA) * (D / 2) + (D == 128 ? 16u * t : 4u * t);
        const uint32_t a_off = 4u * tokA;                           // scalars of tokens tokA (and + 8: 32 bytes on)
        // value codes of row group g: word g of the row at d = 128; bytes 3g .. 3g+2 of the 24-byte row at d = 96, read as the two
        // aligned words around them and one byte-permute (v_sel)
        const uint32_t v_grp = D == 128 ? 4u * g : (3u * g) & ~3u;
        const uint32_t v_sel = 0x3210u + 0x1111u * ((3u * g) & 3u);
        const uint32_t v_off0 = uint32_t(tokV0) * (D / 4) + v_grp, v_off1 = uint32_t(tokV1) * (D / 4) + v_grp;
        const uint32_t p_off = 4u * tokP, q_off = 4u * tokQ;

        BitConsts kc;
        kc.sign_mask = reg_const(0x80008000u); kc.minus_ones = reg_const(0xBC00BC00u); kc.lo_nibbles = reg_const(0x0F0F0F0Fu);
        const int tail_ti = (c_len & (TILE - 1)) ? n_tiles - 1 : -1;          // the tile that reaches past the end of the cache
        int a = int(T0 / n_tiles), ti = int(T0 - int64_t(a) * n_tiles);       // lane and tile being computed
        int slot = wg - int((int64_t(a) * n_tiles) / p.st_range);            // partial slot = this warp's rank among the lane's warps
        int heads_here = 0;
        uint32_t bq[D / 16][2];
        uint32_t bu[QM / 16][2];
        auto load_query = [&]() {
            heads_here = heads_of(a);
            const __half* qh = p.st_q16 + (qhead_of(a) + g) * QS;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                // this thread's bytes 2ks, 2ks+1 of a key row: coordinates 2 * kb .. 2 * kb + 3
                const int kb = D == 128 ? 16 * t + 2 * ks : 16 * (ks >> 1) + 4 * t + 2 * (ks & 1);
                // (written by the launch before this one while this grid may already have been resident: read at L2, never through a non-coherent path)
                bq[ks][0] = g < heads_here ? __ldcg(reinterpret_cast<const uint32_t*>(qh + 2 * kb)) : 0u;
                bq[ks][1] = g < heads_here ? __ldcg(reinterpret_cast<const uint32_t*>(qh + 2 * kb + 2)) : 0u;
            }
            if (QJL) {
                // k slot (ks, register hh, half e) of lane t stands for sketch row 4t + 2ks + hh + 16e: the halves of an
                // operand register are then bits 16 apart in a token's sign word
#pragma unroll
                for (int ks = 0; ks < QM / 16; ++ks)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        const int pi = 4 * t + 2 * ks + hh;
                        bu[ks][hh] = 0u;
                        if (g < heads_here) {
                            const unsigned short lo16 = __ldcg(reinterpret_cast<const unsigned short*>(qh + 2 * D + pi));
                            const unsigned short hi16 = __ldcg(reinterpret_cast<const unsigned short*>(qh + 2 * D + pi + 16));
                            bu[ks][hh] = uint32_t(lo16) | (uint32_t(hi16) << 16);
                        }
                    }
            }
        };
        WarpAcc<D, NZ> st;
        st.init();
        load_query();
        auto flush = [&]() {       // one partial: (lane a, slot)
            st.finish();
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], off);
                st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], off);
            }
            float* pp = p.st_part + (int64_t(a) * n_slots + slot) * p.slots * PS;
            if (2 * t < heads_here) {
                const bool two = 2 * t + 1 < heads_here;
                float* h0 = pp + (2 * t) * PS;
                float* h1 = h0 + PS;
#pragma unroll
                for (int mt = 0; mt < D / 16; ++mt) {              // rows g, g + 8 of m-tile mt: coordinates (D/8) g + 2mt, + 1
                    const int c = (D / 8) * g + 2 * mt;
                    *reinterpret_cast<float2*>(h0 + c) = make_float2(st.o[mt][0], st.o[mt][2]);
                    if (two) *reinterpret_cast<float2*>(h1 + c) = make_float2(st.o[mt][1], st.o[mt][3]);
                }
#pragma unroll
                for (int mz = 0; mz < NZ; ++mz) {
                    h0[D + 16 * mz + g] = st.z[mz][0]; h0[D + 16 * mz + g + 8] = st.z[mz][2];
                    if (two) { h1[D + 16 * mz + g] = st.z[mz][1]; h1[D + 16 * mz + g + 8] = st.z[mz][3]; }
                }
                if (g == 0) {
                    h0[D + QM] = st.m[0]; h0[D + QM + 1] = st.l[0];
                    if (two) { h1[D + QM] = st.m[1]; h1[D + QM + 1] = st.l[1]; }
                }
            }
        };

#pragma unroll (Ring<D>::UNROLL)
        for (int n = 0; n < n_my; ++n) {
            const int stage = n % NS;
            const uint32_t sa = my_area + uint32_t(stage) * P::STAGE;
            if (!__all_sync(0xffffffffu, mbar_wait(bar0 + 8u * stage, uint32_t(n / NS) & 1u))) {
                // the copies never landed: record it, drain what is still in flight (bounded), stop - nothing may land in
                // this CTA's memory after it has gone
                atomicCAS(p.status, 0, ERR_RING);
                failed = true;
                for (int m = n + 1; m < min(n_my, n + NS); ++m) mbar_wait(bar0 + 8u * (m % NS), uint32_t(m / NS) & 1u);
                break;
            }
            const bool partial = ti == tail_ti;

            // ---- scores: S[token][head] = K . q^T, keys straight from the byte table ----
            uint32_t kwa[KW], kwb[KW];
            {
                const uint32_t ka = sa + k_off;
                if constexpr (D == 128) {
                    const uint4 x = ring128o<0>(ka), y = ring128o<8 * (D / 2)>(ka);
                    kwa[0] = x.x; kwa[1] = x.y; kwa[KW - 2] = x.z; kwa[KW - 1] = x.w;
                    kwb[0] = y.x; kwb[1] = y.y; kwb[KW - 2] = y.z; kwb[KW - 1] = y.w;
                } else {
                    kwa[0] = ring32o<0>(ka); kwa[1] = ring32o<16>(ka); kwa[KW - 1] = ring32o<32>(ka);
                    kwb[0] = ring32o<8 * (D / 2)>(ka); kwb[1] = ring32o<8 * (D / 2) + 16>(ka); kwb[KW - 1] = ring32o<8 * (D / 2) + 32>(ka);
                }
            }
            float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t w0 = kwa[ks >> 1], w1 = kwb[ks >> 1];
                const int b0 = (ks & 1) * 2;
                const uint32_t a0 = lut32(__byte_perm(w0, c4, 0x7604 | (b0 << 4)));
                const uint32_t a1 = lut32(__byte_perm(w1, c4, 0x7604 | (b0 << 4)));
                const uint32_t a2 = lut32(__byte_perm(w0, c4, 0x7604 | ((b0 + 1) << 4)));
                const uint32_t a3 = lut32(__byte_perm(w1, c4, 0x7604 | ((b0 + 1) << 4)));
                mma16816(s, a0, a1, a2, a3, bq[ks][0], bq[ks][1]);
            }
            const uint32_t aa = sa + a_off;
            const float kn0 = ring_f32o<P::O_KN>(aa), kn1 = ring_f32o<P::O_KN + 32>(aa);
            float vn0 = ring_f32o<P::O_VN>(aa), vn1 = ring_f32o<P::O_VN + 32>(aa);
            float gv0 = 0.f, gv1 = 0.f;
            if (QJL) {
                // sketch term: (c/d) gamma_k * sum_p sign_p (S q)[p]; signs of rows 4t + q (+ 16) sit at bits 12 + q, 28 + q after one shift
                const uint32_t zs0 = ring32o<P::O_KB>(aa) << (12 - 4 * t), zs1 = ring32o<P::O_KB + 32>(aa) << (12 - 4 * t);
                float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < QM / 16; ++ks)
                    mma16816(sq, sign_pair16(zs0 << (3 - 2 * ks), kc), sign_pair16(zs1 << (3 - 2 * ks), kc), sign_pair16(zs0 << (2 - 2 * ks), kc),
                             sign_pair16(zs1 << (2 - 2 * ks), kc), bu[ks][0], bu[ks][1]);
                const float gk0 = ring_f32o<P::O_KG>(aa) * (QJL_C / D), gk1 = ring_f32o<P::O_KG + 32>(aa) * (QJL_C / D);
                s[0] = fmaf(s[0], kn0, sq[0] * gk0); s[1] = fmaf(s[1], kn0, sq[1] * gk0);
                s[2] = fmaf(s[2], kn1, sq[2] * gk1); s[3] = fmaf(s[3], kn1, sq[3] * gk1);
                gv0 = ring_f32o<P::O_VG>(aa); gv1 = ring_f32o<P::O_VG + 32>(aa);
            } else {
                s[0] *= kn0; s[1] *= kn0; s[2] *= kn1; s[3] *= kn1;
            }
            if (partial) {
                // the last tile of a lane reaches past the end of the cache: its missing tokens (arbitrary bytes) get no weight.
                // A real branch (the barrier keeps it one): once per lane, not a dozen selects per tile.
                __syncwarp();
                const bool ok0 = ti * TILE + tokA < c_len, ok1 = ti * TILE + tokA + 8 < c_len;
                vn0 = ok0 ? vn0 : 0.f; vn1 = ok1 ? vn1 : 0.f; gv0 = ok0 ? gv0 : 0.f; gv1 = ok1 ? gv1 : 0.f;
                s[0] = ok0 ? s[0] : -INFINITY; s[1] = ok0 ? s[1] : -INFINITY;
                s[2] = ok1 ? s[2] : -INFINITY; s[3] = ok1 ? s[3] : -INFINITY;
            }
            uint32_t bp[2];
            float pr[4];
            softmax_stream<D, NZ>(s, vn0, vn1, fmaxf(gv0, gv1), st, bp, pr);

            // ---- values: O^T[coordinate][head] += V^T . P^T ----
            {
                uint32_t va, vb, vc, vd;
                if constexpr (D == 128) {
                    va = ring32o<P::O_V>(sa + v_off0); vb = ring32o<P::O_V>(sa + v_off1);
                    vc = ring32o<P::O_V + 8 * (D / 4)>(sa + v_off0); vd = ring32o<P::O_V + 8 * (D / 4)>(sa + v_off1);
                } else {
                    va = __byte_perm(ring32o<P::O_V>(sa + v_off0), ring32o<P::O_V + 4>(sa + v_off0), v_sel);
                    vb = __byte_perm(ring32o<P::O_V>(sa + v_off1), ring32o<P::O_V + 4>(sa + v_off1), v_sel);
                    vc = __byte_perm(ring32o<P::O_V + 8 * (D / 4)>(sa + v_off0), ring32o<P::O_V + 8 * (D / 4) + 4>(sa + v_off0), v_sel);
                    vd = __byte_perm(ring32o<P::O_V + 8 * (D / 4)>(sa + v_off1), ring32o<P::O_V + 8 * (D / 4) + 4>(sa + v_off1), v_sel);
                }
                // pair the nibbles (two adjacent coordinates) of the two tokens: byte j of z0 = (first word, nibble 2j) |
                // (second word, nibble 2j) << 4, z1 the odd nibbles; one 64-bit lookup yields the two operand registers of
                // rows g and g + 8 (the two coordinates, the token pair in each)
                const uint32_t z0 = nibble_mix(va, vb << 4, kc), z1 = nibble_mix(va >> 4, vb, kc);
                const uint32_t w0 = nibble_mix(vc, vd << 4, kc), w1 = nibble_mix(vc >> 4, vd, kc);
#pragma unroll
                for (int k = 0; k < D / 32; ++k) {
                    const uint2 e01 = lut64(__byte_perm(z0, c2, 0x7604 | (k << 4)));   // m-tile 2k:   k slots 2t, 2t+1
                    const uint2 e23 = lut64(__byte_perm(w0, c2, 0x7604 | (k << 4)));   //             k slots 2t+8, 2t+9
                    const uint2 f01 = lut64(__byte_perm(z1, c2, 0x7604 | (k << 4)));   // m-tile 2k+1
                    const uint2 f23 = lut64(__byte_perm(w1, c2, 0x7604 | (k << 4)));
                    mma16816(st.o[2 * k], e01.x, e01.y, e23.x, e23.y, bp[0], bp[1]);
                    mma16816(st.o[2 * k + 1], f01.x, f01.y, f23.x, f23.y, bp[0], bp[1]);
                }
            }
            if (QJL) {
                // sketch rows of the output: z[row][head] += sum_t sign_row(t) * (p_t * gamma_v[t])
                const uint32_t bz0 = movm_t(pack_h2(pr[0] * gv0, pr[1] * gv0));
                const uint32_t bz1 = movm_t(pack_h2(pr[2] * gv1, pr[3] * gv1));
                const uint32_t zv0 = ring32o<P::O_VB>(sa + p_off), zv1 = ring32o<P::O_VB>(sa + q_off);
                const uint32_t zv2 = ring32o<P::O_VB + 32>(sa + p_off), zv3 = ring32o<P::O_VB + 32>(sa + q_off);
                // put the two tokens' half-words side by side (row r of the first at bit r, of the second at bit r + 16)
                const uint32_t x01 = __byte_perm(zv0, zv1, 0x5410) << (7 - g), y01 = __byte_perm(zv0, zv1, 0x7632) << (7 - g);
                const uint32_t x23 = __byte_perm(zv2, zv3, 0x5410) << (7 - g), y23 = __byte_perm(zv2, zv3, 0x7632) << (7 - g);
                mma16816(st.z[0], sign_pair16(x01 << 8, kc), sign_pair16(x01, kc), sign_pair16(x23 << 8, kc), sign_pair16(x23, kc), bz0, bz1);
                mma16816(st.z[NZ ? 1 : 0], sign_pair16(y01 << 8, kc), sign_pair16(y01, kc), sign_pair16(y23 << 8, kc), sign_pair16(y23, kc), bz0, bz1);
            }

            // ---- the stage is free: ask for the tile NS further on ----
            if (n + NS < n_my) {
                __syncwarp();
                issue(stage);
            }
            if (++ti == n_tiles) {       // the next tile belongs to the next lane
                flush();
                ti = 0; ++a; slot = 0;
                if (n + 1 < n_my) { st.init(); load_query(); }
            }
        }
        if (ti != 0 && !failed) flush();
    }
}

// ---- launch 3: merge --------------------------------------------------------------------------------------
// A thread per (lane, query head, coordinate); a block takes as many lanes (sequence, KV head, head group) as fit some
// 512 threads.  R and S are staged in shared memory once per block, so the rotation back costs shared-memory reads
// instead of a chain of L2 round trips.
constexpr int MERGE_SETS = 10;      // (lane, head) pairs per block at most: 1024 threads / 96
template <int D> __host__ __device__ constexpr size_t merge_smem() { return (size_t(D + QM) * D + size_t(MERGE_SETS) * (2 * MAX_PARTS + D + QM)) * sizeof(float); }
inline int merge_lanes_per_block(int slots, int d) { return std::max(1, 512 / (slots * d)); }
template <int D, bool QJL>
__global__ void __launch_bounds__(1024) stream_merge_kernel(DecodeParams p, int lpb) {
    extern __shared__ __align__(16) unsigned char smem_m[];
    constexpr int PS = part_stride(D);
    float* rs = reinterpret_cast<float*>(smem_m);                 // [D][D] R, then [32][D] S
    const int tid = threadIdx.x, set = tid / D, c = tid - set * D, sub = set / p.slots, h = set - sub * p.slots;
    float* s_m = rs + (D + QM) * D + set * (2 * MAX_PARTS + D + QM);
    float* s_l = s_m + MAX_PARTS;
    float* s_rot = s_l + MAX_PARTS;
    float* s_z = s_rot + D;
    pdl_trigger();
    const int rows = D + (QJL ? QM : 0);
    for (int i = tid; i < rows * (D / 4); i += blockDim.x) {      // constants: before the wait
        const int r = i / (D / 4), k4 = i - r * (D / 4);
        *reinterpret_cast<float4*>(rs + r * D + 4 * k4) = __ldg(reinterpret_cast<const float4*>(r < D ? p.rot + int64_t(r) * D : p.qjl_proj + int64_t(r - D) * D) + k4);
    }
    pdl_wait();
    const int L = p.B * p.Hkv * p.HG;
    const int a = min(blockIdx.x * lpb + sub, L - 1);
    const int kvl = a / p.HG, hg = a - kvl * p.HG, b = kvl / p.Hkv, hkv = kvl - b * p.Hkv;
    const int heads_here = min(HPG, p.G - hg * HPG);
    const bool live = blockIdx.x * lpb + sub < L && h < heads_here;
    const int64_t qhead0 = int64_t(b) * p.Hq + int64_t(hkv) * p.G + hg * HPG;
    const int n_tiles = int((p.c_len + TILE - 1) / TILE);
    const int n_slots = p.st_npp + p.st_nd;
    // the warps whose runs touch this lane's tiles [a * n_tiles, (a + 1) * n_tiles)
    const int fw = int((int64_t(a) * n_tiles) / p.st_range), lw = int((int64_t(a + 1) * n_tiles - 1) / p.st_range);
    const int n_pp = n_tiles > 0 ? lw - fw + 1 : 0;
    const float inv_vs = 1.f / p.v_scale_hi;
    const float* ph = p.st_part + (int64_t(a) * n_slots * p.slots + h) * PS;
    const int64_t sstride = int64_t(p.slots) * PS;
    if (c < n_slots) {
        const bool valid = h < heads_here && (c < n_pp || c >= p.st_npp);
        s_m[c] = valid ? __ldcg(ph + c * sstride + D + QM) : -INFINITY;
        s_l[c] = valid ? __ldcg(ph + c * sstride + D + QM + 1) : 0.f;
    }
    __syncthreads();
    float M = -INFINITY;
    for (int i = 0; i < n_slots; ++i) M = fmaxf(M, s_m[i]);
    float Lsum = 0.f, ar = 0.f, ad = 0.f, az = 0.f;
#pragma unroll 8
    for (int i = 0; i < n_slots; ++i) {
        const float mi = s_m[i];
        const float w = mi == -INFINITY ? 0.f : ex2(mi - M);
        const float v = mi == -INFINITY ? 0.f : __ldcg(ph + i * sstride + c);
        Lsum = fmaf(w, s_l[i], Lsum);
        if (i < p.st_npp) {
            ar = fmaf(w, v, ar);
            if (QJL && c < QM && mi != -INFINITY) az = fmaf(w, __ldcg(ph + i * sstride + D + c), az);
        } else {
            ad = fmaf(w, v, ad);
        }
    }
    s_rot[c] = ar * inv_vs;
    if (QJL && c < QM) s_z[c] = az * (QJL_C / D);
    __syncthreads();
    // undo the rotation of the packed part (y @ R, rotation.py:68-78) and add (c/d) z @ S (qjl.py:89-92)
    float v = ad;
#pragma unroll 8
    for (int j = 0; j < D; ++j) v = fmaf(s_rot[j], rs[j * D + c], v);
    if (QJL) {
#pragma unroll 8
        for (int i = 0; i < QM; ++i) v = fmaf(s_z[i], rs[(D + i) * D + c], v);
    }
    if (live) store_from_f32(p.out, p.out_dtype, (qhead0 + h) * D + c, v / Lsum);
}

// ---- host side ------------------------------------------------------------------------------------------------
template <int D, bool QJL> static bool fits() {
    const unsigned sb = dd::probe_smem_base();
    if (sb == ~0u || sb > LO_BASE || (sb & 15u)) return false;
    int dev = 0, max_optin = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return false;
    return size_t(Plan<D, QJL>::SMEM_END - sb) <= size_t(max_optin);
}

template <int D, bool QJL> static int launch(const DecodeParams& p, cudaStream_t s) {
    const unsigned sb = dd::probe_smem_base();
    const size_t smem = Plan<D, QJL>::SMEM_END - sb;
    static std::atomic<bool> set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(decode_stream_kernel<D, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(stream_query_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(query_smem<D>()));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(stream_merge_kernel<D, QJL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(merge_smem<D>()));
        if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: shared memory %zu B: %s", smem, cudaGetErrorString(e));
        set[dev].store(true, std::memory_order_release);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = p.pdl ? 1 : 0;
    cudaLaunchConfig_t cfg{};
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int64_t n_q = int64_t(p.B) * p.Hq;
    cfg.gridDim = dim3(unsigned((n_q + QPB - 1) / QPB));
    cfg.blockDim = dim3(QNT);
    cfg.dynamicSmemBytes = query_smem<D>();
    cudaError_t e = cudaLaunchKernelEx(&cfg, stream_query_kernel<D>, p);
    if (e == cudaSuccess) {
        cfg.gridDim = dim3(unsigned(p.st_grid));
        cfg.blockDim = dim3(NT);
        cfg.dynamicSmemBytes = smem;
        e = cudaLaunchKernelEx(&cfg, decode_stream_kernel<D, QJL>, p);
    }
    if (e == cudaSuccess) {
        const int lpb = merge_lanes_per_block(p.slots, D);
        cfg.gridDim = dim3(unsigned((p.B * p.Hkv * p.HG + lpb - 1) / lpb));
        cfg.blockDim = dim3(unsigned(lpb * p.slots * D));
        cfg.dynamicSmemBytes = merge_smem<D>();
        e = cudaLaunchKernelEx(&cfg, stream_merge_kernel<D, QJL>, p, lpb);
    }
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn: %s", cudaGetErrorString(e));
    return TQ_OK;
}

}  // namespace ds

bool stream_supported(int d, bool qjl) {
    if (d == 96) return qjl ? ds::fits<96, true>() : ds::fits<96, false>();
    if (d == 128) return qjl ? ds::fits<128, true>() : ds::fits<128, false>();
    return false;
}

StreamPlan stream_plan(int batch, int n_q_heads, int n_kv_heads, int d, int64_t c_len, int64_t dense_len, int sms) {
    StreamPlan s{};
    const int G = n_q_heads / n_kv_heads, hg = (G + HPG - 1) / HPG;
    const int64_t L = int64_t(batch) * n_kv_heads * hg;
    const int64_t p_tiles = (c_len + TILE - 1) / TILE, d_tiles = (dense_len + TILE - 1) / TILE;
    s.grid = sms;
    const int64_t n_warps = int64_t(s.grid) * ds::NW;
    s.range = std::max<int64_t>((L * p_tiles + n_warps - 1) / n_warps, 1);
    s.npp = int((p_tiles + s.range - 1) / s.range) + 1;
    if (d_tiles > 0) {
        int64_t nd = std::min<int64_t>(d_tiles, std::max<int64_t>(n_warps / L, 1));
        s.dt = int((d_tiles + nd - 1) / nd);
        s.nd = int((d_tiles + s.dt - 1) / s.dt);
    }
    s.q16_bytes = (size_t(batch) * n_q_heads * ds::q_stride(d) * sizeof(__half) + 255) / 256 * 256;
    s.part_bytes = size_t(L) * size_t(s.npp + s.nd) * size_t(std::min(G, HPG)) * ds::part_stride(d) * sizeof(float);
    return s;
}

int launch_decode_stream(const DecodeParams& p, cudaStream_t s) {
    const bool qjl = p.qjl_proj != nullptr;
    if (p.D == 96) return qjl ? ds::launch<96, true>(p, s) : ds::launch<96, false>(p, s);
    return qjl ? ds::launch<128, true>(p, s) : ds::launch<128, false>(p, s);
}

}  // namespace tq
