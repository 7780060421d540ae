// tq_decode_attn_static: the decode-attention kernel of decode.cu, run on scratch memory that is part of the
// library image instead of a buffer the caller supplies.
//
// Who needs this.  tq_decode_attn asks its caller for a workspace.  Some callers have none to give and cannot
// create one when the call is made: a serving process that handed all device memory to its own arena when it
// started and must not go back to the driver afterwards, or a step loop whose latency budget rules out a driver
// allocation (which may synchronise the whole device).  For them the scratch lives in a fixed-size device array
// compiled into this library: TQ_DECODE_STATIC_SCRATCH_BYTES on every GPU that loads the library, held until
// the process exits.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// Set-up.  Host code cannot use the array's name as a device address (it names a host-side stand-in; a kernel
// given it would fault or touch the wrong memory), so the first call on each device, with that device current,
// resolves the real address once with cudaGetSymbolAddress and keeps it.  Make that first call outside any
// stream capture.  With CUDA's default lazy module loading that first look-up is also the moment the driver
// loads this module and reserves the array's bytes on the device: a process that is about to hand all remaining
// device memory to its own pool must make the first call (or set CUDA_MODULE_LOADING=EAGER) before it does so.
// If the reservation fails the call reports it and allocates nothing else.
//
// Sharing.  All calls on a device use the same array and find in it whatever the previous call left.  The kernel
// needs its arrival counters at zero; every call clears them on the caller's stream before the launch.  Two calls
// that run on the GPU at the same time (different streams, no ordering) would race on the array: order them.
#include <atomic>

#include "decode.cuh"

namespace tq {

static __device__ __align__(256) unsigned char g_decode_scratch[TQ_DECODE_STATIC_SCRATCH_BYTES];

static int static_scratch_ptr(void** out) {
    // one slot per device; filled at most once (compare-and-swap: concurrent first calls resolve the same address)
    static std::atomic<void*> ptrs[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(TQ_ERR_LAUNCH, "tq_decode_attn_static: cudaGetDevice: %s", cudaGetErrorString(e));
    void* p = ptrs[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            return fail(TQ_ERR_LAUNCH, "tq_decode_attn_static: the device has no room left for the library's %zu-byte scratch array "
                        "(the module is loaded at the first call: make it before a memory pool takes the device, or set CUDA_MODULE_LOADING=EAGER)",
                        size_t(TQ_DECODE_STATIC_SCRATCH_BYTES));
        }
        if (e != cudaSuccess || p == nullptr) return fail(TQ_ERR_LAUNCH, "tq_decode_attn_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        void* expected = nullptr;
        ptrs[dev].compare_exchange_strong(expected, p, std::memory_order_acq_rel);
    }
    *out = p;
    return TQ_OK;
}

}  // namespace tq

using namespace tq;

extern "C" int tq_decode_attn_static(const tq_decode_args* a, void* stream) {
    if (!a) return fail(TQ_ERR_INVALID, "tq_decode_attn_static: null args");
    // (the persistent streaming kernel is taken only where its larger scratch fits the array too)
    const size_t need = decode_workspace_bytes_split_kernels(a->batch, a->n_q_heads, a->n_kv_heads, a->d, a->c_len, a->sink_len + a->res_len);
    if (need == 0) return fail(TQ_ERR_INVALID, "tq_decode_attn_static: bad sizes");
    if (need > size_t(TQ_DECODE_STATIC_SCRATCH_BYTES))
        return fail(TQ_ERR_UNSUPPORTED, "tq_decode_attn_static: these sizes need %zu bytes of scratch, the built-in array holds %zu; "
                    "use tq_decode_attn with a caller-provided workspace", need, size_t(TQ_DECODE_STATIC_SCRATCH_BYTES));
    void* scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    DecodeParams p;
    bool direct = false;
    rc = decode_prepare(a, scratch, size_t(TQ_DECODE_STATIC_SCRATCH_BYTES), &p, &direct);
    if (rc) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's bytes; the arrival counters are the only part that must start at zero
    const size_t counter_bytes = size_t(p.B) * p.Hkv * p.HG * sizeof(int);
    cudaError_t e = cudaMemsetAsync(p.counters, 0, counter_bytes, s);
    if (e != cudaSuccess) return fail(TQ_ERR_LAUNCH, "tq_decode_attn_static: clearing counters: %s", cudaGetErrorString(e));
    return decode_launch(p, direct, s);
}
