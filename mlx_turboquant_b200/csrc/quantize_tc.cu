// Tensor-core (tcgen05) quantize kernel for fp16 rows, d = 128.  Placeholder dispatcher: reports
// "not handled" so the caller takes the general CUDA-core path.
#include "common.cuh"

int tq_quantize_pack_tc(const tq_quantize_args*, cudaStream_t, bool* handled) {
    *handled = false;
    return TQ_OK;
}
