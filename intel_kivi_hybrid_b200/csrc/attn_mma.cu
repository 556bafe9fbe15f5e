// Tensor-core decode attention (placeholder until the kernel lands).
#include "kivi_common.cuh"

namespace kivi {

bool attn_mma_supported(const kivi_layer*, int, int) { return false; }

int run_attn_mma(const kivi_layer*, int64_t, int, int, const void*, int, int, float, int, int, int,
                 float*, float*, cudaStream_t) {
    set_error("tensor-core decode attention is not built");
    return KIVI_ERR_UNSUPPORTED;
}

}  // namespace kivi
