// gemv_mma_f16x2: tensor-core skinny kernel for decode-shaped Q4_K calls (placeholder until the kernel lands).
#include "internal.h"

namespace halo_cuda {
bool gemv_mma_supports(const GemvCall&) { return false; }
int launch_gemv_mma(HaloCudaCtx*, const GemvCall&, cudaStream_t) {
    return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_f16x2 is not built");
}
}  // namespace halo_cuda
