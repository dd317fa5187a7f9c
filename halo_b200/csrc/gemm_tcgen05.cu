// gemm_tcgen05: prefill GEMM (placeholder until the kernel lands).
#include "internal.h"

namespace halo_cuda {
bool gemm_tcgen05_supports(const GemvCall&) { return false; }
int launch_gemm_tcgen05(HaloCudaCtx*, const GemvCall&, bool, cudaStream_t) {
    return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemm_tcgen05 is not built");
}
}  // namespace halo_cuda
