// gemv_mma_i8x2: the int8 tensor-core skinny kernels over raw Q4_K rows.
#include "gemv_i8_launch.cuh"

namespace halo_cuda {
bool gemv_i8_supports(const GemvCall& c) { return i8::supports_format<i8::Q4Ki>(c); }
int launch_gemv_i8(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) { return i8::launch_format<i8::Q4Ki>(ctx, c, s); }
}  // namespace halo_cuda
