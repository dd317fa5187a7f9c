// Balanced tensor-core skinny kernels, instantiated for one weight format (see gemv_mma_sk.cuh).
#include "gemv_mma_sk_launch.cuh"

namespace halo_cuda {

int launch_gemv_sk_q40r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) { return sk::launch_format<mma::Q40r>(ctx, c, s); }

}  // namespace halo_cuda
