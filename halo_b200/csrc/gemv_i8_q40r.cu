// gemv_mma_i8x2_r: the int8 tensor-core skinny kernels over repacked Q4_0 rows.
#include "gemv_i8_launch.cuh"

namespace halo_cuda {
bool gemv_i8_q40r_supports(const GemvCall& c) { return i8::supports_format<i8::Q40i>(c); }
bool gemv_i8_q40r_fits(uint32_t cols) { return i8::fits_format<i8::Q40i>(cols); }
int launch_gemv_i8_q40r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) { return i8::launch_format<i8::Q40i>(ctx, c, s); }
uint32_t gemv_i8_q40r_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table) { return i8::plan_for<i8::Q40i>(rows, cols, sm_count, table); }
}  // namespace halo_cuda
