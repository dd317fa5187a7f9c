// gemv_mma_i8x2_r: the int8 tensor-core skinny kernels over repacked Q8_0 rows.
#include "gemv_i8_launch.cuh"

namespace halo_cuda {
bool gemv_i8_q80r_supports(const GemvCall& c) { return i8::supports_format<i8::Q80i>(c); }
bool gemv_i8_q80r_fits(uint32_t cols) { return i8::fits_format<i8::Q80i>(cols); }
int launch_gemv_i8_q80r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) { return i8::launch_format<i8::Q80i>(ctx, c, s); }
uint32_t gemv_i8_q80r_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table) { return i8::plan_for<i8::Q80i>(rows, cols, sm_count, table); }
}  // namespace halo_cuda
