// gemv_mma_i8x2: the int8 tensor-core skinny kernels over raw Q4_K rows.
#include "gemv_i8_launch.cuh"

namespace halo_cuda {
bool gemv_i8_supports(const GemvCall& c) { return i8::supports_format<i8::Q4Ki>(c); }
int launch_gemv_i8(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) { return i8::launch_format<i8::Q4Ki>(ctx, c, s); }
uint32_t gemv_i8_q4k_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table) { return i8::plan_for<i8::Q4Ki>(rows, cols, sm_count, table); }
void gemv_i8_q4k_tiles(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* out) {
    i8::fill_tiles(i8::tile_plan_for<i8::Q4Ki>(rows, cols, n_vec, sm_count), out);
}
}  // namespace halo_cuda
