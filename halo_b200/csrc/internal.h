// Internal declarations shared by the translation units of libhalo_cuda.so.  Not part of the ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "halo_cuda.h"

namespace halo_cuda {

/// Records the calling thread's failure message and returns `status` (for `return fail(...)`).
int fail(int status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define HC_CUDA(expr)                                                                                     \
    do {                                                                                                  \
        cudaError_t e_ = (expr);                                                                          \
        if (e_ != cudaSuccess)                                                                            \
            return ::halo_cuda::fail(e_ == cudaErrorMemoryAllocation ? HALO_CUDA_E_MEMORY : HALO_CUDA_E_BACKEND, \
                                     "%s: %s", #expr, cudaGetErrorString(e_));                            \
    } while (0)

struct TypeInfo {
    uint32_t block_elems, block_bytes;
};
/// Block geometry of a supported weight type (src/tensor/dtype.cpp:19-51); false for any other id.
bool type_info(uint32_t wtype, TypeInfo* out);

struct PlanEntry {
    uint32_t wtype, rows, cols, n_vec_lo, n_vec_hi, variant_id;
};

}  // namespace halo_cuda

struct HaloCudaCtx {
    int device = 0;
    cudaDeviceProp prop{};
    bool lost = false;
    // Scratch for kernels that need global memory beyond their operands (activation staging, split-K
    // partials).  Grown on demand and reused in stream order, so every stream has a set of its own: calls on different
    // streams of one context may overlap on the device without sharing counters, partials or staged x.  One thread drives a context.
    // Slot 0 serves the matmul kernels, slot 1 the LM head (its logits and argmax partials live across a matmul),
    // slot 2 the row-block counters of the balanced kernels (zeroed when allocated, left zeroed by every kernel),
    // slot 3 their partial sums.
    struct Scratch {
        void* block[4] = {nullptr, nullptr, nullptr, nullptr};
        uint64_t bytes[4] = {0, 0, 0, 0};
    };
    std::unordered_map<cudaStream_t, Scratch> scratch;
    std::vector<halo_cuda::PlanEntry> plan;
    // One word of mapped pinned host memory that kernels OR error bits into (bit 0: a bounded device-side wait
    // expired).  The host reads it after every stream wait; a set bit marks the context lost.
    uint32_t* error_word_host = nullptr;
    uint32_t* error_word_dev = nullptr;
    // halo_cuda_malloc serves from a memory pool that never gives memory back to the driver while the context lives, on a
    // stream of its own: an allocation costs microseconds, not a driver call.  `pooled` holds what came from the pool
    // (shareable allocations come from cudaMalloc, which inter-process handles need).
    cudaMemPool_t pool = nullptr;
    cudaStream_t pool_stream = nullptr;
    std::unordered_set<void*> pooled;
    // Two pinned host buffers the weight loader fills in turn, each cut into up to eight lanes (one per host thread), and the
    // event behind the last device copy out of each lane.
    void* staging[2] = {nullptr, nullptr};
    uint64_t staging_bytes = 0;
    cudaEvent_t staging_done[2][8] = {};
    // Kernels whose dynamic shared-memory limit has been raised on THIS device (the attribute is per device, so the
    // bookkeeping is per context, not per process).
    std::unordered_set<const void*> smem_raised;
    // How often the reduction kernel of a row split re-reads a peer's word (about 0.2 us apart) before it declares the sender lost
    // (about a second by default; halo_cuda_ctx_set_peer_wait_polls lowers it, which is how the tests make the wait run out).
    uint32_t peer_wait_polls = 1u << 22;
};

namespace halo_cuda {

/// Makes ctx's device current; E_API for a null ctx, E_DEVICE once the context is lost.
int enter(HaloCudaCtx* ctx);
/// Returns ctx scratch of at least `bytes` (grows with cudaMalloc; earlier contents are dropped; `zeroed` clears a
/// newly allocated block in stream order).
int workspace(HaloCudaCtx* ctx, int slot, uint64_t bytes, cudaStream_t stream, void** out, bool zeroed = false);
/// Raises the dynamic shared-memory limit of `kernel` to `bytes` on ctx's device, once per context.
int allow_dynamic_smem(HaloCudaCtx* ctx, const void* kernel, uint32_t bytes);
/// The bookkeeping of allow_dynamic_smem without the driver call: true when (ctx, kernel) was not yet recorded.
bool note_smem_raised(HaloCudaCtx* ctx, const void* kernel);

/// A validated gemv: strides resolved to bytes, geometry checked.
struct GemvCall {
    uint32_t wtype, rows, cols, n_vec, flags;
    const uint8_t* w;
    const float* x;
    float* y;
    uint64_t w_stride, x_stride, y_stride;  // bytes
    uint64_t row_bytes;
    const HaloCudaPeerReduce* peer = nullptr;  // row-split tensor parallelism: push the result rows to the peers instead of storing y
    const float* norm_w = nullptr;             // fused input norm (single-row calls): x is the raw row, the kernel multiplies by rms and norm_w
    float norm_eps = 0.0f;
    // GDN gates epilogue (GemvArgs::gates): rows == 2 * n_v; row r < n_v stores sigmoid(y), row n_v + j stores
    // a[j] * softplus(y + dt_bias[j]) instead of y
    const float* gate_dt_bias = nullptr;
    const float* gate_a = nullptr;
    uint32_t gate_n_v = 0;
};
int validate_gemv(const HaloCudaGemv* a, const char* op, bool y_optional, GemvCall* out);
uint32_t resolve_variant(const HaloCudaCtx* ctx, const GemvCall& c, uint32_t requested);
int lm_head_outputs_disjoint(const GemvCall& c, const void* result, const void* ids, const char* op);

/// What a kernel stores for row `n` of a matmul with the GDN gates epilogue (n_v != 0), else y unchanged: the CPU backend's
/// gdn_gates (beta_out = sigmoid(beta); g_out = a * softplus(alpha + dt_bias); backends/cpu/kernel_common.h:31-33) applied
/// to the two row halves.  expf / log1pf are the device's (a few ulp from the host's).
__device__ __forceinline__ float gated_value(float y, uint32_t n, uint32_t n_v, const float* __restrict__ dt_bias, const float* __restrict__ a) {
    if (n_v == 0) return y;
    if (n < n_v) return 1.0f / (1.0f + expf(-y));
    const uint32_t j = n - n_v;
    const float t = y + dt_bias[j];
    return a[j] * (t > 20.0f ? t : log1pf(expf(t)));
}

// kernel launchers (one per translation unit); each returns a status
int launch_gemv_exact8(const GemvCall& c, cudaStream_t s);
int launch_gemv_warp_f32(const GemvCall& c, cudaStream_t s);
bool gemv_warp_f32_supports(const GemvCall& c);
int launch_gemv_mma(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_mma_m1(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
bool gemv_mma_supports(const GemvCall& c);
int launch_gemm_tcgen05(HaloCudaCtx* ctx, const GemvCall& c, bool bf16, bool repacked, cudaStream_t s);
int launch_gemv_sk_q4k(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_sk_q40r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_sk_q80r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_sk_q6kr(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_peer_finish(HaloCudaCtx* ctx, const HaloCudaPeerReduce& p, float* y, uint64_t y_stride, uint32_t rows, uint32_t n_vec, cudaStream_t s);
int launch_gemv_mma_r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_i8(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
bool gemv_i8_supports(const GemvCall& c);
int launch_gemv_i8_q6kr(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_i8_q80r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
int launch_gemv_i8_q40r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s);
bool gemv_i8_q6kr_supports(const GemvCall& c);
bool gemv_i8_q80r_supports(const GemvCall& c);
bool gemv_i8_q40r_supports(const GemvCall& c);
bool gemv_i8_r_supports(const GemvCall& c);   // the three above by weight type
namespace mma {
struct SkTable;
}
uint32_t gemv_i8_q4k_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table);
uint32_t gemv_i8_q6kr_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table);
uint32_t gemv_i8_q80r_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table);
uint32_t gemv_i8_q40r_plan(uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table);
void gemv_i8_q4k_tiles(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* out);
void gemv_i8_q6kr_tiles(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* out);
void gemv_i8_q80r_tiles(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* out);
void gemv_i8_q40r_tiles(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* out);
uint32_t gemv_i8_plan(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table);  // by weight type
bool gemv_i8_q6kr_fits(uint32_t cols);
bool gemv_i8_q80r_fits(uint32_t cols);
bool gemv_i8_q40r_fits(uint32_t cols);
/// The variant a repacked tensor of this type and (largest local) K travels with: the int8 family where its x records fit in
/// shared memory, else the fp16 family's repacked kernel (which can stream x).
uint32_t repacked_variant(uint32_t wtype, uint32_t cols);
bool reads_repacked_rows(uint32_t variant_id);  // the W operand of this variant is in the layout of halo_cuda_repack_rows
bool gemv_mma_r_supports(const GemvCall& c);
uint64_t repacked_row_bytes(uint32_t wtype, uint64_t cols);  // 0 for a type without a repacked layout
int launch_repack(uint32_t wtype, const void* src, uint64_t src_stride, void* dst, uint64_t dst_stride, uint32_t rows, uint32_t cols, cudaStream_t s);
bool gemm_tcgen05_supports(const GemvCall& c, bool repacked = false);
int launch_get_rows(const HaloCudaGetRows& a, uint64_t row_bytes, uint64_t table_stride, uint64_t out_stride, cudaStream_t s);
int launch_argmax(const float* logits, uint64_t stride_elems, uint32_t n, uint32_t n_vec, uint32_t valid, uint32_t row_offset,
                  uint32_t* result, int32_t* ids, void* scratch, cudaStream_t s);
uint64_t argmax_scratch_bytes(uint32_t n, uint32_t n_vec);

}  // namespace halo_cuda
