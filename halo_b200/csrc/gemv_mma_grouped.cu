// gemv_mma_r: tensor-core skinny kernel for Q6_K, Q8_0 and Q4_0 weights in the REPACKED row layout of halo_cuda_repack.
//
// Why a repacked layout: the GGUF blocks of these formats are 210 / 34 / 18 bytes, so their rows cannot be fetched by
// the copy engine (tile coordinates and row pitches must be multiples of 16 bytes) and their quant words are only
// 2-byte aligned.  The reference makes the same move for its Vulkan matvecs (include/halo/tensor/repack.h:11-36; the
// layout is a kernel variant, include/halo/backend/backend.h:178-183).  Repacking is a pure byte permutation of each
// 256-weight group (plus padding): every quant code and scale is bit-identical, which the tests check by unpacking the
// repacked rows back.  Layout of one group of 256 weights (rows are sequences of groups):
//   Q4_0r  144 B: d[8] fp16 | for chunk c<2, thread t<4: the quant word (bytes 4t..4t+3) of blocks 4c..4c+3
//   Q8_0r  272 B: d[8] fp16 | for chunk c<4, thread t<4: words (block 2c, k-step 0/1), (block 2c+1, k-step 0/1);
//                 a k-step is 16 elements, the word holds elements 16*step + 4t .. +3
//   Q6_Kr  224 B: scales[16] int8 | d fp16, 14 B pad | for half n<2, thread t<4: ql words (b, lh) = bytes
//                 64n + 32b + 16lh + 4t..+3 | for thread t<4: qh words (n, lh) = bytes 32n + 16lh + 4t..+3
// i.e. the four words one thread needs next to each other, so a fragment is one 16-byte shared-memory load.
//
// Arithmetic (the same scheme as gemv_mma_f16x2): A holds the unsigned quant code as an fp16 subnormal (code * 2^-24,
// exact), B holds x as fp16 hi + lo columns, one m16n8k16 MMA per 16 elements.  Every scale group (a 32-element block,
// or 16 elements of Q6_K) gets a fresh fp32 accumulator, and the group's scale and zero point are applied in fp32:
//     y += scale_g * (acc_g - zero * sum_g(x))        zero = 8 / 128 / 32, sum_g(x) in fp32 from the staging pass.
// Rows do not depend on the batch size; results are bounded against the CPU backend, not bitwise.
//
// Roofline: HBM.  Algorithmic bytes = rows * row_bytes + 4 * n_vec * cols + 4 * n_vec * rows.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {
namespace {

using namespace mma;

// ---- repack: raw GGUF rows -> grouped rows (one thread per 32-bit output word) ---------------------------------------------
__device__ __forceinline__ uint32_t ld_u32_bytes(const uint8_t* p) {
    return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) | (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24);
}

/// Word `wi` of repacked group `grp` of a row whose raw bytes start at `raw` (any alignment).
__device__ uint32_t repack_word(uint32_t wtype, const uint8_t* raw, uint32_t grp, uint32_t wi) {
    if (wtype == HALO_CUDA_T_Q4_0) {
        const uint8_t* g = raw + grp * 144u;  // 8 blocks of 18 bytes
        if (wi < 4) return static_cast<uint32_t>(g[(2 * wi) * 18]) | (static_cast<uint32_t>(g[(2 * wi) * 18 + 1]) << 8) |
                           (static_cast<uint32_t>(g[(2 * wi + 1) * 18]) << 16) | (static_cast<uint32_t>(g[(2 * wi + 1) * 18 + 1]) << 24);
        const uint32_t k = wi - 4, c = k >> 4, t = (k >> 2) & 3u, j = k & 3u;  // chunk, thread, block inside the chunk
        return ld_u32_bytes(g + (4 * c + j) * 18 + 2 + 4 * t);
    }
    if (wtype == HALO_CUDA_T_Q8_0) {
        const uint8_t* g = raw + grp * 272u;  // 8 blocks of 34 bytes
        if (wi < 4) return static_cast<uint32_t>(g[(2 * wi) * 34]) | (static_cast<uint32_t>(g[(2 * wi) * 34 + 1]) << 8) |
                           (static_cast<uint32_t>(g[(2 * wi + 1) * 34]) << 16) | (static_cast<uint32_t>(g[(2 * wi + 1) * 34 + 1]) << 24);
        const uint32_t k = wi - 4, c = k >> 4, t = (k >> 2) & 3u, j = k & 3u;  // j = (block parity) * 2 + k-step
        return ld_u32_bytes(g + (2 * c + (j >> 1)) * 34 + 2 + 16 * (j & 1u) + 4 * t);
    }
    // Q6_K: 210 raw bytes -> 224
    const uint8_t* g = raw + grp * 210u;
    if (wi < 4) return ld_u32_bytes(g + 192 + 4 * wi);                                                                  // scales
    if (wi == 4) return static_cast<uint32_t>(g[208]) | (static_cast<uint32_t>(g[209]) << 8);                          // d
    if (wi < 8) return 0u;                                                                                              // pad
    if (wi < 40) {
        const uint32_t k = wi - 8, n = k >> 4, t = (k >> 2) & 3u, j = k & 3u;  // j = b * 2 + lh
        return ld_u32_bytes(g + 64 * n + 32 * (j >> 1) + 16 * (j & 1u) + 4 * t);
    }
    const uint32_t k = wi - 40, t = k >> 2, j = k & 3u;  // j = n * 2 + lh
    return ld_u32_bytes(g + 128 + 32 * (j >> 1) + 16 * (j & 1u) + 4 * t);
}

__global__ void __launch_bounds__(256) repack_kernel(uint32_t wtype, const uint8_t* __restrict__ src, uint64_t src_stride, uint32_t* __restrict__ dst,
                                                     uint64_t dst_stride, uint32_t rows, uint32_t groups, uint32_t words_per_group) {
    const uint64_t total = uint64_t{rows} * groups * words_per_group;
    for (uint64_t i = uint64_t{blockIdx.x} * blockDim.x + threadIdx.x; i < total; i += uint64_t{gridDim.x} * blockDim.x) {
        const uint32_t wi = static_cast<uint32_t>(i % words_per_group);
        const uint64_t gr = i / words_per_group;
        const uint32_t grp = static_cast<uint32_t>(gr % groups), r = static_cast<uint32_t>(gr / groups);
        reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(dst) + uint64_t{r} * dst_stride)[grp * words_per_group + wi] =
            repack_word(wtype, src + uint64_t{r} * src_stride, grp, wi);
    }
}

uint32_t group_bytes(uint32_t wtype) {
    return wtype == HALO_CUDA_T_Q4_0 ? 144u : wtype == HALO_CUDA_T_Q8_0 ? 272u : wtype == HALO_CUDA_T_Q6_K ? 224u : 0u;
}

}  // namespace

uint64_t repacked_row_bytes(uint32_t wtype, uint64_t cols) { return cols / 256u * group_bytes(wtype); }

bool gemv_mma_r_supports(const GemvCall& c) {
    if (group_bytes(c.wtype) == 0 || c.cols == 0 || c.cols % 256u != 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // tensor-map base and pitch
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) == 0;  // the kernels keep partial sums and staged x in context scratch
}

int launch_gemv_mma_r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    switch (c.wtype) {
        case HALO_CUDA_T_Q4_0: return launch_gemv_sk_q40r(ctx, c, s);
        case HALO_CUDA_T_Q8_0: return launch_gemv_sk_q80r(ctx, c, s);
        case HALO_CUDA_T_Q6_K: return launch_gemv_sk_q6kr(ctx, c, s);
        default: return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_r takes repacked Q4_0 / Q8_0 / Q6_K weights");
    }
}

int launch_repack(uint32_t wtype, const void* src, uint64_t src_stride, void* dst, uint64_t dst_stride, uint32_t rows, uint32_t cols, cudaStream_t s) {
    const uint32_t groups = cols / 256u, words = group_bytes(wtype) / 4u;
    const uint64_t total = uint64_t{rows} * groups * words;
    if (total == 0) return 0;
    const uint32_t blocks = static_cast<uint32_t>(total / 256 + 1 < 148 * 16 ? total / 256 + 1 : 148 * 16);
    repack_kernel<<<blocks, 256, 0, s>>>(wtype, static_cast<const uint8_t*>(src), src_stride, static_cast<uint32_t*>(dst), dst_stride, rows, groups, words);
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace halo_cuda
