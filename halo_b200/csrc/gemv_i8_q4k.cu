// Host side of the int8 tensor-core skinny kernels (gemv_i8.cuh) for raw Q4_K rows: token tiles, scratch, launch.
#include "gemv_i8.cuh"
#include "gemv_mma_sk_launch.cuh"

namespace halo_cuda {
namespace i8 {

constexpr int kRing = 2;    // stages of a warp's weight ring: deeper rings measured slower (more row segments in flight at a time)
constexpr int kMaxTok = 8;  // x rows per launch: two MMA column groups; larger batches run in tiles of eight

template <class F, int NTOK, int KS>
constexpr bool fits(uint32_t nb) {
    return Layout<F, NTOK, kRing, KS>::bytes(nb) <= kSmemBudget;
}

template <class F, int NTOK, int KS>
int launch_tile(HaloCudaCtx* ctx, const GemvCall& c, const sk::Geometry& g, uint32_t tok0, cudaStream_t s) {
    constexpr bool PRE = NTOK >= 2;
    using L = Layout<F, NTOK, kRing, KS>;
    const uint32_t smem_bytes = L::bytes(g.nb);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    CUtensorMap wmap;
    if (int rc = sk::weight_map<F>(c, &wmap)) return rc;
    const uint8_t* xstage = nullptr;
    if constexpr (PRE) {
        void* ws = nullptr;
        if (int rc = workspace(ctx, 0, stage_scratch_bytes(g.nb, NTOK), s, &ws)) return rc;
        cudaLaunchAttribute sattr[1];
        cudaLaunchConfig_t scfg = sk::pdl_config(NTOK, 0, s, sattr);
        scfg.gridDim = dim3(NTOK, (g.nb + 15u) / 16u);
        HC_CUDA(cudaLaunchKernelEx(&scfg, stage_x_i8_kernel, x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, static_cast<uint32_t>(NTOK)));
        xstage = static_cast<const uint8_t*>(ws);
    }
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = sk::pdl_config(g.table.parts, smem_bytes, s, attr);
    if (c.norm_w != nullptr) {
        if constexpr (NTOK == 1) {
            auto kern = gemv_i8_kernel<F, 1, kRing, KS, false, true>;
            if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
            HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, static_cast<float*>(g.partials),
                                       static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), c.norm_w, c.norm_eps));
            return 0;
        } else {
            return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row");
        }
    }
    auto kern = gemv_i8_kernel<F, NTOK, kRing, KS, PRE, false>;
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
    HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, static_cast<float*>(g.partials),
                               static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), static_cast<const float*>(nullptr),
                               0.0f));
    return 0;
}

/// n rows starting at tok0 (n <= the largest tile whose records fit in shared memory)
template <class F, int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > kMaxTok) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n != NTOK) return launch_tokens<F, NTOK + 1>(ctx, c, tok0, n, s);
        sk::Geometry g{};
        if (int rc = sk::geometry<F, NTOK>(ctx, c, s, &g)) return rc;
        if (g.ks == 2) return launch_tile<F, NTOK, 2>(ctx, c, g, tok0, s);
        return launch_tile<F, NTOK, 1>(ctx, c, g, tok0, s);
    }
}

/// The largest token tile (<= kMaxTok) whose x records fit next to the ring for `nb` super-blocks; 0: not even one row.
template <class F>
uint32_t max_tile(uint32_t nb) {
    // the one-slice layout (no slice sums) is the smaller one; the two-slice layout adds at most 4 KB
    const uint64_t fixed = Layout<F, 8, kRing, 2>::kOffDigits + 1024;
    for (uint32_t n = kMaxTok; n >= 1; --n)
        if (fixed + uint64_t{nb} * rec_bytes(n) <= kSmemBudget) return n;
    return 0;
}

}  // namespace i8

bool gemv_i8_supports(const GemvCall& c) {
    if (c.wtype != HALO_CUDA_T_Q4_K || c.cols == 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // tensor-map base and pitch
    if (c.w_stride >= (uint64_t{1} << 40) || c.row_bytes >= (uint64_t{1} << 32)) return false;
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return i8::max_tile<i8::Q4Ki>(c.cols / 256u) != 0;                                       // one row's records must fit in shared memory
}

int launch_gemv_i8(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    const uint32_t tile = i8::max_tile<i8::Q4Ki>(c.cols / 256u);
    if (tile == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_i8x2 keeps x in shared memory; %u columns do not fit", c.cols);
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += tile) {
        const uint32_t n = c.n_vec - t0 < tile ? c.n_vec - t0 : tile;
        if (int rc = i8::launch_tokens<i8::Q4Ki, 1>(ctx, c, t0, n, s)) return rc;
    }
    return 0;
}

}  // namespace halo_cuda
