// Host side of the int8 tensor-core skinny kernels (gemv_i8.cuh): token tiles, scratch, launch.  Included by one .cu per
// weight format so that the formats compile in parallel.
#pragma once
#include "gemv_i8.cuh"
#include "gemv_mma_sk_launch.cuh"

namespace halo_cuda {
namespace i8 {

constexpr int kRing = 2;    // stages of a warp's weight ring: deeper rings measured slower (more row segments in flight at a time)

template <class F, int NTOK, int KS>
int launch_tile(HaloCudaCtx* ctx, const GemvCall& c, const sk::Geometry& g, uint32_t tok0, cudaStream_t s) {
    constexpr bool PRE = NTOK >= 2;
    using L = Layout<F, NTOK, kRing, KS>;
    const uint32_t n_rec = sk::resident_records(g), smem_bytes = L::bytes(n_rec);
    if (smem_bytes > kSmemBudget) return fail(HALO_CUDA_E_KERNEL, "MATMUL: %u x records of %d rows do not fit in shared memory", n_rec, NTOK);
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
        HC_CUDA(cudaLaunchKernelEx(&scfg, stage_x_i8_kernel, x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, static_cast<uint32_t>(NTOK), F::kPermX ? 1u : 0u));
        xstage = static_cast<const uint8_t*>(ws);
    }
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = sk::pdl_config(g.table.parts, smem_bytes, s, attr);
    if (c.norm_w != nullptr) {
        if constexpr (NTOK == 1) {
            auto kern = gemv_i8_kernel<F, 1, kRing, KS, false, true>;
            if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
            HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, n_rec, static_cast<float*>(g.partials),
                                       static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), c.norm_w, c.norm_eps));
            return 0;
        } else {
            return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row");
        }
    }
    auto kern = gemv_i8_kernel<F, NTOK, kRing, KS, PRE, false>;
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
    HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, n_rec, static_cast<float*>(g.partials),
                               static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), static_cast<const float*>(nullptr),
                               0.0f));
    return 0;
}

/// n rows starting at tok0 (n <= the largest tile whose records fit in shared memory)
template <class F, int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > F::kMaxTok) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n != NTOK) return launch_tokens<F, NTOK + 1>(ctx, c, tok0, n, s);
        sk::Geometry g{};
        if (int rc = sk::geometry<F, NTOK>(ctx, c, s, &g)) return rc;
        if constexpr (F::kAllowSlices) {
            if (g.ks == 2) return launch_tile<F, NTOK, 2>(ctx, c, g, tok0, s);
        }
        return launch_tile<F, NTOK, 1>(ctx, c, g, tok0, s);
    }
}

/// The largest token tile (<= F::kMaxTok) whose x records (n_rec super-blocks resident) fit next to the ring; 0: not even one row.
template <class F>
uint32_t max_tile(uint32_t n_rec) {
    // the one-slice layout (no slice sums) is the smaller one; the two-slice layout adds at most 4 KB
    const uint64_t fixed = Layout<F, F::kMaxTok, kRing, 2>::kOffDigits + 1024;
    for (uint32_t n = F::kMaxTok; n >= 1; --n)
        if (fixed + uint64_t{n_rec} * rec_bytes(n) <= kSmemBudget) return n;
    return 0;
}

template <class F>
bool supports_format(const GemvCall& c) {
    if (c.wtype != F::kType || c.cols == 0 || c.cols % 256u != 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // tensor-map base and pitch
    if (c.w_stride >= (uint64_t{1} << 40) || c.row_bytes >= (uint64_t{1} << 32)) return false;
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return max_tile<F>(c.cols / 256u) != 0;                                                 // one row's records must fit whatever the partition
}

template <class F>
int launch_format(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    const uint32_t nb = c.cols / 256u;
    if (max_tile<F>(nb) == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the int8 kernels keep x in shared memory; %u columns do not fit", c.cols);
    // The partition (a function of the shape alone) decides how many records a CTA holds, and that the token tile.
    sk::Geometry g{};
    g.nb = nb;
    g.ks = plan_partition(c.rows, nb, static_cast<uint32_t>(ctx->prop.multiProcessorCount), F::kAllowSlices, &g.table);
    const uint32_t tile = max_tile<F>(sk::resident_records(g));
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += tile) {
        const uint32_t n = c.n_vec - t0 < tile ? c.n_vec - t0 : tile;
        if (int rc = launch_tokens<F, 1>(ctx, c, t0, n, s)) return rc;
    }
    return 0;
}

}  // namespace i8
}  // namespace halo_cuda
