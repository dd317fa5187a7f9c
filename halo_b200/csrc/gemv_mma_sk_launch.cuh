// Host side of the balanced skinny kernels: tensor map, scratch, kernel choice.  Included by one .cu per weight format
// (so the formats compile in parallel); each defines its launch_gemv_sk_<format>().
#pragma once
#include "gemv_mma_sk.cuh"

namespace halo_cuda {
namespace sk {

constexpr int kResidentMaxTok = 8;  // larger batches always stream x (sixteen rows of records do not fit next to any ring)
// Stages of a warp's weight ring.  Two (one tile being read, one in flight) measured faster than three or four on every
// shape: the per-warp streams already keep far more bytes in flight than the memory system needs, and deeper rings
// only spread the DRAM accesses over more rows at a time.
constexpr int kRingStages = 2;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/// The weight matrix as a 2-D tensor {row elements, rows} with row pitch w_stride, tiled (slot pitch) x 16 rows.
/// Tiles reaching past the end of a row or of the matrix are zero-filled by the copy engine.
template <class F>
int weight_map(const GemvCall& c, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        HC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail(HALO_CUDA_E_BACKEND, "cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {c.row_bytes / F::kMapElemBytes, c.rows};
    const cuuint64_t strides[1] = {c.w_stride};
    const cuuint32_t box[2] = {F::kBoxInner, 16};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(out, F::kMapElemBytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2,
                              const_cast<uint8_t*>(c.w), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HALO_CUDA_E_KERNEL, "MATMUL: cannot describe the weight matrix to the copy engine (CUresult %d)", (int)r);
    return 0;
}

inline cudaLaunchConfig_t pdl_config(uint32_t grid, uint32_t smem, cudaStream_t s, cudaLaunchAttribute* attr) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kSkWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

/// The x conversion of a batched call: one warp per super-block, launched so that it overlaps the tail of the kernel before it.
inline int launch_stage(const float* x, uint64_t x_stride, uint8_t* scratch, uint32_t nb, uint32_t n_tok, bool split_halves, cudaStream_t s) {
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(n_tok, 0, s, attr);
    cfg.gridDim = dim3(n_tok, (nb + 15u) / 16u);
    HC_CUDA(cudaLaunchKernelEx(&cfg, stage_x_rec_kernel, x, x_stride, scratch, nb, n_tok, split_halves ? 1u : 0u));
    return 0;
}

/// The kernel-side view of a call's peer description (none: world = 0).
inline PeerPush peer_push(const GemvCall& c, uint32_t tok0) {
    PeerPush pp{};
    if (c.peer == nullptr) return pp;
    pp.tok0 = tok0;
    pp.world = c.peer->world, pp.rank = c.peer->rank, pp.capacity = c.peer->capacity;
    for (uint32_t i = 0; i < c.peer->world && i < kMaxPeers; ++i) pp.slots[i] = static_cast<unsigned long long*>(c.peer->slots[i]);
    pp.epoch = c.peer->epoch;
    return pp;
}

/// The partition of one call: which K slicing, the column ranges of the CTAs, and the scratch of the reduction.
struct Geometry {
    uint32_t nb, ks;
    SkTable table;
    void *counters, *partials;
    // int8 family, calls of several token tiles: the x records of ALL tiles, written by one conversion launch (tile i of
    // `staged_tile` rows at staged + i * nb * rec_bytes(staged_tile)); null: every tile sees to its own
    const uint8_t* staged = nullptr;
    uint32_t staged_tile = 0;
};

/// x records a CTA of the resident kernels holds in shared memory: under a one-slice partition whose every CTA walks less
/// than a unit's columns, the longest range; otherwise all super-blocks.
inline uint32_t resident_records(const Geometry& g) {
    if (g.ks != 1) return g.nb;
    uint32_t longest = 0;
    for (uint32_t c = 0; c < g.table.parts; ++c) longest = std::max(longest, g.table.start[c + 1] - g.table.start[c]);
    return longest < g.table.cols_per_unit ? longest : g.nb;
}

template <class F, int NTOK>
int geometry(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s, Geometry* g) {
    constexpr int G = (NTOK + 3) / 4;
    g->nb = c.cols / 256u;
    const uint64_t n_rb = (uint64_t{c.rows} + 15) / 16;
    if (n_rb * g->nb >= (1ull << 30)) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: more than 2^30 (16-row, 256-column) tiles");
    g->ks = plan_partition(c.rows, g->nb, static_cast<uint32_t>(ctx->prop.multiProcessorCount), F::kAllowSlices, &g->table);
    if (int rc = workspace(ctx, 2, n_rb * 4, s, &g->counters, /*zeroed=*/true)) return rc;
    return workspace(ctx, 3, uint64_t{g->table.parts} * 2 * kSkWarps * 32 * 2 * G * 4, s, &g->partials);
}

template <class F, int NTOK, int NS, int KS>
int launch_resident(HaloCudaCtx* ctx, const GemvCall& c, const Geometry& g, uint32_t tok0, cudaStream_t s) {
    constexpr bool PRE = NTOK >= 2;
    using L = SkLayout<F, NTOK, NS, KS>;
    if constexpr (L::kOffData >= kSmemBudget) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: ring of %d stages does not fit", NS);
    } else {
        const uint32_t smem_bytes = L::kOffData + resident_records(g) * L::kRec;
        if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(gemv_sk_resident_kernel<F, NTOK, NS, KS, PRE>), kSmemBudget)) return rc;
        const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
        float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
        CUtensorMap wmap;
        if (int rc = weight_map<F>(c, &wmap)) return rc;
        const uint8_t* xstage = nullptr;
        if constexpr (PRE) {
            void* ws = nullptr;
            if (int rc = workspace(ctx, 0, stage_rec_scratch_bytes(g.nb, NTOK), s, &ws)) return rc;
            if (int rc = launch_stage(x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, NTOK, F::kXLaneBytes == 8, s)) return rc;
            xstage = static_cast<const uint8_t*>(ws);
        }
        cudaLaunchAttribute attr[1];
        const cudaLaunchConfig_t cfg = pdl_config(g.table.parts, smem_bytes, s, attr);
        if (c.norm_w != nullptr) {
            if constexpr (NTOK == 1) {
                if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(gemv_sk_resident_kernel<F, NTOK, NS, KS, PRE, true>), kSmemBudget)) return rc;
                HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_sk_resident_kernel<F, NTOK, NS, KS, PRE, true>, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows,
                                           g.nb, static_cast<float*>(g.partials), static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage,
                                           peer_push(c, tok0), c.norm_w, c.norm_eps));
                return 0;
            } else {
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row");
            }
        }
        HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_sk_resident_kernel<F, NTOK, NS, KS, PRE>, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb,
                                   static_cast<float*>(g.partials), static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, peer_push(c, tok0),
                                   static_cast<const float*>(nullptr), 0.0f));
        return 0;
    }
}

template <class F, int NTOK, int KS>
int launch_streamed(HaloCudaCtx* ctx, const GemvCall& c, const Geometry& g, uint32_t tok0, cudaStream_t s) {
    constexpr int NS = kRingStages;
    using L = SkLayout<F, NTOK, NS, KS>;
    constexpr uint32_t kXSlot = KS * L::kRec;
    static_assert(L::kOffData + 2 * kXSlot <= kSmemBudget, "two columns of x must fit next to the ring");
    if (c.norm_w != nullptr) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL with a fused input norm: %u columns of x do not fit in shared memory", c.cols);
    const uint32_t xs_cols = std::min<uint32_t>(kMaxXSlots / 2, (kSmemBudget - L::kOffData) / kXSlot / 2);
    const uint32_t smem_bytes = L::kOffData + 2 * xs_cols * kXSlot;
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(gemv_sk_streamed_kernel<F, NTOK, NS, KS>), kSmemBudget)) return rc;
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    CUtensorMap wmap;
    if (int rc = weight_map<F>(c, &wmap)) return rc;
    void* ws = nullptr;
    if (int rc = workspace(ctx, 0, stage_rec_scratch_bytes(g.nb, NTOK), s, &ws)) return rc;
    if (int rc = launch_stage(x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, NTOK, F::kXLaneBytes == 8, s)) return rc;
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = pdl_config(g.table.parts, smem_bytes, s, attr);
    HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_sk_streamed_kernel<F, NTOK, NS, KS>, wmap, g.table, y, c.y_stride, c.rows, g.nb, xs_cols,
                               static_cast<float*>(g.partials), static_cast<uint32_t*>(g.counters), ctx->error_word_dev,
                               static_cast<const uint8_t*>(ws), peer_push(c, tok0)));
    return 0;
}

/// n rows starting at tok0: the resident kernel when all of x fits next to the ring, else the streamed one.
template <class F, int NTOK, int KS>
int launch_sliced(HaloCudaCtx* ctx, const GemvCall& c, const Geometry& g, uint32_t tok0, cudaStream_t s) {
    if constexpr (NTOK <= kResidentMaxTok) {
        const uint64_t x_bytes = uint64_t{resident_records(g)} * XRec<NTOK>::kBytes;
        if (SkLayout<F, NTOK, kRingStages, KS>::kOffData + x_bytes <= kSmemBudget) return launch_resident<F, NTOK, kRingStages, KS>(ctx, c, g, tok0, s);
    }
    return launch_streamed<F, NTOK, KS>(ctx, c, g, tok0, s);
}

template <class F, int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > 16) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n != NTOK) return launch_tokens<F, NTOK + 1>(ctx, c, tok0, n, s);
        Geometry g{};
        if (int rc = geometry<F, NTOK>(ctx, c, s, &g)) return rc;
        if constexpr (F::kAllowSlices) {
            if (g.ks == 2) return launch_sliced<F, NTOK, 2>(ctx, c, g, tok0, s);
        }
        return launch_sliced<F, NTOK, 1>(ctx, c, g, tok0, s);
    }
}

template <class F>
int launch_format(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    // Token tiles of 16 (four MMA column groups); the remainder takes the smallest instantiation that holds it.
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += 16) {
        const uint32_t n = c.n_vec - t0 < 16 ? c.n_vec - t0 : 16;
        if (int rc = launch_tokens<F, 1>(ctx, c, t0, n, s)) return rc;
    }
    return 0;
}

}  // namespace sk
}  // namespace halo_cuda
