// Host side of the int8 tensor-core skinny kernels (gemv_i8.cuh): partition, token tiles, scratch, launch.  Included by
// one .cu per weight format so that the formats compile in parallel.
#pragma once
#include "gemv_i8.cuh"
#include "gemv_mma_sk_launch.cuh"

namespace halo_cuda {
namespace i8 {

constexpr int kRing = 2;  // stages of a warp's weight ring: deeper rings measured slower (more row segments in flight at a time)

/// Shared memory of a launch with n_tok x rows, n_rec resident records and 2^ks_shift slices (Layout<F, n_tok, kRing>::bytes
/// for a batch size known only at run time).
template <class F>
uint32_t smem_bytes(uint32_t n_tok, uint32_t n_rec, uint32_t ks_shift) {
    const uint32_t G = (n_tok + 3) / 4, off_slices = kOffRing + kSkWarps * kRing * 16 * F::kPitch;
    const uint32_t red = (kSkWarps - (kSkWarps >> ks_shift)) * 32u * 2u * G * 4u;
    return ((off_slices + red + 127u) & ~127u) + (n_tok == 1 ? 576u : 0u) + n_rec * rec_bytes(n_tok);
}

constexpr int kStreamFrom = 2;  // the streamed form takes any batch: a long K under a partition that keeps many records per CTA (a large N under
                                // the even split, a long K under slices) leaves the resident form room for one or two rows only

/// Shared memory of the streamed form: the double buffer of x records (two halves of `stretch` columns) in place of the resident ones.
template <class F>
uint32_t smem_bytes_streamed(uint32_t n_tok, uint32_t ks_shift, uint32_t stretch = 2) {
    return smem_bytes<F>(n_tok, 0, ks_shift) + 2u * stretch * (1u << ks_shift) * rec_bytes(n_tok);
}

/// Columns per stretch of a streamed launch: the most that fit, from two (which always do where the form is chosen) to the format's
/// kStretchMax.  Longer stretches mean fewer block barriers: 128256 x 8192 Q4_K at 8 rows 174 -> 161 us, 32768 x 28672 Q4_0 144 -> 129;
/// Q8_0, whose streamed launches already run near the HBM rate, measured 3 - 5 % slower beyond three columns.
template <class F>
uint32_t stretch_columns(uint32_t n_tok, uint32_t ks_shift) {
    uint32_t xc = 2;
    while (xc < F::kStretchMax && smem_bytes_streamed<F>(n_tok, ks_shift, xc + 1) <= kSmemBudget) ++xc;
    return xc;
}

inline uint32_t log2_of(uint32_t ks) {
    uint32_t s = 0;
    while ((1u << s) < ks) ++s;
    return s;
}

/// In-CTA slices need every x record of a row resident; they are on offer where that holds for a tile of eight x rows.
template <class F>
bool slices_fit(uint32_t nb) {
    return smem_bytes<F>(8, nb, 4) <= kSmemBudget;
}

/// The partition of a shape (a function of rows, cols and the SM count alone: every batch size gets the same one).
template <class F>
void plan(const HaloCudaCtx* ctx, const GemvCall& c, sk::Geometry* g) {
    g->nb = c.cols / 256u;
    g->ks = plan_partition_i8(c.rows, g->nb, static_cast<uint32_t>(ctx->prop.multiProcessorCount), slices_fit<F>(g->nb), &g->table);
}

/// The same plan for inspection: slice count and table for a device with `sm_count` SMs.
template <class F>
uint32_t plan_for(uint32_t rows, uint32_t cols, uint32_t sm_count, SkTable* table) {
    return plan_partition_i8(rows, cols / 256u, sm_count, slices_fit<F>(cols / 256u), table);
}

/// Whether a resident launch of n_tok (>= 2) x rows converts them itself instead of reading the records a conversion launch wrote.
/// The conversion launch costs a dependent launch on the chain (about 3 us); converting in the kernel costs every CTA its
/// n_rec * n_tok (record, row) pairs before its first tile.  Measured break-even: near 96 pairs where the CTAs read different
/// columns of x (partial residency: 5120 x 17408 at 8 rows is 80 pairs, 24.5 us against 26.4), near 48 where all of them read
/// all of x (K = 5120 at 2 rows is 40 pairs, 12.3 us against 13.4; at 4 rows the two forms tie, at 8 the launch wins by 3 us).
inline bool converts_in_kernel(const sk::Geometry& g, uint32_t n_rec, uint32_t n_tok) {
    return n_rec * n_tok <= (n_rec < g.nb ? 96u : 48u);
}

/// Whether a tile of n_tok rows reads records a conversion launch wrote (the streamed form always does).
inline bool tile_needs_stage(const sk::Geometry& g, uint32_t n_tok, bool streamed) {
    return n_tok >= 2 && (streamed || !converts_in_kernel(g, sk::resident_records(g), n_tok));
}

/// The conversion launch: `total` x rows from `x` on, as consecutive tiles of `tile_rows` rows, into `scratch`.
inline int launch_stage(const float* x, uint64_t x_stride, uint8_t* scratch, uint32_t nb, uint32_t tile_rows, uint32_t total, bool perm, cudaStream_t s) {
    cudaLaunchAttribute sattr[1];
    cudaLaunchConfig_t scfg = sk::pdl_config(total, 0, s, sattr);
    scfg.gridDim = dim3(total, (nb + 15u) / 16u);
    HC_CUDA(cudaLaunchKernelEx(&scfg, stage_x_i8_kernel, x, x_stride, scratch, nb, tile_rows, total, perm ? 1u : 0u));
    return 0;
}

template <class F, int NTOK, int KSC, int XC = 0>
int launch_tile(HaloCudaCtx* ctx, const GemvCall& c, const sk::Geometry& g, uint32_t tok0, cudaStream_t s) {
    constexpr bool PRE = NTOK >= 2;
    using L = Layout<F, NTOK, kRing>;
    // n_rec: the resident records, or (streamed form) the columns per stretch
    const uint32_t ks_shift = log2_of(g.ks), n_rec = XC == 1 ? stretch_columns<F>(NTOK, ks_shift) : sk::resident_records(g);
    const uint32_t smem_bytes = XC == 1 ? smem_bytes_streamed<F>(NTOK, ks_shift, n_rec) : L::bytes(n_rec, ks_shift);
    if (smem_bytes > kSmemBudget) return fail(HALO_CUDA_E_KERNEL, "MATMUL: %u x records of %d rows do not fit in shared memory", n_rec, NTOK);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    CUtensorMap wmap;
    if (int rc = sk::weight_map<F>(c, &wmap)) return rc;
    const uint8_t* xstage = nullptr;
    if (PRE && g.staged != nullptr) {  // the call's one conversion launch has written this tile's records
        xstage = g.staged + uint64_t{tok0 / g.staged_tile} * g.nb * rec_bytes(g.staged_tile);
    } else if (PRE && tile_needs_stage(g, NTOK, XC == 1)) {
        void* ws = nullptr;
        if (int rc = workspace(ctx, 0, stage_scratch_bytes(g.nb, NTOK), s, &ws)) return rc;
        if (int rc = launch_stage(x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, NTOK, NTOK, F::kPermX, s)) return rc;
        xstage = static_cast<const uint8_t*>(ws);
    }
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = sk::pdl_config(g.table.parts, smem_bytes, s, attr);
    if (c.norm_w != nullptr) {
        if constexpr (NTOK == 1) {
            auto kern = gemv_i8_kernel<F, 1, kRing, KSC, false, true>;
            if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
            HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, n_rec, ks_shift, static_cast<float*>(g.partials),
                                       static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), c.norm_w, c.norm_eps));
            return 0;
        } else {
            return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row");
        }
    }
    auto kern = gemv_i8_kernel<F, NTOK, kRing, KSC, PRE, false, XC>;
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kSmemBudget)) return rc;
    HC_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, g.table, x, c.x_stride, y, c.y_stride, c.rows, g.nb, n_rec, ks_shift, static_cast<float*>(g.partials),
                               static_cast<uint32_t*>(g.counters), ctx->error_word_dev, xstage, sk::peer_push(c, tok0), static_cast<const float*>(nullptr),
                               0.0f));
    return 0;
}

/// n rows starting at tok0 (n <= the largest tile whose records fit in shared memory)
template <class F, int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, sk::Geometry& g, uint32_t tok0, uint32_t n, bool streamed, cudaStream_t s) {
    if constexpr (NTOK > F::kMaxTok) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n != NTOK) return launch_tokens<F, NTOK + 1>(ctx, c, g, tok0, n, streamed, s);
        // scratch of the cross-CTA reduction: a zeroed counter per row block, two partial records per CTA and row-block slot
        constexpr int G = (NTOK + 3) / 4;
        const uint64_t n_rb = (uint64_t{c.rows} + 15) / 16;
        if (int rc = workspace(ctx, 2, n_rb * 4, s, &g.counters, /*zeroed=*/true)) return rc;
        if (int rc = workspace(ctx, 3, uint64_t{g.table.parts} * 2 * kSkWarps * 32 * 2 * G * 4, s, &g.partials)) return rc;
        if constexpr (NTOK >= kStreamFrom) {
            if (streamed) {
                if (c.norm_w != nullptr) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row");
                if (g.ks == 2) return launch_tile<F, NTOK, 2, 1>(ctx, c, g, tok0, s);
                return launch_tile<F, NTOK, 0, 1>(ctx, c, g, tok0, s);
            }
        }
        if constexpr (F::kPipedConversion && NTOK >= 2) {
            // a launch that converts more than three rounds of (record, row) pairs itself does the later rounds behind its first tiles
            // (three rounds -- 5120 x 17408 at 4 rows -- measured 1 % slower that way)
            if (g.staged == nullptr && !tile_needs_stage(g, NTOK, false) && sk::resident_records(g) * NTOK > 3 * kSkWarps) {
                if (g.ks == 2) return launch_tile<F, NTOK, 2, 2>(ctx, c, g, tok0, s);
                return launch_tile<F, NTOK, 0, 2>(ctx, c, g, tok0, s);
            }
        }
        if (g.ks == 2) return launch_tile<F, NTOK, 2>(ctx, c, g, tok0, s);  // the partition of the large shapes: slice count folded into the code
        return launch_tile<F, NTOK, 0>(ctx, c, g, tok0, s);
    }
}

/// The largest token tile (<= F::kMaxTok) whose x records (n_rec super-blocks resident) fit next to the ring; 0: not even one row.
template <class F>
uint32_t max_tile(uint32_t n_rec, uint32_t ks_shift) {
    for (uint32_t n = F::kMaxTok; n >= 1; --n)
        if (smem_bytes<F>(n, n_rec, ks_shift) <= kSmemBudget) return n;
    return 0;
}

template <class F>
bool supports_format(const GemvCall& c) {
    if (c.wtype != F::kType || c.cols == 0 || c.cols % 256u != 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // tensor-map base and pitch
    if (c.w_stride >= (uint64_t{1} << 40) || c.row_bytes >= (uint64_t{1} << 32)) return false;
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    if ((uint64_t{c.rows} + 15) / 16 * (c.cols / 256u) >= (1ull << 30)) return false;      // (16-row, 256-column) tiles
    return max_tile<F>(c.cols / 256u, 0) != 0;  // one row's records must fit whatever the partition
}

/// Whether rows of `cols` columns can run at all: one row's records next to the ring (a function of the format and K alone).
template <class F>
bool fits_format(uint32_t cols) {
    return cols != 0 && cols % 256u == 0 && max_tile<F>(cols / 256u, 0) != 0;
}

/// How a call of n_vec x rows is cut into launches: a function of the partition and the format alone (host arithmetic).
struct TilePlan {
    uint32_t tile = 0;      // x rows of every launch but the last (0: not even one row's records fit)
    uint32_t cap_res = 0;   // the most rows the resident form holds
    bool streamed = false;  // tiles of two rows and up stream x
    bool one_stage = false; // one conversion launch writes the records of every tile
    uint32_t launches = 0, conversions = 0, stretch = 0;  // matmul launches, conversion launches, columns per stretch (streamed)
};

template <class F>
TilePlan tile_plan(const sk::Geometry& g, uint32_t n_vec) {
    TilePlan p;
    // The partition decides how many records a CTA holds, and that the token tile; a batch is cut into equal tiles
    // (whole MMA column groups of four rows where that still fits).
    const uint32_t ks_shift = log2_of(g.ks);
    p.cap_res = max_tile<F>(sk::resident_records(g), ks_shift);
    if (p.cap_res == 0 || n_vec == 0) return p;
    // A batch larger than the resident form holds in one tile streams x instead, where that makes the tile larger: the weights
    // are then read once (same tiles, same order, same bits).
    uint32_t cap = p.cap_res;
    // (only where a CTA walks at least eight columns: on short walks the stretch barriers cost more than the second pass over
    // weights that are still in L2 -- 5120 x 5120 at 16 rows measured 21.7 us streamed against 19.0 us in two resident tiles)
    uint32_t longest = 0;
    for (uint32_t cc = 0; cc < g.table.parts; ++cc) longest = std::max(longest, g.table.start[cc + 1] - g.table.start[cc]);
    if (n_vec > p.cap_res && static_cast<uint32_t>(F::kMaxTok) > p.cap_res && longest >= 8) {
        uint32_t cap_s = 0;
        for (uint32_t n = F::kMaxTok; n >= static_cast<uint32_t>(kStreamFrom) && cap_s == 0; --n)
            if (smem_bytes_streamed<F>(n, ks_shift) <= kSmemBudget) cap_s = n;
        if (cap_s > p.cap_res && n_vec >= static_cast<uint32_t>(kStreamFrom)) cap = cap_s, p.streamed = true;
    }
    const uint32_t n_tiles = (n_vec + cap - 1) / cap;
    p.tile = (n_vec + n_tiles - 1) / n_tiles;
    if ((p.tile + 3u) / 4u * 4u <= cap) p.tile = (p.tile + 3u) / 4u * 4u;
    if (p.streamed && p.tile < static_cast<uint32_t>(kStreamFrom)) p.tile = std::min<uint32_t>(cap, kStreamFrom);
    p.tile = std::min(p.tile, n_vec);  // (a call of fewer rows than the rounded tile is one launch of its own size)
    if (p.streamed) p.stretch = stretch_columns<F>(std::min(p.tile, n_vec), ks_shift);
    // Every tile but the last has `tile` rows, so tile i starts at row i * tile; a last tile of one row is converted in its kernel.
    uint32_t staged_tiles = 0;
    for (uint32_t t0 = 0; t0 < n_vec; t0 += p.tile) {
        const uint32_t left = n_vec - t0, n = std::min(left, p.tile);
        ++p.launches;
        if (tile_needs_stage(g, n, p.streamed && left >= static_cast<uint32_t>(kStreamFrom))) ++staged_tiles;
    }
    // A call of several tiles converts all of its x rows in ONE launch where any tile wants the records made for it: every further
    // conversion launch would be another dependent launch on the chain (two tiles of eight rows: 5120 x 5120 19.2 -> 17.0 us,
    // 1024 x 5120 13.2 -> 11.2).
    p.one_stage = n_vec > p.tile && staged_tiles != 0;
    p.conversions = p.one_stage ? 1u : staged_tiles;
    return p;
}

/// The same for inspection: the plan of a rows x cols matmul at n_vec x rows on a device with `sm_count` SMs.
template <class F>
TilePlan tile_plan_for(uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count) {
    sk::Geometry g{};
    g.nb = cols / 256u;
    g.ks = plan_for<F>(rows, cols, sm_count, &g.table);
    return tile_plan<F>(g, n_vec);
}

inline void fill_tiles(const TilePlan& p, HaloCudaGemvTiles* out) {
    *out = HaloCudaGemvTiles{};
    out->tile_rows = p.tile, out->launches = p.launches, out->conversions = p.conversions, out->streamed = p.streamed ? 1u : 0u;
    out->stretch_cols = p.stretch, out->resident_rows = p.cap_res;
}

template <class F>
int launch_format(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    sk::Geometry g{};
    plan<F>(ctx, c, &g);
    const TilePlan p = tile_plan<F>(g, c.n_vec);
    if (p.cap_res == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the int8 kernels keep x in shared memory; %u columns do not fit", c.cols);
    if (p.one_stage) {
        const uint32_t tiles_all = (c.n_vec + p.tile - 1) / p.tile;
        void* ws = nullptr;
        if (int rc = workspace(ctx, 0, uint64_t{tiles_all} * stage_scratch_bytes(g.nb, p.tile), s, &ws)) return rc;
        if (int rc = launch_stage(c.x, c.x_stride, static_cast<uint8_t*>(ws), g.nb, p.tile, c.n_vec, F::kPermX, s)) return rc;
        g.staged = static_cast<const uint8_t*>(ws), g.staged_tile = p.tile;
    }
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += p.tile) {
        const uint32_t left = c.n_vec - t0, n = std::min(left, p.tile);
        // (a last tile of one row runs the single-row kernel)
        if (int rc = launch_tokens<F, 1>(ctx, c, g, t0, n, p.streamed && left >= static_cast<uint32_t>(kStreamFrom), s)) return rc;
    }
    return 0;
}

}  // namespace i8
}  // namespace halo_cuda
