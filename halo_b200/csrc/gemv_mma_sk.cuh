// The two balanced tensor-core skinny kernels, for any weight format of mma_formats.cuh.
//
// Both run a persistent grid of at most one 16-warp CTA per SM over the partition of mma_common.cuh: every warp of a
// CTA walks the CTA's run of (unit, column) pairs for its own row block and K slice, streaming its 16-row tiles through
// a private ring of TMA tile copies (bounded mbarrier waits); the K slices of a row block are added through shared
// memory, and row blocks whose K range is shared between CTAs are finished by the last-arriver reduction, so every
// sum has one fixed order.  The kernels differ only in how x reaches the MMAs:
//
//   resident  x (all of K, every row of the call) sits in shared memory for the whole kernel: converted in the kernel
//             for a single row, else fetched from the pre-staged records with bulk copies.  Warps run freely.
//   streamed  for calls whose x does not fit: the warps of a CTA walk their columns together, so only a short ring of
//             x records (one per column, bulk-copied from the pre-staged scratch, refilled behind a block barrier
//             every few columns) is resident.
//
// Both use the same partition, the same per-item arithmetic and the same x records, so a row's bits depend neither on
// the batch size nor on which of the two kernels computed it.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "internal.h"
#include "mma_formats.cuh"

namespace halo_cuda {
namespace sk {

using namespace mma;

constexpr uint32_t kOffXFull = 272;  // mbarriers of the x ring (streamed kernel): after the partial maxima
constexpr uint32_t kMaxXSlots = 16;

template <class F>
__device__ __forceinline__ void tma_item_g2s(uint32_t dst, const CUtensorMap* map, uint32_t sb, uint32_t row, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(sb * F::kItemCoord), "r"(row), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void linger_after_loss() {  // copies may still be in flight towards this CTA's shared memory
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
}

/// Position in a CTA's run of columns: the producer (ring fill) and the consumer walk it independently.
struct ColumnWalk {
    uint32_t col, end, unit, k;
    __device__ __forceinline__ void init(uint32_t lo, uint32_t hi, uint32_t cpu) { col = lo, end = hi, unit = lo / cpu, k = lo - unit * cpu; }
    __device__ __forceinline__ void step(uint32_t cpu) {
        ++col;
        if (++k == cpu) k = 0, ++unit;
    }
};

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

/// End of a unit (or of the CTA's share of it): the KS slices of the row block are added in ks order through shared
/// memory (`red`: [r][ks - 1][lane][2G] floats), then slice 0 hands the sums over.
template <int G, int NTOK, int KS>
__device__ __forceinline__ void finish_block(float (&yacc)[G][2], uint32_t unit, uint32_t r, uint32_t ks, float* red, const SkTable& tb, uint32_t cta,
                                             float* part, uint32_t* counters, float* y, uint64_t y_stride, uint32_t rows,
                                             uint32_t lane, uint32_t row, const PeerPush& peer) {
    constexpr int R = kSkWarps / KS;
    if constexpr (KS > 1) {
        if (ks != 0) {
            float2* mine = reinterpret_cast<float2*>(red) + ((r * (KS - 1) + (ks - 1)) * 32 + lane) * G;
#pragma unroll
            for (int gi = 0; gi < G; ++gi) mine[gi] = make_float2(yacc[gi][0], yacc[gi][1]);
        }
        named_barrier(1 + r, KS * 32);
        if (ks == 0) {
            for (int k = 1; k < KS; ++k) {
                const float2* p = reinterpret_cast<const float2*>(red) + ((r * (KS - 1) + (k - 1)) * 32 + lane) * G;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) yacc[gi][0] += p[gi].x, yacc[gi][1] += p[gi].y;
            }
        }
        named_barrier(1 + r, KS * 32);  // the slices may overwrite `red` at their next block only after slice 0 has read it
    }
    if (ks == 0) sk_flush<G, NTOK, R>(yacc, unit, r, tb, cta, part, counters, y, y_stride, rows, lane, row, peer);
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;
}

// Shared-memory layout of both kernels: header (mma_common.cuh) | weight ring | slice sums (KS > 1) | zeros | x
template <class F, int NTOK, int NS, int KS>
struct SkLayout {
    static constexpr int G = (NTOK + 3) / 4;
    static constexpr uint32_t kSlot = 16 * F::kPitch, kRec = XRec<NTOK>::kBytes;
    static constexpr uint32_t kOffSlices = kOffRing + kSkWarps * NS * kSlot;
    static constexpr uint32_t kRedBytes = KS > 1 ? (kSkWarps / KS) * (KS - 1) * 32 * 2 * G * 4 : 0;
    static constexpr uint32_t kOffZero = (kOffSlices + kRedBytes + 127u) & ~127u;  // zeros read by single-row items
    static constexpr uint32_t kZeroBytes = NTOK == 1 ? F::kZeroBytes : 0;
    static constexpr uint32_t kOffData = kOffZero + kZeroBytes;
};

// ---- resident x -------------------------------------------------------------------------------------------------------------------
// NORM (single-row calls only): x is the raw row; the kernel normalises it by its rms and norm_w while converting it.
template <class F, int NTOK, int NS, int KS, bool PRE, bool NORM = false>
__global__ void __launch_bounds__(kSkWarps * 32, 1)
gemv_sk_resident_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ SkTable tb, const float* __restrict__ x, uint64_t x_stride,
                        float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t nb, float* __restrict__ partials,
                        uint32_t* __restrict__ counters, uint32_t* __restrict__ error_word, const uint8_t* __restrict__ xstage,
                        const __grid_constant__ PeerPush peer, const float* __restrict__ norm_w, float norm_eps) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    using L = SkLayout<F, NTOK, NS, KS>;
    constexpr int G = L::G, R = kSkWarps / KS;
    constexpr uint32_t kThreads = kSkWarps * 32, kWarps = kSkWarps, kSlot = L::kSlot, kRec = L::kRec, kOffData = L::kOffData;
    static_assert(kWarps <= kMaxWarps && NS <= 6, "shared-memory header layout");
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t r = warp % R, ks = warp / R;
    const uint32_t n_rb = (rows + 15u) / 16u, cpu = tb.cols_per_unit;
    const uint32_t cta = blockIdx.x;  // the grid has exactly tb.parts CTAs

    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlot;
    asm volatile("griddepcontrol.launch_dependents;");  // the next kernel in the stream may start filling its ring
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    ColumnWalk prod;
    prod.init(tb.start[cta], tb.start[cta + 1], cpu);
    uint32_t fill_slot = 0;
    auto refill = [&]() {  // the tile of the producer's column -> slot fill_slot (positions past the matrix have no tiles)
        if (prod.col >= prod.end) return;
        const uint32_t prb = prod.unit * R + r, psb = prod.k * KS + ks;
        if (prb < n_rb && psb < nb) {
            if (lane == 0) {
                mbar_expect_tx(bars + fill_slot * 8u, kSlot);
                tma_item_g2s<F>(ring + fill_slot * kSlot, &wmap, psb, prb * 16u, bars + fill_slot * 8u);
            }
            fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        }
        prod.step(cpu);
    };
#pragma unroll
    for (int it = 0; it < NS; ++it) refill();
    // The weights never depend on the kernel before this one, so the ring is filled first; only now wait for it.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const uint32_t xbar = smem_base + kOffXBar;
    bool lost = false;
    for (uint32_t i = tid; i < L::kZeroBytes / 4; i += kThreads) reinterpret_cast<uint32_t*>(smem + L::kOffZero)[i] = 0u;  // before the barriers below
    if constexpr (PRE) {
        if (tid == 0) {
            mbar_init(xbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            // the records of the super-blocks this CTA walks: all of them, or -- for a range shorter than a unit's columns --
            // the cyclic run that starts where the range starts, i.e. at most two contiguous pieces
            const uint32_t c_begin = tb.start[cta], c_count = tb.start[cta + 1] - c_begin;
            uint32_t lo[2] = {0u, 0u}, hi[2] = {nb, 0u}, at[2] = {0u, 0u};  // super-blocks [lo, hi) go to records at, at + 1, ...
            if (KS == 1 && c_count < cpu) {  // two-slice partitions give every CTA whole units
                const uint32_t first = (c_begin % cpu) * KS, last = first + c_count * KS, wrap = cpu * KS;
                lo[0] = min(first, nb), hi[0] = min(min(last, wrap), nb);
                lo[1] = 0u, hi[1] = last > wrap ? min(last - wrap, nb) : 0u, at[1] = wrap - first;
            }
            mbar_expect_tx(xbar, ((hi[0] - lo[0]) + (hi[1] - lo[1])) * kRec);
#pragma unroll
            for (int p = 0; p < 2; ++p)
                for (uint32_t off = 0; off < (hi[p] - lo[p]) * kRec; off += 32768u)  // records are multiples of 16 bytes
                    bulk_g2s(smem_base + kOffData + at[p] * kRec + off, xstage + lo[p] * kRec + off, min(32768u, (hi[p] - lo[p]) * kRec - off), xbar);
        }
        __syncthreads();
        if (!mbar_wait(xbar, 0)) {
            if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
            lost = true;
        }
    } else {
        // A CTA whose range is shorter than a unit's columns walks only those columns (super-blocks k * KS + ks for its
        // columns k, cyclically from where its range starts): it converts just that part of x.  Wider ranges take all of it.
        const uint32_t c_begin = tb.start[cta], c_count = tb.start[cta + 1] - c_begin;
        float inv = 1.0f;
        // fused input norm (single row): the row's rms first (one more block barrier); the conversion then multiplies every
        // element by it and by norm_w
        if constexpr (NORM) inv = block_inv_rms<kWarps>(x, nb * 256u, norm_eps, reinterpret_cast<float*>(smem + kOffRed), tid);
        // every warp converts whole super-blocks of x on its own (scale included): one pass, one barrier
        if (KS == 1 && c_count < cpu) {  // two-slice partitions give every CTA whole units
            for (uint32_t tk = 0; tk < NTOK; ++tk)
                stage_row_rec<NORM, true>(smem + kOffData, reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride),
                                          nb, NTOK, tk, warp, kWarps, lane, F::kXLaneBytes == 8, norm_w, inv, (c_begin % cpu) * KS, c_count * KS, cpu * KS);
        } else {
            for (uint32_t tk = 0; tk < NTOK; ++tk)
                stage_row_rec<NORM, false>(smem + kOffData, reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride),
                                           nb, NTOK, tk, warp, kWarps, lane, F::kXLaneBytes == 8, norm_w, inv);
        }
        __syncthreads();
    }

    // Under a partial conversion record j holds the super-block of the j-th column of this CTA's range, not super-block j.
    const uint32_t run_begin = tb.start[cta];
    const bool run_part = KS == 1 && tb.start[cta + 1] - run_begin < cpu;
    const XLane<G> xl = make_xlane<NTOK, F::kXLaneBytes>(g, t);
    // fragment row g of the MMA reads slot row F::slot_row(g) (a format may permute the rows of a tile against bank conflicts)
    const uint32_t row = F::slot_row(g);
    const uint8_t* slot0 = smem + kOffRing + warp * NS * kSlot + row * F::kPitch;
    float* red = reinterpret_cast<float*>(smem + L::kOffSlices);
    float yacc[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;

    uint32_t slot = 0, parity = 0;
    ColumnWalk cons;
    cons.init(tb.start[cta], tb.start[cta + 1], cpu);
    // A warp that lost a copy keeps walking (without computing): its siblings wait for it at the block barriers.
    while (cons.col < cons.end) {
        const uint32_t rb = cons.unit * R + r, sb = cons.k * KS + ks;
        if (rb < n_rb) {
            if (sb < nb && !lost) {
                if (!mbar_wait(bars + slot * 8u, parity)) {
                    if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                    lost = true;  // warp-uniform: every lane polled the same barrier
                } else {
                    F::template item<G, NTOK>(slot0 + slot * kSlot, t, smem + kOffData + (KS == 1 && run_part ? cons.col - run_begin : sb) * kRec, xl, smem + L::kOffZero, yacc, [&]() {
                        __syncwarp();
                        slot = slot + 1 == NS ? 0 : slot + 1;
                        parity ^= (slot == 0);
                        refill();
                    });
                }
            } else {
                refill();  // keeps the producer in step
            }
            if (cons.k + 1 == cpu || cons.col + 1 == cons.end)  // the row block, or this CTA's share of it, is done
                finish_block<G, NTOK, KS>(yacc, cons.unit, r, ks, red, tb, cta, partials, counters, y, y_stride, rows, lane, row, peer);
        } else {
            refill();
        }
        cons.step(cpu);
    }
    if (lost) linger_after_loss();
}

// ---- streamed x -------------------------------------------------------------------------------------------------------------------
// xs_cols: columns between two block barriers; the x ring holds 2 * xs_cols slots of KS records (one column of x).
template <class F, int NTOK, int NS, int KS>
__global__ void __launch_bounds__(kSkWarps * 32, 1)
gemv_sk_streamed_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ SkTable tb, float* __restrict__ y, uint64_t y_stride,
                        uint32_t rows, uint32_t nb, uint32_t xs_cols, float* __restrict__ partials, uint32_t* __restrict__ counters,
                        uint32_t* __restrict__ error_word, const uint8_t* __restrict__ xstage, const __grid_constant__ PeerPush peer) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    using L = SkLayout<F, NTOK, NS, KS>;
    constexpr int G = L::G, R = kSkWarps / KS;
    constexpr uint32_t kSlot = L::kSlot, kRec = L::kRec, kOffData = L::kOffData, kXSlot = KS * kRec;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t r = warp % R, ks = warp / R;
    const uint32_t n_rb = (rows + 15u) / 16u, cpu = tb.cols_per_unit;
    const uint32_t cta = blockIdx.x;
    const uint32_t col_lo = tb.start[cta], col_hi = tb.start[cta + 1];
    const uint32_t x_slots = 2u * xs_cols;

    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlot;
    asm volatile("griddepcontrol.launch_dependents;");
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        if (warp == 0)
            for (uint32_t s = 0; s < x_slots; ++s) mbar_init(smem_base + kOffXFull + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    ColumnWalk prod;
    prod.init(col_lo, col_hi, cpu);
    uint32_t fill_slot = 0;
    auto refill = [&]() {
        if (prod.col >= prod.end) return;
        const uint32_t prb = prod.unit * R + r, psb = prod.k * KS + ks;
        if (prb < n_rb && psb < nb) {
            if (lane == 0) {
                mbar_expect_tx(bars + fill_slot * 8u, kSlot);
                tma_item_g2s<F>(ring + fill_slot * kSlot, &wmap, psb, prb * 16u, bars + fill_slot * 8u);
            }
            fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        }
        prod.step(cpu);
    };
#pragma unroll
    for (int it = 0; it < NS; ++it) refill();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    for (uint32_t i = tid; i < L::kZeroBytes / 4; i += kSkWarps * 32) reinterpret_cast<uint32_t*>(smem + L::kOffZero)[i] = 0u;
    __syncthreads();  // barriers initialised, zeros in place
    // x ring: column c of this CTA (super-blocks k * KS .. k * KS + KS - 1 of x) goes to slot (c - col_lo) % x_slots
    auto fetch_x = [&](uint32_t c) {  // called by thread 0
        const uint32_t xs = (c - col_lo) % x_slots, sb0 = (c % cpu) * KS, bytes = min(static_cast<uint32_t>(KS), nb - sb0) * kRec;
        mbar_expect_tx(smem_base + kOffXFull + xs * 8u, bytes);
        bulk_g2s(smem_base + kOffData + xs * kXSlot, xstage + uint64_t{sb0} * kRec, bytes, smem_base + kOffXFull + xs * 8u);
    };
    if (tid == 0)
        for (uint32_t c = col_lo; c < col_lo + x_slots && c < col_hi; ++c) fetch_x(c);

    const XLane<G> xl = make_xlane<NTOK, F::kXLaneBytes>(g, t);
    // fragment row g of the MMA reads slot row F::slot_row(g) (a format may permute the rows of a tile against bank conflicts)
    const uint32_t row = F::slot_row(g);
    const uint8_t* slot0 = smem + kOffRing + warp * NS * kSlot + row * F::kPitch;
    float* red = reinterpret_cast<float*>(smem + L::kOffSlices);
    float yacc[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;

    uint32_t slot = 0, parity = 0;
    ColumnWalk cons;
    cons.init(col_lo, col_hi, cpu);
    bool lost = false;
    for (uint32_t c0 = col_lo; c0 < col_hi; c0 += xs_cols) {
        const uint32_t c1 = min(c0 + xs_cols, col_hi);
        for (uint32_t c = c0; c < c1; ++c) {
            const uint32_t rb = cons.unit * R + r, sb = cons.k * KS + ks;
            if (rb < n_rb) {
                if (sb < nb && !lost) {
                    const uint32_t n = c - col_lo, xs = n % x_slots;
                    if (!mbar_wait(smem_base + kOffXFull + xs * 8u, (n / x_slots) & 1u) || !mbar_wait(bars + slot * 8u, parity)) {
                        if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                        lost = true;
                    } else {
                        F::template item<G, NTOK>(slot0 + slot * kSlot, t, smem + kOffData + xs * kXSlot + ks * kRec, xl, smem + L::kOffZero, yacc, [&]() {
                            __syncwarp();
                            slot = slot + 1 == NS ? 0 : slot + 1;
                            parity ^= (slot == 0);
                            refill();
                        });
                    }
                } else {
                    refill();
                }
                if (cons.k + 1 == cpu || c + 1 == col_hi)
                    finish_block<G, NTOK, KS>(yacc, cons.unit, r, ks, red, tb, cta, partials, counters, y, y_stride, rows, lane, row, peer);
            } else {
                refill();
            }
            cons.step(cpu);
        }
        __syncthreads();  // every warp is done with the x records of this stretch: refill them two stretches ahead
        if (tid == 0)
            for (uint32_t c = c0 + x_slots; c < c1 + x_slots && c < col_hi; ++c) fetch_x(c);
    }
    if (lost) linger_after_loss();
}

}  // namespace sk
}  // namespace halo_cuda
