// The statically partitioned tensor-core skinny kernels for Q4_K: what gemv_mma_f16x2 runs under
// HALO_CUDA_GEMV_FLAG_NO_SCRATCH (no context scratch: each CTA owns 128 W rows and converts x itself), and the
// single-row specialist gemv_mma_m1.  Every other call of gemv_mma_f16x2 takes the balanced kernels of gemv_mma_sk.cuh.
//
// Why tensor cores for a matrix-vector product: at 0.5625 bytes per weight the B200 streams ~11.6 T weights/s from
// HBM while the CUDA cores issue ~36 T lane-instructions/s, so a kernel may spend about three instructions per
// weight in total.  Unpacking a nibble to fp32 and multiplying it costs more than that; handing the multiply-adds
// to mma.sync leaves the CUDA cores with nothing but the unpacking (about one instruction per weight).
//
// Arithmetic.  One warp owns 16 consecutive W rows (the A operand of m16n8k16, fp16 in, fp32 accumulate).
//   * A holds the INTEGER q * sc of each weight (4-bit quant times 6-bit sub-block scale, <= 945) encoded as an fp16
//     subnormal: the masked nibble pair is already the bit pattern of (q * 2^-24, q' * 2^-24), and one packed fp16
//     multiply by (sc, sc) keeps it exact.  No int-to-float conversion and no rounding happen on the weight side.
//   * B holds x.  Each token takes two of the eight columns: x * s rounded to fp16 (hi) and the fp16 remainder (lo),
//     where s is a power of two that puts the row's largest magnitude near 2^13; hi + lo carries ~22 bits of x.
//   * The min term dmin * sum_s m_s * (sum of x over sub-block s) runs through one extra MMA per super-block whose
//     A holds the 6-bit min codes and whose B holds the per-sub-block sums of x (again hi + lo).
//   * Per super-block the two fp32 accumulators are folded into the row sum with d and dmin in fp32.
// Every output column is an independent chain of MMAs over K in a fixed order, so a row's bits do not depend on how
// many rows share the call (include/halo/backend/backend.h:300-304).  The result differs from the CPU's in the last
// bits (different summation order, x carried as hi + lo): bounded, not bitwise.
//
// Data movement.  Weights go HBM -> shared memory by bulk asynchronous copies (cp.async.bulk, the 1-D TMA path): each
// warp keeps a ring of stages, one super-block (144 B) of its 16 rows per stage, filled several steps ahead and
// tracked by one mbarrier per stage.  x is converted once per CTA into shared memory in MMA-fragment order (chunked
// over K when n_vec * cols is large), so the inner loop reads its B fragments with one conflict-free 16-byte load
// per sub-block.  Every mbarrier wait is bounded: on expiry the warp raises the context's error word and leaves.
//
// Roofline: HBM.  Algorithmic bytes = rows * row_bytes + 4 * n_vec * cols + 4 * n_vec * rows.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {

namespace {

using namespace mma;


// NTOK: x rows of this launch (1..16), i.e. 2 * NTOK B columns in G = ceil(NTOK / 4) MMA column groups.
// KS: warps sharing one 16-row block; warp ks takes the super-blocks sb = ks (mod KS), a split that depends on
// nothing but KS, and the KS partial sums are added in ks order.  NS: ring stages per warp.
// The CTA converts its chunks of x itself: the kernel needs no scratch memory (the balanced kernels of gemv_mma_sk.cuh
// serve every call that may use context scratch).
template <int NTOK, int KS, int NS>
__global__ void __launch_bounds__(kRowBlocks * KS * 32, kRowBlocks >= 8 ? 1 : 2)
gemv_mma_q4k_kernel(const __grid_constant__ CUtensorMap wmap, const float* __restrict__ x, uint64_t x_stride,
                    float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t nb, uint32_t chunk_sb,
                    uint32_t* __restrict__ error_word) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    constexpr int G = (NTOK + 3) / 4;
    constexpr uint32_t kThreads = kRowBlocks * KS * 32;
    constexpr uint32_t kWarps = kRowBlocks * KS;
    static_assert(kWarps <= kMaxWarps && NS <= 6, "shared-memory header layout");
    constexpr uint32_t kOffData = kOffRing + kWarps * NS * kSlotBytes;
    constexpr uint32_t kCols = 2 * NTOK;             // B columns that carry a token
    constexpr uint32_t kSubStride = kCols * 64u;     // xs bytes per 32-element sub-block
    constexpr uint32_t kSbStride = kCols * 16u;      // sx bytes per super-block
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rbl = warp % kRowBlocks, ks = warp / kRowBlocks;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t cols = nb * 256u;

    // ---- this warp's rows; fill the ring before anything else so HBM is busy during the x prologue ------------------
    const uint32_t rb = blockIdx.x * kRowBlocks + rbl;
    const bool active = rb * 16u < rows;
    const uint32_t n_items = active && nb > ks ? (nb - ks + KS - 1) / KS : 0;  // super-blocks ks, ks+KS, ...
    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlotBytes;
    uint32_t next_x = ks * 144u;  // byte column of the next super-block to fetch
    asm volatile("griddepcontrol.launch_dependents;");  // the next kernel in the stream may start filling its ring
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t fill_slot = 0, issued = 0;
    auto refill = [&]() {  // next super-block of this warp -> slot fill_slot
        if (lane == 0) {
            mbar_expect_tx(bars + fill_slot * 8u, kStageTx);
            tma_tile_g2s(ring + fill_slot * kSlotBytes, &wmap, next_x, rb * 16u, bars + fill_slot * 8u);
        }
        next_x += KS * 144u;
        fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        ++issued;
    };
    for (uint32_t it = 0; it < NS && it < n_items; ++it) refill();
    // Programmatic dependent launch: the weights never depend on the kernel before this one, so the ring is filled
    // first; only now wait for that kernel's results (x may be one of them, and y may still be read by it).
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- per-token power-of-two scale from the row's largest magnitude ------------------------------------------------
    float* s_scale = reinterpret_cast<float*>(smem + kOffScale);
    float* s_inv = reinterpret_cast<float*>(smem + kOffInv);
    float* s_red = reinterpret_cast<float*>(smem + kOffRed);  // kWarps partial maxima
    for (uint32_t tk = 0; tk < NTOK; ++tk) {
        const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride);
        float m = 0.0f;
        for (uint32_t i = tid; i < cols / 4; i += kThreads) {
            const float4 v = xr[i];
            m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        if (lane == 0) s_red[warp] = m;
        __syncthreads();
        if (tid == 0) {
            float a = 0.0f;
            for (uint32_t i = 0; i < kWarps; ++i) a = fmaxf(a, s_red[i]);
            row_scale(a, s_scale[tk], s_inv[tk]);
        }
        __syncthreads();
    }

    // ---- B fragment pointers.  MMA columns are independent, so a lane whose column carries no token simply reads
    // the last real column: what it computes lands in accumulator columns that are never stored. ---------------------
    const uint8_t* xs_ptr[G];
    const uint8_t* sx_ptr[G];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t col = min(8u * gi + g, kCols - 1);
        xs_ptr[gi] = smem + kOffData + col * 64u + t * 16u;
        sx_ptr[gi] = smem + kOffData + chunk_sb * 8u * kSubStride + col * 16u + t * 4u;
    }

    // thread-constant selector for the pair of 6-bit min codes this thread feeds to the min-term MMA
    const uint32_t m_sel = (2 * t) | ((2 * t) << 4) | ((2 * t + 1) << 8) | ((2 * t + 1) << 12);
    // this thread's fragment base inside a ring slot: rows g (and g+8, 8 * kSlotRow further), 8 bytes per 32-byte group
    const uint8_t* frag = smem + kOffRing + warp * NS * kSlotBytes + g * kSlotRow + t * 8u;
    const uint8_t* hdr = smem + kOffRing + warp * NS * kSlotBytes + g * kSlotRow;

    float yacc[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;

    uint32_t slot = 0, parity = 0, done = 0;  // ring read position, and super-blocks consumed so far
    bool lost = false;
    for (uint32_t c0 = 0; c0 < nb; c0 += chunk_sb) {
        const uint32_t n_sb = min(chunk_sb, nb - c0);
        if (c0 != 0) __syncthreads();  // everyone is done reading the previous chunk
        // ---- x[:, chunk] as fp16 hi / lo in slot order, and the sub-block sums ------------------------------------------------
        for (uint32_t tk = 0; tk < NTOK; ++tk)
            stage_row(smem + kOffData, smem + kOffData + chunk_sb * 8u * kSubStride,
                      reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride), s_scale[tk], c0, n_sb,
                      kSubStride, kSbStride, 2 * tk * 64u, tid, kThreads);
        __syncthreads();
        if (!active || lost) continue;

        // this warp's super-blocks inside the chunk: sb = ks (mod KS), in increasing order
        for (uint32_t i = (ks + KS - c0 % KS) % KS; i < n_sb; i += KS) {
            if (!mbar_wait(bars + slot * 8u, parity)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;  // warp-uniform: every lane polled the same barrier
                break;
            }
            const uint8_t* fq = frag + slot * kSlotBytes;
            const uint8_t* fh = hdr + slot * kSlotBytes;

            // ---- 6-bit codes of both rows, four per word (SWAR form of src/tensor/quant.cpp:236-244) -------------------------
            uint32_t sc_lo[2], sc_hi[2], mpair[2];
            float dq[2], dmn[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint4 h = *reinterpret_cast<const uint4*>(fh + r * 8 * kSlotRow);
                sc_lo[r] = h.y & 0x3F3F3F3Fu;                                       // sc0..sc3
                sc_hi[r] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);        // sc4..sc7
                const uint32_t m_lo = h.z & 0x3F3F3F3Fu;                            // m0..m3
                const uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);  // m4..m7
                mpair[r] = prmt(m_lo, m_hi, m_sel) & 0x00FF00FFu;                   // (m_2t, m_2t+1) as fp16 subnormals
                const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
                dq[r] = __low2float(dd) * 16777216.0f;           // d * 2^24: undoes the subnormal encoding of A
                dmn[r] = __high2float(dd) * (16777216.0f * 32.0f);  // dmin * 2^24 * 32: and the /32 of the sums
            }

            // kChains independent accumulator chains per column group keep the tensor pipe from waiting on its own
            // result; MMA n of every 64-element group goes to chain n % kChains, and the chains are added in a fixed order.
            float cq[G][kChains][4], cm[G][4];
            const uint8_t* xb[G];
#pragma unroll
            for (int gi = 0; gi < G; ++gi) xb[gi] = xs_ptr[gi] + i * (8u * kSubStride);

#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // (sc, sc) for the low-nibble sub-block 2j and (sc/16, sc/16) for the high-nibble sub-block 2j+1, per row
                uint32_t sA[2], sB[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint32_t src = j < 2 ? sc_lo[r] : sc_hi[r];
                    const uint32_t ia = (j & 1) * 2, ib = ia + 1;
                    const uint32_t ba = prmt(src, 0x64646464u, ia | (4u << 4) | (ia << 8) | (4u << 12));  // 1024 + sc, twice
                    const uint32_t bb = prmt(src, 0x64646464u, ib | (4u << 4) | (ib << 8) | (4u << 12));
                    sA[r] = hsub2_bits(ba, 0x64006400u);                     // (sc, sc)
                    sB[r] = hfma2_bits(bb, 0x2C002C00u, 0xD400D400u);        // (1024 + sc) / 16 - 64 = sc / 16
                }
                uint32_t aLo[2][4], aHi[2][4];  // [row][lo02(qA), lo13(qA), lo02(qB), lo13(qB)] and the high-nibble twins
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const uint2 q = *reinterpret_cast<const uint2*>(fq + r * 8 * kSlotRow + 16 + j * 32);
                    const uint32_t qa = q.x, qb = q.y;
                    const uint32_t qa8 = qa >> 8, qb8 = qb >> 8;
                    aLo[r][0] = hmul2_bits(qa & 0x000F000Fu, sA[r]);
                    aLo[r][1] = hmul2_bits(qa8 & 0x000F000Fu, sA[r]);
                    aLo[r][2] = hmul2_bits(qb & 0x000F000Fu, sA[r]);
                    aLo[r][3] = hmul2_bits(qb8 & 0x000F000Fu, sA[r]);
                    aHi[r][0] = hmul2_bits(qa & 0x00F000F0u, sB[r]);
                    aHi[r][1] = hmul2_bits(qa8 & 0x00F000F0u, sB[r]);
                    aHi[r][2] = hmul2_bits(qb & 0x00F000F0u, sB[r]);
                    aHi[r][3] = hmul2_bits(qb8 & 0x00F000F0u, sB[r]);
                }
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const uint4 bl = *reinterpret_cast<const uint4*>(xb[gi] + (2 * j) * kSubStride);
                    const uint4 bh = *reinterpret_cast<const uint4*>(xb[gi] + (2 * j + 1) * kSubStride);
                    if (j == 0) mma16816_first(cq[gi][0], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    else mma16816(cq[gi][0], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    if (j == 0 && kChains > 1) mma16816_first(cq[gi][1 % kChains], aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                    else mma16816(cq[gi][1 % kChains], aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                    if (j == 0 && kChains > 2) mma16816_first(cq[gi][2 % kChains], aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                    else mma16816(cq[gi][2 % kChains], aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                    if (j == 0 && kChains > 3) mma16816_first(cq[gi][3 % kChains], aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
                    else mma16816(cq[gi][3 % kChains], aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
                }
            }
            // every byte of the slot has been consumed by the instructions above: hand it back to the copy engine
            __syncwarp();
            ++done;
            slot = slot + 1 == NS ? 0 : slot + 1;
            parity ^= (slot == 0);
            if (issued < n_items) refill();
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const uint32_t bs = *reinterpret_cast<const uint32_t*>(sx_ptr[gi] + i * kSbStride);
                mma16816_first(cm[gi], mpair[0], mpair[1], 0u, 0u, bs, 0u);
                float cs[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if constexpr (kChains == 1) cs[k] = cq[gi][0][k];
                    else if constexpr (kChains == 2) cs[k] = cq[gi][0][k] + cq[gi][1][k];
                    else cs[k] = (cq[gi][0][k] + cq[gi][1][k]) + (cq[gi][2][k] + cq[gi][3][k]);
                }
                yacc[gi][0] = fmaf(dq[0], cs[0] + cs[1], yacc[gi][0]);
                yacc[gi][0] = fmaf(-dmn[0], cm[gi][0] + cm[gi][1], yacc[gi][0]);
                yacc[gi][1] = fmaf(dq[1], cs[2] + cs[3], yacc[gi][1]);
                yacc[gi][1] = fmaf(-dmn[1], cm[gi][2] + cm[gi][3], yacc[gi][1]);
            }
        }
    }

    if constexpr (KS > 1) {
        // fold the KS partial sums of each row block in ks order (the x staging area is free by now)
        __syncthreads();
        float* red = reinterpret_cast<float*>(smem + kOffData);
        if (active && ks != 0) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                red[(((ks - 1) * kRowBlocks + rbl) * 32 + lane) * (2 * G) + 2 * gi + 0] = yacc[gi][0];
                red[(((ks - 1) * kRowBlocks + rbl) * 32 + lane) * (2 * G) + 2 * gi + 1] = yacc[gi][1];
            }
        }
        __syncthreads();
        if (ks != 0) return;
        if (active) {
            for (int k = 1; k < KS; ++k) {
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    yacc[gi][0] += red[(((k - 1) * kRowBlocks + rbl) * 32 + lane) * (2 * G) + 2 * gi + 0];
                    yacc[gi][1] += red[(((k - 1) * kRowBlocks + rbl) * 32 + lane) * (2 * G) + 2 * gi + 1];
                }
            }
        }
    }
    if (lost) {
        // copies may still be in flight towards this CTA's shared memory: give them a bounded time to land
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
        return;
    }
    if (!active) return;
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t tk = 4u * gi + t;
        if (tk < NTOK) {
            const float inv = s_inv[tk];
            float* yr = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{tk} * y_stride);
            const uint32_t n0 = rb * 16u + g, n1 = n0 + 8u;
            if (n0 < rows) yr[n0] = yacc[gi][0] * inv;
            if (n1 < rows) yr[n1] = yacc[gi][1] * inv;
        }
    }
}

// ---- the single-row specialist (variant gemv_mma_m1) -----------------------------------------------------------------
// With one x row the eight MMA columns are free, and they are spent on the eight sub-blocks of a super-block: for
// the MMAs of sub-block s only column s of B carries x (every other column reads zeros), so accumulator column s
// ends up holding sum_{k in s} q_k x_k.  The weight side then needs NO multiply at all -- the masked nibble pair goes
// straight into the A fragment -- and the 6-bit scales are applied to 2 accumulator columns per thread in fp32
// (thread t of a quad owns sub-blocks 2t and 2t+1).  High-nibble sub-blocks carry 16 q, so their x is staged
// pre-divided by 16 (exact).  x is again fp16 hi + lo (two MMAs per k-step).  The min term uses the exact fp32
// sub-block sums of x.  A row's arithmetic differs from gemv_mma_f16x2, so the two are different numerics families.
template <int KS, int NS>
__global__ void __launch_bounds__(kRowBlocks * KS * 32, kRowBlocks >= 8 ? 1 : 2)
gemv_mma_q4k_m1_kernel(const __grid_constant__ CUtensorMap wmap, const float* __restrict__ x, float* __restrict__ y, uint32_t rows,
                       uint32_t nb, uint32_t chunk_sb, uint32_t* __restrict__ error_word) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    constexpr uint32_t kThreads = kRowBlocks * KS * 32;
    constexpr uint32_t kWarps = kRowBlocks * KS;
    static_assert(kWarps <= kMaxWarps && NS <= 6, "shared-memory header layout");
    constexpr uint32_t kOffData = kOffRing + kWarps * NS * kSlotBytes;  // its first 128 bytes stay zero
    constexpr uint32_t kOffXs = kOffData + 128;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rbl = warp % kRowBlocks, ks = warp / kRowBlocks;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t cols = nb * 256u;

    const uint32_t rb = blockIdx.x * kRowBlocks + rbl;
    const bool active = rb * 16u < rows;
    const uint32_t n_items = active && nb > ks ? (nb - ks + KS - 1) / KS : 0;
    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlotBytes;
    uint32_t next_x = ks * 144u;
    asm volatile("griddepcontrol.launch_dependents;");  // the next kernel in the stream may start filling its ring
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t fill_slot = 0, issued = 0;
    auto refill = [&]() {
        if (lane == 0) {
            mbar_expect_tx(bars + fill_slot * 8u, kStageTx);
            tma_tile_g2s(ring + fill_slot * kSlotBytes, &wmap, next_x, rb * 16u, bars + fill_slot * 8u);
        }
        next_x += KS * 144u;
        fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        ++issued;
    };
    for (uint32_t it = 0; it < NS && it < n_items; ++it) refill();
    // Programmatic dependent launch: the weights never depend on the kernel before this one, so the ring is filled
    // first; only now wait for that kernel's results (x may be one of them, and y may still be read by it).
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- power-of-two scale from the largest magnitude of x -------------------------------------------------------------
    float* s_scale = reinterpret_cast<float*>(smem + kOffScale);
    float* s_inv = reinterpret_cast<float*>(smem + kOffInv);
    float* s_red = reinterpret_cast<float*>(smem + kOffRed);
    if (tid < 32) reinterpret_cast<uint32_t*>(smem + kOffData)[tid] = 0u;
    {
        const float4* xr = reinterpret_cast<const float4*>(x);
        float m = 0.0f;
        for (uint32_t i = tid; i < cols / 4; i += kThreads) {
            const float4 v = xr[i];
            m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        if (lane == 0) s_red[warp] = m;
        __syncthreads();
        if (tid == 0) {
            float a = 0.0f;
            for (uint32_t i = 0; i < kWarps; ++i) a = fmaxf(a, s_red[i]);
            row_scale(a, s_scale[0], s_inv[0]);
        }
        __syncthreads();
    }

    // ---- per-lane B addressing: this lane feeds column g, which is live only for sub-block g of each super-block; for
    // the other seven sub-blocks it reads the 16 zero bytes (step 0) ---------------------------------------------------
    uint32_t b_base[8], b_step[8];
#pragma unroll
    for (int sblk = 0; sblk < 8; ++sblk) {
        const bool mine = g == static_cast<uint32_t>(sblk);
        b_base[sblk] = mine ? smem_base + kOffXs + sblk * 128u + t * 16u : smem_base + kOffData;
        b_step[sblk] = mine ? 8u * 128u : 0u;
    }
    const uint32_t sx_base = smem_base + kOffXs + chunk_sb * 8u * 128u + t * 8u;  // fp32 sums of sub-blocks 2t, 2t+1

    const uint32_t code_sel = (2 * t) | ((2 * t) << 4) | ((2 * t + 1) << 8) | ((2 * t + 1) << 12);
    const uint8_t* frag = smem + kOffRing + warp * NS * kSlotBytes + g * kSlotRow + t * 8u;
    const uint8_t* hdr = smem + kOffRing + warp * NS * kSlotBytes + g * kSlotRow;

    float yacc0 = 0.0f, yacc1 = 0.0f;
    uint32_t slot = 0, parity = 0;
    bool lost = false;
    for (uint32_t c0 = 0; c0 < nb; c0 += chunk_sb) {
        const uint32_t n_sb = min(chunk_sb, nb - c0);
        if (c0 != 0) __syncthreads();
        {
            const float4* xr = reinterpret_cast<const float4*>(x) + c0 * 64u;
            const float s = s_scale[0];
            for (uint32_t qd = tid; qd < n_sb * 64u; qd += kThreads) {
                float4 v = xr[qd];
                v.x *= s; v.y *= s; v.z *= s; v.w *= s;
                const uint32_t sub = qd >> 3, in = qd & 7u;
                float sum = (v.x + v.y) + (v.z + v.w);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
                if (in == 0) *reinterpret_cast<float*>(smem + kOffXs + chunk_sb * 8u * 128u + sub * 4u) = sum;
                if (sub & 1u) {  // a high-nibble sub-block: its A entries are 16 q
                    v.x *= 0.0625f; v.y *= 0.0625f; v.z *= 0.0625f; v.w *= 0.0625f;
                }
                uint2 hi, lo;
                split4(v, hi, lo);
                uint8_t* dst = smem + kOffXs + sub * 128u + in * 8u;
                *reinterpret_cast<uint2*>(dst) = hi;
                *reinterpret_cast<uint2*>(dst + 64) = lo;
            }
        }
        __syncthreads();
        if (!active || lost) continue;

        for (uint32_t i = (ks + KS - c0 % KS) % KS; i < n_sb; i += KS) {
            if (!mbar_wait(bars + slot * 8u, parity)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;
                break;
            }
            const uint8_t* fq = frag + slot * kSlotBytes;
            const uint8_t* fh = hdr + slot * kSlotBytes;
            float c[4];
#pragma unroll
            for (int sblk = 0; sblk < 8; ++sblk) {
                const int j = sblk >> 1;
                const uint32_t ba = b_base[sblk] + i * b_step[sblk];
                uint4 bh, bl;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(bh.x), "=r"(bh.y), "=r"(bh.z), "=r"(bh.w) : "r"(ba));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+64];" : "=r"(bl.x), "=r"(bl.y), "=r"(bl.z), "=r"(bl.w) : "r"(ba));
                const uint2 q0 = *reinterpret_cast<const uint2*>(fq + 16 + j * 32);
                const uint2 q1 = *reinterpret_cast<const uint2*>(fq + 8 * kSlotRow + 16 + j * 32);
                const uint32_t mask = (sblk & 1) ? 0x00F000F0u : 0x000F000Fu;
                const uint32_t a0 = q0.x & mask, a1 = q1.x & mask, a2 = (q0.x >> 8) & mask, a3 = (q1.x >> 8) & mask;
                const uint32_t e0 = q0.y & mask, e1 = q1.y & mask, e2 = (q0.y >> 8) & mask, e3 = (q1.y >> 8) & mask;
                if (sblk == 0) mma16816_first(c, a0, a1, a2, a3, bh.x, bh.y);
                else mma16816(c, a0, a1, a2, a3, bh.x, bh.y);
                mma16816(c, e0, e1, e2, e3, bh.z, bh.w);
                mma16816(c, a0, a1, a2, a3, bl.x, bl.y);
                mma16816(c, e0, e1, e2, e3, bl.z, bl.w);
            }
            // ---- scales of this thread's two sub-blocks (2t, 2t+1), both rows, as fp32 --------------------------------------
            const float2 sx = *reinterpret_cast<const float2*>(smem + (sx_base - smem_base) + i * 32u);
            float part[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint4 h = *reinterpret_cast<const uint4*>(fh + r * 8 * kSlotRow);
                const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                const uint32_t m_lo = h.z & 0x3F3F3F3Fu, m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
                const uint32_t scp = prmt(sc_lo, sc_hi, code_sel), mp = prmt(m_lo, m_hi, code_sel);  // bytes 0 and 2 = codes 2t, 2t+1
                // 0x4B000000 | code is the float 2^23 + code
                const float sc0 = __uint_as_float(prmt(scp, 0x4B000000u, 0x7650u)) - 8388608.0f;
                const float sc1 = __uint_as_float(prmt(scp, 0x4B000000u, 0x7652u)) - 8388608.0f;
                const float m0 = __uint_as_float(prmt(mp, 0x4B000000u, 0x7650u)) - 8388608.0f;
                const float m1 = __uint_as_float(prmt(mp, 0x4B000000u, 0x7652u)) - 8388608.0f;
                const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
                const float dq = __low2float(dd) * 16777216.0f;  // undoes the 2^-24 of the subnormal encoding
                const float dmn = __high2float(dd);
                const float tq = fmaf(sc1, c[2 * r + 1], sc0 * c[2 * r]);
                const float tm = fmaf(m1, sx.y, m0 * sx.x);
                part[r] = fmaf(-dmn, tm, dq * tq);
            }
            yacc0 += part[0];
            yacc1 += part[1];
            __syncwarp();
            slot = slot + 1 == NS ? 0 : slot + 1;
            parity ^= (slot == 0);
            if (issued < n_items) refill();
        }
    }
    // the four threads of a quad hold the partial sums of different sub-block pairs: add them in a fixed order
    yacc0 += __shfl_xor_sync(0xFFFFFFFFu, yacc0, 1);
    yacc0 += __shfl_xor_sync(0xFFFFFFFFu, yacc0, 2);
    yacc1 += __shfl_xor_sync(0xFFFFFFFFu, yacc1, 1);
    yacc1 += __shfl_xor_sync(0xFFFFFFFFu, yacc1, 2);
    if constexpr (KS > 1) {
        __syncthreads();
        float* red = reinterpret_cast<float*>(smem + kOffXs);
        if (active && ks != 0) {
            red[(((ks - 1) * kRowBlocks + rbl) * 32 + lane) * 2 + 0] = yacc0;
            red[(((ks - 1) * kRowBlocks + rbl) * 32 + lane) * 2 + 1] = yacc1;
        }
        __syncthreads();
        if (ks != 0) return;
        if (active) {
            for (int k = 1; k < KS; ++k) {
                yacc0 += red[(((k - 1) * kRowBlocks + rbl) * 32 + lane) * 2 + 0];
                yacc1 += red[(((k - 1) * kRowBlocks + rbl) * 32 + lane) * 2 + 1];
            }
        }
    }
    if (lost) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {
        }
        return;
    }
    if (!active || t != 0) return;
    const float inv = s_inv[0];
    const uint32_t n0 = rb * 16u + g, n1 = n0 + 8u;
    if (n0 < rows) y[n0] = yacc0 * inv;
    if (n1 < rows) y[n1] = yacc1 * inv;
}

struct Plan {
    uint32_t chunk_sb;
    uint32_t smem_bytes;
};

Plan plan_for(uint32_t nb, uint32_t n_tok, uint32_t off_data, uint32_t reduce_bytes) {
    const uint32_t ncols = 2 * n_tok;
    const uint32_t per_sb = 8u * ncols * 64u + ncols * 16u;
    uint32_t chunk = (kSmemBudget - off_data) / per_sb;
    if (chunk > nb) chunk = nb;
    if (chunk == 0) chunk = 1;
    const uint32_t data = chunk * per_sb;  // the K-split reduction reuses this area
    return {chunk, off_data + (data > reduce_bytes ? data : reduce_bytes)};
}

/// Launch configuration with programmatic stream serialization: the kernel may begin (and prefetch weights) while the
/// kernel before it in the stream drains; it orders itself with griddepcontrol.wait before touching x or y.
cudaLaunchConfig_t pdl_config(uint32_t grid, uint32_t block, uint32_t smem, cudaStream_t s, cudaLaunchAttribute* attr) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cfg;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/// The weight matrix as a 2-D byte tensor {row_bytes, rows} with row pitch w_stride, tiled 160 x 16.
int weight_map(const GemvCall& c, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        HC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail(HALO_CUDA_E_BACKEND, "cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {c.row_bytes, c.rows};
    const cuuint64_t strides[1] = {c.w_stride};
    const cuuint32_t box[2] = {kSlotRow, 16};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(c.w), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HALO_CUDA_E_KERNEL, "MATMUL: cannot describe the weight matrix to the copy engine (CUresult %d)", (int)r);
    return 0;
}

template <int NTOK, int KS, int NS>
int launch_n(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, cudaStream_t s) {
    constexpr int G = (NTOK + 3) / 4;
    const uint32_t nb = c.cols / 256u;
    const Plan p = plan_for(nb, NTOK, kOffRing + kRowBlocks * KS * NS * kSlotBytes, (KS - 1) * kRowBlocks * 32 * 2 * G * 4);
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(gemv_mma_q4k_kernel<NTOK, KS, NS>), kSmemBudget)) return rc;
    const uint32_t grid = (c.rows + 16u * kRowBlocks - 1) / (16u * kRowBlocks);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    CUtensorMap wmap;
    if (int rc = weight_map(c, &wmap)) return rc;
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = pdl_config(grid, kRowBlocks * KS * 32, p.smem_bytes, s, attr);
    HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_mma_q4k_kernel<NTOK, KS, NS>, wmap, x, c.x_stride, y, c.y_stride, c.rows, nb, p.chunk_sb,
                               ctx->error_word_dev));
    return 0;
}

// The K split (2 warps per row block) and the ring depth are the same for every token count: the split is part
// of a row's arithmetic, and must not move with the batch size.
template <int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > 16) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
#ifndef HALO_MMA_KS
#define HALO_MMA_KS 2
#define HALO_MMA_NS 3
#endif
        if (n == NTOK) {
            return launch_n<NTOK, HALO_MMA_KS, HALO_MMA_NS>(ctx, c, tok0, s);
        }
        return launch_tokens<NTOK + 1>(ctx, c, tok0, n, s);
    }
}

template <int KS, int NS>
int launch_m1(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok, cudaStream_t s) {
    const uint32_t nb = c.cols / 256u;
    constexpr uint32_t off_xs = kOffRing + kRowBlocks * KS * NS * kSlotBytes + 128;
    const uint32_t per_sb = 8u * 128u + 32u;
    uint32_t chunk = (kSmemBudget - off_xs) / per_sb;
    if (chunk > nb) chunk = nb;
    const uint32_t data = chunk * per_sb, red = (KS - 1) * kRowBlocks * 32 * 2 * 4;
    const uint32_t smem_bytes = off_xs + (data > red ? data : red);
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(gemv_mma_q4k_m1_kernel<KS, NS>), kSmemBudget)) return rc;
    CUtensorMap wmap;
    if (int rc = weight_map(c, &wmap)) return rc;
    const uint32_t grid = (c.rows + 16u * kRowBlocks - 1) / (16u * kRowBlocks);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok} * c.y_stride);
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = pdl_config(grid, kRowBlocks * KS * 32, smem_bytes, s, attr);
    HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_mma_q4k_m1_kernel<KS, NS>, wmap, x, y, c.rows, nb, chunk, ctx->error_word_dev));
    return 0;
}

}  // namespace

int launch_gemv_mma_m1(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    // One launch per x row: the single-row kernel re-reads the weights for every row, which keeps each row bitwise
    // its own n_vec == 1 result; batches belong to gemv_mma_f16x2.
#ifndef HALO_M1_KS
#define HALO_M1_KS 2
#define HALO_M1_NS 3
#endif
    for (uint32_t t = 0; t < c.n_vec; ++t) {
        if (int rc = launch_m1<HALO_M1_KS, HALO_M1_NS>(ctx, c, t, s)) return rc;
    }
    return 0;
}

bool gemv_mma_supports(const GemvCall& c) {
    if (c.wtype != HALO_CUDA_T_Q4_K || c.cols == 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // tensor-map base and pitch
    if (c.w_stride >= (uint64_t{1} << 40) || c.row_bytes >= (uint64_t{1} << 32)) return false;
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return true;
}

int launch_gemv_mma(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    // Token tiles of 16 (four MMA column groups); the remainder takes the smallest instantiation that holds it.
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += 16) {
        const uint32_t n = c.n_vec - t0 < 16 ? c.n_vec - t0 : 16;
        const int rc = launch_tokens<1>(ctx, c, t0, n, s);
        if (rc != 0) return rc;
    }
    return 0;
}

}  // namespace halo_cuda
