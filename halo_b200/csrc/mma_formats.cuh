// Weight formats of the balanced tensor-core skinny kernels: for each, how one 16-row x 256-column tile ("item") sits
// in a ring slot and the arithmetic that folds it into the row sums.  The kernels around these (gemv_mma_sk.cu) only
// move data and walk the partition.
//
// Shared arithmetic: A holds unsigned quant codes as fp16 subnormals (code * 2^-24, exact), B holds x as fp16 hi + lo
// columns, fp32 accumulation in mma.sync m16n8k16; a lane (g = lane / 4, t = lane % 4) owns rows g and g + 8 of the
// tile and the B columns 2t, 2t + 1 of every 8-column group.
//
// x is scaled per super-block (256 elements, what one warp converts at a time): s = the power of two that puts the
// super-block's largest magnitude near 2^13, so the conversion needs no pass over the whole row and no block-wide
// reduction, and an item folds 1 / s into its final multiply.
// x record of one super-block for NTOK rows (what stage_superblock writes and an item reads):
//   [sub-block 0..7][column 0..2*NTOK-1][64 B]   fp16 hi (even column) / lo (odd column) of x * s, in quads of 8 bytes; for
//                                                the formats that read 8 bytes per lane and k-step the two 16-element halves
//                                                of a sub-block are kept apart instead: [half][column][32 B], so that the
//                                                four columns a half warp reads together fall on different banks
//   [column][16 B]                               sum of each 32-element sub-block / 32 as fp16 hi / lo (Q4_K min term)
//   [16-element group 0..15][row] fp32           sums of x * s over 16 elements (zero points of the other formats)
//   [row] fp32                                   1 / s (padded to 16 bytes)
#pragma once
#include "halo_cuda.h"
#include "mma_common.cuh"

namespace halo_cuda {
namespace mma {

template <int NTOK>
struct XRec {
    static constexpr uint32_t kCols = 2 * NTOK, kSubStride = kCols * 64u, kSbStride = kCols * 16u, kSx16Bytes = 64u * NTOK;
    static constexpr uint32_t kOffSums = 8u * kSubStride, kOffSx16 = kOffSums + kSbStride, kOffInv = kOffSx16 + kSx16Bytes;
    static constexpr uint32_t kBytes = kOffInv + ((4u * NTOK + 15u) & ~15u);
};
inline constexpr uint32_t xrec_bytes(uint32_t n_tok) { return 1120u * n_tok + ((4u * n_tok + 15u) & ~15u); }

/// Lane-constant byte offsets into an x record: B fragments and sums of this lane's column in each column group.
/// A lane whose column carries no row reads the last real column; what it computes is never stored.
template <int G>
struct XLane {
    uint32_t xs[G], sums[G], tok[G], g, t;
};
template <int NTOK, uint32_t LaneBytes>
__device__ __forceinline__ XLane<(NTOK + 3) / 4> make_xlane(uint32_t g, uint32_t t) {
    XLane<(NTOK + 3) / 4> xl;
    xl.g = g, xl.t = t;
#pragma unroll
    for (int gi = 0; gi < (NTOK + 3) / 4; ++gi) {
        const uint32_t col = min(8u * gi + g, XRec<NTOK>::kCols - 1);
        xl.xs[gi] = LaneBytes == 8 ? col * 32u + t * 8u : col * 64u + t * 16u;
        xl.sums[gi] = XRec<NTOK>::kOffSums + col * 16u + t * 4u;
        xl.tok[gi] = min(4u * gi + t, static_cast<uint32_t>(NTOK - 1));
    }
    return xl;
}

/// One super-block (index sb) of an x row into its record at `area`, by one warp: lane l holds quads l and l + 32
/// (elements 4l .. 4l + 3 and 128 + 4l .. ) in v; the scale comes from the largest magnitude among the 64 quads.
__device__ __forceinline__ void stage_superblock(uint8_t* area, const float4 (&v)[2], uint32_t sb, uint32_t n_tok, uint32_t tok, uint32_t lane,
                                                 bool split_halves) {
    const uint32_t rec = xrec_bytes(n_tok), sub_stride = 128u * n_tok;
    float m = 0.0f;
#pragma unroll
    for (int h = 0; h < 2; ++h) m = fmaxf(fmaxf(m, fmaxf(fabsf(v[h].x), fabsf(v[h].y))), fmaxf(fabsf(v[h].z), fabsf(v[h].w)));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    float s, inv;
    row_scale(m, s, inv);
    uint8_t* base = area + sb * rec;
    uint8_t* sums = base + 8u * sub_stride;
    float* sx16 = reinterpret_cast<float*>(sums + 32u * n_tok);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float4 u = v[h];
        u.x *= s; u.y *= s; u.z *= s; u.w *= s;
        uint2 hi, lo;
        split4(u, hi, lo);
        const uint32_t qd = 32u * h + lane, sub = qd >> 3, in = qd & 7u;  // 8 quads per 32-element sub-block
        if (split_halves) {
            uint8_t* dst = base + sub * sub_stride + (in >> 2) * (64u * n_tok) + tok * 64u + (in & 3u) * 8u;
            *reinterpret_cast<uint2*>(dst) = hi;
            *reinterpret_cast<uint2*>(dst + 32) = lo;
        } else {
            uint8_t* dst = base + sub * sub_stride + tok * 128u + in * 8u;
            *reinterpret_cast<uint2*>(dst) = hi;
            *reinterpret_cast<uint2*>(dst + 64) = lo;
        }
        float sum = (u.x + u.y) + (u.z + u.w);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if ((in & 3u) == 0) sx16[(sub * 2u + (in >> 2)) * n_tok + tok] = sum;
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        if (in == 0) {
            sum *= 0.03125f;  // keeps the fp16 copy in range: |sum| <= 32 * 2^14
            const __half hh = __float2half_rn(sum);
            const __half ll = __float2half_rn(sum - __half2float(hh));
            uint8_t* sd = sums + tok * 32u + sub * 2u;
            *reinterpret_cast<__half*>(sd) = hh;
            *reinterpret_cast<__half*>(sd + 16) = ll;
        }
    }
    if (lane == 0) (sx16 + 16u * n_tok)[tok] = inv;
}

/// Converts super-blocks [0, n_sb) of one x row into records starting at `area`: warp w of `n_warps` takes super-blocks
/// w, w + n_warps, ..., four at a time so that their loads overlap.  The arithmetic does not depend on who calls it.
/// NORM: the row is normalised on the way, element i becomes (x[i] * inv) * norm_w[i] -- the arithmetic of the CPU backend's
/// rms_norm (backends/cpu/ops_basic.cpp:28-30) with `inv` = 1 / sqrt(mean of squares + eps) supplied by the caller.
/// PART: only the super-blocks (first + j) mod wrap for j < count are converted (a CTA that walks a few columns of K needs
/// no more) and record j of the area belongs to the j-th of them; otherwise all are converted, record sb to super-block sb.
template <bool NORM = false, bool PART = false>
__device__ __forceinline__ void stage_row_rec(uint8_t* area, const float* xrow, uint32_t n_sb, uint32_t n_tok, uint32_t tok, uint32_t warp,
                                              uint32_t n_warps, uint32_t lane, bool split_halves, const float* norm_w = nullptr, float inv = 1.0f,
                                              uint32_t first = 0, uint32_t count = 0, uint32_t wrap = 0) {
    constexpr uint32_t kAhead = 4;
    const float4* xr = reinterpret_cast<const float4*>(xrow);
    const float4* wr = reinterpret_cast<const float4*>(norm_w);
    if constexpr (!PART) count = n_sb;
    auto sb_of = [&](uint32_t j) {  // the j-th super-block to convert; n_sb (= none) past the end or past the row
        if constexpr (!PART) {
            return j;
        } else {
            if (j >= count) return n_sb;
            uint32_t sb = first + j;
            if (sb >= wrap) sb -= wrap;
            return sb;
        }
    };
    for (uint32_t j0 = warp; j0 < count; j0 += kAhead * n_warps) {
        float4 v[kAhead][2];
#pragma unroll
        for (uint32_t j = 0; j < kAhead; ++j) {
            const uint32_t sb = sb_of(j0 + j * n_warps);
            if (sb < n_sb) v[j][0] = xr[sb * 64u + lane], v[j][1] = xr[sb * 64u + 32u + lane];
        }
        if constexpr (NORM) {
#pragma unroll
            for (uint32_t j = 0; j < kAhead; ++j) {
                const uint32_t sb = sb_of(j0 + j * n_warps);
                if (sb < n_sb) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float4 w = wr[sb * 64u + h * 32u + lane];
                        v[j][h].x = __fmul_rn(__fmul_rn(v[j][h].x, inv), w.x);
                        v[j][h].y = __fmul_rn(__fmul_rn(v[j][h].y, inv), w.y);
                        v[j][h].z = __fmul_rn(__fmul_rn(v[j][h].z, inv), w.z);
                        v[j][h].w = __fmul_rn(__fmul_rn(v[j][h].w, inv), w.w);
                    }
                }
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < kAhead; ++j) {
            const uint32_t sb = sb_of(j0 + j * n_warps);
            // a partial conversion stores its records compactly, in the order of the run
            if (sb < n_sb) stage_superblock(area, v[j], PART ? j0 + j * n_warps : sb, n_tok, tok, lane, split_halves);
        }
    }
}

/// 1 / sqrt(mean of squares + eps) of a row of n floats (n a multiple of 4, 16-byte aligned), computed by the whole block
/// in a fixed order: thread-strided partial sums, a shuffle tree per warp, the warps' sums added in warp order by every
/// thread.  `red` is shared memory for one float per warp.  Contains one block barrier.
template <uint32_t kWarps>
__device__ __forceinline__ float block_inv_rms(const float* xrow, uint32_t n, float eps, float* red, uint32_t tid) {
    const float4* xr = reinterpret_cast<const float4*>(xrow);
    float s = 0.0f;
    constexpr uint32_t kAhead = 4, kStride = kWarps * 32u;  // four loads in flight per thread; the additions stay in index order
    for (uint32_t i0 = tid; i0 < n / 4u; i0 += kAhead * kStride) {
        float4 v[kAhead];
#pragma unroll
        for (uint32_t j = 0; j < kAhead; ++j)
            if (i0 + j * kStride < n / 4u) v[j] = xr[i0 + j * kStride];
#pragma unroll
        for (uint32_t j = 0; j < kAhead; ++j) {
            if (i0 + j * kStride < n / 4u) {
                s = fmaf(v[j].x, v[j].x, s);
                s = fmaf(v[j].y, v[j].y, s);
                s = fmaf(v[j].z, v[j].z, s);
                s = fmaf(v[j].w, v[j].w, s);
            }
        }
    }
#pragma unroll
    for (uint32_t d = 16; d != 0; d >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, d);
    if ((tid & 31u) == 0) red[tid >> 5] = s;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (uint32_t w = 0; w < kWarps; ++w) total += red[w];
    return 1.0f / sqrtf(total / static_cast<float>(n) + eps);
}

/// Bytes of global scratch stage_x_rec_kernel fills: the records of all super-blocks.
inline uint64_t stage_rec_scratch_bytes(uint32_t nb, uint32_t n_tok) { return uint64_t{nb} * xrec_bytes(n_tok); }

/// grid (x rows, blocks of 16 super-blocks): every warp converts one super-block; nothing is shared between warps.
static __global__ void __launch_bounds__(512) stage_x_rec_kernel(const float* __restrict__ x, uint64_t x_stride, uint8_t* __restrict__ scratch,
                                                                 uint32_t nb, uint32_t n_tok, uint32_t split_halves) {
    // Programmatic dependent launch on both sides: the matmul behind this kernel may start filling its weight ring
    // now; x and the scratch records belong to the kernels before this one until they have completed.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t tk = blockIdx.x, sb = blockIdx.y * 16u + (threadIdx.x >> 5);
    if (sb >= nb) return;
    const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride);
    const uint32_t lane = threadIdx.x & 31u;
    const float4 v[2] = {xr[sb * 64u + lane], xr[sb * 64u + 32u + lane]};
    stage_superblock(scratch, v, sb, n_tok, tk, lane, split_halves != 0);
}

// ---- Q4_K: raw GGUF super-blocks (144 B), fetched as 160-byte slot rows ----------------------------------------------------
// A holds the bare 4-bit codes (low nibbles as q * 2^-24, high nibbles in place as 16 q * 2^-24).  Every 32-element
// sub-block s gets a fresh fp32 accumulator S_s (two MMAs), and the 6-bit scales enter in fp32:
//     a_p = fma(w_{4+p}, S_{4+p}, w_p * S_p)   p = 0..3      (w_s = sc_s, or sc_s / 16 for the high-nibble sub-blocks)
//     T   = (a_0 + a_1) + (a_2 + a_3)
//     y  += (d * 2^24 / s) * T  -  (dmin * 2^24 * 32 / s) * M      s = the scale of this super-block of x
// where M, the min term sum_s m_s * (sum of x over sub-block s) / 32, comes from one extra MMA whose A holds the 6-bit min
// codes and whose B holds the sub-block sums of x.  That operation order is the same for every batch size; a call
// with ONE x row gets it with a quarter of the scale work by placing x in the column pair (2p, 2p + 1) of B for the
// sub-blocks s = p (mod 4) (the other columns read zeros), so that one accumulator tile carries four sub-blocks and
// lane t of a row finishes sub-blocks t and 4 + t; two shuffles build T.  Adding exact zeros leaves S_s bit-identical.
struct Q4Kf {
    static constexpr uint32_t kType = HALO_CUDA_T_Q4_K, kPitch = 160, kItemCoord = 144, kBoxInner = 160, kMapElemBytes = 1, kXLaneBytes = 16;
    static constexpr bool kAllowSlices = format_allows_slices(kType);
    static constexpr uint32_t kZeroBytes = 1024;  // zeros a single-row call reads for the B columns that carry nothing
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return g; }

    /// int byte `idx` of `word` as float (times 1/16 with `sixteenth`) through a 2^23 (2^19) + code bit pattern: exact.
    __device__ static __forceinline__ float code_to_float(uint32_t word, uint32_t idx, bool sixteenth) {
        const uint32_t bits = prmt(word, sixteenth ? 0x49000000u : 0x4B000000u, idx | (4u << 4) | (5u << 8) | (7u << 12));
        return __uint_as_float(bits) - (sixteenth ? 524288.0f : 8388608.0f);
    }

    template <int G, int NTOK, class Release>
    __device__ static __forceinline__ void item(const uint8_t* row, uint32_t t, const uint8_t* rec, const XLane<G>& xl, const uint8_t* zeros,
                                                float (&yacc)[G][2], Release&& release) {
        constexpr uint32_t kSubStride = XRec<NTOK>::kSubStride;
        const uint8_t* fq = row + t * 8u;
        const uint32_t m_sel = (2 * t) | ((2 * t) << 4) | ((2 * t + 1) << 8) | ((2 * t + 1) << 12);
        // 6-bit codes of both rows, four per word (SWAR form of src/tensor/quant.cpp:236-244)
        uint32_t sc_lo[2], sc_hi[2], mpair[2];
        float dq[2], dmn[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint4 h = *reinterpret_cast<const uint4*>(row + r * 8 * kPitch);
            sc_lo[r] = h.y & 0x3F3F3F3Fu;                                 // sc0..sc3
            sc_hi[r] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);  // sc4..sc7
            const uint32_t m_lo = h.z & 0x3F3F3F3Fu;
            const uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            mpair[r] = prmt(m_lo, m_hi, m_sel) & 0x00FF00FFu;  // (m_2t, m_2t+1) as fp16 subnormals
            const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
            dq[r] = __low2float(dd) * 16777216.0f;              // d * 2^24: undoes the subnormal encoding of A
            dmn[r] = __high2float(dd) * (16777216.0f * 32.0f);  // dmin * 2^24 * 32: and the / 32 of the sums
        }
        // A fragments of sub-block pair j: [row][quad-pair registers], low nibbles (sub-block 2j) and high (2j + 1)
        auto load_a = [&](int j, uint32_t (&aLo)[2][4], uint32_t (&aHi)[2][4]) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint2 q = *reinterpret_cast<const uint2*>(fq + r * 8 * kPitch + 16 + j * 32);
                const uint32_t qa = q.x, qb = q.y, qa8 = qa >> 8, qb8 = qb >> 8;
                aLo[r][0] = qa & 0x000F000Fu, aLo[r][1] = qa8 & 0x000F000Fu, aLo[r][2] = qb & 0x000F000Fu, aLo[r][3] = qb8 & 0x000F000Fu;
                aHi[r][0] = qa & 0x00F000F0u, aHi[r][1] = qa8 & 0x00F000F0u, aHi[r][2] = qb & 0x00F000F0u, aHi[r][3] = qb8 & 0x00F000F0u;
            }
        };
        const float* invp = reinterpret_cast<const float*>(rec + XRec<NTOK>::kOffInv);
        float T[G][2];  // the item's scaled sums per column group: rows g, g + 8
        if constexpr (NTOK == 1) {
            // B base per sub-block phase p: the lane whose column pair is p reads x (hi for even g, lo for odd g), the others zeros
            const uint8_t* real = rec + (xl.g & 1u) * 64u + t * 16u;
            const uint8_t* zb = zeros + t * 16u;
            const uint8_t* bp[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) bp[p] = (xl.g >> 1) == static_cast<uint32_t>(p) ? real : zb;
            float c[2][4];  // tile h: sub-blocks 4h .. 4h + 3
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t aLo[2][4], aHi[2][4];
                load_a(j, aLo, aHi);
                const int h = j >> 1, pl = (2 * j) & 3, ph = (2 * j + 1) & 3;
                const uint4 bl = *reinterpret_cast<const uint4*>(bp[pl] + (2 * j) * kSubStride);
                const uint4 bh = *reinterpret_cast<const uint4*>(bp[ph] + (2 * j + 1) * kSubStride);
                if ((j & 1) == 0) mma16816_first(c[h], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                else mma16816(c[h], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                mma16816(c[h], aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                mma16816(c[h], aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                mma16816(c[h], aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
            }
            release();  // every byte of the slot has been consumed
            // lane t holds S_t (tile 0) and S_{4+t} (tile 1) of rows g and g + 8 in its column pair (hi, lo)
            const bool odd = (t & 1u) != 0;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float w0 = code_to_float(sc_lo[r], t, odd), w1 = code_to_float(sc_hi[r], t, odd);
                float a = fmaf(w1, c[1][2 * r] + c[1][2 * r + 1], w0 * (c[0][2 * r] + c[0][2 * r + 1]));
                a += __shfl_xor_sync(0xFFFFFFFFu, a, 1);
                a += __shfl_xor_sync(0xFFFFFFFFu, a, 2);
                T[0][r] = a;
            }
        } else {
            float a[G][2][4];  // a_p per column group and row half: w_p * S_p after sub-block p, completed by sub-block 4 + p
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t aLo[2][4], aHi[2][4];
                load_a(j, aLo, aHi);
                float wl[2], wh[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    wl[r] = code_to_float(j < 2 ? sc_lo[r] : sc_hi[r], (2 * j) & 3, false);
                    wh[r] = code_to_float(j < 2 ? sc_lo[r] : sc_hi[r], (2 * j + 1) & 3, true);
                }
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const uint4 bl = *reinterpret_cast<const uint4*>(rec + xl.xs[gi] + (2 * j) * kSubStride);
                    const uint4 bh = *reinterpret_cast<const uint4*>(rec + xl.xs[gi] + (2 * j + 1) * kSubStride);
                    float cl[4], ch[4];
                    mma16816_first(cl, aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    mma16816(cl, aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                    mma16816_first(ch, aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                    mma16816(ch, aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
                    const int pl = (2 * j) & 3, ph = (2 * j + 1) & 3;
                    if (j < 2) {
                        a[gi][0][pl] = wl[0] * (cl[0] + cl[1]), a[gi][1][pl] = wl[1] * (cl[2] + cl[3]);
                        a[gi][0][ph] = wh[0] * (ch[0] + ch[1]), a[gi][1][ph] = wh[1] * (ch[2] + ch[3]);
                    } else {
                        a[gi][0][pl] = fmaf(wl[0], cl[0] + cl[1], a[gi][0][pl]), a[gi][1][pl] = fmaf(wl[1], cl[2] + cl[3], a[gi][1][pl]);
                        a[gi][0][ph] = fmaf(wh[0], ch[0] + ch[1], a[gi][0][ph]), a[gi][1][ph] = fmaf(wh[1], ch[2] + ch[3], a[gi][1][ph]);
                    }
                }
            }
            release();
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                T[gi][0] = (a[gi][0][0] + a[gi][0][1]) + (a[gi][0][2] + a[gi][0][3]);
                T[gi][1] = (a[gi][1][0] + a[gi][1][1]) + (a[gi][1][2] + a[gi][1][3]);
            }
        }
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const uint32_t bs = *reinterpret_cast<const uint32_t*>(rec + xl.sums[gi]);
            float cm[4];
            mma16816_first(cm, mpair[0], mpair[1], 0u, 0u, bs, 0u);
            const float inv = invp[xl.tok[gi]];  // 1 / s of this super-block of the column group's x row: a power of two
            yacc[gi][0] = fmaf(dq[0] * inv, T[gi][0], yacc[gi][0]);
            yacc[gi][0] = fmaf(-dmn[0] * inv, cm[0] + cm[1], yacc[gi][0]);
            yacc[gi][1] = fmaf(dq[1] * inv, T[gi][1], yacc[gi][1]);
            yacc[gi][1] = fmaf(-dmn[1] * inv, cm[2] + cm[3], yacc[gi][1]);
        }
    }
};

// ---- repacked formats (layouts: gemv_mma_grouped.cu) ------------------------------------------------------------------------
// Every scale group sg (a 32-element block, or 16 elements of Q6_K) gets a fresh fp32 accumulator S_sg; the group's
// scale and zero point are applied in fp32, in this order for every batch size:
//     P_p = sum over the groups sg = p (mod 4), ascending, of m_sg * (S_sg - zero * 2^-24 * sum_sg(x))     (an fma chain)
//     y  += ((P_0 + P_1) + (P_2 + P_3)) / s                         m_sg = scale_sg * 2^24, s = the scale of this super-block of x
// A call with ONE x row places x in the column pair (2p, 2p + 1) of B for the groups sg = p (mod 4) (the other columns
// read zeros), so one accumulator tile carries four groups and lane t of a row owns P_t; two shuffles build the sum.
template <class T>
struct GroupedItem {
    static constexpr uint32_t kZeroBytes = 1024;
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return g; }

    template <int G, int NTOK, class Release>
    __device__ static __forceinline__ void item(const uint8_t* r0, uint32_t t, const uint8_t* rec, const XLane<G>& xl, const uint8_t* zeros,
                                                float (&yacc)[G][2], Release&& release) {
        constexpr uint32_t kSubStride = XRec<NTOK>::kSubStride;
        constexpr int kGroups = static_cast<int>(T::kScaleGroups), kSteps = static_cast<int>(T::kStepsPerGroup);
        constexpr float kZ = -T::kZero / 16777216.0f;
        constexpr uint32_t kHalfStride = XRec<NTOK>::kCols * 32u;  // the two 16-element halves of a sub-block are [half][column][32 B]
        const uint8_t* r1 = r0 + 8 * T::kPitch;
        typename T::Frag f0, f1;
        T::load(f0, r0, t);
        T::load(f1, r1, t);
        typename T::Scales s0, s1;
        T::load_scales(s0, r0);
        T::load_scales(s1, r1);
        release();  // fragments and scales are in registers
        const float* sx16 = reinterpret_cast<const float*>(rec + XRec<NTOK>::kOffSx16);
        // the 16 elements of step s of group sg inside x: 32-element sub-block `sub`, half `lh`
        auto sub_of = [](int sg, int s) { return kSteps == 2 ? sg : sg >> 1; };
        auto lh_of = [](int sg, int s) { return kSteps == 2 ? s : sg & 1; };
        if constexpr (NTOK == 1) {
            const uint8_t* real = rec + (xl.g & 1u) * 32u + t * 8u;
            const uint8_t* zb = zeros + t * 8u;
            const uint8_t* bp[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) bp[p] = (xl.g >> 1) == static_cast<uint32_t>(p) ? real : zb;
            float P0 = 0.0f, P1 = 0.0f;  // this lane's P_t for rows g and g + 8
#pragma unroll
            for (int q = 0; q < kGroups / 4; ++q) {
                float c[4];
#pragma unroll
                for (int p = 0; p < 4; ++p) {
#pragma unroll
                    for (int s = 0; s < kSteps; ++s) {
                        const int sg = 4 * q + p;
                        uint32_t a0, a1, a2, a3;
                        T::pairs(f0, sg, s, a0, a2);
                        T::pairs(f1, sg, s, a1, a3);
                        const uint2 b = *reinterpret_cast<const uint2*>(bp[p] + sub_of(sg, s) * kSubStride + lh_of(sg, s) * kHalfStride);
                        if (p == 0 && s == 0) mma16816_first(c, a0, a1, a2, a3, b.x, b.y);
                        else mma16816(c, a0, a1, a2, a3, b.x, b.y);
                    }
                }
                // lane t finishes group 4q + t
                const float m0 = T::scale_lane(s0, q, t), m1 = T::scale_lane(s1, q, t);
                float sx;
                if constexpr (kSteps == 2) sx = sx16[2 * (4 * q + t)] + sx16[2 * (4 * q + t) + 1];
                else sx = sx16[4 * q + t];
                const float z = __fmul_rn(sx, kZ);
                if (q == 0) P0 = __fmul_rn(m0, (c[0] + c[1]) + z), P1 = __fmul_rn(m1, (c[2] + c[3]) + z);
                else P0 = fmaf(m0, (c[0] + c[1]) + z, P0), P1 = fmaf(m1, (c[2] + c[3]) + z, P1);
            }
            P0 += __shfl_xor_sync(0xFFFFFFFFu, P0, 1);
            P1 += __shfl_xor_sync(0xFFFFFFFFu, P1, 1);
            P0 += __shfl_xor_sync(0xFFFFFFFFu, P0, 2);
            P1 += __shfl_xor_sync(0xFFFFFFFFu, P1, 2);
            const float inv = reinterpret_cast<const float*>(rec + XRec<NTOK>::kOffInv)[0];  // 1 / s of this super-block of x
            yacc[0][0] = fmaf(inv, P0, yacc[0][0]);
            yacc[0][1] = fmaf(inv, P1, yacc[0][1]);
        } else {
            float P[G][2][4];
#pragma unroll
            for (int sg = 0; sg < kGroups; ++sg) {
                float c[G][4];
#pragma unroll
                for (int s = 0; s < kSteps; ++s) {
                    uint32_t a0, a1, a2, a3;
                    T::pairs(f0, sg, s, a0, a2);
                    T::pairs(f1, sg, s, a1, a3);
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) {
                        const uint2 b = *reinterpret_cast<const uint2*>(rec + xl.xs[gi] + sub_of(sg, s) * kSubStride + lh_of(sg, s) * kHalfStride);
                        if (s == 0) mma16816_first(c[gi], a0, a1, a2, a3, b.x, b.y);
                        else mma16816(c[gi], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                const float m0 = T::scale(s0, sg), m1 = T::scale(s1, sg);
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    float sx;
                    if constexpr (kSteps == 2) sx = sx16[(2 * sg) * NTOK + xl.tok[gi]] + sx16[(2 * sg + 1) * NTOK + xl.tok[gi]];
                    else sx = sx16[sg * NTOK + xl.tok[gi]];
                    const float z = __fmul_rn(sx, kZ);
                    if (sg < 4) {
                        P[gi][0][sg & 3] = __fmul_rn(m0, (c[gi][0] + c[gi][1]) + z);
                        P[gi][1][sg & 3] = __fmul_rn(m1, (c[gi][2] + c[gi][3]) + z);
                    } else {
                        P[gi][0][sg & 3] = fmaf(m0, (c[gi][0] + c[gi][1]) + z, P[gi][0][sg & 3]);
                        P[gi][1][sg & 3] = fmaf(m1, (c[gi][2] + c[gi][3]) + z, P[gi][1][sg & 3]);
                    }
                }
            }
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const float inv = reinterpret_cast<const float*>(rec + XRec<NTOK>::kOffInv)[xl.tok[gi]];
                yacc[gi][0] = fmaf(inv, (P[gi][0][0] + P[gi][0][1]) + (P[gi][0][2] + P[gi][0][3]), yacc[gi][0]);
                yacc[gi][1] = fmaf(inv, (P[gi][1][0] + P[gi][1][1]) + (P[gi][1][2] + P[gi][1][3]), yacc[gi][1]);
            }
        }
    }
};

struct Q40r : GroupedItem<Q40r> {
    static constexpr uint32_t kType = HALO_CUDA_T_Q4_0, kGroupBytes = 144, kPitch = 192, kScaleGroups = 8, kStepsPerGroup = 2;
    static constexpr uint32_t kItemCoord = kGroupBytes / 4, kBoxInner = kPitch / 4, kMapElemBytes = 4, kXLaneBytes = 8;
    static constexpr bool kAllowSlices = format_allows_slices(kType);
    static constexpr float kZero = 8.0f;
    struct Frag {
        uint4 q[2];  // chunk c: words of blocks 4c..4c+3
    };
    struct Scales {
        uint4 d;  // eight fp16
    };
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.q[0] = *reinterpret_cast<const uint4*>(row + 16 + t * 16);
        f.q[1] = *reinterpret_cast<const uint4*>(row + 16 + 64 + t * 16);
    }
    __device__ static void load_scales(Scales& s, const uint8_t* row) { s.d = *reinterpret_cast<const uint4*>(row); }
    /// A pair registers (elements 4t+0, 4t+2 | 4t+1, 4t+3) of scale group g, k-step s (0: low nibbles, 1: high nibbles)
    __device__ static void pairs(const Frag& f, int g, int s, uint32_t& p02, uint32_t& p13) {
        const uint4 c = f.q[g >> 2];
        const uint32_t w = (g & 3) == 0 ? c.x : (g & 3) == 1 ? c.y : (g & 3) == 2 ? c.z : c.w;
        p02 = (w >> (4 * s)) & 0x000F000Fu;
        p13 = (w >> (8 + 4 * s)) & 0x000F000Fu;
    }
    __device__ static float scale(const Scales& s, int g) {
        const uint32_t w = (g >> 1) == 0 ? s.d.x : (g >> 1) == 1 ? s.d.y : (g >> 1) == 2 ? s.d.z : s.d.w;
        return __half2float(__ushort_as_half(static_cast<unsigned short>(g & 1 ? w >> 16 : w & 0xFFFFu))) * 16777216.0f;
    }
    /// scale(s, 4 * q + t) for a lane-dependent t
    __device__ static float scale_lane(const Scales& s, int q, uint32_t t) {
        const uint32_t w = q == 0 ? (t & 2u ? s.d.y : s.d.x) : (t & 2u ? s.d.w : s.d.z);
        return __half2float(__ushort_as_half(static_cast<unsigned short>(t & 1u ? w >> 16 : w & 0xFFFFu))) * 16777216.0f;
    }
};

struct Q80r : GroupedItem<Q80r> {
    static constexpr uint32_t kType = HALO_CUDA_T_Q8_0, kGroupBytes = 272, kPitch = 320, kScaleGroups = 8, kStepsPerGroup = 2;
    static constexpr uint32_t kItemCoord = kGroupBytes / 4, kBoxInner = kPitch / 4, kMapElemBytes = 4, kXLaneBytes = 8;
    static constexpr bool kAllowSlices = format_allows_slices(kType);
    static constexpr float kZero = 128.0f;
    struct Frag {
        uint4 q[4];  // chunk c: (block 2c, step 0), (block 2c, step 1), (block 2c+1, step 0), (block 2c+1, step 1)
    };
    using Scales = Q40r::Scales;
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
#pragma unroll
        for (int c = 0; c < 4; ++c) f.q[c] = *reinterpret_cast<const uint4*>(row + 16 + c * 64 + t * 16);
    }
    __device__ static void load_scales(Scales& s, const uint8_t* row) { s.d = *reinterpret_cast<const uint4*>(row); }
    __device__ static void pairs(const Frag& f, int g, int s, uint32_t& p02, uint32_t& p13) {
        const uint4 c = f.q[g >> 1];
        const int i = (g & 1) * 2 + s;
        const uint32_t w = i == 0 ? c.x : i == 1 ? c.y : i == 2 ? c.z : c.w;
        // int8 + 128 as an unsigned byte: flip the sign bit; the 128 comes back out through the zero point
        p02 = (w & 0x00FF00FFu) ^ 0x00800080u;
        p13 = ((w >> 8) & 0x00FF00FFu) ^ 0x00800080u;
    }
    __device__ static float scale(const Scales& s, int g) { return Q40r::scale(s, g); }
    __device__ static float scale_lane(const Scales& s, int q, uint32_t t) { return Q40r::scale_lane(s, q, t); }
};

struct Q6Kr : GroupedItem<Q6Kr> {
    static constexpr uint32_t kType = HALO_CUDA_T_Q6_K, kGroupBytes = 224, kPitch = 224, kScaleGroups = 16, kStepsPerGroup = 1;
    static constexpr uint32_t kItemCoord = kGroupBytes / 4, kBoxInner = kPitch / 4, kMapElemBytes = 4, kXLaneBytes = 8;
    static constexpr bool kAllowSlices = format_allows_slices(kType);
    static constexpr float kZero = 32.0f;
    /// The 224-byte slot rows put rows g and g + 1 on overlapping banks; fragment rows 0..7 take slot rows 0,2,4,6,1,3,5,7
    /// instead (rows two apart are 64 bytes apart modulo the 128-byte bank span), and y is stored accordingly.
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return ((2u * g) & 7u) | (g >> 2); }
    struct Frag {
        uint4 ql[2];  // half n: words (b, lh) = (0,0), (0,1), (1,0), (1,1)
        uint4 qh;     // words (n, lh) = (0,0), (0,1), (1,0), (1,1)
    };
    struct Scales {
        uint4 sc;   // sixteen int8
        float d24;  // d * 2^24
    };
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.ql[0] = *reinterpret_cast<const uint4*>(row + 32 + t * 16);
        f.ql[1] = *reinterpret_cast<const uint4*>(row + 32 + 64 + t * 16);
        f.qh = *reinterpret_cast<const uint4*>(row + 32 + 128 + t * 16);
    }
    __device__ static void load_scales(Scales& s, const uint8_t* row) {
        s.sc = *reinterpret_cast<const uint4*>(row);
        s.d24 = __half2float(*reinterpret_cast<const __half*>(row + 16)) * 16777216.0f;
    }
    /// scale group g = 8n + 2*quarter + lh: elements 128n + 32*quarter + 16*lh + (4t .. 4t+3)
    __device__ static void pairs(const Frag& f, int g, int /*s*/, uint32_t& p02, uint32_t& p13) {
        const int n = g >> 3, quarter = (g >> 1) & 3, lh = g & 1, b = quarter & 1, nib = quarter >> 1;
        const uint4 c = f.ql[n];
        const int wi = b * 2 + lh, hi = n * 2 + lh;
        const uint32_t w = wi == 0 ? c.x : wi == 1 ? c.y : wi == 2 ? c.z : c.w;
        const uint32_t h = hi == 0 ? f.qh.x : hi == 1 ? f.qh.y : hi == 2 ? f.qh.z : f.qh.w;
        // the four 6-bit codes of this lane as bytes: nibble | two high bits << 4 (byte j of h holds element j's high bits
        // of all four quarters, two bits each), then the byte pairs (0, 2) and (1, 3) as 16-bit lanes
        const uint32_t wn = nib ? w >> 4 : w;
        const uint32_t hs = quarter == 0 ? h << 4 : quarter == 1 ? h << 2 : quarter == 2 ? h : h >> 2;
        const uint32_t codes = (wn & 0x0F0F0F0Fu) | (hs & 0x30303030u);
        p02 = prmt(codes, 0u, 0x4240u);
        p13 = prmt(codes, 0u, 0x4341u);
    }
    /// d * 2^24 * sc_g; the int8 goes to float through the 2^23 + 128 + sc bit pattern (exact, no conversion instruction)
    __device__ static float scale(const Scales& s, int g) {
        const uint32_t w = (g >> 2) == 0 ? s.sc.x : (g >> 2) == 1 ? s.sc.y : (g >> 2) == 2 ? s.sc.z : s.sc.w;
        const uint32_t bits = prmt(w ^ 0x80808080u, 0x4B000000u, (g & 3) | (4u << 4) | (5u << 8) | (7u << 12));
        return (__uint_as_float(bits) - 8388736.0f) * s.d24;
    }
    __device__ static float scale_lane(const Scales& s, int q, uint32_t t) {
        const uint32_t w = q == 0 ? s.sc.x : q == 1 ? s.sc.y : q == 2 ? s.sc.z : s.sc.w;
        const uint32_t bits = prmt(w ^ 0x80808080u, 0x4B000000u, t | (4u << 4) | (5u << 8) | (7u << 12));
        return (__uint_as_float(bits) - 8388736.0f) * s.d24;
    }
};

}  // namespace mma
}  // namespace halo_cuda
