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

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {
namespace {

using namespace mma;

// ---- per-format traits --------------------------------------------------------------------------------------------
struct Q40r {
    static constexpr uint32_t kType = HALO_CUDA_T_Q4_0, kGroupBytes = 144, kPitch = 192, kScaleGroups = 8, kStepsPerGroup = 2;
    static constexpr float kZero = 8.0f;
    struct Frag {
        uint4 q[2];  // chunk c: words of blocks 4c..4c+3
    };
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.q[0] = *reinterpret_cast<const uint4*>(row + 16 + t * 16);
        f.q[1] = *reinterpret_cast<const uint4*>(row + 16 + 64 + t * 16);
    }
    /// A pair registers (elements 4t+0, 4t+2 | 4t+1, 4t+3) of scale group g, k-step s (0: low nibbles, 1: high nibbles)
    __device__ static void pairs(const Frag& f, int g, int s, uint32_t& p02, uint32_t& p13) {
        const uint4 c = f.q[g >> 2];
        const uint32_t w = (g & 3) == 0 ? c.x : (g & 3) == 1 ? c.y : (g & 3) == 2 ? c.z : c.w;
        p02 = (w >> (4 * s)) & 0x000F000Fu;
        p13 = (w >> (8 + 4 * s)) & 0x000F000Fu;
    }
    __device__ static float scale(const uint8_t* row, int g) { return __half2float(reinterpret_cast<const __half*>(row)[g]); }
};

struct Q80r {
    static constexpr uint32_t kType = HALO_CUDA_T_Q8_0, kGroupBytes = 272, kPitch = 320, kScaleGroups = 8, kStepsPerGroup = 2;
    static constexpr float kZero = 128.0f;
    struct Frag {
        uint4 q[4];  // chunk c: (block 2c, step 0), (block 2c, step 1), (block 2c+1, step 0), (block 2c+1, step 1)
    };
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
#pragma unroll
        for (int c = 0; c < 4; ++c) f.q[c] = *reinterpret_cast<const uint4*>(row + 16 + c * 64 + t * 16);
    }
    __device__ static void pairs(const Frag& f, int g, int s, uint32_t& p02, uint32_t& p13) {
        const uint4 c = f.q[g >> 1];
        const int i = (g & 1) * 2 + s;
        const uint32_t w = i == 0 ? c.x : i == 1 ? c.y : i == 2 ? c.z : c.w;
        // int8 + 128 as an unsigned byte: flip the sign bit; the 128 comes back out through the zero point
        p02 = (w & 0x00FF00FFu) ^ 0x00800080u;
        p13 = ((w >> 8) & 0x00FF00FFu) ^ 0x00800080u;
    }
    __device__ static float scale(const uint8_t* row, int g) { return __half2float(reinterpret_cast<const __half*>(row)[g]); }
};

struct Q6Kr {
    static constexpr uint32_t kType = HALO_CUDA_T_Q6_K, kGroupBytes = 224, kPitch = 224, kScaleGroups = 16, kStepsPerGroup = 1;
    static constexpr float kZero = 32.0f;
    struct Frag {
        uint4 ql[2];  // half n: words (b, lh) = (0,0), (0,1), (1,0), (1,1)
        uint4 qh;     // words (n, lh) = (0,0), (0,1), (1,0), (1,1)
    };
    __device__ static void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.ql[0] = *reinterpret_cast<const uint4*>(row + 32 + t * 16);
        f.ql[1] = *reinterpret_cast<const uint4*>(row + 32 + 64 + t * 16);
        f.qh = *reinterpret_cast<const uint4*>(row + 32 + 128 + t * 16);
    }
    /// scale group g = 8n + 2*quarter + lh: elements 128n + 32*quarter + 16*lh + (4t .. 4t+3)
    __device__ static void pairs(const Frag& f, int g, int /*s*/, uint32_t& p02, uint32_t& p13) {
        const int n = g >> 3, quarter = (g >> 1) & 3, lh = g & 1, b = quarter & 1, nib = quarter >> 1;
        const uint4 c = f.ql[n];
        const int wi = b * 2 + lh, hi = n * 2 + lh;
        const uint32_t w = wi == 0 ? c.x : wi == 1 ? c.y : wi == 2 ? c.z : c.w;
        const uint32_t h = hi == 0 ? f.qh.x : hi == 1 ? f.qh.y : hi == 2 ? f.qh.z : f.qh.w;
        // 6-bit code = nibble | two high bits << 4, both halves of a pair at once
        const int sh02 = 2 * quarter - 4, sh13 = 8 + 2 * quarter - 4;
        const uint32_t h02 = sh02 >= 0 ? h >> sh02 : h << -sh02;
        const uint32_t h13 = h >> sh13;
        p02 = ((w >> (4 * nib)) & 0x000F000Fu) | (h02 & 0x00300030u);
        p13 = ((w >> (8 + 4 * nib)) & 0x000F000Fu) | (h13 & 0x00300030u);
    }
    __device__ static float scale(const uint8_t* row, int g) {
        const float d = __half2float(*reinterpret_cast<const __half*>(row + 16));
        return d * static_cast<float>(reinterpret_cast<const int8_t*>(row)[g]);
    }
};

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

/// One tile of a tensor map over 32-bit words: words [x, x + box) of rows [y, y + 16).
__device__ __forceinline__ void tma_words_g2s(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// T: format traits.  NTOK / KS / NS / PRE as in gemv_mma_q4k_kernel.
template <class T, int NTOK, int KS, int NS, bool PRE>
__global__ void __launch_bounds__(kRowBlocks * KS * 32, 1)
gemv_mma_grouped_kernel(const __grid_constant__ CUtensorMap wmap, const float* __restrict__ x, uint64_t x_stride, float* __restrict__ y,
                        uint64_t y_stride, uint32_t rows, uint32_t nb, uint32_t chunk_sb, uint32_t* __restrict__ error_word,
                        const uint8_t* __restrict__ xstage) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    constexpr int G = (NTOK + 3) / 4;
    constexpr uint32_t kThreads = kRowBlocks * KS * 32, kWarps = kRowBlocks * KS;
    static_assert(kWarps <= kMaxWarps && NS <= 6, "shared-memory header layout");
    constexpr uint32_t kSlot = 16 * T::kPitch;
    constexpr uint32_t kOffData = kOffRing + kWarps * NS * kSlot;
    constexpr uint32_t kCols = 2 * NTOK, kSubStride = kCols * 64u, kSbStride = kCols * 16u, kSx16Stride = 16u * NTOK * 4u;  // per super-block
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rbl = warp % kRowBlocks, ks = warp / kRowBlocks;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t cols = nb * 256u;

    const uint32_t rb = blockIdx.x * kRowBlocks + rbl;
    const bool active = rb * 16u < rows;
    const uint32_t n_items = active && nb > ks ? (nb - ks + KS - 1) / KS : 0;
    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlot;
    uint32_t next_x = ks * (T::kGroupBytes / 4);  // word column of the next group to fetch
    asm volatile("griddepcontrol.launch_dependents;");
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t fill_slot = 0, issued = 0;
    auto refill = [&]() {
        if (lane == 0) {
            mbar_expect_tx(bars + fill_slot * 8u, kSlot);
            tma_words_g2s(ring + fill_slot * kSlot, &wmap, next_x, rb * 16u, bars + fill_slot * 8u);
        }
        next_x += KS * (T::kGroupBytes / 4);
        fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        ++issued;
    };
    for (uint32_t it = 0; it < NS && it < n_items; ++it) refill();
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float* s_scale = reinterpret_cast<float*>(smem + kOffScale);
    float* s_inv = reinterpret_cast<float*>(smem + kOffInv);
    float* s_red = reinterpret_cast<float*>(smem + kOffRed);
    const uint32_t xbar = smem_base + kOffXBar;
    uint8_t* const xs_area = smem + kOffData;
    uint8_t* const sxh_area = xs_area + chunk_sb * 8u * kSubStride;       // fp16 sums (written by the staging code, not read here)
    float* const sx16_area = reinterpret_cast<float*>(sxh_area + chunk_sb * kSbStride);
    if constexpr (PRE) {
        if (tid == 0) {
            mbar_init(xbar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        if (tid < NTOK) s_inv[tid] = reinterpret_cast<const float*>(xstage + uint64_t{nb} * (8u * kSubStride + kSbStride))[tid];
        __syncthreads();
    } else {
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
    }

    // B fragment base per column group (a lane whose column carries no token reads the last real column, see gemv_mma.cu)
    const uint8_t* xs_ptr[G];
    uint32_t tok[G];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t col = min(8u * gi + g, kCols - 1);
        xs_ptr[gi] = xs_area + col * 64u + t * 8u;
        tok[gi] = min(4u * gi + t, static_cast<uint32_t>(NTOK - 1));
    }
    const uint8_t* slot0 = smem + kOffRing + warp * NS * kSlot + g * T::kPitch;

    float yacc[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;

    uint32_t slot = 0, parity = 0;
    bool lost = false;
    for (uint32_t c0 = 0; c0 < nb; c0 += chunk_sb) {
        const uint32_t n_sb = min(chunk_sb, nb - c0);
        if (c0 != 0) __syncthreads();
        if constexpr (PRE) {
            if (tid == 0) {
                const uint32_t xs_bytes = n_sb * 8u * kSubStride, sx_bytes = n_sb * kSx16Stride;
                mbar_expect_tx(xbar, xs_bytes + sx_bytes);
                bulk_g2s(smem_base + kOffData, xstage + uint64_t{c0} * 8u * kSubStride, xs_bytes, xbar);
                bulk_g2s(smem_base + kOffData + chunk_sb * (8u * kSubStride + kSbStride),
                         xstage + uint64_t{nb} * (8u * kSubStride + kSbStride) + 64 + uint64_t{c0} * kSx16Stride, sx_bytes, xbar);
            }
            if (!mbar_wait(xbar, (c0 / chunk_sb) & 1u)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;
            }
        } else {
            for (uint32_t tk = 0; tk < NTOK; ++tk)
                stage_row(xs_area, sxh_area, reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride),
                          s_scale[tk], c0, n_sb, kSubStride, kSbStride, 2 * tk * 64u, tid, kThreads, sx16_area, NTOK, tk);
        }
        __syncthreads();
        if (!active || lost) continue;

        for (uint32_t i = (ks + KS - c0 % KS) % KS; i < n_sb; i += KS) {
            if (!mbar_wait(bars + slot * 8u, parity)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;
                break;
            }
            const uint8_t* r0 = slot0 + slot * kSlot;
            const uint8_t* r1 = r0 + 8 * T::kPitch;
            typename T::Frag f0, f1;
            T::load(f0, r0, t);
            T::load(f1, r1, t);
            const uint8_t* xb[G];
#pragma unroll
            for (int gi = 0; gi < G; ++gi) xb[gi] = xs_ptr[gi] + i * (8u * kSubStride);
            const float* sxi = sx16_area + i * (16u * NTOK);
#pragma unroll
            for (int sg = 0; sg < static_cast<int>(T::kScaleGroups); ++sg) {
                float c[G][4];
#pragma unroll
                for (int s = 0; s < static_cast<int>(T::kStepsPerGroup); ++s) {
                    uint32_t a0, a1, a2, a3;
                    T::pairs(f0, sg, s, a0, a2);
                    T::pairs(f1, sg, s, a1, a3);
                    // the 16 elements of this step inside x: 32-element sub-block `sub`, half `lh`
                    const int sub = T::kStepsPerGroup == 2 ? sg : sg >> 1, lh = T::kStepsPerGroup == 2 ? s : sg & 1;
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) {
                        const uint2 b = *reinterpret_cast<const uint2*>(xb[gi] + sub * kSubStride + lh * 32);
                        if (s == 0) mma16816_first(c[gi], a0, a1, a2, a3, b.x, b.y);
                        else mma16816(c[gi], a0, a1, a2, a3, b.x, b.y);
                    }
                }
                // scale and zero point of this group, both rows, in fp32; 2^24 undoes the subnormal encoding of A
                const float sc0 = T::scale(r0, sg), sc1 = T::scale(r1, sg);
                const float m0 = sc0 * 16777216.0f, m1 = sc1 * 16777216.0f, z0 = -sc0 * T::kZero, z1 = -sc1 * T::kZero;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    float sx;
                    if constexpr (T::kStepsPerGroup == 2) sx = sxi[(2 * sg) * NTOK + tok[gi]] + sxi[(2 * sg + 1) * NTOK + tok[gi]];
                    else sx = sxi[sg * NTOK + tok[gi]];
                    yacc[gi][0] = fmaf(m0, c[gi][0] + c[gi][1], yacc[gi][0]);
                    yacc[gi][0] = fmaf(z0, sx, yacc[gi][0]);
                    yacc[gi][1] = fmaf(m1, c[gi][2] + c[gi][3], yacc[gi][1]);
                    yacc[gi][1] = fmaf(z1, sx, yacc[gi][1]);
                }
            }
            __syncwarp();
            slot = slot + 1 == NS ? 0 : slot + 1;
            parity ^= (slot == 0);
            if (issued < n_items) refill();
        }
    }

    if constexpr (KS > 1) {
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

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/// The repacked weight matrix as a 2-D tensor of 32-bit words {row words, rows}, tiled `pitch / 4` words x 16 rows.
int weight_map_words(const GemvCall& c, uint32_t pitch, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        HC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail(HALO_CUDA_E_BACKEND, "cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {c.row_bytes / 4, c.rows};
    const cuuint64_t strides[1] = {c.w_stride};
    const cuuint32_t box[2] = {pitch / 4, 16};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint8_t*>(c.w), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HALO_CUDA_E_KERNEL, "MATMUL: cannot describe the repacked weight matrix to the copy engine (CUresult %d)", (int)r);
    return 0;
}

cudaLaunchConfig_t pdl_config_r(uint32_t grid, uint32_t block, uint32_t smem, cudaStream_t s, cudaLaunchAttribute* attr) {
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

template <class T, int NTOK, int KS, int NS>
int launch_r(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, cudaStream_t s) {
    constexpr bool PRE = NTOK >= 2;
    constexpr int G = (NTOK + 3) / 4;
    constexpr uint32_t kSlot = 16 * T::kPitch;
    constexpr uint32_t off_data = kOffRing + kRowBlocks * KS * NS * kSlot;
    const uint32_t nb = c.cols / 256u;
    const uint32_t per_sb = 8u * (2 * NTOK) * 64u + (2 * NTOK) * 16u + 16u * NTOK * 4u;
    uint32_t chunk = (kSmemBudget - off_data) / per_sb;
    if (chunk > nb) chunk = nb;
    if (chunk == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_r has no shared memory left for %d x rows", NTOK);
    const uint32_t red = (KS - 1) * kRowBlocks * 32 * 2 * G * 4, data = chunk * per_sb;
    const uint32_t smem_bytes = off_data + (data > red ? data : red);
    static bool attr_set = false;
    if (!attr_set) {
        HC_CUDA(cudaFuncSetAttribute(gemv_mma_grouped_kernel<T, NTOK, KS, NS, PRE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kSmemBudget)));
        attr_set = true;
    }
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    CUtensorMap wmap;
    if (int rc = weight_map_words(c, T::kPitch, &wmap)) return rc;
    const uint8_t* xstage = nullptr;
    if constexpr (PRE) {
        void* ws = nullptr;
        if (int rc = workspace(ctx, 0, stage_scratch_bytes(nb, NTOK), s, &ws)) return rc;
        stage_x_kernel<<<NTOK, 512, 0, s>>>(x, c.x_stride, static_cast<uint8_t*>(ws), nb, NTOK);
        HC_CUDA(cudaGetLastError());
        xstage = static_cast<const uint8_t*>(ws);
    }
    const uint32_t grid = (c.rows + 16u * kRowBlocks - 1) / (16u * kRowBlocks);
    cudaLaunchAttribute attr[1];
    const cudaLaunchConfig_t cfg = pdl_config_r(grid, kRowBlocks * KS * 32, smem_bytes, s, attr);
    HC_CUDA(cudaLaunchKernelEx(&cfg, gemv_mma_grouped_kernel<T, NTOK, KS, NS, PRE>, wmap, x, c.x_stride, y, c.y_stride, c.rows, nb, chunk,
                               ctx->error_word_dev, xstage));
    return 0;
}

// Two warps per row block; the ring depth follows the slot size so that ring + x staging fit in shared memory.
template <class T, int NTOK>
int launch_tokens_r(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > 16) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n == NTOK) return launch_r<T, NTOK, 2, T::kPitch <= 224 ? 3 : 2>(ctx, c, tok0, s);
        return launch_tokens_r<T, NTOK + 1>(ctx, c, tok0, n, s);
    }
}

template <class T>
int launch_type_r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += 16) {
        const uint32_t n = c.n_vec - t0 < 16 ? c.n_vec - t0 : 16;
        if (int rc = launch_tokens_r<T, 1>(ctx, c, t0, n, s)) return rc;
    }
    return 0;
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
    return (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) == 0 || c.n_vec == 1;
}

int launch_gemv_mma_r(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    switch (c.wtype) {
        case HALO_CUDA_T_Q4_0: return launch_type_r<Q40r>(ctx, c, s);
        case HALO_CUDA_T_Q8_0: return launch_type_r<Q80r>(ctx, c, s);
        case HALO_CUDA_T_Q6_K: return launch_type_r<Q6Kr>(ctx, c, s);
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
