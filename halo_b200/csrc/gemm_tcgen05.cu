// gemm_tcgen05_{f16,bf16}[_r]: the prefill GEMM, Y[M x N] = X[M x K] * dequant(W)[N x K]^T, M >= 64, for raw Q4_K rows and
// (the _r variants) for Q6_K / Q8_0 / Q4_0 rows in the repacked layout of halo_cuda_repack_rows (gemv_mma_grouped.cu).
//
// The reference's own GEMM path rounds x and dequant(W) to fp16 and accumulates in fp32
// (backends/vulkan/shaders/common/matmul_cm_main.glsl:1-6); a caller opts in with GemvArgs::allow_gemm
// (include/halo/backend/backend.h:300-304).  Same numerics here: W is dequantized in fp32 exactly as
// tensor::dequantize_row does ((d*sc)*q - dmin*m, src/tensor/quant.cpp:247-269; (d*s)*(q-32), :302-327; d*q, :143-151;
// d*(q-8), :79-90) and rounded ONCE to the 16-bit type.
//
// Structure (one 256-token x 256-row output tile per CTA, 576 threads):
//   warp 0      TMA producer: two 128 x 64 boxes of the 16-bit copy of X per stage (128-byte swizzle)
//   warp 1      allocates TMEM, issues tcgen05.mma (M=128, N=256, K=16; two accumulators = all 512 TMEM columns)
//   warps 2-17  two threads per W row: each reads 16 bytes of quants + the block header and writes 32 dequantized
//               16-bit values, together one 128-byte swizzled row of the B tile; afterwards the same warps run the epilogue
//               (tcgen05.ld -> fp32 y)
// A three-stage ring of {A0, A1, B} tiles is tracked by mbarriers: full_a (TMA bytes), full_b (16 warp arrivals after
// a proxy fence), empty (tcgen05.commit).  Each CTA dequantizes its W tile once for 256 tokens, which keeps the
// CUDA-core work below the tensor-pipe time of the two MMAs it feeds.
//
// The K order inside every group of 8 elements is permuted to (0,2,1,3,4,6,5,7) in BOTH operands -- the cast kernel
// writes X that way -- because that is the order in which masked nibble pairs fall out of a 32-bit word.
//
// Every mbarrier wait is bounded; a role that gives up raises the context error word, and all roles still meet at
// the final barrier so that TMEM is released before the CTA exits.
//
// Roofline: tensor pipe, 2*M*N*K flops per call.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace halo_cuda {
namespace {

constexpr uint32_t kBM = 256, kBN = 256, kBK = 64, kStages = 3;
constexpr uint32_t kTileA = 128 * kBK * 2;          // one 128-token box: 16 KiB
constexpr uint32_t kTileB = kBN * kBK * 2;          // 32 KiB
constexpr uint32_t kStageBytes = 2 * kTileA + kTileB;  // 64 KiB
constexpr uint32_t kDeqWarps = 16;                  // two threads per W row: each unpacks 16 of the 32 quant bytes
constexpr uint32_t kGemmThreads = 64 + kDeqWarps * 32;
constexpr uint32_t kGemmSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kGemmWaitSpins = 1u << 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void g_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void g_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void g_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool g_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kGemmWaitSpins; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void g_tma_2d(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows and 128-byte swizzle: start address / 16,
// leading byte offset (unused for swizzled K-major, 1), stride byte offset 1024 / 16 (one 8-row swizzle atom),
// descriptor version 1 (bits 46-47), layout type 2 = SWIZZLE_128B (bits 61-63).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return static_cast<uint64_t>((addr & 0x3FFFFu) >> 4) | (uint64_t{1} << 16) | (uint64_t{64} << 32) | (uint64_t{1} << 46) |
           (uint64_t{2} << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

/// fp32 -> 16-bit copy of X with the K order of every 8-element group permuted to (0,2,1,3,4,6,5,7).
template <bool BF16>
__global__ void __launch_bounds__(256) cast_x_kernel(const float* __restrict__ x, uint64_t x_stride, uint16_t* __restrict__ out,
                                                     uint32_t n_vec, uint32_t cols) {
    const uint32_t groups = cols / 8;
    for (uint64_t i = uint64_t{blockIdx.x} * blockDim.x + threadIdx.x; i < uint64_t{n_vec} * groups; i += uint64_t{gridDim.x} * blockDim.x) {
        const uint32_t t = static_cast<uint32_t>(i / groups), gidx = static_cast<uint32_t>(i % groups);
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{t} * x_stride) + gidx * 2;
        const float4 a = src[0], b = src[1];
        const float v[8] = {a.x, a.z, a.y, a.w, b.x, b.z, b.y, b.w};
        uint32_t p[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if constexpr (BF16) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
                p[k] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                const __half2 h = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
                p[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(out + (uint64_t{t} * cols + uint64_t{gidx} * 8)) = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

/// Two dequantized weights (fp32, the reference's expression) -> one packed 16-bit pair, rounded once.
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    if constexpr (BF16) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    } else {
        const __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
}

/// A masked nibble pair (two quants in bits 0-3 or 4-7 of each half) -> two fp32 dequantized weights -> packed pair.
/// 0x6400 | q is the half 1024 + q (1024 + 16 q for a high nibble, whose scale arrives pre-divided by 16).
template <bool BF16>
__device__ __forceinline__ uint32_t deq_pair(uint32_t masked, float scale, float minv) {
    const uint32_t h = masked | 0x64006400u;
    const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&h), __half2half2(__ushort_as_half(0x6400)));
    const float2 f = __half22float2(q);
    // d1 * q is exact in fp32 (11-bit scale x 6-bit code x 4-bit quant), so the fused form rounds like mul-then-sub
    return pack2<BF16>(fmaf(scale, f.x, -minv), fmaf(scale, f.y, -minv));
}

// ---- what a dequant thread does per K block of 64 weights, by weight format -------------------------------------------------------
// Thread (row r, half hf) of the B tile owns 32 of the row's 64 weights of the block and writes four 16-byte chunks (8 values
// each) of the row's 128 bytes; chunk position p holds weights 8p .. 8p+7 of the block in the order (0,2,1,3,4,6,5,7), which is
// how byte pairs (0,2) and (1,3) fall out of a masked 32-bit word.  fetch() requests the bytes one K block ahead.
__device__ __forceinline__ void store_chunk(uint8_t* dst, uint32_t pos, uint32_t sw, const uint4& v) {
    *reinterpret_cast<uint4*>(dst + ((pos ^ sw) << 4)) = v;
}

struct GemmQ4K {  // raw rows of 144-byte super-blocks: K block j of a super-block = sub-blocks 2j (low nibbles) and 2j + 1 (high)
    struct Regs {
        uint4 h, q;
    };
    __device__ static __forceinline__ void fetch(Regs& r, const uint8_t* row, uint32_t kb, uint32_t hf) {
        const uint8_t* blk = row + (kb >> 2) * 144u;
        r.h = *reinterpret_cast<const uint4*>(blk);
        r.q = *reinterpret_cast<const uint4*>(blk + 16 + (kb & 3u) * 32 + hf * 16);
    }
    template <bool BF16>
    __device__ static __forceinline__ void emit(const Regs& r, uint32_t kb, uint32_t hf, uint8_t* dst, uint32_t sw) {
        const uint32_t j = kb & 3u;
        // 6-bit codes of sub-blocks 2j (low nibbles) and 2j+1 (high nibbles), src/tensor/quant.cpp:236-244
        const uint32_t s0 = r.h.y, s1 = r.h.z, s2 = r.h.w;
        uint32_t sc0, mn0, sc1, mn1;
        if (j < 2) {
            sc0 = (s0 >> (16 * j)) & 63u;       mn0 = (s1 >> (16 * j)) & 63u;
            sc1 = (s0 >> (16 * j + 8)) & 63u;   mn1 = (s1 >> (16 * j + 8)) & 63u;
        } else {
            const uint32_t sh = 16 * (j - 2);
            sc0 = ((s2 >> sh) & 0x0Fu) | (((s0 >> (sh + 6)) & 3u) << 4);
            mn0 = ((s2 >> (sh + 4)) & 0x0Fu) | (((s1 >> (sh + 6)) & 3u) << 4);
            sc1 = ((s2 >> (sh + 8)) & 0x0Fu) | (((s0 >> (sh + 14)) & 3u) << 4);
            mn1 = ((s2 >> (sh + 12)) & 0x0Fu) | (((s1 >> (sh + 14)) & 3u) << 4);
        }
        const __half2 dd = *reinterpret_cast<const __half2*>(&r.h.x);
        const float d = __low2float(dd), dmin = __high2float(dd);
        const float d1 = d * static_cast<float>(sc0), m1 = dmin * static_cast<float>(mn0);
        const float d2 = d * static_cast<float>(sc1) * 0.0625f, m2 = dmin * static_cast<float>(mn1);
        const uint32_t q[4] = {r.q.x, r.q.y, r.q.z, r.q.w};
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {  // 16-byte chunk c: elements 8c..8c+7 of the low-nibble sub-block, c+4: of the high one
            const uint32_t c = 2 * hf + cc;
            const uint32_t u0 = q[2 * cc], u1 = q[2 * cc + 1];
            uint4 lo, hi;
            lo.x = deq_pair<BF16>(u0 & 0x000F000Fu, d1, m1);
            lo.y = deq_pair<BF16>((u0 >> 8) & 0x000F000Fu, d1, m1);
            lo.z = deq_pair<BF16>(u1 & 0x000F000Fu, d1, m1);
            lo.w = deq_pair<BF16>((u1 >> 8) & 0x000F000Fu, d1, m1);
            hi.x = deq_pair<BF16>(u0 & 0x00F000F0u, d2, m2);
            hi.y = deq_pair<BF16>((u0 >> 8) & 0x00F000F0u, d2, m2);
            hi.z = deq_pair<BF16>(u1 & 0x00F000F0u, d2, m2);
            hi.w = deq_pair<BF16>((u1 >> 8) & 0x00F000F0u, d2, m2);
            store_chunk(dst, c, sw, lo);
            store_chunk(dst, c + 4, sw, hi);
        }
    }
};

/// One 8-value chunk from two words whose bytes are the unsigned codes of weights 0..3 and 4..7 (each < 1024 as a 16-bit lane).
template <bool BF16>
__device__ __forceinline__ uint4 chunk_of_bytes(uint32_t w0, uint32_t w1, float scale, float minv) {
    uint4 v;
    v.x = deq_pair<BF16>(w0 & 0x00FF00FFu, scale, minv);
    v.y = deq_pair<BF16>((w0 >> 8) & 0x00FF00FFu, scale, minv);
    v.z = deq_pair<BF16>(w1 & 0x00FF00FFu, scale, minv);
    v.w = deq_pair<BF16>((w1 >> 8) & 0x00FF00FFu, scale, minv);
    return v;
}

struct GemmQ80R {  // repacked groups of 272 B: d[8] fp16 | chunk c < 4, thread t < 4: words (block 2c, step 0/1), (block 2c+1, step 0/1)
    struct Regs {
        uint2 w[4];  // thread t: the words (step 0, step 1) of this thread's block
        float d;
    };
    __device__ static __forceinline__ void fetch(Regs& r, const uint8_t* row, uint32_t kb, uint32_t hf) {
        const uint8_t* grp = row + (kb >> 2) * 272u;
        const uint8_t* chunk = grp + 16 + (kb & 3u) * 64 + hf * 8;
#pragma unroll
        for (int t = 0; t < 4; ++t) r.w[t] = *reinterpret_cast<const uint2*>(chunk + t * 16);
        r.d = __half2float(*reinterpret_cast<const __half*>(grp + 2 * (2 * (kb & 3u) + hf)));
    }
    template <bool BF16>
    __device__ static __forceinline__ void emit(const Regs& r, uint32_t kb, uint32_t hf, uint8_t* dst, uint32_t sw) {
        const float minv = 128.0f * r.d;  // int8 + 128 as an unsigned byte; d * (u - 128) = fma(d, u, -128 d), rounded once
#pragma unroll
        for (int g = 0; g < 4; ++g) {     // weights 8g .. 8g+7 of the block: step g / 2, threads 2 (g % 2) and + 1
            const int t0 = 2 * (g & 1);
            const uint32_t w0 = (g >> 1 ? r.w[t0].y : r.w[t0].x) ^ 0x80808080u, w1 = (g >> 1 ? r.w[t0 + 1].y : r.w[t0 + 1].x) ^ 0x80808080u;
            store_chunk(dst, 4 * hf + g, sw, chunk_of_bytes<BF16>(w0, w1, r.d, minv));
        }
    }
};

struct GemmQ40R {  // repacked groups of 144 B: d[8] fp16 | chunk c < 2, thread t < 4: the quant word (bytes 4t..4t+3) of blocks 4c..4c+3
    struct Regs {
        uint32_t w[4];  // thread t's word of this thread's block: low nibbles = weights 4t.., high nibbles = weights 16 + 4t..
        float d;
    };
    __device__ static __forceinline__ void fetch(Regs& r, const uint8_t* row, uint32_t kb, uint32_t hf) {
        const uint8_t* grp = row + (kb >> 2) * 144u;
        const uint32_t b = 2 * (kb & 3u) + hf;  // block of the group
        const uint8_t* at = grp + 16 + (b >> 2) * 64 + (b & 3u) * 4;
#pragma unroll
        for (int t = 0; t < 4; ++t) r.w[t] = *reinterpret_cast<const uint32_t*>(at + t * 16);
        r.d = __half2float(*reinterpret_cast<const __half*>(grp + 2 * b));
    }
    template <bool BF16>
    __device__ static __forceinline__ void emit(const Regs& r, uint32_t kb, uint32_t hf, uint8_t* dst, uint32_t sw) {
        const float minv = 8.0f * r.d, d16 = r.d * 0.0625f;  // a high nibble arrives as 16 q
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // weights 8g .. 8g+7: g < 2 the low nibbles of words 2g, 2g+1; else the high nibbles of words 2(g-2), +1
            const uint32_t w0 = r.w[2 * (g & 1)], w1 = r.w[2 * (g & 1) + 1];
            uint4 v;
            if (g < 2) {
                v.x = deq_pair<BF16>(w0 & 0x000F000Fu, r.d, minv);
                v.y = deq_pair<BF16>((w0 >> 8) & 0x000F000Fu, r.d, minv);
                v.z = deq_pair<BF16>(w1 & 0x000F000Fu, r.d, minv);
                v.w = deq_pair<BF16>((w1 >> 8) & 0x000F000Fu, r.d, minv);
            } else {
                v.x = deq_pair<BF16>(w0 & 0x00F000F0u, d16, minv);
                v.y = deq_pair<BF16>((w0 >> 8) & 0x00F000F0u, d16, minv);
                v.z = deq_pair<BF16>(w1 & 0x00F000F0u, d16, minv);
                v.w = deq_pair<BF16>((w1 >> 8) & 0x00F000F0u, d16, minv);
            }
            store_chunk(dst, 4 * hf + g, sw, v);
        }
    }
};

struct GemmQ6KR {  // repacked groups of 224 B: scales[16] int8 | d fp16, pad | half n < 2, thread t < 4: ql words (b, lh) | thread t: qh words (n, lh)
    struct Regs {
        uint2 ql[4], qh[4];  // thread t: the words (lh 0, lh 1) of this thread's quarter
        float ds[2];         // d * scale of the quarter's two 16-weight groups
    };
    __device__ static __forceinline__ void fetch(Regs& r, const uint8_t* row, uint32_t kb, uint32_t hf) {
        const uint8_t* grp = row + (kb >> 2) * 224u;
        const uint32_t n = (kb >> 1) & 1u, quarter = 2 * (kb & 1u) + hf;  // weights 128 n + 32 quarter .. + 31
        const uint8_t* ql = grp + 32 + n * 64 + (quarter & 1u) * 8, *qh = grp + 32 + 128 + n * 8;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            r.ql[t] = *reinterpret_cast<const uint2*>(ql + t * 16);
            r.qh[t] = *reinterpret_cast<const uint2*>(qh + t * 16);
        }
        const float d = __half2float(*reinterpret_cast<const __half*>(grp + 16));
        const char2 sc = *reinterpret_cast<const char2*>(grp + 8 * n + 2 * quarter);
        r.ds[0] = d * static_cast<float>(sc.x), r.ds[1] = d * static_cast<float>(sc.y);
    }
    template <bool BF16>
    __device__ static __forceinline__ void emit(const Regs& r, uint32_t kb, uint32_t hf, uint8_t* dst, uint32_t sw) {
        const uint32_t quarter = 2 * (kb & 1u) + hf, nib = (quarter >> 1) * 4, hsh = 2 * quarter;
#pragma unroll
        for (int g = 0; g < 4; ++g) {  // weights 8g .. 8g+7 of the quarter: lh = g / 2, threads 2 (g % 2) and + 1
            const int t0 = 2 * (g & 1), lh = g >> 1;
            auto codes = [&](int t) {
                const uint32_t l = lh ? r.ql[t].y : r.ql[t].x, h = lh ? r.qh[t].y : r.qh[t].x;
                return ((l >> nib) & 0x0F0F0F0Fu) | (((h >> hsh) & 0x03030303u) << 4);
            };
            const float ds = r.ds[lh];
            store_chunk(dst, 4 * hf + g, sw, chunk_of_bytes<BF16>(codes(t0), codes(t0 + 1), ds, 32.0f * ds));  // (d*s)*(q-32), rounded once
        }
    }
};

template <bool BF16, class F>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap xmap, const uint8_t* __restrict__ w, uint64_t w_stride,
                        float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t n_vec, uint32_t nkb,
                        uint32_t* __restrict__ error_word) {
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment (one swizzle atom)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t{1023});
    const uint32_t tiles = smem_u32(smem);
    const uint32_t bars = tiles + kStages * kStageBytes;  // full_a[3], full_b[3], empty[3], accum, then the TMEM base word
    auto full_a = [&](uint32_t s) { return bars + s * 8u; };
    auto full_b = [&](uint32_t s) { return bars + (kStages + s) * 8u; };
    auto empty = [&](uint32_t s) { return bars + (2 * kStages + s) * 8u; };
    const uint32_t accum_bar = bars + 3 * kStages * 8u;
    volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(smem + kStages * kStageBytes + 3 * kStages * 8 + 8);
    volatile uint32_t* abort_word = tmem_word + 1;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            g_mbar_init(full_a(s), 1);
            g_mbar_init(full_b(s), kDeqWarps);
            g_mbar_init(empty(s), 1);
        }
        g_mbar_init(accum_bar, 1);
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: all 512 columns (two 128 x 256 fp32 accumulators); one CTA per SM, so nobody else asks
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(tmem_word))), "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_word;

    if (warp == 0) {
        // ---- TMA producer: X tiles -----------------------------------------------------------------------------------
        if (lane == 0) {
            for (uint32_t kb = 0; kb < nkb; ++kb) {
                const uint32_t s = kb % kStages, use = kb / kStages;
                if (use > 0 && !g_mbar_wait(empty(s), (use - 1) & 1u)) {
                    *abort_word = 1;
                    break;
                }
                g_mbar_expect_tx(full_a(s), 2 * kTileA);
                g_tma_2d(tiles + s * kStageBytes, &xmap, kb * kBK, m0, full_a(s));
                g_tma_2d(tiles + s * kStageBytes + kTileA, &xmap, kb * kBK, m0 + 128, full_a(s));
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----------------------------------------------------------------------------------------------------
        if (lane == 0) {
            // instruction descriptor: D = fp32 (bits 4-5 = 1), A / B format (bits 7-9 / 10-12: 0 = f16, 1 = bf16), both
            // K-major (bits 15, 16 = 0), N / 8 at bits 17-22, M / 16 at bits 24-28
            const uint32_t fmt = BF16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((kBN >> 3) << 17) | ((128u >> 4) << 24);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
                const uint32_t s = kb % kStages, parity = (kb / kStages) & 1u;
                ok = g_mbar_wait(full_a(s), parity) && g_mbar_wait(full_b(s), parity);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a0 = tiles + s * kStageBytes, a1 = a0 + kTileA, b = a0 + 2 * kTileA;
#pragma unroll
                for (uint32_t k = 0; k < kBK / 16; ++k) {  // 16 elements = 32 bytes along K inside the swizzled row
                    const uint32_t acc = (kb | k) != 0 ? 1u : 0u;
                    umma_f16(tmem_base, smem_desc(a0 + k * 32), smem_desc(b + k * 32), idesc, acc);
                    umma_f16(tmem_base + 256, smem_desc(a1 + k * 32), smem_desc(b + k * 32), idesc, acc);
                }
                umma_commit(empty(s));  // arrives once the MMAs above have finished reading this stage
            }
            if (ok) umma_commit(accum_bar);
            else *abort_word = 1;
        }
    } else {
        // ---- dequant producers: thread r writes W row n0 + r of the B tile ------------------------------------------------------
        const uint32_t r = (threadIdx.x - 64) >> 1, hf = threadIdx.x & 1u;  // row of the tile, and which 16 quant bytes
        const bool valid = n0 + r < rows;
        const uint8_t* row = w + uint64_t{valid ? n0 + r : 0} * w_stride;
        const uint32_t sw = r & 7u;
        bool ok = true;
        // the quants of the next K block are requested one iteration ahead, so that their latency hides behind the
        // unpacking of the current block and the wait for a free stage
        typename F::Regs next{};
        if (valid) F::fetch(next, row, 0, hf);
        for (uint32_t kb = 0; kb < nkb; ++kb) {
            const uint32_t s = kb % kStages, use = kb / kStages;
            const typename F::Regs cur = next;
            if (valid && kb + 1 < nkb) F::fetch(next, row, kb + 1, hf);
            if (use > 0) {
                ok = g_mbar_wait(empty(s), (use - 1) & 1u);
                ok = __all_sync(0xFFFFFFFFu, ok);
                if (!ok) break;
            }
            uint8_t* dst = smem + s * kStageBytes + 2 * kTileA + r * 128u;
            if (valid) {
                F::template emit<BF16>(cur, kb, hf, dst, sw);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + ((4 * hf + c) << 4)) = make_uint4(0, 0, 0, 0);
            }
            // make the generic-proxy stores visible to the tensor core's (async-proxy) reads, then one arrival per warp
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) g_mbar_arrive(full_b(s));
        }
        // ---- epilogue: TMEM -> registers -> y --------------------------------------------------------------------------------
        if (ok) {
            ok = g_mbar_wait(accum_bar, 0);
            ok = __all_sync(0xFFFFFFFFu, ok);
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // TMEM lanes 32*quarter.. (fixed by warp id % 4), accumulator `half`, and which 128 of its 256 columns
            const uint32_t quarter = warp & 3u, half = ((warp - 2) >> 2) & 1u, chalf = (warp - 2) >> 3;
            const uint32_t token = m0 + half * 128u + quarter * 32u + lane;
            float* yr = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{token} * y_stride) + n0;
#pragma unroll 1
            for (uint32_t c = chalf * (kBN / 64); c < (chalf + 1) * (kBN / 64); ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + half * 256u + c * 32u;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (token < n_vec) {
                    const uint32_t nn = n0 + c * 32u;
                    if (nn + 32u <= rows && (reinterpret_cast<uintptr_t>(yr + c * 32u) & 15u) == 0) {
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            *reinterpret_cast<uint4*>(yr + c * 32u + 4 * k) = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
                    } else {
                        for (uint32_t k = 0; k < 32u && nn + k < rows; ++k) yr[c * 32u + k] = __uint_as_float(v[k]);
                    }
                }
            }
        } else if (lane == 0) {
            *abort_word = 1;
        }
    }
    // ---- everyone meets here, also after a failed wait, so that TMEM is always released -----------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && *abort_word != 0 && error_word != nullptr) atomicOr(error_word, 2u);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

/// The 16-bit copy of X as a 2-D tensor {cols, n_vec}, boxes of 64 x 128 elements with the 128-byte swizzle UMMA expects.
int x_map(void* x16, uint32_t n_vec, uint32_t cols, bool bf16, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        HC_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return fail(HALO_CUDA_E_BACKEND, "cuTensorMapEncodeTiled is not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {cols, n_vec};
    const cuuint64_t strides[1] = {uint64_t{cols} * 2};
    const cuuint32_t box[2] = {kBK, 128};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x16, dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(HALO_CUDA_E_KERNEL, "MATMUL: cannot describe x to the copy engine (CUresult %d)", (int)r);
    return 0;
}

template <bool BF16, class F>
int launch_t(HaloCudaCtx* ctx, const GemvCall& c, cudaStream_t s) {
    void* ws = nullptr;
    if (int rc = workspace(ctx, 0, uint64_t{c.n_vec} * c.cols * 2, s, &ws)) return rc;
    const uint64_t groups = uint64_t{c.n_vec} * (c.cols / 8);
    const uint32_t cast_blocks = static_cast<uint32_t>(groups / 256 + 1 < 148 * 8 ? groups / 256 + 1 : 148 * 8);
    cast_x_kernel<BF16><<<cast_blocks, 256, 0, s>>>(c.x, c.x_stride, static_cast<uint16_t*>(ws), c.n_vec, c.cols);
    HC_CUDA(cudaGetLastError());
    CUtensorMap xmap;
    if (int rc = x_map(ws, c.n_vec, c.cols, BF16, &xmap)) return rc;
    auto kern = gemm_tcgen05_kernel<BF16, F>;
    if (int rc = allow_dynamic_smem(ctx, reinterpret_cast<const void*>(kern), kGemmSmem)) return rc;
    const dim3 grid((c.rows + kBN - 1) / kBN, (c.n_vec + kBM - 1) / kBM);
    kern<<<grid, kGemmThreads, kGemmSmem, s>>>(xmap, c.w, c.w_stride, c.y, c.y_stride, c.rows, c.n_vec, c.cols / kBK, ctx->error_word_dev);
    HC_CUDA(cudaGetLastError());
    return 0;
}

template <class F>
int launch_f(HaloCudaCtx* ctx, const GemvCall& c, bool bf16, cudaStream_t s) {
    return bf16 ? launch_t<true, F>(ctx, c, s) : launch_t<false, F>(ctx, c, s);
}

}  // namespace

/// repacked: W is in the layout of halo_cuda_repack_rows (Q6_K / Q8_0 / Q4_0); else raw Q4_K rows.
bool gemm_tcgen05_supports(const GemvCall& c, bool repacked) {
    const bool type_ok = repacked ? (c.wtype == HALO_CUDA_T_Q6_K || c.wtype == HALO_CUDA_T_Q8_0 || c.wtype == HALO_CUDA_T_Q4_0) : c.wtype == HALO_CUDA_T_Q4_K;
    if (!type_ok || c.cols == 0 || c.rows == 0 || c.cols % 256u != 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // 16-byte block loads
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return (c.rows + kBN - 1) / kBN <= 0x7FFFFFFFu && (c.n_vec + kBM - 1) / kBM <= 65535u;
}

int launch_gemm_tcgen05(HaloCudaCtx* ctx, const GemvCall& c, bool bf16, bool repacked, cudaStream_t s) {
    if (!repacked) return launch_f<GemmQ4K>(ctx, c, bf16, s);
    switch (c.wtype) {
        case HALO_CUDA_T_Q6_K: return launch_f<GemmQ6KR>(ctx, c, bf16, s);
        case HALO_CUDA_T_Q8_0: return launch_f<GemmQ80R>(ctx, c, bf16, s);
        case HALO_CUDA_T_Q4_0: return launch_f<GemmQ40R>(ctx, c, bf16, s);
        default: return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: no repacked GEMM for weight type id %u", c.wtype);
    }
}

}  // namespace halo_cuda
