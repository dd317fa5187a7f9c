// gemv_warp_f32: the fp32 CUDA-core streaming kernel for decode-shaped calls, all four block formats.
//
// One warp owns one W row.  The row is cut into 16- or 32-weight chunks; lane L takes chunks L, L+32, ... so a
// warp-wide load walks the row front to back in runs of whole sectors.  Inside a chunk the sub-block scale is
// factored out (the reference's Vulkan matvec does the same, backends/vulkan/shaders/common/matvec_q4_k_main.glsl:72-90):
//     Q4_K: d*sc*sum(q*x) - dmin*m*sum(x)     Q6_K: (d*s)*sum((q-32)*x)     Q8_0 / Q4_0: d*sum(q*x)
// with every sum in fp32.  The 32 lane partials are added by a fixed xor-shuffle tree.  The split of K over the
// lanes and the order of every addition depend on the shape only, never on the batch size: each x row is bitwise
// its own n_vec == 1 result (the batch-invariance contract of include/halo/backend/backend.h:300-304).
//
// Roofline: HBM.  Algorithmic bytes per call = rows*row_bytes + 4*n_vec*cols + 4*n_vec*rows
// (the reference's own accounting, include/halo/backends/cpu/traffic.h:94-99).
#include "internal.h"
#include "quant_dev.cuh"

namespace halo_cuda {

namespace {

constexpr int kWarpsPerBlock = 4;

__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t* p) {  // 2-byte aligned
    const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
    return static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 16);
}

__device__ __forceinline__ float4 ld_x4(const float* p) { return *reinterpret_cast<const float4*>(p); }

template <int MT>
struct XRows {
    const float* r[MT];
};

// ---- per-format chunk bodies: add chunk c of `row` times x into acc[t] -------------------------------------------

template <int MT>
__device__ __forceinline__ void chunk_q4k(const uint8_t* row, uint32_t c, const XRows<MT>& x, float (&acc)[MT]) {
    // chunk = 8 bytes of qs: 8 low nibbles (sub-block 2g) + 8 high nibbles (sub-block 2g+1), same positions
    const uint32_t b = c >> 4, g = (c >> 2) & 3u, ir = c & 3u;
    const uint8_t* blk = row + b * 144u;
    const uint32_t dm = *reinterpret_cast<const uint32_t*>(blk);
    const float d = f16_bits_to_f32(dm & 0xFFFFu), dmin = f16_bits_to_f32(dm >> 16);
    uint32_t sc0, mn0, sc1, mn1;
    q4k_codes(2 * g, blk + 4, sc0, mn0);
    q4k_codes(2 * g + 1, blk + 4, sc1, mn1);
    const float d0 = d * static_cast<float>(sc0), m0 = dmin * static_cast<float>(mn0);
    const float d1 = d * static_cast<float>(sc1), m1 = dmin * static_cast<float>(mn1);
    const uint2 q = *reinterpret_cast<const uint2*>(blk + 16 + g * 32u + ir * 8u);
    float ql[8], qh[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        ql[i] = static_cast<float>((q.x >> (8 * i)) & 0x0Fu);
        qh[i] = static_cast<float>((q.x >> (8 * i + 4)) & 0x0Fu);
        ql[4 + i] = static_cast<float>((q.y >> (8 * i)) & 0x0Fu);
        qh[4 + i] = static_cast<float>((q.y >> (8 * i + 4)) & 0x0Fu);
    }
    const uint32_t e0 = b * 256u + g * 64u + ir * 8u;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        const float4 a0 = ld_x4(x.r[t] + e0), a1 = ld_x4(x.r[t] + e0 + 4);
        const float4 b0 = ld_x4(x.r[t] + e0 + 32), b1 = ld_x4(x.r[t] + e0 + 36);
        float sl = ql[0] * a0.x;
        sl = fmaf(ql[1], a0.y, sl); sl = fmaf(ql[2], a0.z, sl); sl = fmaf(ql[3], a0.w, sl);
        sl = fmaf(ql[4], a1.x, sl); sl = fmaf(ql[5], a1.y, sl); sl = fmaf(ql[6], a1.z, sl); sl = fmaf(ql[7], a1.w, sl);
        float sh = qh[0] * b0.x;
        sh = fmaf(qh[1], b0.y, sh); sh = fmaf(qh[2], b0.z, sh); sh = fmaf(qh[3], b0.w, sh);
        sh = fmaf(qh[4], b1.x, sh); sh = fmaf(qh[5], b1.y, sh); sh = fmaf(qh[6], b1.z, sh); sh = fmaf(qh[7], b1.w, sh);
        const float xl = ((a0.x + a0.y) + (a0.z + a0.w)) + ((a1.x + a1.y) + (a1.z + a1.w));
        const float xh = ((b0.x + b0.y) + (b0.z + b0.w)) + ((b1.x + b1.y) + (b1.z + b1.w));
        float a = acc[t];
        a = fmaf(d0, sl, a);
        a = fmaf(-m0, xl, a);
        a = fmaf(d1, sh, a);
        a = fmaf(-m1, xh, a);
        acc[t] = a;
    }
}

template <int MT>
__device__ __forceinline__ void chunk_q6k(const uint8_t* row, uint32_t c, const XRows<MT>& x, float (&acc)[MT]) {
    // chunk = positions l0..l0+3 of one 128-element half: 4 quants from each of its four 32-element runs
    const uint32_t b = c >> 4, half = (c >> 3) & 1u, p = c & 7u, l0 = p * 4u;
    const uint8_t* blk = row + b * 210u;
    const uint32_t qa = ld_u32_a2(blk + half * 64u + l0);
    const uint32_t qb = ld_u32_a2(blk + half * 64u + 32u + l0);
    const uint32_t qh = ld_u32_a2(blk + 128u + half * 32u + l0);
    const float d = f16_at(blk + 208);
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + half * 8u + (p >> 2));
    float ds[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) ds[r] = d * static_cast<float>(sc[2 * r]);
    float q[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t la = (qa >> (8 * i)) & 0xFFu, lb = (qb >> (8 * i)) & 0xFFu, h = (qh >> (8 * i)) & 0xFFu;
        q[0][i] = static_cast<float>(static_cast<int>((la & 0x0Fu) | ((h & 3u) << 4)) - 32);
        q[1][i] = static_cast<float>(static_cast<int>((lb & 0x0Fu) | (((h >> 2) & 3u) << 4)) - 32);
        q[2][i] = static_cast<float>(static_cast<int>((la >> 4) | (((h >> 4) & 3u) << 4)) - 32);
        q[3][i] = static_cast<float>(static_cast<int>((lb >> 4) | (((h >> 6) & 3u) << 4)) - 32);
    }
    const uint32_t e0 = b * 256u + half * 128u + l0;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        float a = acc[t];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const float4 v = ld_x4(x.r[t] + e0 + 32 * r);
            float s = q[r][0] * v.x;
            s = fmaf(q[r][1], v.y, s); s = fmaf(q[r][2], v.z, s); s = fmaf(q[r][3], v.w, s);
            a = fmaf(ds[r], s, a);
        }
        acc[t] = a;
    }
}

template <int MT>
__device__ __forceinline__ void chunk_q80(const uint8_t* row, uint32_t c, const XRows<MT>& x, float (&acc)[MT]) {
    // chunk = half a block: 16 int8 quants
    const uint8_t* blk = row + (c >> 1) * 34u;
    const uint32_t h = c & 1u;
    const float d = f16_at(blk);
    float q[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t v = ld_u32_a2(blk + 2 + h * 16u + 4 * i);
#pragma unroll
        for (int j = 0; j < 4; ++j) q[4 * i + j] = static_cast<float>(static_cast<int8_t>((v >> (8 * j)) & 0xFFu));
    }
    const uint32_t e0 = (c >> 1) * 32u + h * 16u;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = ld_x4(x.r[t] + e0 + 4 * i);
            s = fmaf(q[4 * i + 0], v.x, s); s = fmaf(q[4 * i + 1], v.y, s);
            s = fmaf(q[4 * i + 2], v.z, s); s = fmaf(q[4 * i + 3], v.w, s);
        }
        acc[t] = fmaf(d, s, acc[t]);
    }
}

template <int MT>
__device__ __forceinline__ void chunk_q40(const uint8_t* row, uint32_t c, const XRows<MT>& x, float (&acc)[MT]) {
    // chunk = one block: 16 bytes, low nibbles are elements 0..15, high nibbles 16..31
    const uint8_t* blk = row + c * 18u;
    const float d = f16_at(blk);
    float ql[16], qh[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t v = ld_u32_a2(blk + 2 + 4 * i);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            ql[4 * i + j] = static_cast<float>(static_cast<int>((v >> (8 * j)) & 0x0Fu) - 8);
            qh[4 * i + j] = static_cast<float>(static_cast<int>((v >> (8 * j + 4)) & 0x0Fu) - 8);
        }
    }
    const uint32_t e0 = c * 32u;
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = ld_x4(x.r[t] + e0 + 4 * i);
            s = fmaf(ql[4 * i + 0], v.x, s); s = fmaf(ql[4 * i + 1], v.y, s);
            s = fmaf(ql[4 * i + 2], v.z, s); s = fmaf(ql[4 * i + 3], v.w, s);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = ld_x4(x.r[t] + e0 + 16 + 4 * i);
            s = fmaf(qh[4 * i + 0], v.x, s); s = fmaf(qh[4 * i + 1], v.y, s);
            s = fmaf(qh[4 * i + 2], v.z, s); s = fmaf(qh[4 * i + 3], v.w, s);
        }
        acc[t] = fmaf(d, s, acc[t]);
    }
}

template <uint32_t WT, int MT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) gemv_warp_kernel(const uint8_t* __restrict__ w, uint64_t w_stride,
                                                                       const float* __restrict__ x, uint64_t x_stride,
                                                                       float* __restrict__ y, uint64_t y_stride, uint32_t rows,
                                                                       uint32_t cols, uint32_t n_vec, const float* __restrict__ gate_dt_bias,
                                                                       const float* __restrict__ gate_a, uint32_t gate_n_v) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (n >= rows) return;  // whole warps leave together
    const uint32_t t0 = blockIdx.y * MT;
    const uint8_t* row = w + uint64_t{n} * w_stride;
    XRows<MT> xr;
    float acc[MT];
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        const uint32_t tt = t0 + t < n_vec ? t0 + t : n_vec - 1;
        xr.r[t] = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tt} * x_stride);
        acc[t] = 0.0f;
    }
    constexpr uint32_t kChunkElems = WT == HALO_CUDA_T_Q4_0 ? 32u : 16u;
    const uint32_t n_chunks = cols / kChunkElems;
    for (uint32_t c = lane; c < n_chunks; c += 32) {
        if constexpr (WT == HALO_CUDA_T_Q4_K) chunk_q4k<MT>(row, c, xr, acc);
        else if constexpr (WT == HALO_CUDA_T_Q6_K) chunk_q6k<MT>(row, c, xr, acc);
        else if constexpr (WT == HALO_CUDA_T_Q8_0) chunk_q80<MT>(row, c, xr, acc);
        else chunk_q40<MT>(row, c, xr, acc);
    }
#pragma unroll
    for (int t = 0; t < MT; ++t) {
        float a = acc[t];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, off);
        if (lane == 0 && t0 + t < n_vec)
            reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{t0 + t} * y_stride)[n] = gated_value(a, n, gate_n_v, gate_dt_bias, gate_a);
    }
}

template <uint32_t WT>
int launch_t(const GemvCall& c, cudaStream_t s) {
    const uint32_t gx = (c.rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    // Token tiles of 4, 2 and 1 rows of x: the tile width changes how often a weight chunk is re-read from L2,
    // never a row's arithmetic.
    uint32_t t = 0;
    auto offset = [&](uint32_t first) {
        GemvCall d = c;
        d.x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{first} * c.x_stride);
        d.y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{first} * c.y_stride);
        return d;
    };
    if (c.n_vec - t >= 4) {
        const uint32_t tiles = (c.n_vec - t) / 4;
        if (tiles > 65535u) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: n_vec %u exceeds the launch limit", c.n_vec);
        const GemvCall d = offset(t);
        gemv_warp_kernel<WT, 4><<<dim3(gx, tiles), kWarpsPerBlock * 32, 0, s>>>(d.w, d.w_stride, d.x, d.x_stride, d.y, d.y_stride, d.rows,
                                                                                d.cols, tiles * 4, d.gate_dt_bias, d.gate_a, d.gate_n_v);
        t += tiles * 4;
    }
    if (c.n_vec - t >= 2) {
        const GemvCall d = offset(t);
        gemv_warp_kernel<WT, 2><<<dim3(gx, 1), kWarpsPerBlock * 32, 0, s>>>(d.w, d.w_stride, d.x, d.x_stride, d.y, d.y_stride, d.rows, d.cols, 2,
                                                                            d.gate_dt_bias, d.gate_a, d.gate_n_v);
        t += 2;
    }
    if (c.n_vec - t >= 1) {
        const GemvCall d = offset(t);
        gemv_warp_kernel<WT, 1><<<dim3(gx, 1), kWarpsPerBlock * 32, 0, s>>>(d.w, d.w_stride, d.x, d.x_stride, d.y, d.y_stride, d.rows, d.cols, 1,
                                                                            d.gate_dt_bias, d.gate_a, d.gate_n_v);
    }
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

bool gemv_warp_f32_supports(const GemvCall& c) {
    // vector loads: x rows 16-byte aligned; Q4_K blocks read as 32/64-bit words, the other formats as 16-bit words
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;
    const auto wa = reinterpret_cast<uintptr_t>(c.w);
    switch (c.wtype) {
        case HALO_CUDA_T_Q4_K: return wa % 8 == 0 && c.w_stride % 8 == 0;
        case HALO_CUDA_T_Q6_K:
        case HALO_CUDA_T_Q8_0:
        case HALO_CUDA_T_Q4_0: return wa % 2 == 0 && c.w_stride % 2 == 0;
        default: return false;
    }
}

int launch_gemv_warp_f32(const GemvCall& c, cudaStream_t s) {
    switch (c.wtype) {
        case HALO_CUDA_T_Q4_0: return launch_t<HALO_CUDA_T_Q4_0>(c, s);
        case HALO_CUDA_T_Q8_0: return launch_t<HALO_CUDA_T_Q8_0>(c, s);
        case HALO_CUDA_T_Q4_K: return launch_t<HALO_CUDA_T_Q4_K>(c, s);
        case HALO_CUDA_T_Q6_K: return launch_t<HALO_CUDA_T_Q6_K>(c, s);
        default: return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_warp_f32 takes Q4_0 / Q8_0 / Q4_K / Q6_K weights");
    }
}

}  // namespace halo_cuda
