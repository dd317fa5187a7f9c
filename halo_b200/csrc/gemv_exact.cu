// Bit-exact kernels: the CPU-order gemv (variant gemv_exact8), the GET_ROWS-shaped dequantizer and the
// two-stage argmax of the LM head.
//
// gemv_exact8 reproduces the reference's detail::dot (backends/cpu/kernel_common.h:16-27) on the device: eight
// lanes per W row hold the eight interleaved partial sums, lane j adds the products of elements i = j (mod 8)
// in increasing i with the multiply and the add rounded separately, and the lanes are combined as
// ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)) followed by the sequential tail.  Its output is bitwise the CPU backend's.
// It is the acceptance anchor and the autotuner's validation reference, not the fast path: HBM traffic is the
// algorithmic minimum (every weight byte once per token tile) but the per-element unpacking is issue-bound.
#include "internal.h"
#include "quant_dev.cuh"

namespace halo_cuda {

namespace {

constexpr int kExactRowsPerBlock = 32;  // 32 rows x 8 lanes = 256 threads
constexpr int kExactTokens = 4;         // x rows sharing one unpacked weight

template <uint32_t WT>
__global__ void __launch_bounds__(256) gemv_exact8_kernel(const uint8_t* __restrict__ w, uint64_t w_stride,
                                                          const float* __restrict__ x, uint64_t x_stride,
                                                          float* __restrict__ y, uint64_t y_stride, uint32_t rows,
                                                          uint32_t cols, uint32_t n_vec, const float* __restrict__ gate_dt_bias,
                                                          const float* __restrict__ gate_a, uint32_t gate_n_v) {
    const uint32_t lane8 = threadIdx.x & 7u;
    const uint32_t n = blockIdx.x * kExactRowsPerBlock + (threadIdx.x >> 3);
    const uint32_t t0 = blockIdx.y * kExactTokens;
    // Rows past the end still take part in the shuffles below (with a clamped row), they only skip the store.
    const uint32_t nc = n < rows ? n : rows - 1;
    const uint8_t* row = w + uint64_t{nc} * w_stride;
    const float* xr[kExactTokens];
    float acc[kExactTokens];
#pragma unroll
    for (int t = 0; t < kExactTokens; ++t) {
        const uint32_t tt = t0 + t < n_vec ? t0 + t : n_vec - 1;
        xr[t] = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tt} * x_stride);
        acc[t] = 0.0f;
    }
    const uint32_t k8 = cols & ~7u;
    for (uint32_t i = lane8; i < k8; i += 8) {
        const float wv = weight_elem<WT>(row, i);
#pragma unroll
        for (int t = 0; t < kExactTokens; ++t) acc[t] = __fadd_rn(acc[t], __fmul_rn(xr[t][i], wv));
    }
#pragma unroll
    for (int t = 0; t < kExactTokens; ++t) {
        float a = acc[t];
        a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, 4));  // a_j + a_{j+4}
        a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, 1));  // (a0+a4)+(a1+a5) | (a2+a6)+(a3+a7)
        a = __fadd_rn(a, __shfl_xor_sync(0xFFFFFFFFu, a, 2));
        float tail = 0.0f;
        for (uint32_t i = k8; i < cols; ++i) tail = __fadd_rn(tail, __fmul_rn(xr[t][i], weight_elem<WT>(row, i)));
        if (lane8 == 0 && n < rows && t0 + t < n_vec) {
            float* yr = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{t0 + t} * y_stride);
            yr[n] = gated_value(__fadd_rn(a, tail), n, gate_n_v, gate_dt_bias, gate_a);
        }
    }
}

template <uint32_t WT>
__global__ void __launch_bounds__(256) get_rows_kernel(const uint8_t* __restrict__ table, uint64_t table_stride,
                                                       const int32_t* __restrict__ ids, float* __restrict__ out,
                                                       uint64_t out_stride, uint32_t n_rows, uint32_t cols,
                                                       uint32_t* __restrict__ status) {
    const uint32_t i = blockIdx.y;
    int64_t id = ids != nullptr ? ids[i] : static_cast<int64_t>(i);
    if (id < 0 || id >= static_cast<int64_t>(n_rows)) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && status != nullptr) atomicOr(status, 8u);  // kStatusBadIndex
        return;
    }
    const uint8_t* row = table + static_cast<uint64_t>(id) * table_stride;
    float* o = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(out) + uint64_t{i} * out_stride);
    for (uint32_t e = blockIdx.x * blockDim.x + threadIdx.x; e < cols; e += gridDim.x * blockDim.x) o[e] = weight_elem<WT>(row, e);
}

// ---- argmax ---------------------------------------------------------------------------------------------------
// "Larger value first, then lower index" is a strict total order (backends/cpu/matmul.cpp:19-22), so any reduction
// tree returns the index a sequential scan returns.  NaN is never ordered: it only raises the vector's flag.
struct ArgPart {
    float value;
    uint32_t index;  // 0xFFFFFFFF = no candidate
    uint32_t nan;
    uint32_t pad;
};
constexpr uint32_t kNoIndex = 0xFFFFFFFFu;
constexpr int kArgmaxThreads = 256;
constexpr uint32_t kArgmaxChunk = 8192;  // logits per first-stage block

__device__ __forceinline__ bool ranks_before(float va, uint32_t ia, float vb, uint32_t ib) {
    if (ia == kNoIndex) return false;
    if (ib == kNoIndex) return true;
    return va > vb || (va == vb && ia < ib);
}

__device__ __forceinline__ void block_reduce_part(float& v, uint32_t& idx, uint32_t& nan) {
    __shared__ float sv[kArgmaxThreads / 32];
    __shared__ uint32_t si[kArgmaxThreads / 32], sn[kArgmaxThreads / 32];
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, off);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
        nan |= __shfl_xor_sync(0xFFFFFFFFu, nan, off);
        if (ranks_before(ov, oi, v, idx)) {
            v = ov;
            idx = oi;
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        sv[warp] = v;
        si[warp] = idx;
        sn[warp] = nan;
    }
    __syncthreads();
    if (warp == 0) {
        v = lane < kArgmaxThreads / 32 ? sv[lane] : 0.0f;
        idx = lane < kArgmaxThreads / 32 ? si[lane] : kNoIndex;
        nan = lane < kArgmaxThreads / 32 ? sn[lane] : 0u;
        for (int off = 4; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
            nan |= __shfl_xor_sync(0xFFFFFFFFu, nan, off);
            if (ranks_before(ov, oi, v, idx)) {
                v = ov;
                idx = oi;
            }
        }
    }
}

__global__ void __launch_bounds__(kArgmaxThreads) argmax_stage1(const float* __restrict__ logits, uint64_t stride, uint32_t n,
                                                                uint32_t limit, ArgPart* __restrict__ parts) {
    const uint32_t t = blockIdx.y;
    const float* row = logits + uint64_t{t} * stride;
    const uint32_t begin = blockIdx.x * kArgmaxChunk;
    const uint32_t end = min(n, begin + kArgmaxChunk);
    float v = 0.0f;
    uint32_t idx = kNoIndex, nan = 0;
    for (uint32_t c = begin + threadIdx.x; c < end; c += kArgmaxThreads) {
        const float f = row[c];
        if (f != f) {
            nan = 1;
        } else if (c < limit && ranks_before(f, c, v, idx)) {
            v = f;
            idx = c;
        }
    }
    block_reduce_part(v, idx, nan);
    if (threadIdx.x == 0) parts[uint64_t{t} * gridDim.x + blockIdx.x] = {v, idx, nan, 0u};
}

__global__ void __launch_bounds__(kArgmaxThreads) argmax_stage2(const ArgPart* __restrict__ parts, uint32_t n_parts, uint32_t row_offset,
                                                                uint32_t* __restrict__ result, int32_t* __restrict__ ids) {
    const uint32_t t = blockIdx.x;
    float v = 0.0f;
    uint32_t idx = kNoIndex, nan = 0;
    for (uint32_t p = threadIdx.x; p < n_parts; p += kArgmaxThreads) {
        const ArgPart a = parts[uint64_t{t} * n_parts + p];
        nan |= a.nan;
        if (ranks_before(a.value, a.index, v, idx)) {
            v = a.value;
            idx = a.index;
        }
    }
    block_reduce_part(v, idx, nan);
    if (threadIdx.x == 0) {
        // {index, value bits, nan}: a poisoned vector reports {-1, quiet NaN, 1} and the dense id 0
        // (src/backend/cpu_backend.cpp:751-758, 825-833).
        const bool poisoned = nan != 0;
        const uint32_t out_idx = poisoned || idx == kNoIndex ? kNoIndex : idx + row_offset;
        result[3 * t + 0] = out_idx;
        result[3 * t + 1] = poisoned ? 0x7FC00000u : __float_as_uint(v);
        result[3 * t + 2] = poisoned ? 1u : 0u;
        if (ids != nullptr) ids[t] = out_idx == kNoIndex ? 0 : static_cast<int32_t>(out_idx);
    }
}

template <uint32_t WT>
int launch_exact_t(const GemvCall& c, cudaStream_t s) {
    const dim3 grid((c.rows + kExactRowsPerBlock - 1) / kExactRowsPerBlock, (c.n_vec + kExactTokens - 1) / kExactTokens);
    gemv_exact8_kernel<WT><<<grid, 256, 0, s>>>(c.w, c.w_stride, c.x, c.x_stride, c.y, c.y_stride, c.rows, c.cols, c.n_vec, c.gate_dt_bias,
                                                c.gate_a, c.gate_n_v);
    HC_CUDA(cudaGetLastError());
    return 0;
}

template <uint32_t WT>
int launch_get_rows_t(const HaloCudaGetRows& a, uint64_t ts, uint64_t os, cudaStream_t s) {
    const uint32_t bx = min((a.cols + 255u) / 256u, 64u);
    get_rows_kernel<WT><<<dim3(bx, a.n_ids), 256, 0, s>>>(static_cast<const uint8_t*>(a.table), ts, a.ids, a.out, os, a.n_rows, a.cols,
                                                          a.status);
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

int launch_gemv_exact8(const GemvCall& c, cudaStream_t s) {
    if (c.n_vec > 65535u * kExactTokens) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: n_vec %u exceeds the launch limit", c.n_vec);
    switch (c.wtype) {
        case HALO_CUDA_T_F32: return launch_exact_t<HALO_CUDA_T_F32>(c, s);
        case HALO_CUDA_T_Q4_0: return launch_exact_t<HALO_CUDA_T_Q4_0>(c, s);
        case HALO_CUDA_T_Q8_0: return launch_exact_t<HALO_CUDA_T_Q8_0>(c, s);
        case HALO_CUDA_T_Q4_K: return launch_exact_t<HALO_CUDA_T_Q4_K>(c, s);
        case HALO_CUDA_T_Q6_K: return launch_exact_t<HALO_CUDA_T_Q6_K>(c, s);
        default: return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: weight type id %u", c.wtype);
    }
}

int launch_get_rows(const HaloCudaGetRows& a, uint64_t /*row_bytes*/, uint64_t ts, uint64_t os, cudaStream_t s) {
    if (a.n_ids > 65535u) return fail(HALO_CUDA_E_UNSUPPORTED, "GET_ROWS: n_ids %u exceeds the launch limit", a.n_ids);
    switch (a.type) {
        case HALO_CUDA_T_F32: return launch_get_rows_t<HALO_CUDA_T_F32>(a, ts, os, s);
        case HALO_CUDA_T_Q4_0: return launch_get_rows_t<HALO_CUDA_T_Q4_0>(a, ts, os, s);
        case HALO_CUDA_T_Q8_0: return launch_get_rows_t<HALO_CUDA_T_Q8_0>(a, ts, os, s);
        case HALO_CUDA_T_Q4_K: return launch_get_rows_t<HALO_CUDA_T_Q4_K>(a, ts, os, s);
        case HALO_CUDA_T_Q6_K: return launch_get_rows_t<HALO_CUDA_T_Q6_K>(a, ts, os, s);
        default: return fail(HALO_CUDA_E_UNSUPPORTED, "GET_ROWS: type id %u", a.type);
    }
}

uint64_t argmax_scratch_bytes(uint32_t n, uint32_t n_vec) {
    const uint64_t parts = (uint64_t{n} + kArgmaxChunk - 1) / kArgmaxChunk;
    return (parts == 0 ? 1 : parts) * n_vec * sizeof(ArgPart);
}

int launch_argmax(const float* logits, uint64_t stride_elems, uint32_t n, uint32_t n_vec, uint32_t valid, uint32_t row_offset,
                  uint32_t* result, int32_t* ids, void* scratch, cudaStream_t s) {
    if (n_vec > 65535u) return fail(HALO_CUDA_E_UNSUPPORTED, "LM_HEAD: n_vec %u exceeds the launch limit", n_vec);
    const uint32_t parts = (n + kArgmaxChunk - 1) / kArgmaxChunk;
    const uint32_t limit = valid > 0 && valid < n ? valid : n;
    ArgPart* p = static_cast<ArgPart*>(scratch);
    if (parts != 0) {
        argmax_stage1<<<dim3(parts, n_vec), kArgmaxThreads, 0, s>>>(logits, stride_elems, n, limit, p);
        HC_CUDA(cudaGetLastError());
    }
    argmax_stage2<<<n_vec, kArgmaxThreads, 0, s>>>(p, parts, row_offset, result, ids);
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace halo_cuda
