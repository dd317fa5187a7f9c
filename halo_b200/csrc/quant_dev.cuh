// Device-side readers of the GGUF block formats.  Every float expression keeps the evaluation order of the
// reference's scalar dequantizers (src/tensor/quant.cpp), with products and sums rounded separately
// (__fmul_rn / __fsub_rn are never contracted into an FMA), so the unpacked values are bit-identical.
#pragma once
#include <cuda_fp16.h>

#include <cstdint>

#include "halo_cuda.h"

namespace halo_cuda {

__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half(static_cast<unsigned short>(h))); }

/// fp16 field at any byte address (blocks are packed: Q6_K's d sits at byte 208 of 210).
__device__ __forceinline__ float f16_at(const uint8_t* p) {
    return f16_bits_to_f32(static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8));
}

/// The 6-bit (scale, min) codes of Q4_K sub-block j from the 12 packed bytes (src/tensor/quant.cpp:236-244).
__device__ __forceinline__ void q4k_codes(int j, const uint8_t* s, uint32_t& sc, uint32_t& mn) {
    if (j < 4) {
        sc = s[j] & 63u;
        mn = s[j + 4] & 63u;
    } else {
        sc = (s[j + 4] & 0x0Fu) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/// Element `e` (0..255) of one Q4_K super-block: (d*sc)*q - dmin*m (src/tensor/quant.cpp:247-269).
__device__ __forceinline__ float q4k_elem(const uint8_t* blk, int e) {
    const int sub = e >> 5, l = e & 31;
    uint32_t sc, mn;
    q4k_codes(sub, blk + 4, sc, mn);
    const float d1 = __fmul_rn(f16_at(blk), static_cast<float>(sc));
    const float m1 = __fmul_rn(f16_at(blk + 2), static_cast<float>(mn));
    const uint32_t byte = blk[16 + (sub >> 1) * 32 + l];
    const uint32_t q = (sub & 1) ? (byte >> 4) : (byte & 0x0Fu);
    return __fsub_rn(__fmul_rn(d1, static_cast<float>(q)), m1);
}

/// Element `e` (0..255) of one Q6_K super-block: (d*scale)*(q-32) (src/tensor/quant.cpp:302-327).
__device__ __forceinline__ float q6k_elem(const uint8_t* blk, int e) {
    const int half = e >> 7, r = e & 127, quarter = r >> 5, l = r & 31;
    const uint8_t* ql = blk + half * 64;
    const uint8_t* qh = blk + 128 + half * 32;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + half * 8);
    const uint32_t lo = ql[l + ((quarter & 1) ? 32 : 0)];
    const uint32_t nib = (quarter & 2) ? (lo >> 4) : (lo & 0x0Fu);
    const int q = static_cast<int>(nib | (((qh[l] >> (2 * quarter)) & 3u) << 4)) - 32;
    const float ds = __fmul_rn(f16_at(blk + 208), static_cast<float>(sc[(l >> 4) + 2 * quarter]));
    return __fmul_rn(ds, static_cast<float>(q));
}

/// Element `e` (0..31) of one Q8_0 block: q*d (src/tensor/quant.cpp:143-151).
__device__ __forceinline__ float q80_elem(const uint8_t* blk, int e) {
    return __fmul_rn(static_cast<float>(static_cast<int8_t>(blk[2 + e])), f16_at(blk));
}

/// Element `e` (0..31) of one Q4_0 block: (q-8)*d, low nibbles first (src/tensor/quant.cpp:79-90).
__device__ __forceinline__ float q40_elem(const uint8_t* blk, int e) {
    const uint32_t byte = blk[2 + (e & 15)];
    const int q = static_cast<int>((e & 16) ? (byte >> 4) : (byte & 0x0Fu)) - 8;
    return __fmul_rn(static_cast<float>(q), f16_at(blk));
}

/// Element i of a weight row of type WT, exactly as tensor::dequantize_row produces it.
template <uint32_t WT>
__device__ __forceinline__ float weight_elem(const uint8_t* row, uint32_t i) {
    if constexpr (WT == HALO_CUDA_T_F32) {
        return reinterpret_cast<const float*>(row)[i];
    } else if constexpr (WT == HALO_CUDA_T_Q4_K) {
        return q4k_elem(row + (i >> 8) * 144u, i & 255);
    } else if constexpr (WT == HALO_CUDA_T_Q6_K) {
        return q6k_elem(row + (i >> 8) * 210u, i & 255);
    } else if constexpr (WT == HALO_CUDA_T_Q8_0) {
        return q80_elem(row + (i >> 5) * 34u, i & 31);
    } else {
        return q40_elem(row + (i >> 5) * 18u, i & 31);
    }
}

}  // namespace halo_cuda
