// gemv_mma_f16x2: tensor-core skinny kernel for decode-shaped Q4_K calls (M = 1 ... 16 and beyond in token tiles).
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
// Data movement.  Weights go HBM -> registers with 16- and 8-byte loads, one super-block (144 B) per row per step,
// the next step's loads in flight while the current one is unpacked.  x is converted once per CTA into shared
// memory in MMA-fragment order (chunked over K when n_vec * cols is large), so the inner loop reads its B fragments
// with one conflict-free 16-byte load per sub-block.
//
// Roofline: HBM.  Algorithmic bytes = rows * row_bytes + 4 * n_vec * cols + 4 * n_vec * rows.
#include <cuda_fp16.h>

#include "internal.h"

namespace halo_cuda {

namespace {

constexpr int kRowBlocks = 8;         // 16-row blocks per CTA: a CTA covers 128 W rows
constexpr uint32_t kSmemBudget = 200 * 1024;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_bits(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg64_stream(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

/// fp16 hi / lo split of four scaled activations, packed in MMA slot order (e0, e2 | e1, e3).
__device__ __forceinline__ void split4(float4 v, uint2& hi, uint2& lo) {
    const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y), h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
    const __half l0 = __float2half_rn(v.x - __half2float(h0)), l1 = __float2half_rn(v.y - __half2float(h1));
    const __half l2 = __float2half_rn(v.z - __half2float(h2)), l3 = __float2half_rn(v.w - __half2float(h3));
    hi.x = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h2)) << 16);
    hi.y = static_cast<uint32_t>(__half_as_ushort(h1)) | (static_cast<uint32_t>(__half_as_ushort(h3)) << 16);
    lo.x = static_cast<uint32_t>(__half_as_ushort(l0)) | (static_cast<uint32_t>(__half_as_ushort(l2)) << 16);
    lo.y = static_cast<uint32_t>(__half_as_ushort(l1)) | (static_cast<uint32_t>(__half_as_ushort(l3)) << 16);
}

struct Weights {  // one super-block of the warp's 16 rows, as this thread sees it
    uint4 hdr[2];   // row g / row g+8: d | dmin, scales[12]
    uint2 q[2][4];  // row, 64-element group: 8 bytes of qs
};

__device__ __forceinline__ void load_weights(Weights& w, const uint8_t* row0, const uint8_t* row1, uint32_t sb, uint32_t t) {
    const uint8_t* b0 = row0 + sb * 144u;
    const uint8_t* b1 = row1 + sb * 144u;
    w.hdr[0] = ldg128_stream(b0);
    w.hdr[1] = ldg128_stream(b1);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        w.q[0][j] = ldg64_stream(b0 + 16 + j * 32 + t * 8);
        w.q[1][j] = ldg64_stream(b1 + 16 + j * 32 + t * 8);
    }
}

// Shared-memory layout (byte offsets from the dynamic base), for `ncols` = 2 * tokens columns:
//   [0, 16)                        zeros (read by lanes whose column holds no token)
//   [16, 16 + 64)                  per-token scale s and 1/s (16 tokens x 2 floats... kept as two 64-byte arrays below)
//   xs:  [sub-block][column][64 B] fp16 x in slot order    sx: [super-block][column][16 B] sub-block sums / 32
constexpr uint32_t kOffZero = 0, kOffScale = 16, kOffInv = 16 + 64, kOffRed = 16 + 128, kOffData = 16 + 128 + 64;

// G: MMA column groups (4 tokens each).  KS: warps sharing one 16-row block; warp ks takes the super-blocks
// sb = ks (mod KS), a split that depends on nothing but KS, and the KS partial sums are added in ks order.
template <int G, int KS>
__global__ void __launch_bounds__(kRowBlocks * KS * 32, 1)
gemv_mma_q4k_kernel(const uint8_t* __restrict__ w, uint64_t w_stride, const float* __restrict__ x, uint64_t x_stride,
                    float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t nb, uint32_t n_vec, uint32_t chunk_sb) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    constexpr uint32_t kThreads = kRowBlocks * KS * 32;
    constexpr uint32_t kWarps = kRowBlocks * KS;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t rbl = warp % kRowBlocks, ks = warp / kRowBlocks;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t ncols = 2 * n_vec;  // n_vec <= 4 * G here
    const uint32_t cols = nb * 256u;

    // ---- this warp's rows, and the first super-block's loads in flight before anything else ----------------------
    const uint32_t rb = blockIdx.x * kRowBlocks + rbl;
    const bool active = rb * 16u < rows;
    const uint32_t r0 = min(rb * 16u + g, rows - 1), r1 = min(rb * 16u + 8u + g, rows - 1);
    const uint8_t* row0 = w + uint64_t{r0} * w_stride;
    const uint8_t* row1 = w + uint64_t{r1} * w_stride;
    Weights cur, nxt;
    if (active && ks < nb) load_weights(cur, row0, row1, ks, t);

    // ---- per-token power-of-two scale from the row's largest magnitude ------------------------------------------------
    float* s_scale = reinterpret_cast<float*>(smem + kOffScale);
    float* s_inv = reinterpret_cast<float*>(smem + kOffInv);
    float* s_red = reinterpret_cast<float*>(smem + kOffRed);  // kWarps partial maxima
    if (tid < 4) reinterpret_cast<uint32_t*>(smem + kOffZero)[tid] = 0u;
    for (uint32_t tk = 0; tk < n_vec; ++tk) {
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
            // s = 2^(13 - floor(log2 a)) for a normal finite a, else 1; exponent clamped so that s and 1/s stay normal
            int e = static_cast<int>((__float_as_uint(a) >> 23) & 0xFFu) - 127;
            int se = (a > 0.0f && e < 128) ? 13 - e : 0;
            se = max(-100, min(100, se));
            s_scale[tk] = __uint_as_float(static_cast<uint32_t>(127 + se) << 23);
            s_inv[tk] = __uint_as_float(static_cast<uint32_t>(127 - se) << 23);
        }
        __syncthreads();
    }

    // ---- fragment addresses: lanes whose column carries no token read the zero word forever ------------------------------
    uint32_t xs_addr[G], xs_step[G], sx_addr[G], sx_step[G];
    const uint32_t xs_base = smem_base + kOffData;
    const uint32_t sx_base = xs_base + chunk_sb * 8u * ncols * 64u;
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t col = 8u * gi + g;
        const bool valid = col < ncols;
        xs_addr[gi] = valid ? xs_base + col * 64u + t * 16u : smem_base + kOffZero;
        xs_step[gi] = valid ? ncols * 64u : 0u;   // per sub-block
        sx_addr[gi] = valid ? sx_base + col * 16u + t * 4u : smem_base + kOffZero;
        sx_step[gi] = valid ? ncols * 16u : 0u;   // per super-block
    }

    // thread-constant selectors for the 6-bit codes (see the SWAR unpack below)
    const uint32_t m_sel = (2 * t) | ((2 * t) << 4) | ((2 * t + 1) << 8) | ((2 * t + 1) << 12);

    float yacc[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) yacc[gi][0] = yacc[gi][1] = 0.0f;

    for (uint32_t c0 = 0; c0 < nb; c0 += chunk_sb) {
        const uint32_t n_sb = min(chunk_sb, nb - c0);
        if (c0 != 0) __syncthreads();  // everyone is done reading the previous chunk
        // ---- stage x[:, chunk] as fp16 hi / lo in slot order, and the sub-block sums ------------------------------------------
        for (uint32_t tk = 0; tk < n_vec; ++tk) {
            const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride) + c0 * 64u;
            const float s = s_scale[tk];
            for (uint32_t qd = tid; qd < n_sb * 64u; qd += kThreads) {
                float4 v = xr[qd];
                v.x *= s; v.y *= s; v.z *= s; v.w *= s;
                uint2 hi, lo;
                split4(v, hi, lo);
                const uint32_t sub = qd >> 3, in = qd & 7u;  // 8 quads per 32-element sub-block
                uint8_t* dst = smem + kOffData + (sub * ncols + 2 * tk) * 64u + in * 8u;
                *reinterpret_cast<uint2*>(dst) = hi;
                *reinterpret_cast<uint2*>(dst + 64) = lo;
                float sum = (v.x + v.y) + (v.z + v.w);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
                sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
                if (in == 0) {
                    sum *= 0.03125f;  // keeps the fp16 copy in range: |sum| <= 32 * 2^14
                    const __half h = __float2half_rn(sum);
                    const __half l = __float2half_rn(sum - __half2float(h));
                    uint8_t* sd = smem + kOffData + chunk_sb * 8u * ncols * 64u + ((sub >> 3) * ncols + 2 * tk) * 16u + (sub & 7u) * 2u;
                    *reinterpret_cast<__half*>(sd) = h;
                    *reinterpret_cast<__half*>(sd + 16) = l;
                }
            }
        }
        __syncthreads();
        if (!active) continue;

        for (uint32_t sb = c0 + (ks + KS - c0 % KS) % KS; sb < c0 + n_sb; sb += KS) {
            const uint32_t i = sb - c0;
            if (sb + KS < nb) load_weights(nxt, row0, row1, sb + KS, t);

            // ---- 6-bit codes of both rows, four per word (SWAR form of src/tensor/quant.cpp:236-244) -------------------------
            uint32_t sc_lo[2], sc_hi[2], mpair[2];
            float dq[2], dmn[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint4 h = cur.hdr[r];
                sc_lo[r] = h.y & 0x3F3F3F3Fu;                                       // sc0..sc3
                sc_hi[r] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);        // sc4..sc7
                const uint32_t m_lo = h.z & 0x3F3F3F3Fu;                            // m0..m3
                const uint32_t m_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);  // m4..m7
                mpair[r] = prmt(m_lo, m_hi, m_sel) & 0x00FF00FFu;                   // (m_2t, m_2t+1) as fp16 subnormals
                const __half2 dd = *reinterpret_cast<const __half2*>(&h.x);
                dq[r] = __low2float(dd) * 16777216.0f;           // d * 2^24: undoes the subnormal encoding of A
                dmn[r] = __high2float(dd) * (16777216.0f * 32.0f);  // dmin * 2^24 * 32: and the /32 of the sums
            }

            float cq[G][4], cm[G][4];
#pragma unroll
            for (int gi = 0; gi < G; ++gi)
#pragma unroll
                for (int k = 0; k < 4; ++k) cq[gi][k] = cm[gi][k] = 0.0f;

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
                    const uint32_t qa = cur.q[r][j].x, qb = cur.q[r][j].y;
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
                    const uint32_t sub = i * 8u + 2u * j;
                    const uint4 bl = lds128(xs_addr[gi] + sub * xs_step[gi]);
                    const uint4 bh = lds128(xs_addr[gi] + (sub + 1u) * xs_step[gi]);
                    mma16816(cq[gi], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    mma16816(cq[gi], aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                    mma16816(cq[gi], aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                    mma16816(cq[gi], aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
                }
            }
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const uint32_t bs = lds32(sx_addr[gi] + i * sx_step[gi]);
                mma16816(cm[gi], mpair[0], mpair[1], 0u, 0u, bs, 0u);
                yacc[gi][0] = fmaf(dq[0], cq[gi][0] + cq[gi][1], yacc[gi][0]);
                yacc[gi][0] = fmaf(-dmn[0], cm[gi][0] + cm[gi][1], yacc[gi][0]);
                yacc[gi][1] = fmaf(dq[1], cq[gi][2] + cq[gi][3], yacc[gi][1]);
                yacc[gi][1] = fmaf(-dmn[1], cm[gi][2] + cm[gi][3], yacc[gi][1]);
            }
            cur = nxt;
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
    if (!active) return;
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t tk = 4u * gi + t;
        if (tk < n_vec) {
            const float inv = s_inv[tk];
            float* yr = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{tk} * y_stride);
            const uint32_t n0 = rb * 16u + g, n1 = n0 + 8u;
            if (n0 < rows) yr[n0] = yacc[gi][0] * inv;
            if (n1 < rows) yr[n1] = yacc[gi][1] * inv;
        }
    }
}

struct Plan {
    uint32_t chunk_sb;
    uint32_t smem_bytes;
};

Plan plan_for(uint32_t nb, uint32_t n_tok, uint32_t reduce_bytes) {
    const uint32_t ncols = 2 * n_tok;
    const uint32_t per_sb = 8u * ncols * 64u + ncols * 16u;
    uint32_t chunk = (kSmemBudget - kOffData) / per_sb;
    if (chunk > nb) chunk = nb;
    if (chunk == 0) chunk = 1;
    const uint32_t data = chunk * per_sb;  // the K-split reduction reuses this area
    return {chunk, kOffData + (data > reduce_bytes ? data : reduce_bytes)};
}

template <int G, int KS>
int launch_g(const GemvCall& c, uint32_t tok0, uint32_t n_tok, cudaStream_t s) {
    const uint32_t nb = c.cols / 256u;
    const Plan p = plan_for(nb, n_tok, (KS - 1) * kRowBlocks * 32 * 2 * G * 4);
    static bool attr_set = false;
    if (!attr_set) {
        HC_CUDA(cudaFuncSetAttribute(gemv_mma_q4k_kernel<G, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBudget)));
        attr_set = true;
    }
    const uint32_t grid = (c.rows + 16u * kRowBlocks - 1) / (16u * kRowBlocks);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    gemv_mma_q4k_kernel<G, KS><<<grid, kRowBlocks * KS * 32, p.smem_bytes, s>>>(c.w, c.w_stride, x, c.x_stride, y, c.y_stride, c.rows, nb, n_tok, p.chunk_sb);
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace

bool gemv_mma_supports(const GemvCall& c) {
    if (c.wtype != HALO_CUDA_T_Q4_K || c.cols == 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // 16-byte header loads
    if (reinterpret_cast<uintptr_t>(c.x) % 16 != 0 || c.x_stride % 16 != 0) return false;  // float4 reads of x
    return true;
}

int launch_gemv_mma(HaloCudaCtx* /*ctx*/, const GemvCall& c, cudaStream_t s) {
    // Token tiles of 16 (four MMA column groups); the remainder takes the smallest instantiation that holds it.
    for (uint32_t t0 = 0; t0 < c.n_vec; t0 += 16) {
        const uint32_t n = c.n_vec - t0 < 16 ? c.n_vec - t0 : 16;
        int rc;
        // The K split (2 warps per row block) is the same for every token count: it is part of a row's arithmetic.
        if (n <= 4) rc = launch_g<1, 2>(c, t0, n, s);
        else if (n <= 8) rc = launch_g<2, 2>(c, t0, n, s);
        else if (n <= 12) rc = launch_g<3, 2>(c, t0, n, s);
        else rc = launch_g<4, 2>(c, t0, n, s);
        if (rc != 0) return rc;
    }
    return 0;
}

}  // namespace halo_cuda
