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
// Data movement.  Weights go HBM -> shared memory by bulk asynchronous copies (cp.async.bulk, the 1-D TMA path): each
// warp keeps a ring of stages, one super-block (144 B) of its 16 rows per stage, filled several steps ahead and
// tracked by one mbarrier per stage.  x is converted once per CTA into shared memory in MMA-fragment order (chunked
// over K when n_vec * cols is large), so the inner loop reads its B fragments with one conflict-free 16-byte load
// per sub-block.  Every mbarrier wait is bounded: on expiry the warp raises the context's error word and leaves.
//
// Roofline: HBM.  Algorithmic bytes = rows * row_bytes + 4 * n_vec * cols + 4 * n_vec * rows.
#include <cuda_fp16.h>

#include "internal.h"

namespace halo_cuda {

namespace {

constexpr int kRowBlocks = 8;         // 16-row blocks per CTA: a CTA covers 128 W rows
constexpr uint32_t kSmemBudget = 220 * 1024;

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

/// The first MMA of a chain: C = 0 comes from the zero register, no accumulator clearing needed.
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
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

// ---- shared-memory weight ring -------------------------------------------------------------------------------------
// Each warp streams its own rows: per pipeline stage, 16 bulk copies (cp.async.bulk, one 144-byte super-block per W
// row) land in a 16 x 160-byte slot and complete on that stage's mbarrier.  The 16-byte row padding makes the
// fragment reads below conflict-free.  Nothing but the owning warp touches a slot, so the only synchronisation is
// the mbarrier (data arrived) and program order (slot consumed before it is refilled).
constexpr uint32_t kSlotRow = 160, kSlotBytes = 16 * kSlotRow, kStageTx = 16 * 144;
constexpr uint32_t kWaitSpins = 1u << 20;  // try_wait polls (each blocks for a short hardware-defined time) before a stage is declared lost

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
/// Bounded wait: false after kWaitSpins polls (the caller then raises the error word and leaves).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitSpins; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory layout (byte offsets from the dynamic base), for `ncols` = 2 * tokens columns:
//   [0, 16) unused | scales | partial maxima | mbarriers | weight ring |
//   xs:  [sub-block][column][64 B] fp16 x in slot order    sx: [super-block][column][16 B] sub-block sums / 32
constexpr uint32_t kOffScale = 16, kOffInv = 16 + 64, kOffRed = 16 + 128, kOffBars = 256, kOffRing = 1024;

// NTOK: x rows of this launch (1..16), i.e. 2 * NTOK B columns in G = ceil(NTOK / 4) MMA column groups.
// KS: warps sharing one 16-row block; warp ks takes the super-blocks sb = ks (mod KS), a split that depends on
// nothing but KS, and the KS partial sums are added in ks order.  NS: ring stages per warp.
template <int NTOK, int KS, int NS>
__global__ void __launch_bounds__(kRowBlocks * KS * 32, 1)
gemv_mma_q4k_kernel(const uint8_t* __restrict__ w, uint64_t w_stride, const float* __restrict__ x, uint64_t x_stride,
                    float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t nb, uint32_t chunk_sb,
                    uint32_t* __restrict__ error_word) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    constexpr int G = (NTOK + 3) / 4;
    constexpr uint32_t kThreads = kRowBlocks * KS * 32;
    constexpr uint32_t kWarps = kRowBlocks * KS;
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
    // lanes 0..15 each own one W row of the block (clamped: rows past the end re-read the last row and are not stored)
    const uint8_t* next_src = w + uint64_t{min(rb * 16u + (lane & 15u), rows - 1)} * w_stride + ks * 144u;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    uint32_t fill_slot = 0, issued = 0;
    auto refill = [&]() {  // next super-block of this warp -> slot fill_slot
        if (lane == 0) mbar_expect_tx(bars + fill_slot * 8u, kStageTx);
        __syncwarp();
        if (lane < 16) bulk_g2s(ring + fill_slot * kSlotBytes + lane * kSlotRow, next_src, 144u, bars + fill_slot * 8u);
        next_src += KS * 144u;
        fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        ++issued;
    };
    for (uint32_t it = 0; it < NS && it < n_items; ++it) refill();

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
            // s = 2^(13 - floor(log2 a)) for a normal finite a, else 1; exponent clamped so that s and 1/s stay normal
            int e = static_cast<int>((__float_as_uint(a) >> 23) & 0xFFu) - 127;
            int se = (a > 0.0f && e < 128) ? 13 - e : 0;
            se = max(-100, min(100, se));
            s_scale[tk] = __uint_as_float(static_cast<uint32_t>(127 + se) << 23);
            s_inv[tk] = __uint_as_float(static_cast<uint32_t>(127 - se) << 23);
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
        // ---- stage x[:, chunk] as fp16 hi / lo in slot order, and the sub-block sums ------------------------------------------
        for (uint32_t tk = 0; tk < NTOK; ++tk) {
            const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tk} * x_stride) + c0 * 64u;
            const float s = s_scale[tk];
            for (uint32_t qd = tid; qd < n_sb * 64u; qd += kThreads) {
                float4 v = xr[qd];
                v.x *= s; v.y *= s; v.z *= s; v.w *= s;
                uint2 hi, lo;
                split4(v, hi, lo);
                const uint32_t sub = qd >> 3, in = qd & 7u;  // 8 quads per 32-element sub-block
                uint8_t* dst = smem + kOffData + sub * kSubStride + (2 * tk) * 64u + in * 8u;
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
                    uint8_t* sd = smem + kOffData + chunk_sb * 8u * kSubStride + (sub >> 3) * kSbStride + (2 * tk) * 16u + (sub & 7u) * 2u;
                    *reinterpret_cast<__half*>(sd) = h;
                    *reinterpret_cast<__half*>(sd + 16) = l;
                }
            }
        }
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

            float cq[G][4], cm[G][4];
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
                    if (j == 0) mma16816_first(cq[gi], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    else mma16816(cq[gi], aLo[0][0], aLo[1][0], aLo[0][1], aLo[1][1], bl.x, bl.y);
                    mma16816(cq[gi], aLo[0][2], aLo[1][2], aLo[0][3], aLo[1][3], bl.z, bl.w);
                    mma16816(cq[gi], aHi[0][0], aHi[1][0], aHi[0][1], aHi[1][1], bh.x, bh.y);
                    mma16816(cq[gi], aHi[0][2], aHi[1][2], aHi[0][3], aHi[1][3], bh.z, bh.w);
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
                yacc[gi][0] = fmaf(dq[0], cq[gi][0] + cq[gi][1], yacc[gi][0]);
                yacc[gi][0] = fmaf(-dmn[0], cm[gi][0] + cm[gi][1], yacc[gi][0]);
                yacc[gi][1] = fmaf(dq[1], cq[gi][2] + cq[gi][3], yacc[gi][1]);
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

template <int NTOK, int KS, int NS>
int launch_n(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, cudaStream_t s) {
    constexpr int G = (NTOK + 3) / 4;
    const uint32_t nb = c.cols / 256u;
    const Plan p = plan_for(nb, NTOK, kOffRing + kRowBlocks * KS * NS * kSlotBytes, (KS - 1) * kRowBlocks * 32 * 2 * G * 4);
    static bool attr_set = false;
    if (!attr_set) {
        HC_CUDA(cudaFuncSetAttribute(gemv_mma_q4k_kernel<NTOK, KS, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kSmemBudget)));
        attr_set = true;
    }
    const uint32_t grid = (c.rows + 16u * kRowBlocks - 1) / (16u * kRowBlocks);
    const float* x = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(c.x) + uint64_t{tok0} * c.x_stride);
    float* y = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(c.y) + uint64_t{tok0} * c.y_stride);
    gemv_mma_q4k_kernel<NTOK, KS, NS><<<grid, kRowBlocks * KS * 32, p.smem_bytes, s>>>(c.w, c.w_stride, x, c.x_stride, y, c.y_stride, c.rows,
                                                                                       nb, p.chunk_sb, ctx->error_word_dev);
    HC_CUDA(cudaGetLastError());
    return 0;
}

// The K split (2 warps per row block) and the ring depth are the same for every token count: the split is part
// of a row's arithmetic, and must not move with the batch size.
template <int NTOK>
int launch_tokens(HaloCudaCtx* ctx, const GemvCall& c, uint32_t tok0, uint32_t n, cudaStream_t s) {
    if constexpr (NTOK > 16) {
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: token tile of %u", n);
    } else {
        if (n == NTOK) return launch_n<NTOK, 2, 3>(ctx, c, tok0, s);
        return launch_tokens<NTOK + 1>(ctx, c, tok0, n, s);
    }
}

}  // namespace

bool gemv_mma_supports(const GemvCall& c) {
    if (c.wtype != HALO_CUDA_T_Q4_K || c.cols == 0) return false;
    if (reinterpret_cast<uintptr_t>(c.w) % 16 != 0 || c.w_stride % 16 != 0) return false;  // 16-byte header loads
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
