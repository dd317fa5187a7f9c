// The int8 tensor-core skinny kernels (variants gemv_mma_i8x2 over raw Q4_K rows and gemv_mma_i8x2_r over repacked Q6_K / Q8_0 /
// Q4_0 rows): x travels as two signed 8-bit digits per element, the quant codes go into the MMA as bytes, and every sum up to
// the per-group scale is an exact integer.  The Q4_K arithmetic is spelled out here; the other formats say theirs at their structs.
//
// x is quantised per super-block (256 elements, what one warp converts at a time): s = the power of two that puts the
// super-block's largest magnitude in (2^14, 32639], xq = rint(x * s) = 256 * hi + lo with hi, lo in [-128, 127].  The
// error of the product is therefore |x * s - xq| <= 1/2 per element, i.e. at most 2^-15 of the super-block's largest
// magnitude; everything behind it is exact until the fp32 epilogue:
//     S_s  = sum over the 32 elements of sub-block s of q * xq                      (int32, mma.sync m16n8k32 u8 x s8)
//     A_p  = sc_p * S_p + sc_{4+p} * S_{4+p},   M_p = m_p * X_p + m_{4+p} * X_{4+p}    (int32; X_s = sum of xq over sub-block s)
//     u_p  = fma(-dmin, float(M_p), d * float(A_p))                                  p = 0 .. 3
//     P_p  = fma(1 / s, u_p, P_p)                                                    over the super-blocks of the walk, in order
//     y    = (P_0 + P_1) + (P_2 + P_3),  then the K slices and the CTAs' partials as in the other balanced kernels.
// That order is the same for every batch size, so a row's bits do not depend on how many rows share the call
// (include/halo/backend/backend.h:300-304).  A call with ONE x row gets it with a quarter of the MMA work per sub-block:
// x sits in the column pair (2p, 2p + 1) of B for the sub-blocks s = p (mod 4) (hi digit, lo digit; the other columns
// read zeros), so one accumulator tile carries four sub-blocks and lane t of a row finishes P_t; two shuffles add them.
//
// The per-warp TMA weight ring and the cross-CTA reduction are those of gemv_mma_sk.cuh; the partition (1 to 16 in-CTA K slices,
// a launch parameter) is plan_partition_i8 of mma_common.cuh.
#pragma once
#include <cuda.h>

#include <algorithm>

#include "gemv_mma_sk.cuh"

namespace halo_cuda {
namespace i8 {

using namespace mma;

__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
/// The first MMA of a chain: C = 0 comes from the zero register.
__device__ __forceinline__ void imma0(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Two fp32 operations in one instruction (rows g and g + 8 of a lane's sums share every step of the epilogue): each half is
// the IEEE operation of the scalar form, so the bits are those of __fmaf_rn / __fmul_rn.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// x records of NTOK rows, per super-block:
//   digits  [sub-block 0..7][column 0..2 * NTOK - 1][32 B]   column 2 * tok = hi digits, 2 * tok + 1 = lo digits of row tok;
//                                                            byte i of a column = element i of the sub-block
//                                                            (formats whose weight words hold elements 4t .. 4t+3 and 16+4t .. of a
//                                                            32-element block keep a column PERMUTED: element e at byte
//                                                            8 * ((e % 16) / 4) + 4 * (e / 16) + e % 4, so that a lane's two B
//                                                            registers are one 8-byte load)
//   meta    [row][48 B]                                      int32 pairs (X_p, X_{4+p}) for p = 0..3 (sums of xq over 32 elements: what
//                                                            Q4_K's mins multiply), 1 / s as fp32 at byte 32
// The digit area and the meta area are separate arrays (all super-blocks of one, then all of the other), in shared
// memory as in the scratch the conversion kernel (stage_x_i8_kernel) fills.
constexpr uint32_t kDigitBytes = 512, kMetaBytes = 48;
__host__ __device__ inline constexpr uint32_t rec_bytes(uint32_t n_tok) { return (kDigitBytes + kMetaBytes) * n_tok; }
inline uint64_t stage_scratch_bytes(uint32_t nb, uint32_t n_tok) { return uint64_t{nb} * rec_bytes(n_tok); }

/// One super-block (index sb) of x row `tok` into the records at `digits` / `meta`, by one warp: lane l holds elements
/// 8 l .. 8 l + 7 in (v0, v1).  A super-block with a NaN or an infinity gets 1 / s = NaN, which poisons exactly the sums it
/// enters (the reference's per-row NaN, src/backend/backend.cpp:91-96).
__device__ __forceinline__ void stage_superblock(uint8_t* digits, uint8_t* meta, float4 v0, float4 v1, uint32_t sb, uint32_t n_tok, uint32_t tok,
                                                 uint32_t lane, bool perm = false) {
    float m = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                    fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    const bool finite = m < __int_as_float(0x7F800000);  // false for NaN too (fmaxf drops NaNs: checked per element below)
    const int e = static_cast<int>((__float_as_uint(m) >> 23) & 0xFFu) - 127;
    int se = (m > 0.0f && finite) ? 14 - e : 0;
    se = max(-100, min(100, se));
    float s = __uint_as_float(static_cast<uint32_t>(127 + se) << 23);
    if (m * s > 32639.0f) se -= 1, s = __uint_as_float(static_cast<uint32_t>(127 + se) << 23);
    // |f * s| <= 32639 for every element by the choice of s (a power of two: the product is exact), so the conversion needs no
    // clamp.  A super-block with an infinity is multiplied by 0 instead: inf * 0 and NaN * anything are NaN, which converts to 0.
    const float mul = finite ? s : 0.0f;
    const float f[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    int q[8], h[8], sum = 0;
    bool bad = !finite;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        bad |= f[i] != f[i];
        q[i] = __float2int_rn(f[i] * mul);
        h[i] = (q[i] + 128) >> 8;
        sum += q[i];
    }
    bad = __any_sync(0xFFFFFFFFu, bad);
    // hi digits h; lo digits q - 256 h are the low bytes of q (two's complement)
    uint2 hi, lo;
    hi.x = prmt(prmt(h[0], h[1], 0x0040), prmt(h[2], h[3], 0x0040), 0x5410);
    hi.y = prmt(prmt(h[4], h[5], 0x0040), prmt(h[6], h[7], 0x0040), 0x5410);
    lo.x = prmt(prmt(q[0], q[1], 0x0040), prmt(q[2], q[3], 0x0040), 0x5410);
    lo.y = prmt(prmt(q[4], q[5], 0x0040), prmt(q[6], q[7], 0x0040), 0x5410);
    const uint32_t sub = lane >> 2, pos = (lane & 3u) * 8u;
    uint8_t* d = digits + uint64_t{sb} * (kDigitBytes * n_tok) + sub * (64u * n_tok) + tok * 64u;
    if (!perm) {
        *reinterpret_cast<uint2*>(d + pos) = hi;
        *reinterpret_cast<uint2*>(d + pos + 32) = lo;
    } else {  // elements 8 (l & 3) .. + 3 and .. + 4 .. + 7: k-step half (l & 3) >> 1, threads 2 (l & 1) and 2 (l & 1) + 1
        const uint32_t at = 16u * (lane & 1u) + 4u * ((lane & 3u) >> 1);
        *reinterpret_cast<uint32_t*>(d + at) = hi.x;
        *reinterpret_cast<uint32_t*>(d + at + 8) = hi.y;
        *reinterpret_cast<uint32_t*>(d + at + 32) = lo.x;
        *reinterpret_cast<uint32_t*>(d + at + 40) = lo.y;
    }
    uint8_t* mt = meta + uint64_t{sb} * (kMetaBytes * n_tok) + tok * kMetaBytes;
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if ((lane & 3u) == 0) reinterpret_cast<int*>(mt)[(sub & 3u) * 2u + (sub >> 2)] = sum;
    if (lane == 0) reinterpret_cast<float*>(mt)[8] = bad ? __int_as_float(0x7FC00000) : __uint_as_float(static_cast<uint32_t>(127 - se) << 23);
}

/// grid (x rows, blocks of 16 super-blocks): every warp converts one super-block of one row into the scratch records.  The `total`
/// rows are those of consecutive token tiles of `tile_rows` rows (the last one may be shorter); tile i's records start at
/// scratch + i * nb * rec_bytes(tile_rows) and are laid out for that tile's own row count.
static __global__ void __launch_bounds__(512) stage_x_i8_kernel(const float* __restrict__ x, uint64_t x_stride, uint8_t* __restrict__ scratch, uint32_t nb,
                                                                uint32_t tile_rows, uint32_t total, uint32_t perm) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t row = blockIdx.x, sb = blockIdx.y * 16u + (threadIdx.x >> 5);
    if (sb >= nb) return;
    const uint32_t tile = row / tile_rows, tok = row - tile * tile_rows, n_tok = min(tile_rows, total - tile * tile_rows);
    uint8_t* region = scratch + uint64_t{tile} * nb * rec_bytes(tile_rows);
    const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{row} * x_stride);
    const uint32_t lane = threadIdx.x & 31u;
    stage_superblock(region, region + uint64_t{nb} * kDigitBytes * n_tok, xr[sb * 64u + 2u * lane], xr[sb * 64u + 2u * lane + 1u], sb, n_tok, tok, lane, perm != 0);
}

// ---- Q4_K: raw GGUF super-blocks (144 B), fetched as 160-byte slot rows (the extra 16 bytes keep the fragment reads conflict-free)
struct Q4Ki {
    // (144-byte slot rows with permuted tile rows, as the repacked formats below have them, measured the same for one x row and 2 - 4 %
    // slower for batches)
    static constexpr uint32_t kType = HALO_CUDA_T_Q4_K, kPitch = 160, kItemCoord = 144, kBoxInner = 160, kMapElemBytes = 1;
    static constexpr bool kPermX = false;
    static constexpr int kMaxTok = 16;  // x rows per launch (four MMA column groups); larger batches, or records that do not fit, run in tiles
    static constexpr uint32_t kStretchMax = 8;  // columns per stretch of streamed x
    static constexpr bool kPipedConversion = false;
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return g; }

    /// Lane constants of the single-row form.
    struct One {
        const uint8_t* bp[4];  // B base per sub-block phase: this lane's digits, or zeros
        uint32_t bstep[4];     // bytes per super-block of that base (0 for the zeros)
        uint32_t sel, sh;      // byte selector of this lane's scale codes; 4 where its sub-blocks come from the high nibbles
    };
    __device__ static __forceinline__ One make_one(const uint8_t* digits, const uint8_t* zeros, uint32_t g, uint32_t t) {
        One o;
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {
            const bool real = (g >> 1) == static_cast<uint32_t>(ph);
            o.bp[ph] = real ? digits + (g & 1u) * 32u + t * 8u : zeros + t * 8u;
            o.bstep[ph] = real ? kDigitBytes : 0u;
        }
        o.sel = t | 0x4440u;
        o.sh = (t & 1u) * 4u;
        return o;
    }

    /// One row's share of the epilogue: the 6-bit codes of sub-blocks t and 4 + t (src/tensor/quant.cpp:236-244), the integer
    /// sums, the fp32 step.  S0 / S1: the sub-block sums (already without the high-nibble factor), X: (X_t, X_{4+t}).
    __device__ static __forceinline__ float finish_pair(const uint4 h, uint32_t sel, int S0, int S1, int2 X) {
        const uint32_t by = prmt(h.y, 0u, sel), bz = prmt(h.z, 0u, sel), bw = prmt(h.w, 0u, sel);
        const int sc0 = by & 63u, m0 = bz & 63u;
        const int sc1 = (bw & 15u) | ((by >> 2) & 0x30u), m1 = (bw >> 4) | ((bz >> 2) & 0x30u);
        const int A = sc0 * S0 + sc1 * S1, M = m0 * X.x + m1 * X.y;
        const __half2 dh = *reinterpret_cast<const __half2*>(&h.x);
        return __fmaf_rn(-__high2float(dh), __int2float_rn(M), __fmul_rn(__low2float(dh), __int2float_rn(A)));
    }

    /// A single x row: P[0], P[1] are this lane's P_t of rows g and g + 8.
    template <class Release>
    __device__ static __forceinline__ void item_one(const uint8_t* r0, uint32_t t, const One& o, uint32_t rec, const uint8_t* meta, float (&P)[2],
                                                    Release&& release) {
        const uint8_t* r1 = r0 + 8 * kPitch;
        const uint4 h0 = *reinterpret_cast<const uint4*>(r0), h1 = *reinterpret_cast<const uint4*>(r1);
        const uint8_t* bq[4];
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) bq[ph] = o.bp[ph] + rec * o.bstep[ph];
        int c[2][4];  // tile h: sub-blocks 4h .. 4h + 3, one per column pair
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint2 q0 = *reinterpret_cast<const uint2*>(r0 + 16 + 32 * j + 8 * t);
            const uint2 q1 = *reinterpret_cast<const uint2*>(r1 + 16 + 32 * j + 8 * t);
            const uint2 bl = *reinterpret_cast<const uint2*>(bq[(2 * j) & 3] + (2 * j) * 64);
            const uint2 bh = *reinterpret_cast<const uint2*>(bq[(2 * j + 1) & 3] + (2 * j + 1) * 64);
            if ((j & 1) == 0) imma0(c[j >> 1], q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, bl.x, bl.y);
            else imma(c[j >> 1], q0.x & 0x0F0F0F0Fu, q1.x & 0x0F0F0F0Fu, q0.y & 0x0F0F0F0Fu, q1.y & 0x0F0F0F0Fu, bl.x, bl.y);
            // the high nibbles stay in place: 16 q as an unsigned byte, the factor leaves the sum by an exact shift
            imma(c[j >> 1], q0.x & 0xF0F0F0F0u, q1.x & 0xF0F0F0F0u, q0.y & 0xF0F0F0F0u, q1.y & 0xF0F0F0F0u, bh.x, bh.y);
        }
        release();  // every byte of the slot has been consumed
        const uint8_t* mt = meta + rec * kMetaBytes;
        const int2 X = *reinterpret_cast<const int2*>(mt + t * 8u);
        const float inv = *reinterpret_cast<const float*>(mt + 32);
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const int S0 = (c[0][2 * rr] * 256 + c[0][2 * rr + 1]) >> o.sh, S1 = (c[1][2 * rr] * 256 + c[1][2 * rr + 1]) >> o.sh;
            P[rr] = __fmaf_rn(inv, finish_pair(rr ? h1 : h0, o.sel, S0, S1, X), P[rr]);
        }
    }

    /// 2 .. 16 x rows: P[gi][rr][p] of rows g, g + 8 and x row 4 gi + t.
    template <int G, int NTOK, class Release>
    __device__ static __forceinline__ void item_many(const uint8_t* r0, uint32_t t, uint32_t g, const uint8_t* dig, const uint8_t* meta, float (&P)[G][2][4],
                                                     Release&& release) {
        constexpr uint32_t kSub = 64u * NTOK;
        const uint8_t* r1 = r0 + 8 * kPitch;
        const uint4 hh[2] = {*reinterpret_cast<const uint4*>(r0), *reinterpret_cast<const uint4*>(r1)};
        uint32_t boff[G], moff[G];
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            boff[gi] = min(8u * gi + g, 2u * NTOK - 1u) * 32u + t * 8u;
            moff[gi] = min(4u * gi + t, static_cast<uint32_t>(NTOK - 1)) * kMetaBytes;
        }
        // the 6-bit codes of both rows, four per word: [0] sub-blocks 0..3, [1] sub-blocks 4..7
        uint32_t sc[2][2], mn[2][2];
        float dq[2], dmn[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const uint4 h = hh[rr];
            sc[rr][0] = h.y & 0x3F3F3F3Fu;
            sc[rr][1] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
            mn[rr][0] = h.z & 0x3F3F3F3Fu;
            mn[rr][1] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
            const __half2 dh = *reinterpret_cast<const __half2*>(&h.x);
            dq[rr] = __low2float(dh), dmn[rr] = __high2float(dh);
        }
        auto code = [](uint32_t word, int idx) { return static_cast<int>((word >> (8 * idx)) & 0xFFu); };
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {  // phases p = 2 jj, 2 jj + 1: sub-blocks p, p + 4 (chunks jj and jj + 2)
            int A[G][2][2];
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int j = jj + 2 * half;
                const uint2 q0 = *reinterpret_cast<const uint2*>(r0 + 16 + 32 * j + 8 * t);
                const uint2 q1 = *reinterpret_cast<const uint2*>(r1 + 16 + 32 * j + 8 * t);
                const uint32_t l0 = q0.x & 0x0F0F0F0Fu, l1 = q1.x & 0x0F0F0F0Fu, l2 = q0.y & 0x0F0F0F0Fu, l3 = q1.y & 0x0F0F0F0Fu;
                const uint32_t u0 = q0.x & 0xF0F0F0F0u, u1 = q1.x & 0xF0F0F0F0u, u2 = q0.y & 0xF0F0F0F0u, u3 = q1.y & 0xF0F0F0F0u;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const uint2 bl = *reinterpret_cast<const uint2*>(dig + (2 * j) * kSub + boff[gi]);
                    const uint2 bh = *reinterpret_cast<const uint2*>(dig + (2 * j + 1) * kSub + boff[gi]);
                    int cl[4], ch[4];
                    imma0(cl, l0, l1, l2, l3, bl.x, bl.y);
                    imma0(ch, u0, u1, u2, u3, bh.x, bh.y);
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) {
                        const int Sl = cl[2 * rr] * 256 + cl[2 * rr + 1], Sh = (ch[2 * rr] * 256 + ch[2 * rr + 1]) >> 4;
                        const int wl = code(sc[rr][half], 2 * jj), wh = code(sc[rr][half], 2 * jj + 1);
                        if (half == 0) A[gi][rr][0] = wl * Sl, A[gi][rr][1] = wh * Sh;
                        else A[gi][rr][0] += wl * Sl, A[gi][rr][1] += wh * Sh;
                    }
                }
            }
            if (jj == 1) release();
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const int4 X = *reinterpret_cast<const int4*>(meta + moff[gi] + jj * 16);  // (X_p, X_{4+p}, X_{p+1}, X_{5+p}), p = 2 jj
                const float inv = *reinterpret_cast<const float*>(meta + moff[gi] + 32);
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int M0 = code(mn[rr][0], 2 * jj) * X.x + code(mn[rr][1], 2 * jj) * X.y;
                    const int M1 = code(mn[rr][0], 2 * jj + 1) * X.z + code(mn[rr][1], 2 * jj + 1) * X.w;
                    const float u0 = __fmaf_rn(-dmn[rr], __int2float_rn(M0), __fmul_rn(dq[rr], __int2float_rn(A[gi][rr][0])));
                    const float u1 = __fmaf_rn(-dmn[rr], __int2float_rn(M1), __fmul_rn(dq[rr], __int2float_rn(A[gi][rr][1])));
                    P[gi][rr][2 * jj] = __fmaf_rn(inv, u0, P[gi][rr][2 * jj]);
                    P[gi][rr][2 * jj + 1] = __fmaf_rn(inv, u1, P[gi][rr][2 * jj + 1]);
                }
            }
        }
    }
};

// ---- repacked Q8_0 / Q4_0 rows (layouts: gemv_mma_grouped.cu): eight 32-element blocks per 256-weight group, an fp16 scale each --------
// One MMA (k = 32) per block: a lane's weight word holds elements 4t .. 4t+3 (k-step 0) or 16+4t .. (k-step 1), the x digits are
// kept in the same order (permuted columns).  The A operand is the SIGNED weight times 2^kShift as an s8 (Q8_0: the int8 itself;
// Q4_0: ((nibble ^ 8) << 4) = 16 (q - 8), one or two operations per word), so no zero point is left for the epilogue.  Per block b:
// A_b = sum 2^kShift (q - zero) xq (int32, exact), and per phase p = 0..3
//     u_p = fma(d_{4+p}, float(A_{4+p}), d_p * float(A_p)),   P_p = fma(2^-kShift / s, u_p, P_p),   y = (P_0 + P_1) + (P_2 + P_3).
__device__ __forceinline__ void imma_ss(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma0_ss(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <class T>
struct Blocks32 {
    static constexpr bool kPermX = true;
    /// Slot rows are exactly one item wide (144 or 272 bytes: 16 mod 128), so the copy engine fetches no padding.  A quarter warp's
    /// 16-byte fragment loads cover fragment rows g and g + 1: they take slot rows four apart (64 bytes mod 128), which keeps the
    /// two 64-byte windows on different banks: fragment rows 0..7 read slot rows 0,4,1,5,2,6,3,7.
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return (g >> 1) + 4u * (g & 1u); }

    template <bool FIRST>
    __device__ static __forceinline__ void mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
        if constexpr (FIRST) imma0_ss(c, a0, a1, a2, a3, b0, b1);
        else imma_ss(c, a0, a1, a2, a3, b0, b1);
    }
    /// 1 / s of the x record times the factor the A operand carries (both powers of two: exact)
    __device__ static __forceinline__ float unscale(float inv) { return T::kShift == 0 ? inv : __fmul_rn(inv, 1.0f / static_cast<float>(1 << T::kShift)); }
    /// fp16 number `idx` (compile time) of the eight in `d` as fp32
    __device__ static __forceinline__ float scale(const uint4& d, int idx) {
        const uint32_t w = (idx >> 1) == 0 ? d.x : (idx >> 1) == 1 ? d.y : (idx >> 1) == 2 ? d.z : d.w;
        return __half2float(__ushort_as_half(static_cast<unsigned short>(idx & 1 ? w >> 16 : w & 0xFFFFu)));
    }

    struct One {
        const uint8_t* bp[4];
        uint32_t bstep[4];
        uint32_t sel;  // byte selector that moves fp16 number t of a word pair into the low half
    };
    __device__ static __forceinline__ One make_one(const uint8_t* digits, const uint8_t* zeros, uint32_t g, uint32_t t) {
        One o;
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) {
            const bool real = (g >> 1) == static_cast<uint32_t>(ph);
            o.bp[ph] = real ? digits + (g & 1u) * 32u + t * 8u : zeros + t * 8u;
            o.bstep[ph] = real ? kDigitBytes : 0u;
        }
        o.sel = (2u * t) | ((2u * t + 1u) << 4);
        return o;
    }

    template <class Release>
    __device__ static __forceinline__ void item_one(const uint8_t* r0, uint32_t t, const One& o, uint32_t rec, const uint8_t* meta, float (&P)[2],
                                                    Release&& release) {
        const uint8_t* r1 = r0 + 8 * T::kPitch;
        typename T::Frag f0, f1;
        T::load(f0, r0, t);
        T::load(f1, r1, t);
        const uint4 d0 = *reinterpret_cast<const uint4*>(r0), d1 = *reinterpret_cast<const uint4*>(r1);
        release();  // fragments and scales are in registers
        const uint8_t* bq[4];
#pragma unroll
        for (int ph = 0; ph < 4; ++ph) bq[ph] = o.bp[ph] + rec * o.bstep[ph];
        int c[2][4];  // tile h: blocks 4h .. 4h + 3, one per column pair
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            uint32_t a0, a1, a2, a3;
            T::regs(f0, b, a0, a2);
            T::regs(f1, b, a1, a3);
            const uint2 bx = *reinterpret_cast<const uint2*>(bq[b & 3] + b * 64);
            if ((b & 3) == 0) mma<true>(c[b >> 2], a0, a1, a2, a3, bx.x, bx.y);
            else mma<false>(c[b >> 2], a0, a1, a2, a3, bx.x, bx.y);
        }
        const float inv = unscale(*reinterpret_cast<const float*>(meta + rec * kMetaBytes + 32));
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            const uint4 d = rr ? d1 : d0;
            const uint32_t lo = prmt(d.x, d.y, o.sel), hi = prmt(d.z, d.w, o.sel);  // scales of blocks t and 4 + t in the low halves
            const float s0 = __low2float(*reinterpret_cast<const __half2*>(&lo)), s1 = __low2float(*reinterpret_cast<const __half2*>(&hi));
            const int A0 = c[0][2 * rr] * 256 + c[0][2 * rr + 1], A1 = c[1][2 * rr] * 256 + c[1][2 * rr + 1];
            const float u = __fmaf_rn(s1, __int2float_rn(A1), __fmul_rn(s0, __int2float_rn(A0)));
            P[rr] = __fmaf_rn(inv, u, P[rr]);
        }
    }

    template <int G, int NTOK, class Release>
    __device__ static __forceinline__ void item_many(const uint8_t* r0, uint32_t t, uint32_t g, const uint8_t* dig, const uint8_t* meta, float (&P)[G][2][4],
                                                     Release&& release) {
        constexpr uint32_t kSub = 64u * NTOK;
        const uint8_t* r1 = r0 + 8 * T::kPitch;
        typename T::Frag f0, f1;
        T::load(f0, r0, t);
        T::load(f1, r1, t);
        const uint4 dd[2] = {*reinterpret_cast<const uint4*>(r0), *reinterpret_cast<const uint4*>(r1)};
        release();
        uint32_t boff[G], moff[G];
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            boff[gi] = min(8u * gi + g, 2u * NTOK - 1u) * 32u + t * 8u;
            moff[gi] = min(4u * gi + t, static_cast<uint32_t>(NTOK - 1)) * kMetaBytes;
        }
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {  // phases p = 2 jj, 2 jj + 1: blocks p and p + 4
            [[maybe_unused]] uint64_t U[G][2];    // packed form, [x-row group][e]: (row g, row g + 8)
            [[maybe_unused]] float Uf[G][2][2];  // scalar form, [x-row group][row][e]
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int b = 2 * jj + e + 4 * half;
                    uint32_t a0, a1, a2, a3;
                    T::regs(f0, b, a0, a2);
                    T::regs(f1, b, a1, a3);
                    const float s0 = scale(dd[0], b), s1 = scale(dd[1], b);
                    [[maybe_unused]] const uint64_t sc = pack2(s0, s1);
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) {
                        const uint2 bx = *reinterpret_cast<const uint2*>(dig + b * kSub + boff[gi]);
                        int c[4];
                        mma<true>(c, a0, a1, a2, a3, bx.x, bx.y);
                        const float fa0 = __int2float_rn(c[0] * 256 + c[1]), fa1 = __int2float_rn(c[2] * 256 + c[3]);
                        if constexpr (T::kPackedEpilogue) {
                            U[gi][e] = half == 0 ? mul2(sc, pack2(fa0, fa1)) : fma2(sc, pack2(fa0, fa1), U[gi][e]);
                        } else {
                            Uf[gi][0][e] = half == 0 ? __fmul_rn(s0, fa0) : __fmaf_rn(s0, fa0, Uf[gi][0][e]);
                            Uf[gi][1][e] = half == 0 ? __fmul_rn(s1, fa1) : __fmaf_rn(s1, fa1, Uf[gi][1][e]);
                        }
                    }
                }
            }
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const float inv = unscale(*reinterpret_cast<const float*>(meta + moff[gi] + 32));
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if constexpr (T::kPackedEpilogue) {
                        const uint64_t acc = fma2(pack2(inv, inv), U[gi][e], pack2(P[gi][0][2 * jj + e], P[gi][1][2 * jj + e]));
                        unpack2(acc, P[gi][0][2 * jj + e], P[gi][1][2 * jj + e]);
                    } else {
                        P[gi][0][2 * jj + e] = __fmaf_rn(inv, Uf[gi][0][e], P[gi][0][2 * jj + e]);
                        P[gi][1][2 * jj + e] = __fmaf_rn(inv, Uf[gi][1][e], P[gi][1][2 * jj + e]);
                    }
                }
            }
        }
    }
};

struct Q80i : Blocks32<Q80i> {
    static constexpr uint32_t kType = HALO_CUDA_T_Q8_0, kPitch = 272, kItemCoord = 272 / 4, kBoxInner = 272 / 4, kMapElemBytes = 4;
    static constexpr int kShift = 0, kMaxTok = 16;  // the int8 quants are the operand
    static constexpr uint32_t kStretchMax = 3;
    static constexpr bool kPackedEpilogue = false;  // (measured 1.7 % slower at 8 rows: this format waits on its weights, not on issue slots)
    // A batch that converts its x rows in the kernel does the later rounds behind its first tiles (5120 x 17408 at 8 rows 24.9 -> 22.6 us).
    // The other formats' batch kernels are bound by issue slots and lose 3 - 6 % to the hooks in the tile loop.
    static constexpr bool kPipedConversion = true;
    struct Frag {
        uint4 q[4];  // chunk c: (block 2c, k-step 0), (block 2c, k-step 1), (block 2c + 1, k-step 0), (block 2c + 1, k-step 1)
    };
    __device__ static __forceinline__ void load(Frag& f, const uint8_t* row, uint32_t t) {
#pragma unroll
        for (int c = 0; c < 4; ++c) f.q[c] = *reinterpret_cast<const uint4*>(row + 16 + c * 64 + t * 16);
    }
    __device__ static __forceinline__ void regs(const Frag& f, int b, uint32_t& k0, uint32_t& k1) {
        const uint4 c = f.q[b >> 1];
        k0 = (b & 1) ? c.z : c.x, k1 = (b & 1) ? c.w : c.y;
    }
};

struct Q40i : Blocks32<Q40i> {
    static constexpr uint32_t kType = HALO_CUDA_T_Q4_0, kPitch = 144, kItemCoord = 144 / 4, kBoxInner = 144 / 4, kMapElemBytes = 4;
    static constexpr int kShift = 4, kMaxTok = 16;  // the operand is 16 (q - 8)
    static constexpr uint32_t kStretchMax = 8;
    static constexpr bool kPackedEpilogue = true;  // two-wide fp32 operations in the batch epilogue: 1.5 - 2.4 % fewer microseconds at 16 rows
    static constexpr bool kPipedConversion = false;
    struct Frag {
        uint4 q[2];  // chunk c: the words of blocks 4c .. 4c + 3 (low nibbles: elements 4t .., high nibbles: elements 16 + 4t ..)
    };
    __device__ static __forceinline__ void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.q[0] = *reinterpret_cast<const uint4*>(row + 16 + t * 16);
        f.q[1] = *reinterpret_cast<const uint4*>(row + 16 + 64 + t * 16);
    }
    __device__ static __forceinline__ void regs(const Frag& f, int b, uint32_t& k0, uint32_t& k1) {
        const uint4 c = f.q[b >> 2];
        const uint32_t w = (b & 3) == 0 ? c.x : (b & 3) == 1 ? c.y : (b & 3) == 2 ? c.z : c.w;
        // ((nibble ^ 8) << 4) as a signed byte is 16 (nibble - 8): the zero point rides in the operand
        k0 = ((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u, k1 = (w & 0xF0F0F0F0u) ^ 0x80808080u;
    }
};

// ---- repacked Q6_K rows (224 B per super-block): sixteen 16-element groups with an int8 scale each, one fp16 d per super-block ------
// The 6-bit codes enter as SIGNED bytes 4 (code - 32) = ((code << 2) ^ 0x80), built in the four operations per word it takes to put
// nibble and high bits together, so no zero point is left for the epilogue:  A_g = 4 sum (q - 32) xq  (int32, exact).  Per phase
// p = 0..3 (group g = 4 T + p, T = 0..3 ascending):
//     u_p = sc_p * A_p,  u_p = fma(sc_{4T+p}, A_{4T+p}, u_p)   (fp32; sc converted exactly),   P_p = fma(1 / (4 s), d * u_p, P_p)
// A batch uses one m16n8k16 MMA per group.  A single row uses m16n8k32: a 32-element sub-block holds two groups, which land in
// different column pairs because the B registers of the other half are masked to zero.
__device__ __forceinline__ void imma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};\n"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

struct Q6Ki {
    static constexpr uint32_t kType = HALO_CUDA_T_Q6_K, kPitch = 224, kItemCoord = 224 / 4, kBoxInner = 224 / 4, kMapElemBytes = 4;
    static constexpr bool kPermX = true;
    static constexpr int kMaxTok = 16;
    static constexpr uint32_t kStretchMax = 8;
    static constexpr bool kPipedConversion = false;
    /// 224-byte slot rows put rows g and g + 1 on overlapping banks: fragment rows 0..7 take slot rows 0,2,4,6,1,3,5,7
    __device__ static __forceinline__ uint32_t slot_row(uint32_t g) { return ((2u * g) & 7u) | (g >> 2); }

    struct Frag {
        uint4 ql[2];  // half n: words (b, lh) = (0,0), (0,1), (1,0), (1,1)
        uint4 qh;     // words (n, lh) = (0,0), (0,1), (1,0), (1,1)
    };
    __device__ static __forceinline__ void load(Frag& f, const uint8_t* row, uint32_t t) {
        f.ql[0] = *reinterpret_cast<const uint4*>(row + 32 + t * 16);
        f.ql[1] = *reinterpret_cast<const uint4*>(row + 32 + 64 + t * 16);
        f.qh = *reinterpret_cast<const uint4*>(row + 32 + 128 + t * 16);
    }
    /// The codes of sub-block sub = 4 n + quarter (elements 128 n + 32 quarter ..): k0 = elements 4t .. 4t+3, k1 = 16 + 4t ..
    __device__ static __forceinline__ void regs(const Frag& f, int sub, uint32_t& k0, uint32_t& k1) {
        const int n = sub >> 2, quarter = sub & 3, b = quarter & 1, nib = quarter >> 1;
        const uint4 c = f.ql[n];
        const uint32_t w0 = b ? c.z : c.x, w1 = b ? c.w : c.y;
        const uint32_t h0 = n ? f.qh.z : f.qh.x, h1 = n ? f.qh.w : f.qh.y;
        // 4 code = nibble << 2 | two high bits << 6 (byte j of h holds the high bits of element j for all four quarters, two bits
        // each); flipping bit 7 makes the byte, read as signed, 4 (code - 32)
        auto code = [&](uint32_t w, uint32_t h) {
            const uint32_t wn = nib ? w >> 2 : w << 2;
            const uint32_t hs = quarter == 0 ? h << 6 : quarter == 1 ? h << 4 : quarter == 2 ? h << 2 : h;
            return (wn & 0x3C3C3C3Cu) | ((hs & 0xC0C0C0C0u) ^ 0x80808080u);
        };
        k0 = code(w0, h0), k1 = code(w1, h1);
    }
    __device__ static __forceinline__ uint32_t word(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

    struct One {
        const uint8_t* bp[2];  // B base for the first / second sub-block of a tile: this lane's digits, or zeros
        uint32_t bstep[2];
        uint32_t m0, m1;       // which half of a sub-block this lane's column pair carries
        uint32_t sel;          // sign-extending selector of scale byte t
    };
    __device__ static __forceinline__ One make_one(const uint8_t* digits, const uint8_t* zeros, uint32_t g, uint32_t t) {
        One o;
        const uint32_t ph = g >> 1;  // the column pair's group inside a tile of four
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const bool real = (ph >> 1) == static_cast<uint32_t>(e);
            o.bp[e] = real ? digits + (g & 1u) * 32u + t * 8u : zeros + t * 8u;
            o.bstep[e] = real ? kDigitBytes : 0u;
        }
        o.m0 = (ph & 1u) == 0 ? 0xFFFFFFFFu : 0u;
        o.m1 = ~o.m0;
        o.sel = t | ((8u | t) * 0x1110u);
        return o;
    }

    template <class Release>
    __device__ static __forceinline__ void item_one(const uint8_t* r0, uint32_t t, const One& o, uint32_t rec, const uint8_t* meta, float (&P)[2],
                                                    Release&& release) {
        const uint8_t* r1 = r0 + 8 * kPitch;
        Frag f0, f1;
        load(f0, r0, t);
        load(f1, r1, t);
        const uint4 sw[2] = {*reinterpret_cast<const uint4*>(r0), *reinterpret_cast<const uint4*>(r1)};
        const float d[2] = {__half2float(*reinterpret_cast<const __half*>(r0 + 16)), __half2float(*reinterpret_cast<const __half*>(r1 + 16))};
        release();  // fragments and scales are in registers
        const uint8_t* bq[2] = {o.bp[0] + rec * o.bstep[0], o.bp[1] + rec * o.bstep[1]};
        int c[4][4];  // tile T: groups 4T .. 4T + 3, one per column pair
#pragma unroll
        for (int T = 0; T < 4; ++T) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int sub = 2 * T + e;
                uint32_t a0, a1, a2, a3;
                regs(f0, sub, a0, a2);
                regs(f1, sub, a1, a3);
                const uint2 v = *reinterpret_cast<const uint2*>(bq[e] + sub * 64);
                if (e == 0) imma0_ss(c[T], a0, a1, a2, a3, v.x & o.m0, v.y & o.m1);
                else imma_ss(c[T], a0, a1, a2, a3, v.x & o.m0, v.y & o.m1);
            }
        }
        const float inv = __fmul_rn(*reinterpret_cast<const float*>(meta + rec * kMetaBytes + 32), 0.25f);  // the operand carries a factor 4
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            float u = 0.0f;
#pragma unroll
            for (int T = 0; T < 4; ++T) {
                const float a = __int2float_rn(c[T][2 * rr] * 256 + c[T][2 * rr + 1]);
                const float sc = __int2float_rn(static_cast<int>(prmt(word(sw[rr], T), 0u, o.sel)));
                u = T == 0 ? __fmul_rn(sc, a) : __fmaf_rn(sc, a, u);
            }
            P[rr] = __fmaf_rn(inv, __fmul_rn(d[rr], u), P[rr]);
        }
    }

    template <int G, int NTOK, class Release>
    __device__ static __forceinline__ void item_many(const uint8_t* r0, uint32_t t, uint32_t g, const uint8_t* dig, const uint8_t* meta, float (&P)[G][2][4],
                                                     Release&& release) {
        constexpr uint32_t kSub = 64u * NTOK;
        const uint8_t* r1 = r0 + 8 * kPitch;
        Frag f0, f1;
        load(f0, r0, t);
        load(f1, r1, t);
        const uint4 sw[2] = {*reinterpret_cast<const uint4*>(r0), *reinterpret_cast<const uint4*>(r1)};
        const float d[2] = {__half2float(*reinterpret_cast<const __half*>(r0 + 16)), __half2float(*reinterpret_cast<const __half*>(r1 + 16))};
        release();
        uint32_t boff[G], moff[G];
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            boff[gi] = min(8u * gi + g, 2u * NTOK - 1u) * 32u + t * 8u;
            moff[gi] = min(4u * gi + t, static_cast<uint32_t>(NTOK - 1)) * kMetaBytes;
        }
        // the epilogue runs two-wide over rows g and g + 8 (26.2 -> 25.5 us at 8 rows; the Q4_K form measured mixed and stays scalar)
        uint64_t U[G][4];  // [x-row group][phase]: (row g, row g + 8)
#pragma unroll
        for (int T = 0; T < 4; ++T) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int sub = 2 * T + e;
                uint32_t a0, a1, a2, a3;
                regs(f0, sub, a0, a2);
                regs(f1, sub, a1, a3);
                uint64_t sc[2];
#pragma unroll
                for (int lh = 0; lh < 2; ++lh) {
                    const int p = 2 * e + lh;
                    sc[lh] = pack2(__int2float_rn(static_cast<int>(static_cast<int8_t>(word(sw[0], T) >> (8 * p)))),
                                   __int2float_rn(static_cast<int>(static_cast<int8_t>(word(sw[1], T) >> (8 * p)))));
                }
#pragma unroll
                for (int gi = 0; gi < G; ++gi) {
                    const uint2 bx = *reinterpret_cast<const uint2*>(dig + sub * kSub + boff[gi]);
#pragma unroll
                    for (int lh = 0; lh < 2; ++lh) {
                        const int p = 2 * e + lh;  // group 4 T + p
                        int c[4];
                        imma_k16(c, lh ? a2 : a0, lh ? a3 : a1, lh ? bx.y : bx.x);
                        const uint64_t a = pack2(__int2float_rn(c[0] * 256 + c[1]), __int2float_rn(c[2] * 256 + c[3]));
                        U[gi][p] = T == 0 ? mul2(sc[lh], a) : fma2(sc[lh], a, U[gi][p]);
                    }
                }
            }
        }
        const uint64_t d2 = pack2(d[0], d[1]);
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const float inv = __fmul_rn(*reinterpret_cast<const float*>(meta + moff[gi] + 32), 0.25f);
            const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint64_t acc = fma2(inv2, mul2(d2, U[gi][p]), pack2(P[gi][0][p], P[gi][1][p]));
                unpack2(acc, P[gi][0][p], P[gi][1][p]);
            }
        }
    }
};

// Shared-memory layout: header (mma_common.cuh) | weight ring | slice sums (KS > 1) | zeros (single row) | digits | meta
// KS (1, 2, 4, 8 or 16 in-CTA K slices; R = 16 / KS row blocks per unit) is a launch parameter: one kernel per format and batch size.
template <class F, int NTOK, int NS>
struct Layout {
    static constexpr int G = (NTOK + 3) / 4;
    static constexpr uint32_t kSlot = 16 * F::kPitch;
    static constexpr uint32_t kOffSlices = kOffRing + kSkWarps * NS * kSlot;
    /// slice sums: [r][ks - 1][lane][2 G] floats = (16 - R) warps' worth; ks_shift = log2 of the slice count
    __host__ __device__ static constexpr uint32_t red_bytes(uint32_t ks_shift) { return (kSkWarps - (kSkWarps >> ks_shift)) * 32u * 2u * G * 4u; }
    __host__ __device__ static constexpr uint32_t off_zero(uint32_t ks_shift) { return (kOffSlices + red_bytes(ks_shift) + 127u) & ~127u; }
    // a single row's digits start 64 bytes off the zeros' 128-byte phase: the lanes of a half warp that read x and those that
    // read zeros then never meet on a bank
    __host__ __device__ static constexpr uint32_t off_digits(uint32_t ks_shift) { return off_zero(ks_shift) + (NTOK == 1 ? 512u + 64u : 0u); }
    __host__ __device__ static constexpr uint32_t bytes(uint32_t n_rec, uint32_t ks_shift) { return off_digits(ks_shift) + n_rec * rec_bytes(NTOK); }
};

/// End of a unit (or of the CTA's share of it): the KS slices of the row block are added in ks order through shared memory
/// (`red`: [r][ks - 1][lane][2G] floats), then slice 0 hands the sums over (gemv_mma_sk.cuh's finish_block with KS at run time).
template <int G, int NTOK>
__device__ __forceinline__ void finish_slices(float (&yacc)[G][2], uint32_t unit, uint32_t r, uint32_t ks, uint32_t KS, uint32_t R, float* red, const SkTable& tb,
                                              uint32_t cta, float* part, uint32_t* counters, float* y, uint64_t y_stride, uint32_t rows, uint32_t lane,
                                              uint32_t row, const PeerPush& peer) {
    if (KS > 1) {
        if (ks != 0) {
            float2* mine = reinterpret_cast<float2*>(red) + ((r * (KS - 1) + (ks - 1)) * 32 + lane) * G;
#pragma unroll
            for (int gi = 0; gi < G; ++gi) mine[gi] = make_float2(yacc[gi][0], yacc[gi][1]);
        }
        sk::named_barrier(1 + r, KS * 32);
        if (ks == 0) {
            for (uint32_t k = 1; k < KS; ++k) {
                const float2* p = reinterpret_cast<const float2*>(red) + ((r * (KS - 1) + (k - 1)) * 32 + lane) * G;
#pragma unroll
                for (int gi = 0; gi < G; ++gi) yacc[gi][0] = __fadd_rn(yacc[gi][0], p[gi].x), yacc[gi][1] = __fadd_rn(yacc[gi][1], p[gi].y);
            }
        }
        sk::named_barrier(1 + r, KS * 32);  // the slices may overwrite `red` at their next block only after slice 0 has read it
    }
    if (ks == 0) sk_flush_r<G, NTOK>(yacc, unit, r, R, tb, cta, part, counters, y, y_stride, rows, lane, row, peer);
}

// KSC: the slice count where it is known at compile time (the two-slice partition of the large shapes, whose inner loop
// is the one that runs at memory speed), 0: taken from ks_shift_arg.
// PRE (every launch of two x rows and up): the x records come from `xstage`, where a conversion launch wrote them, or --
// xstage == nullptr -- the kernel converts the rows itself (the host chooses: gemv_i8_launch.cuh).  A single row is always
// converted in the kernel.
// XC == 2: a resident batch launch that converts its x rows itself does so in rounds, the later ones behind its first tiles.
// XC == 1 (batches whose x records do not all fit): x is STREAMED.  The CTA's columns are walked in stretches of n_rec columns (as many
// as fit: fewer block barriers, more room for the warps to run ahead of one another); the records of
// a stretch (KS super-blocks per column, all NTOK rows) sit in one half of a double buffer, the next stretch's are copied into
// the other half meanwhile, and a block barrier ends every stretch.  Same tiles, same order, same arithmetic as the resident
// form: the bits do not change; the weights are read once whatever the batch.
template <class F, int NTOK, int NS, int KSC, bool PRE, bool NORM = false, int XC = 0>
__global__ void __launch_bounds__(kSkWarps * 32, 1)
gemv_i8_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ SkTable tb, const float* __restrict__ x, uint64_t x_stride,
               float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t nb, uint32_t n_rec, uint32_t ks_shift_arg, float* __restrict__ partials,
               uint32_t* __restrict__ counters, uint32_t* __restrict__ error_word, const uint8_t* __restrict__ xstage,
               const __grid_constant__ PeerPush peer, const float* __restrict__ norm_w, float norm_eps) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    using L = Layout<F, NTOK, NS>;
    constexpr int G = L::G;
    constexpr uint32_t kThreads = kSkWarps * 32, kSlot = L::kSlot;
    static_assert(KSC == 0 || KSC == 2, "compile-time slice counts");
    const uint32_t ks_shift = KSC == 2 ? 1u : ks_shift_arg;
    const uint32_t KS = 1u << ks_shift, R = kSkWarps >> ks_shift;  // K slices, row blocks per unit
    static_assert(kSkWarps == 16 && kSkWarps <= kMaxWarps && NS <= 6, "shared-memory header layout; warp -> (r, ks) by shifts");
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t r = warp & (R - 1u), ks = warp >> (4u - ks_shift);
    const uint32_t n_rb = (rows + 15u) / 16u, cpu = tb.cols_per_unit;
    const uint32_t cta = blockIdx.x;  // the grid has exactly tb.parts CTAs
    // n_rec x records are resident: all nb of them (record j = super-block j), or -- when every CTA of a one-slice partition walks
    // fewer columns than a unit has -- only those of the CTA's own columns, record j = its j-th column (super-block (c0 + j) mod nb)
    const uint32_t off_zero = L::off_zero(ks_shift), off_digits = L::off_digits(ks_shift);
    uint8_t* digits = smem + off_digits;
    uint8_t* meta = digits + n_rec * (kDigitBytes * NTOK);

    const uint32_t bars = smem_base + kOffBars + warp * NS * 8u;
    const uint32_t ring = smem_base + kOffRing + warp * NS * kSlot;
    asm volatile("griddepcontrol.launch_dependents;");  // the next kernel in the stream may start filling its ring
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8u, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    // This warp's tiles: for every unit the CTA's column range [c0, c1) touches, the columns k (super-block k * KS + ks) of
    // that unit inside the range, as long as the row block and the super-block exist.  The producer (ring fill) and the
    // consumer walk them independently; later units have later row blocks, so the first row block past the matrix ends both.
    const uint32_t c0 = tb.start[cta], c1 = tb.start[cta + 1];
    const uint32_t kmax = nb > ks ? min(cpu, (nb - ks + KS - 1u) >> ks_shift) : 0u;  // this warp's columns in a whole unit
    const uint32_t unit0 = c0 / cpu;
    auto seg_end = [&](uint32_t unit) { return unit * R + r < n_rb && unit * cpu < c1 ? min(kmax, c1 - unit * cpu) : 0u; };
    uint32_t p_unit = unit0, p_k = c0 - unit0 * cpu, p_end = seg_end(unit0), fill_slot = 0;
    auto settle = [&]() {  // moves the producer to the unit of its next tile, if any
        while (p_k >= p_end && (p_unit + 1) * cpu < c1 && (p_unit + 1) * R + r < n_rb) ++p_unit, p_k = 0, p_end = seg_end(p_unit);
    };
    settle();
    auto refill = [&]() {  // the producer's tile -> slot fill_slot
        if (p_k >= p_end) return;
        if (lane == 0) {
            mbar_expect_tx(bars + fill_slot * 8u, kSlot);
            sk::tma_item_g2s<F>(ring + fill_slot * kSlot, &wmap, p_k * KS + ks, (p_unit * R + r) * 16u, bars + fill_slot * 8u);
        }
        if constexpr (NS == 2) fill_slot ^= 1u;
        else fill_slot = fill_slot + 1 == NS ? 0 : fill_slot + 1;
        if (++p_k >= p_end) settle();
    };
#pragma unroll
    for (int it = 0; it < NS; ++it) refill();
    // The weights never depend on the kernel before this one, so the ring is filled first; only now wait for it.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    bool lost = false;
    // In-kernel conversion of a batch (PRE launches without a conversion launch): pairs to convert, rounds of sixteen, this warp's next round
    [[maybe_unused]] uint32_t cv_first = 0, cv_items = 0, cv_rounds = 0, cv_next = 0, cv_seen = 1;
    [[maybe_unused]] auto cv_src = [&](uint32_t i) {  // this lane's eight floats of pair i
        const uint32_t j = i / NTOK, tok = i - j * NTOK;
        const uint32_t sb = cv_first + j >= nb ? cv_first + j - nb : cv_first + j;  // (a one-slice partition has cpu == nb)
        return reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tok} * x_stride) + sb * 64u + 2u * lane;
    };
    [[maybe_unused]] auto cv_prefetch = [&]() {  // the row of this warp's next pair -> L1, ahead of the tile it is converted behind
        const uint32_t i = warp + cv_next * kSkWarps;
        if (cv_next < cv_rounds && i < cv_items) asm volatile("prefetch.global.L1 [%0];" ::"l"(cv_src(i)));
    };
    [[maybe_unused]] auto cv_step = [&]() {  // converts this warp's pair of round cv_next (if it has one) and arrives on the round's barrier
        const uint32_t i = warp + cv_next * kSkWarps;
        if (i < cv_items) {
            const float4* src = cv_src(i);
            const float4 a = src[0], b = src[1];
            stage_superblock(smem + off_digits, smem + off_digits + n_rec * (kDigitBytes * NTOK), a, b, i / NTOK, NTOK, i % NTOK, lane, F::kPermX);
        }
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(smem_base + kOffRounds + (cv_next - 2u) * 8u) : "memory");
        ++cv_next;
    };
    if constexpr (NTOK == 1)
        for (uint32_t i = tid; i < 512u / 4u; i += kThreads) reinterpret_cast<uint32_t*>(smem + off_zero)[i] = 0u;
    constexpr uint32_t kXFull = kOffRed + 160u;  // two mbarriers of the streamed form (the warp-sum floats before them end at kOffRed + 128)
    if constexpr (XC == 1) {
        static_assert(PRE && NTOK >= 2 && kXFull + 16u <= kOffBars, "streamed x: batches, records from the conversion launch");
        if (tid == 0) {
            mbar_init(smem_base + kXFull, 1);
            mbar_init(smem_base + kXFull + 8u, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    } else if constexpr (PRE) {
        static_assert(!NORM, "the fused input norm takes one x row");
        if (xstage != nullptr) {  // the records were written by the conversion kernel before this launch: copy this CTA's in
            const uint32_t xbar = smem_base + kOffXBar;
            if (tid == 0) {
                mbar_init(xbar, 1);
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                // the records of this CTA's super-blocks: all of them, or the cyclic run of its columns (at most two contiguous pieces)
                const uint32_t xc0 = tb.start[cta], xn = tb.start[cta + 1] - xc0;
                const bool xpart = KS == 1 && n_rec < nb;
                const uint32_t first = xpart ? xc0 % cpu : 0u, count = xpart ? xn : nb;
                const uint32_t n1 = min(count, nb - first), n2 = count - n1;  // super-blocks [first, first + n1) then [0, n2)
                constexpr uint32_t kD = kDigitBytes * NTOK, kM = kMetaBytes * NTOK;
                mbar_expect_tx(xbar, count * (kD + kM));
                const uint8_t* gmeta = xstage + uint64_t{nb} * kD;
                const uint32_t smeta = smem_base + off_digits + n_rec * kD;
                auto copy = [&](uint32_t dst, const uint8_t* src, uint32_t bytes) {
                    for (uint32_t off = 0; off < bytes; off += 32768u) bulk_g2s(dst + off, src + off, min(32768u, bytes - off), xbar);
                };
                copy(smem_base + off_digits, xstage + uint64_t{first} * kD, n1 * kD);
                copy(smeta, gmeta + uint64_t{first} * kM, n1 * kM);
                if (n2 != 0) {
                    copy(smem_base + off_digits + n1 * kD, xstage, n2 * kD);
                    copy(smeta + n1 * kM, gmeta, n2 * kM);
                }
            }
            __syncthreads();
            if (!mbar_wait(xbar, 0)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;
            }
        } else {
            if constexpr (XC == 2) {
                // No conversion launch (the host leaves it out where a CTA has few records to make): the rows are converted here, a
                // (record, row) pair per warp at a time, record-major: pair i = warp + 16 u belongs to ROUND u.  Under a partial
                // residency the records are the super-blocks of the CTA's own columns only; under in-CTA slices every CTA converts all
                // of x.  Rounds 0 and 1 are converted before the first tile (their loads in flight together, a block barrier behind
                // them); a later round is converted by every warp after one of its tiles (the row was prefetched before that tile) and
                // completes behind an mbarrier that only the tiles of its records wait for.
                const uint32_t x_c0 = tb.start[cta], x_cols = tb.start[cta + 1] - x_c0;
                const bool part = KS == 1 && n_rec < nb;
                cv_first = part ? x_c0 % cpu : 0u, cv_items = (part ? x_cols : nb) * NTOK, cv_rounds = (cv_items + kSkWarps - 1u) / kSkWarps;
                if (tid == 0 && cv_rounds > 2u) {
                    for (uint32_t u = 2; u < cv_rounds; ++u) mbar_init(smem_base + kOffRounds + (u - 2u) * 8u, kSkWarps);
                    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                }
                float4 v[2][2];
#pragma unroll
                for (uint32_t u = 0; u < 2; ++u) {
                    const uint32_t i = warp + u * kSkWarps;
                    if (i < cv_items) {
                        const float4* src = cv_src(i);
                        v[u][0] = src[0], v[u][1] = src[1];
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < 2; ++u) {
                    const uint32_t i = warp + u * kSkWarps;
                    if (i < cv_items) stage_superblock(digits, meta, v[u][0], v[u][1], i / NTOK, NTOK, i % NTOK, lane, F::kPermX);
                }
                cv_next = 2;
                __syncthreads();
            } else {
                // No conversion launch (the host leaves it out where a CTA has few records to make): the rows are converted here, a
                // (record, row) pair per warp at a time, record-major, the loads of kAhead pairs in flight together.  Under a partial
                // residency these are the super-blocks of the CTA's own columns only; under in-CTA slices every CTA converts all of x.
                const uint32_t x_c0 = tb.start[cta], x_cols = tb.start[cta + 1] - x_c0;
                const bool part = KS == 1 && n_rec < nb;
                const uint32_t x_first = part ? x_c0 % cpu : 0u, n_items = (part ? x_cols : nb) * NTOK;
                constexpr uint32_t kAhead = 4;  // (eight measured the same or slower)
                for (uint32_t i0 = warp; i0 < n_items; i0 += kAhead * kSkWarps) {
                    float4 v[kAhead][2];
#pragma unroll
                    for (uint32_t u = 0; u < kAhead; ++u) {
                        const uint32_t i = i0 + u * kSkWarps;
                        if (i < n_items) {
                            const uint32_t j = i / NTOK, tok = i - j * NTOK;
                            const uint32_t sb = x_first + j >= nb ? x_first + j - nb : x_first + j;  // (a one-slice partition has cpu == nb)
                            const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const uint8_t*>(x) + uint64_t{tok} * x_stride);
                            v[u][0] = xr[sb * 64u + 2u * lane], v[u][1] = xr[sb * 64u + 2u * lane + 1u];
                        }
                    }
#pragma unroll
                    for (uint32_t u = 0; u < kAhead; ++u) {
                        const uint32_t i = i0 + u * kSkWarps;
                        if (i < n_items) stage_superblock(digits, meta, v[u][0], v[u][1], i / NTOK, NTOK, i % NTOK, lane, F::kPermX);
                    }
                }
                __syncthreads();
            }
        }
    } else {
        static_assert(NTOK == 1, "batches arrive through the branch above");
        // The row is converted in the kernel, one super-block per warp and round.  The first round (super-blocks 0 .. 15) is
        // what every warp's first tiles need: the block waits for it; the later rounds (their loads already in flight) finish
        // behind an mbarrier that only the tiles of super-block 16 and up wait for.
        // Under a partial residency the CTA converts only the super-blocks of its own columns, cyclically from where its range starts.
        const uint32_t x_c0 = tb.start[cta], x_cols = tb.start[cta + 1] - x_c0;
        const bool part = KS == 1 && n_rec < nb;
        const uint32_t x_first = part ? x_c0 % cpu : 0u, x_count = part ? x_cols : nb;
        auto x_sb = [&](uint32_t j) {  // the j-th super-block this CTA converts
            const uint32_t sb = x_first + j;
            return sb >= nb ? sb - nb : sb;  // (a one-slice partition has cpu == nb)
        };
        const uint32_t late_warps = x_count > kSkWarps ? min(x_count - kSkWarps, kSkWarps) : 0u;
        if (tid == 0 && late_warps != 0) {
            mbar_init(smem_base + kOffXBar + 8u, late_warps);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        float inv_rms = 1.0f;
        if constexpr (NORM) inv_rms = block_inv_rms<kSkWarps>(x, nb * 256u, norm_eps, reinterpret_cast<float*>(smem + kOffRed), tid);
        const float4* xr = reinterpret_cast<const float4*>(x);
        const float4* wr = reinterpret_cast<const float4*>(norm_w);
        auto fetch = [&](uint32_t sb, float4 (&v)[2]) {
            v[0] = xr[sb * 64u + 2u * lane], v[1] = xr[sb * 64u + 2u * lane + 1u];
            if constexpr (NORM) {  // the CPU backend's rms_norm arithmetic (backends/cpu/ops_basic.cpp:28-30), unfused multiplies
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const float4 w = wr[sb * 64u + 2u * lane + hf];
                    v[hf].x = __fmul_rn(__fmul_rn(v[hf].x, inv_rms), w.x);
                    v[hf].y = __fmul_rn(__fmul_rn(v[hf].y, inv_rms), w.y);
                    v[hf].z = __fmul_rn(__fmul_rn(v[hf].z, inv_rms), w.z);
                    v[hf].w = __fmul_rn(__fmul_rn(v[hf].w, inv_rms), w.w);
                }
            }
        };
        float4 v0[2], v1[2];
        const bool first = warp < x_count, second = warp + kSkWarps < x_count;
        if (first) fetch(x_sb(warp), v0);
        if (second) fetch(x_sb(warp + kSkWarps), v1);
        if (first) stage_superblock(digits, meta, v0[0], v0[1], warp, 1, 0, lane, F::kPermX);
        __syncthreads();
        if (second) {
            stage_superblock(digits, meta, v1[0], v1[1], warp + kSkWarps, 1, 0, lane, F::kPermX);
            for (uint32_t j = warp + 2 * kSkWarps; j < x_count; j += kSkWarps) {
                fetch(x_sb(j), v0);
                stage_superblock(digits, meta, v0[0], v0[1], j, 1, 0, lane, F::kPermX);
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_base + kOffXBar + 8u) : "memory");
        }
    }
    bool late_ready = false;  // this warp has seen the later rounds of the x conversion complete
    // the record of a tile: its super-block, or (partial residency) its column's distance from the start of the CTA's range
    const bool x_part = KS == 1 && n_rec < nb;

    const uint8_t* slot0 = smem + kOffRing + warp * NS * kSlot + F::slot_row(g) * F::kPitch;
    float* red = reinterpret_cast<float*>(smem + L::kOffSlices);
    [[maybe_unused]] typename F::One one;
    if constexpr (NTOK == 1) one = F::make_one(digits, smem + off_zero, g, t);
    float P[G][2][NTOK == 1 ? 1 : 4];
#pragma unroll
    for (int gi = 0; gi < G; ++gi)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
            for (int p = 0; p < (NTOK == 1 ? 1 : 4); ++p) P[gi][rr][p] = 0.0f;

    uint32_t slot = 0, parity = 0, taken = 0;  // tiles this warp has consumed: slot = taken mod NS, parity = (taken / NS) mod 2
    auto release = [&]() {
        __syncwarp();
        ++taken;
        if constexpr (NS == 2) {
            slot = taken & 1u, parity = (taken >> 1) & 1u;
        } else {
            slot = slot + 1 == NS ? 0 : slot + 1;
            parity ^= (slot == 0);
        }
        refill();
    };
    auto finish_unit = [&](uint32_t unit) {  // the row block, or this CTA's share of it, is done
        float yacc[G][2];
#pragma unroll
        for (int gi = 0; gi < G; ++gi)
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                if constexpr (NTOK == 1) {
                    float v = P[gi][rr][0];
                    v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));  // (P_0 + P_1), (P_2 + P_3)
                    v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
                    yacc[gi][rr] = v;
                    P[gi][rr][0] = 0.0f;
                } else {
                    yacc[gi][rr] = __fadd_rn(__fadd_rn(P[gi][rr][0], P[gi][rr][1]), __fadd_rn(P[gi][rr][2], P[gi][rr][3]));
#pragma unroll
                    for (int p = 0; p < 4; ++p) P[gi][rr][p] = 0.0f;
                }
            }
        finish_slices<G, NTOK>(yacc, unit, r, ks, KS, R, red, tb, cta, partials, counters, y, y_stride, rows, lane, F::slot_row(g), peer);
    };
    if constexpr (XC == 1) {
        constexpr uint32_t kD = kDigitBytes * NTOK, kM = kMetaBytes * NTOK;
        const uint32_t xc = n_rec;  // (streamed form: the parameter carries the columns per stretch)
        const uint32_t col_bytes = KS * (kD + kM), half_bytes = xc * col_bytes;  // a column: KS super-blocks of digits, then KS of meta
        const uint32_t n_str = (c1 - c0 + xc - 1u) / xc;
        const uint8_t* gmeta = xstage + uint64_t{nb} * kD;
        auto issue = [&](uint32_t j) {  // thread 0: the records of stretch j into half j & 1
            const uint32_t bar = smem_base + kXFull + (j & 1u) * 8u, dst0 = smem_base + off_digits + (j & 1u) * half_bytes;
            uint32_t total = 0;
            for (uint32_t i = 0, col = c0 + j * xc; i < xc && col < c1; ++i, ++col) {
                const uint32_t sb0 = (col % cpu) * KS;
                total += (sb0 < nb ? min(KS, nb - sb0) : 0u) * (kD + kM);
            }
            mbar_expect_tx(bar, total);
            for (uint32_t i = 0, col = c0 + j * xc; i < xc && col < c1; ++i, ++col) {
                const uint32_t sb0 = (col % cpu) * KS, cnt = sb0 < nb ? min(KS, nb - sb0) : 0u;
                if (cnt == 0) continue;
                bulk_g2s(dst0 + i * col_bytes, xstage + uint64_t{sb0} * kD, cnt * kD, bar);
                bulk_g2s(dst0 + i * col_bytes + KS * kD, gmeta + uint64_t{sb0} * kM, cnt * kM, bar);
            }
        };
        if (tid == 0) {
            issue(0);
            if (n_str > 1) issue(1);
        }
        uint32_t unit = unit0, kk = c0 - unit0 * cpu;
        for (uint32_t j = 0; j < n_str; ++j) {
            if (!mbar_wait(smem_base + kXFull + (j & 1u) * 8u, (j >> 1) & 1u)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;
            }
            const uint8_t* half = digits + (j & 1u) * half_bytes;
            for (uint32_t i = 0, col = c0 + j * xc; i < xc && col < c1; ++i, ++col) {
                const bool row_ok = unit * R + r < n_rb;
                if (row_ok && kk < kmax) {
                    if (!lost && !mbar_wait(bars + slot * 8u, parity)) {
                        if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                        lost = true;
                    }
                    const uint8_t* colp = half + i * col_bytes;
                    F::template item_many<G, NTOK>(slot0 + slot * kSlot, t, g, colp + ks * kD, colp + KS * kD + ks * kM, P, release);
                }
                if (kk + 1u == cpu || col + 1u == c1) {
                    if (row_ok) finish_unit(unit);
                    kk = 0, ++unit;
                } else {
                    ++kk;
                }
            }
            __syncthreads();  // every warp is done with this half: refill it two stretches ahead
            if (tid == 0 && j + 2u < n_str) issue(j + 2u);
        }
        if (lost) sk::linger_after_loss();
        return;
    }
    // A warp that lost a copy keeps walking (its sums are garbage, the error word says so): its siblings wait for it at the barriers.
    for (uint32_t unit = unit0, k_lo = c0 - unit0 * cpu; unit * cpu < c1; ++unit, k_lo = 0) {
        if (unit * R + r >= n_rb) break;
        const uint32_t k_hi = min(kmax, c1 - unit * cpu);
        for (uint32_t k = k_lo; k < k_hi; ++k) {
            const uint32_t sb = k * KS + ks, rec = x_part ? unit * cpu + k - c0 : sb;
            if constexpr (!PRE) {
                if (rec >= kSkWarps && !late_ready) {
                    if (!mbar_wait(smem_base + kOffXBar + 8u, 0)) {
                        if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                        lost = true;
                    }
                    late_ready = true;
                }
            }
            if constexpr (XC == 2) {
                if (cv_rounds > 2u) {
                    // the round that completes this record; a warp converts its own pairs up to that round before it waits for the others'
                    const uint32_t need = (rec * NTOK + NTOK - 1u) / kSkWarps;
                    if (need > cv_seen) {
                        while (cv_next <= need) cv_step();
                        if (!mbar_wait(smem_base + kOffRounds + (need - 2u) * 8u, 0)) {
                            if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                            lost = true;
                        }
                        cv_seen = need;
                    }
                    cv_prefetch();
                }
            }
            if (!lost && !mbar_wait(bars + slot * 8u, parity)) {
                if (lane == 0 && error_word != nullptr) atomicOr(error_word, 1u);
                lost = true;  // warp-uniform: every lane polled the same barrier
            }
            if constexpr (NTOK == 1) {
                float (&P1)[2] = *reinterpret_cast<float (*)[2]>(&P[0][0][0]);
                static_assert(sizeof(P) == 2 * sizeof(float), "single-row accumulators");
                F::item_one(slot0 + slot * kSlot, t, one, rec, meta, P1, release);
            } else {
                F::template item_many<G, NTOK>(slot0 + slot * kSlot, t, g, digits + rec * (kDigitBytes * NTOK), meta + rec * (kMetaBytes * NTOK), P, release);
                if constexpr (XC == 2) {
                    if (cv_next < cv_rounds) cv_step();
                }
            }
        }
        if constexpr (XC == 2) {  // before it meets its siblings at the unit's end a warp has converted all its pairs: the warps that
            while (cv_next < cv_rounds) cv_step();  // still wait for a round wait for nobody who waits for them
        }
        finish_unit(unit);
    }
    if constexpr (XC == 2) {  // a warp without tiles still owes the other warps its pairs
        while (cv_next < cv_rounds) cv_step();
    }
    if (lost) sk::linger_after_loss();
}

}  // namespace i8
}  // namespace halo_cuda
