// Building blocks shared by the tensor-core gemv kernels: mma.sync wrappers, the fp16 hi / lo staging of x, the
// per-warp TMA weight ring with bounded mbarrier waits, and the shared-memory header layout.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>

namespace halo_cuda {
namespace mma {

#ifndef HALO_MMA_ROWBLOCKS
#define HALO_MMA_ROWBLOCKS 8
#endif
constexpr int kRowBlocks = HALO_MMA_ROWBLOCKS;  // 16-row blocks per CTA (8: a CTA covers 128 W rows)
constexpr uint32_t kSmemBudget = 220 * 1024;
#ifndef HALO_MMA_CHAINS
#define HALO_MMA_CHAINS 2
#endif
constexpr int kChains = HALO_MMA_CHAINS;  // part of a row's arithmetic: the same for every token count

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


/// Power-of-two scale of one x row from its largest magnitude a: s = 2^(13 - floor(log2 a)) for a normal finite a, else 1;
/// the exponent is clamped so that s and 1/s stay normal.
__device__ __forceinline__ void row_scale(float a, float& s, float& inv) {
    int e = static_cast<int>((__float_as_uint(a) >> 23) & 0xFFu) - 127;
    int se = (a > 0.0f && e < 128) ? 13 - e : 0;
    se = max(-100, min(100, se));
    s = __uint_as_float(static_cast<uint32_t>(127 + se) << 23);
    inv = __uint_as_float(static_cast<uint32_t>(127 - se) << 23);
}

/// Converts super-blocks [c0, c0 + n_sb) of one x row into MMA-fragment order: fp16 hi / lo of x * s per 32-element
/// sub-block (`sub_stride` bytes apart, this token's columns at byte `col_off`), and the sub-block sums / 32 as fp16
/// hi / lo (`sb_stride` bytes per super-block, this token's columns at byte `col_off / 4`).  Called by every thread of
/// a CTA (`nthreads` a multiple of 32); the arithmetic does not depend on who calls it or on the chunking.
/// With `sx16` set, the fp32 sums of x * s over every 16 elements are stored too, at sx16[(16-group index) * n_tok + tok].
__device__ __forceinline__ void stage_row(uint8_t* xs, uint8_t* sx, const float* xrow, float s, uint32_t c0, uint32_t n_sb,
                                          uint32_t sub_stride, uint32_t sb_stride, uint32_t col_off, uint32_t tid, uint32_t nthreads,
                                          float* sx16 = nullptr, uint32_t n_tok = 0, uint32_t tok = 0) {
    const float4* xr = reinterpret_cast<const float4*>(xrow) + c0 * 64u;
    for (uint32_t qd = tid; qd < n_sb * 64u; qd += nthreads) {
        float4 v = xr[qd];
        v.x *= s; v.y *= s; v.z *= s; v.w *= s;
        uint2 hi, lo;
        split4(v, hi, lo);
        const uint32_t sub = qd >> 3, in = qd & 7u;  // 8 quads per 32-element sub-block
        uint8_t* dst = xs + sub * sub_stride + col_off + in * 8u;
        *reinterpret_cast<uint2*>(dst) = hi;
        *reinterpret_cast<uint2*>(dst + 64) = lo;
        float sum = (v.x + v.y) + (v.z + v.w);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if (sx16 != nullptr && (in & 3u) == 0) sx16[(sub * 2u + (in >> 2)) * n_tok + tok] = sum;
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
        if (in == 0) {
            sum *= 0.03125f;  // keeps the fp16 copy in range: |sum| <= 32 * 2^14
            const __half h = __float2half_rn(sum);
            const __half l = __float2half_rn(sum - __half2float(h));
            uint8_t* sd = sx + (sub >> 3) * sb_stride + (col_off >> 2) + (sub & 7u) * 2u;
            *reinterpret_cast<__half*>(sd) = h;
            *reinterpret_cast<__half*>(sd + 16) = l;
        }
    }
}

/// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completing on an mbarrier.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- shared-memory weight ring -------------------------------------------------------------------------------------
// Each warp streams its own rows: per pipeline stage one TMA tile copy (cp.async.bulk.tensor.2d over a tensor map of
// the weight matrix as rows of bytes) brings the 144-byte super-block of its 16 W rows into a 16 x 160-byte slot and
// completes on that stage's mbarrier.  The box is 160 bytes wide: the 16 extra bytes (the next block's header, or
// zero fill past the row end) only pad the slot so that the fragment reads below are bank-conflict-free.  Rows past
// the end of the matrix are zero-filled by the copy engine.  Nothing but the owning warp touches a slot, so the
// only synchronisation is the mbarrier (data arrived) and program order (slot consumed before it is refilled).
constexpr uint32_t kSlotRow = 160, kSlotBytes = 16 * kSlotRow, kStageTx = kSlotBytes;
constexpr uint32_t kWaitSpins = 1u << 14;  // try_wait polls (each blocks for a short hardware-defined time) before a stage is declared lost

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
/// One tile of the tensor map: bytes [x, x + 160) of rows [y, y + 16).  x must be a multiple of 16.
__device__ __forceinline__ void tma_tile_g2s(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

// Shared-memory layout (byte offsets from the dynamic base), for `ncols` = 2 * tokens columns:
//   [0, 16) unused | scales | partial maxima | mbarriers | weight ring |
//   xs:  [sub-block][column][64 B] fp16 x in slot order    sx: [super-block][column][16 B] sub-block sums / 32
constexpr uint32_t kOffXBar = 0, kOffScale = 16, kOffInv = 16 + 64, kOffRed = 16 + 128, kOffBars = 512, kOffRing = 2048;
constexpr uint32_t kOffRounds = 1280;  // int8 family (16 warps, <= 6 stages: barriers end at 1280): up to eight mbarriers of the in-kernel x conversion
constexpr int kMaxWarps = 32;  // kOffRed holds one float per warp, kOffBars eight bytes per warp and stage (<= 6 stages)

// ---- balanced work partition -----------------------------------------------------------------------------------------
// The work of a skinny matmul is the grid of items (16-row block, super-block).  A CTA has kSkWarps = 16 warps,
// arranged as R row blocks x KS interleaved K slices (R * KS = 16): warp (r, ks) of a CTA working on unit u owns row
// block u * R + r and, of that block's super-blocks, sb = k * KS + ks for the unit's columns k = 0 .. ceil(nb / KS) - 1.
// The columns of all units form one sequence (unit-major); a persistent grid of at most one CTA per SM cuts it into
// contiguous ranges, one per CTA, given by a table the host computes from (rows, cols, SM count) alone:
//   * whole units per CTA when that keeps the SMs evenly loaded (no row block is shared between CTAs), else
//   * an even split of the columns, where a unit cut by a range boundary is finished by whichever of its CTAs
//     arrives last: each stores its partial sums, bumps the row block's counter, and the last one adds the partials
//     IN CTA ORDER, so the sum does not depend on arrival order.
// Within a CTA the KS slices of a row block are added in ks order through shared memory.  All warps of a CTA walk the
// same columns, so they can share a stream of x.  Nothing here depends on the batch size.
constexpr uint32_t kSkWarps = 16;   // warps per CTA of the persistent kernels
constexpr uint32_t kSkMaxCtas = 160;

struct SkTable {
    uint32_t parts;                   // CTAs of the grid
    uint32_t cols_per_unit;           // ceil(nb / KS)
    uint32_t start[kSkMaxCtas + 1];   // CTA c owns columns [start[c], start[c + 1])
};

/// Whether the kernels of a weight type may cut K into two in-CTA slices: two columns of x records must fit in shared
/// memory next to the weight ring at every batch size, which the 5 KB ring slots of repacked Q8_0 do not allow.
constexpr bool format_allows_slices(uint32_t wtype) { return wtype != 8u /* Q8_0 */; }

/// Host side of the partition: returns the number of K slices (1 or 2) and fills the table.
/// Columns one CTA walks at most under `ks` slices with whole units per CTA (0: not possible) and with an even split.
/// The choice is a function of (rows, cols, SM count) alone, so every batch size of a shape gets the same partition.
inline uint32_t plan_partition(uint32_t rows, uint32_t nb, uint32_t sms, bool allow_slices, SkTable* table) {
    const uint64_t n_rb = (uint64_t{rows} + 15) / 16;
    sms = std::min(sms, kSkMaxCtas);
    // candidate A: 2 slices, whole units per CTA.  candidate B: 1 slice, even split of the columns, where a CTA pays
    // roughly three columns' time for the cross-CTA reduction of the units its range cuts.
    const uint64_t units_a = (n_rb + 7) / 8, cpu_a = (nb + 1) / 2, parts_a = std::min<uint64_t>(sms, units_a);
    const uint64_t time_a = (units_a + parts_a - 1) / parts_a * cpu_a;
    const uint64_t units_b = (n_rb + 15) / 16, cols_b = units_b * nb, parts_b = std::min<uint64_t>(sms, cols_b);
    const uint64_t time_b = (cols_b + parts_b - 1) / parts_b + (parts_b == units_b ? 0 : 3);
    SkTable& t = *table;
    if (allow_slices && nb >= 2 && time_a <= time_b) {
        t.parts = static_cast<uint32_t>(parts_a);
        t.cols_per_unit = static_cast<uint32_t>(cpu_a);
        for (uint32_t c = 0; c <= t.parts; ++c) t.start[c] = static_cast<uint32_t>(uint64_t{c} * units_a / parts_a * cpu_a);
        return 2;
    }
    t.parts = static_cast<uint32_t>(parts_b);
    t.cols_per_unit = nb;
    for (uint32_t c = 0; c <= t.parts; ++c) t.start[c] = static_cast<uint32_t>(uint64_t{c} * cols_b / parts_b);
    return 1;
}

/// The partition of the int8 kernels, whose CTAs cut K into 1, 2, 4, 8 or 16 in-CTA slices (R = 16 / KS row blocks per unit).
/// With whole units per CTA nothing crosses CTAs, and a launch lasts about as long as the tiles one warp walks:
/// ceil(units / CTAs) * ceil(nb / KS).  The fewest tiles win, ties go to fewer slices (more rows per CTA share an x record).
/// Every unit of a sliced partition ends with the slices' sums meeting in shared memory (KS - 1 records added behind two named
/// barriers), charged KS / 16 of a tile: with one or two tiles per unit that is what a launch spends its time on (128256 x 4096
/// under sixteen slices, 55 tiles and 55 such meetings per warp, ran at 0.60 of the HBM rate; under two slices 56 tiles run at 0.9).
/// Slices need every x record of a row resident in shared memory (`slices_ok`: they fit for a tile of eight x rows); without
/// them, and where it walks fewer tiles even with the cross-CTA reduction (about `kReducePenalty` tiles' time), the even
/// split of plan_partition's candidate B.  Returns KS; a function of (rows, cols, SM count) alone.
constexpr uint32_t kReducePenalty = 4;
inline uint32_t plan_partition_i8(uint32_t rows, uint32_t nb, uint32_t sms, bool slices_ok, SkTable* table) {
    const uint64_t n_rb = (uint64_t{rows} + 15) / 16;
    sms = std::min(sms, kSkMaxCtas);
    SkTable& t = *table;
    const uint64_t units_b = (n_rb + 15) / 16, cols_b = units_b * nb, parts_b = std::max<uint64_t>(1, std::min<uint64_t>(sms, cols_b));
    // costs in sixteenths of a tile
    uint64_t best = 16 * ((cols_b + parts_b - 1) / parts_b + (parts_b == units_b ? 0 : kReducePenalty));
    uint32_t best_ks = 1;
    if (slices_ok) {
        for (uint32_t ks = 2; ks <= kSkWarps && ks / 2 < std::max(nb, 1u); ks *= 2) {  // no more slices than the next power of two above nb
            const uint64_t units = (n_rb + kSkWarps / ks - 1) / (kSkWarps / ks), parts = std::max<uint64_t>(1, std::min<uint64_t>(sms, units));
            const uint64_t tiles = (units + parts - 1) / parts * (16 * ((nb + ks - 1) / ks) + ks);
            if (tiles < best) best = tiles, best_ks = ks;
        }
    }
    if (best_ks == 1) {
        t.parts = static_cast<uint32_t>(parts_b);
        t.cols_per_unit = nb;
        for (uint32_t c = 0; c <= t.parts; ++c) t.start[c] = static_cast<uint32_t>(uint64_t{c} * cols_b / parts_b);
        return 1;
    }
    const uint64_t R = kSkWarps / best_ks, units = (n_rb + R - 1) / R, cpu = (nb + best_ks - 1) / best_ks, parts = std::max<uint64_t>(1, std::min<uint64_t>(sms, units));
    t.parts = static_cast<uint32_t>(parts);
    t.cols_per_unit = static_cast<uint32_t>(cpu);
    for (uint32_t c = 0; c <= t.parts; ++c) t.start[c] = static_cast<uint32_t>(uint64_t{c} * units / parts * cpu);
    return best_ks;
}

/// Row-split tensor parallelism: instead of storing a finished row block to y, push it into slot `rank` of every
/// peer's receive buffer (peer-mapped memory, plain stores over NVLink).  Every element travels as one 8-byte word
/// {value bits, number of the reduction}: the word is written and read atomically, so the receiver needs no flag
/// and the sender no fence — an element is valid as soon as its tag is the reduction the receiver is waiting for.
/// world == 0: not in use.  Receive buffer of a rank: [2 ping-pong sets][world slots][capacity] words; *epoch counts
/// the reductions this rank has finished (the sender tags with *epoch + 1).
constexpr uint32_t kMaxPeers = 8;
struct PeerPush {
    uint32_t world, rank, capacity;
    uint32_t tok0;  // first x row of this launch within the call (calls of more than 16 rows run in tiles)
    unsigned long long* slots[kMaxPeers];
    const uint32_t* epoch;
};

__device__ __forceinline__ unsigned long long peer_word(float v, uint32_t tag) {
    return (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(v);
}
/// The push of one tagged word: a relaxed system-scope store, the counterpart of the receiver's relaxed system-scope load
/// (a plain store racing that load would be a data race in the PTX memory model; this costs the same).
__device__ __forceinline__ void peer_store(unsigned long long* p, unsigned long long w) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

/// Sums of one row block (this lane: rows g and g + 8 for its G token columns) -> y: directly when this CTA covered
/// all of the unit's columns, else through the partial store and the last-arriver reduction.  `part` holds 2 records
/// per CTA and row-block slot r (record 0: the unit the CTA's range starts in, record 1: the unit it ends in) of
/// 32 lanes x 2G floats; `counters` one zeroed word per row block, left zeroed.  R: row blocks per unit.
template <int G, int NTOK>
__device__ __forceinline__ void sk_flush_r(const float (&acc)[G][2], uint32_t unit, uint32_t r, uint32_t R, const SkTable& tb, uint32_t cta, float* part,
                                           uint32_t* counters, float* y, uint64_t y_stride, uint32_t rows, uint32_t lane,
                                           uint32_t g /* the W row of the block (0..7, and + 8) this lane's sums belong to */, const PeerPush& peer) {
    const uint32_t t = lane & 3u, rb = unit * R + r;
    const uint32_t u_lo = unit * tb.cols_per_unit, u_hi = u_lo + tb.cols_per_unit;  // the unit's columns
    uint32_t c_lo = cta, c_hi = cta;
    while (c_lo > 0 && tb.start[c_lo] > u_lo) --c_lo;
    while (c_hi + 1 < tb.parts && tb.start[c_hi + 1] < u_hi) ++c_hi;
    auto record = [&](uint32_t c) {
        const uint32_t rec = tb.start[c] >= u_lo ? 0u : 1u;  // the range starts inside this unit, or ends in it
        return reinterpret_cast<float2*>(part) + (((uint64_t{c} * 2 + rec) * R + r) * 32 + lane) * G;
    };
    float sum[G][2];
#pragma unroll
    for (int gi = 0; gi < G; ++gi) sum[gi][0] = acc[gi][0], sum[gi][1] = acc[gi][1];
    if (c_lo != c_hi) {
        float2* mine = record(cta);
#pragma unroll
        for (int gi = 0; gi < G; ++gi) __stcg(mine + gi, make_float2(acc[gi][0], acc[gi][1]));
        // release this warp's record and acquire the others' in one atomic: the barrier before it makes the other lanes'
        // stores part of what lane 0 releases, the one after it orders their loads behind what lane 0 acquired
        __syncwarp();
        uint32_t old = 0;
        if (lane == 0) asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(counters + rb) : "memory");
        old = __shfl_sync(0xFFFFFFFFu, old, 0);
        if (old != c_hi - c_lo) return;  // another CTA will finish this block
        __syncwarp();
        // the partials are added in CTA order; they are fetched kBatch contributors at a time so that the loads overlap
        constexpr uint32_t kBatch = G <= 1 ? 8 : G == 2 ? 4 : 2;
        for (uint32_t c0 = c_lo; c0 <= c_hi; c0 += kBatch) {
            float2 v[kBatch][G];
#pragma unroll
            for (uint32_t i = 0; i < kBatch; ++i) {
                if (c0 + i <= c_hi) {
                    const float2* p = record(c0 + i);
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) v[i][gi] = __ldcg(p + gi);
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < kBatch; ++i) {
                if (c0 + i <= c_hi) {
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) {
                        if (c0 + i == c_lo) sum[gi][0] = v[i][gi].x, sum[gi][1] = v[i][gi].y;
                        else sum[gi][0] += v[i][gi].x, sum[gi][1] += v[i][gi].y;
                    }
                }
            }
        }
        if (lane == 0) counters[rb] = 0;
    }
    if (peer.world != 0) {
        const uint32_t next = *peer.epoch + 1u, set = next & 1u;
        const uint64_t slot = (uint64_t{set} * peer.world + peer.rank) * peer.capacity;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const uint32_t tk = 4u * gi + t;
            if (tk < NTOK) {
                const uint32_t n0 = rb * 16u + g, n1 = n0 + 8u;
                const uint64_t at = slot + uint64_t{peer.tok0 + tk} * rows;  // the pushed rows are dense: [x row][W row]
                const unsigned long long w0 = peer_word(sum[gi][0], next), w1 = peer_word(sum[gi][1], next);
                for (uint32_t p = 0; p < peer.world; ++p) {
                    if (n0 < rows) peer_store(peer.slots[p] + at + n0, w0);
                    if (n1 < rows) peer_store(peer.slots[p] + at + n1, w1);
                }
            }
        }
        return;
    }
#pragma unroll
    for (int gi = 0; gi < G; ++gi) {
        const uint32_t tk = 4u * gi + t;
        if (tk < NTOK) {
            float* yr = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{tk} * y_stride);
            const uint32_t n0 = rb * 16u + g, n1 = n0 + 8u;
            if (n0 < rows) yr[n0] = sum[gi][0];
            if (n1 < rows) yr[n1] = sum[gi][1];
        }
    }
}

template <int G, int NTOK, int R>
__device__ __forceinline__ void sk_flush(const float (&acc)[G][2], uint32_t unit, uint32_t r, const SkTable& tb, uint32_t cta, float* part,
                                         uint32_t* counters, float* y, uint64_t y_stride, uint32_t rows, uint32_t lane, uint32_t g,
                                         const PeerPush& peer) {
    sk_flush_r<G, NTOK>(acc, unit, r, static_cast<uint32_t>(R), tb, cta, part, counters, y, y_stride, rows, lane, g, peer);
}

}  // namespace mma
}  // namespace halo_cuda
