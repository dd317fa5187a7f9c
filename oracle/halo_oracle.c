/*
 * CPU oracle for the quantized weight matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CPU backend for
 * MATMUL / QUANT_GEMV and the fused LM head, so that the CUDA kernels can be checked on a
 * machine where the reference sources are absent.  It is never linked into, imported by or
 * called from the product library; only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark use it.
 *
 * Parity status: PINNED.  The restatement is compared bit for bit with (a) the reference's
 * own CPU backend compiled from its sources (oracle/_ref, see build_ref.sh), (b) gguf-py's
 * dequantizer, and (c) the reference's hand-built known-answer blocks; the outputs of (a)
 * and (b) are committed as fixtures under tests/golden/.
 *
 * Every function names the reference code it follows (paths relative to the reference tree).
 * Build with: gcc -O2 -ffp-contract=off -fPIC -shared -pthread   (no -ffast-math, no FMA
 * contraction: the accumulation order below is part of the result).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HALO_T_F32 0
#define HALO_T_Q4_0 2
#define HALO_T_Q8_0 8
#define HALO_T_Q4_K 12
#define HALO_T_Q6_K 14

#define HALO_ORACLE_OK 0
#define HALO_ORACLE_E_MODEL (-1)       /* element count is not a whole number of blocks */
#define HALO_ORACLE_E_UNSUPPORTED (-8) /* type outside {F32, Q4_0, Q8_0, Q4_K, Q6_K} */
#define HALO_ORACLE_E_KERNEL (-4)      /* shape / stride problem */
#define HALO_ORACLE_E_MEMORY (-2)

/* ---- half precision ------------------------------------------------------------------ */

/* Exact widening of an IEEE binary16 value, subnormals, infinities and NaN payloads
 * included (include/halo/tensor/fp16.h:19-37 gives the same value for every input). */
float halo_oracle_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Round-to-nearest-even narrowing; overflow gives infinity, NaN gives 0x7E00 | sign
 * (include/halo/tensor/fp16.h:39-59). */
uint16_t halo_oracle_fp32_to_fp16(float f) {
    uint32_t w;
    memcpy(&w, &f, 4);
    const uint16_t sign = (uint16_t)((w >> 16) & 0x8000u);
    const uint32_t a = w & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7C00u); /* >= 65536: infinity */
    if (a < 0x33000000u) return sign;                        /* < 2^-25: zero */
    const int e = (int)(a >> 23) - 127;
    uint32_t man = (a & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    int shift;                                   /* bits dropped from the significand */
    uint32_t base;
    if (e < -14) { /* subnormal half: value = man * 2^(e-23), unit 2^-24 */
        shift = -e - 1; /* 13 + (-14 - e) */
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7FFFFFu;
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    /* a carry out of the mantissa moves into the exponent field, which is the right value
     * (and reaches 0x7C00 = infinity for 65520 and above). */
    return (uint16_t)(sign | (base + q));
}

static float f16_at(const uint8_t* p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return halo_oracle_fp16_to_fp32(h);
}

/* ---- block geometry ------------------------------------------------------------------ */

/* ggml type table rows for the five types (src/tensor/dtype.cpp:19-51). */
static int type_geometry(int type, int64_t* block_elems, int64_t* block_bytes) {
    switch (type) {
        case HALO_T_F32: *block_elems = 1; *block_bytes = 4; return 0;
        case HALO_T_Q4_0: *block_elems = 32; *block_bytes = 18; return 0;
        case HALO_T_Q8_0: *block_elems = 32; *block_bytes = 34; return 0;
        case HALO_T_Q4_K: *block_elems = 256; *block_bytes = 144; return 0;
        case HALO_T_Q6_K: *block_elems = 256; *block_bytes = 210; return 0;
        default: return HALO_ORACLE_E_UNSUPPORTED;
    }
}

/* Bytes of a row of n elements, or a negative error (src/tensor/quant.cpp:411-428:
 * n must be non-negative and a whole number of blocks). */
int64_t halo_oracle_row_bytes(int type, int64_t n) {
    int64_t be, bb;
    const int rc = type_geometry(type, &be, &bb);
    if (rc != 0) return rc;
    if (n < 0 || n % be != 0) return HALO_ORACLE_E_MODEL;
    const int64_t nb = n / be;
    if (nb > INT64_MAX / bb) return HALO_ORACLE_E_MODEL;
    return nb * bb;
}

/* ---- dequantizers (float expressions keep the reference's evaluation order) ------------ */

/* {f16 d; u8 qs[16]}: low nibbles are elements 0..15, high nibbles 16..31, y = (q-8)*d
 * (src/tensor/quant.cpp:79-90). */
static void deq_q4_0(const uint8_t* x, float* y, size_t nb) {
    for (size_t i = 0; i < nb; ++i, x += 18, y += 32) {
        const float d = f16_at(x);
        for (int j = 0; j < 16; ++j) {
            y[j] = (float)((int)(x[2 + j] & 0x0F) - 8) * d;
            y[j + 16] = (float)((int)(x[2 + j] >> 4) - 8) * d;
        }
    }
}

/* {f16 d; i8 qs[32]}: y = q*d (src/tensor/quant.cpp:143-151). */
static void deq_q8_0(const uint8_t* x, float* y, size_t nb) {
    for (size_t i = 0; i < nb; ++i, x += 34, y += 32) {
        const float d = f16_at(x);
        for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)x[2 + j] * d;
    }
}

/* The 6-bit (scale, min) code pair of sub-block j from the 12 packed bytes
 * (src/tensor/quant.cpp:236-244). */
static void q4k_codes(int j, const uint8_t* s, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = (uint8_t)(s[j] & 63);
        *mn = (uint8_t)(s[j + 4] & 63);
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]}: per 64 elements the low nibbles of 32 bytes
 * form sub-block 2g and the high nibbles sub-block 2g+1; y = (d*sc)*q - (dmin*m), product
 * and difference rounded separately (src/tensor/quant.cpp:247-269). */
static void deq_q4_k(const uint8_t* x, float* y, size_t nb) {
    for (size_t i = 0; i < nb; ++i, x += 144) {
        const float d = f16_at(x);
        const float dmin = f16_at(x + 2);
        const uint8_t* q = x + 16;
        for (int g = 0; g < 4; ++g, q += 32) {
            uint8_t sc, mn;
            q4k_codes(2 * g, x + 4, &sc, &mn);
            const float d1 = d * (float)sc;
            const float m1 = dmin * (float)mn;
            q4k_codes(2 * g + 1, x + 4, &sc, &mn);
            const float d2 = d * (float)sc;
            const float m2 = dmin * (float)mn;
            for (int l = 0; l < 32; ++l) {
                const float p = d1 * (float)(q[l] & 0x0F);
                *y++ = p - m1;
            }
            for (int l = 0; l < 32; ++l) {
                const float p = d2 * (float)(q[l] >> 4);
                *y++ = p - m2;
            }
        }
    }
}

/* {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}: y = (d*scale)*(q-32), four interleaved
 * 32-element runs per 128-element half (src/tensor/quant.cpp:302-327). */
static void deq_q6_k(const uint8_t* x, float* y, size_t nb) {
    for (size_t i = 0; i < nb; ++i, x += 210) {
        const float d = f16_at(x + 208);
        const uint8_t* ql = x;
        const uint8_t* qh = x + 128;
        const int8_t* sc = (const int8_t*)(x + 192);
        for (int half = 0; half < 2; ++half, y += 128, ql += 64, qh += 32, sc += 8) {
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int q1 = (int)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                const float s0 = d * (float)sc[is + 0];
                const float s2 = d * (float)sc[is + 2];
                const float s4 = d * (float)sc[is + 4];
                const float s6 = d * (float)sc[is + 6];
                y[l + 0] = s0 * (float)q1;
                y[l + 32] = s2 * (float)q2;
                y[l + 64] = s4 * (float)q3;
                y[l + 96] = s6 * (float)q4;
            }
        }
    }
}

/* tensor::dequantize_row (src/tensor/quant.cpp:430-435): n elements, whole blocks only. */
int halo_oracle_dequantize_row(int type, const void* src, float* dst, int64_t n) {
    int64_t be, bb;
    const int rc = type_geometry(type, &be, &bb);
    if (rc != 0) return rc;
    if (n < 0 || n % be != 0) return HALO_ORACLE_E_MODEL;
    const size_t nb = (size_t)(n / be);
    const uint8_t* x = (const uint8_t*)src;
    switch (type) {
        case HALO_T_F32: memcpy(dst, src, (size_t)n * 4); break;
        case HALO_T_Q4_0: deq_q4_0(x, dst, nb); break;
        case HALO_T_Q8_0: deq_q8_0(x, dst, nb); break;
        case HALO_T_Q4_K: deq_q4_k(x, dst, nb); break;
        case HALO_T_Q6_K: deq_q6_k(x, dst, nb); break;
        default: return HALO_ORACLE_E_UNSUPPORTED;
    }
    return HALO_ORACLE_OK;
}

/* ---- the dot product -------------------------------------------------------------------- */

/* Eight interleaved fp32 partial sums over i = j (mod 8) in increasing i, combined as
 * ((a0+a4)+(a1+a5))+((a2+a6)+(a3+a7)), a sequential tail, then s + tail; products and sums
 * are rounded separately (backends/cpu/kernel_common.h:16-27). */
float halo_oracle_dot(const float* a, const float* b, size_t n) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t i = 0;
    for (; i + 8 <= n; i += 8) {
        for (int j = 0; j < 8; ++j) {
            const float p = a[i + j] * b[i + j];
            acc[j] = acc[j] + p;
        }
    }
    float tail = 0.0f;
    for (; i < n; ++i) {
        const float p = a[i] * b[i];
        tail = tail + p;
    }
    const float s = ((acc[0] + acc[4]) + (acc[1] + acc[5])) + ((acc[2] + acc[6]) + (acc[3] + acc[7]));
    return s + tail;
}

/* fp64 accumulation of the dequantized row times x, rounded once to fp32
 * (src/tensor/quant.cpp:447-466); a third opinion for accuracy bounds. */
int halo_oracle_vec_dot_row(int type, const void* row, const float* x, int64_t n, float* out) {
    float* w = (float*)malloc((size_t)(n > 0 ? n : 1) * sizeof(float));
    if (!w) return HALO_ORACLE_E_MEMORY;
    const int rc = halo_oracle_dequantize_row(type, row, w, n);
    if (rc == 0) {
        double acc = 0.0;
        for (int64_t i = 0; i < n; ++i) acc += (double)w[i] * (double)x[i];
        *out = (float)acc;
    }
    free(w);
    return rc;
}

/* ---- matmul ------------------------------------------------------------------------------ */

typedef struct {
    int type;
    const uint8_t* w;
    uint64_t w_stride;
    const float* x;
    uint64_t x_stride; /* elements */
    float* y;
    uint64_t y_stride; /* elements */
    uint32_t rows, cols, n_vec;
    uint32_t row_begin, row_end; /* this worker's W rows */
    int rc;
} gemv_job;

/* One worker: blocks of 16 W rows are dequantized once to fp32 and every x row is dotted
 * with each of them (backends/cpu/matmul.cpp:17, 46-58).  The block size and the split over
 * threads do not change any output bit; they are kept for a like-for-like CPU timing. */
static void* gemv_worker(void* arg) {
    gemv_job* j = (gemv_job*)arg;
    const size_t K = j->cols;
    float* scratch = (float*)malloc(16 * (K ? K : 1) * sizeof(float));
    if (!scratch) {
        j->rc = HALO_ORACLE_E_MEMORY;
        return NULL;
    }
    for (uint32_t n0 = j->row_begin; n0 < j->row_end; n0 += 16) {
        const uint32_t nn = (j->row_end - n0) < 16 ? (j->row_end - n0) : 16;
        const float* wb = scratch;
        size_t wb_stride = K;
        if (j->type == HALO_T_F32) {
            wb = (const float*)(j->w + (uint64_t)n0 * j->w_stride);
            wb_stride = j->w_stride / 4;
        } else {
            for (uint32_t r = 0; r < nn; ++r) {
                const int rc = halo_oracle_dequantize_row(j->type, j->w + (uint64_t)(n0 + r) * j->w_stride,
                                                          scratch + (size_t)r * K, (int64_t)K);
                if (rc != 0) {
                    j->rc = rc;
                    free(scratch);
                    return NULL;
                }
            }
        }
        for (uint32_t t = 0; t < j->n_vec; ++t) {
            const float* xt = j->x + (uint64_t)t * j->x_stride;
            float* yt = j->y + (uint64_t)t * j->y_stride + n0;
            for (uint32_t n = 0; n < nn; ++n) yt[n] = halo_oracle_dot(xt, wb + (size_t)n * wb_stride, K);
        }
    }
    free(scratch);
    return NULL;
}

/* y[t][n] = dot(x[t], dequant(W[n])) for t < n_vec, n < rows (CpuBackend::gemv,
 * src/backend/cpu_backend.cpp:338-351 -> cpu::matmul, backends/cpu/matmul.cpp:37-59).
 * w_stride in bytes (0 = dense rows), x_stride / y_stride in elements (0 = dense).
 * `threads` workers take contiguous ranges of 16-row blocks, like the reference's static
 * partition (include/halo/backends/cpu/thread_pool.h:64-72). */
int halo_oracle_gemv(int type, const void* w, uint64_t w_stride, const float* x, uint64_t x_stride, float* y,
                     uint64_t y_stride, uint32_t rows, uint32_t cols, uint32_t n_vec, int threads) {
    const int64_t rb = halo_oracle_row_bytes(type, (int64_t)cols);
    if (rb < 0) return (int)rb;
    if (w_stride == 0) w_stride = (uint64_t)rb;
    if (x_stride == 0) x_stride = cols;
    if (y_stride == 0) y_stride = rows;
    if ((rows > 1 && w_stride < (uint64_t)rb) || (n_vec > 1 && (x_stride < cols || y_stride < rows)))
        return HALO_ORACLE_E_KERNEL;
    if (rows == 0 || n_vec == 0) return HALO_ORACLE_OK;
    const uint32_t n_blocks = (rows + 15) / 16;
    if (threads < 1) threads = 1;
    if ((uint32_t)threads > n_blocks) threads = (int)n_blocks;
    gemv_job* jobs = (gemv_job*)calloc((size_t)threads, sizeof(gemv_job));
    pthread_t* tids = (pthread_t*)calloc((size_t)threads, sizeof(pthread_t));
    if (!jobs || !tids) {
        free(jobs);
        free(tids);
        return HALO_ORACLE_E_MEMORY;
    }
    const uint32_t base = n_blocks / (uint32_t)threads, extra = n_blocks % (uint32_t)threads;
    uint32_t b = 0;
    for (int i = 0; i < threads; ++i) {
        const uint32_t nb = base + ((uint32_t)i < extra ? 1u : 0u);
        gemv_job j = {type, (const uint8_t*)w, w_stride, x, x_stride, y, y_stride, rows, cols, n_vec, b * 16, 0, 0};
        b += nb;
        j.row_end = b * 16 < rows ? b * 16 : rows;
        jobs[i] = j;
    }
    for (int i = 1; i < threads; ++i) pthread_create(&tids[i], NULL, gemv_worker, &jobs[i]);
    gemv_worker(&jobs[0]); /* the caller runs part 0 */
    int rc = jobs[0].rc;
    for (int i = 1; i < threads; ++i) {
        pthread_join(tids[i], NULL);
        if (rc == 0) rc = jobs[i].rc;
    }
    free(jobs);
    free(tids);
    return rc;
}

/* ---- LM head: gemv over the vocabulary + argmax --------------------------------------------- */

/* CpuBackend::lm_head (src/backend/cpu_backend.cpp:669-770): the logits are exactly those of
 * the gemv; per vector the winner is the first strictly greatest non-NaN value among rows
 * below the limit (valid_rows, 0 = all rows); any NaN logit (at any row, also at or after the
 * limit) poisons that vector only: its triple becomes {0xFFFFFFFF, bits of quiet NaN, 1} and
 * its dense id 0.  result: n_vec triples {index, value bits, nan}; logits (optional): n_vec
 * rows of `rows` floats, logits_stride elements apart; ids (optional): n_vec int32. */
int halo_oracle_lm_head(int type, const void* w, uint64_t w_stride, const float* x, uint64_t x_stride,
                        float* logits, uint64_t logits_stride, uint32_t* result, int32_t* ids, uint32_t rows,
                        uint32_t cols, uint32_t n_vec, uint32_t valid_rows, int threads) {
    if (n_vec == 0) return HALO_ORACLE_OK;
    float* buf = logits;
    uint64_t stride = logits_stride ? logits_stride : rows;
    if (!buf) {
        buf = (float*)malloc((size_t)n_vec * (rows ? rows : 1) * sizeof(float));
        if (!buf) return HALO_ORACLE_E_MEMORY;
        stride = rows;
    }
    const int rc = halo_oracle_gemv(type, w, w_stride, x, x_stride, buf, stride, rows, cols, n_vec, threads);
    if (rc == 0) {
        const uint32_t limit = valid_rows > 0 && valid_rows < rows ? valid_rows : rows;
        for (uint32_t t = 0; t < n_vec; ++t) {
            const float* row = buf + (uint64_t)t * stride;
            int32_t best = -1;
            float best_v = 0.0f;
            int nan = 0;
            for (uint32_t c = 0; c < rows; ++c) {
                if (isnan(row[c])) {
                    nan = 1;
                    continue;
                }
                if (c < limit && (best < 0 || row[c] > best_v)) {
                    best = (int32_t)c;
                    best_v = row[c];
                }
            }
            uint32_t bits;
            if (nan) {
                best = -1;
                bits = 0x7FC00000u;
            } else {
                memcpy(&bits, &best_v, 4);
            }
            result[3 * t + 0] = (uint32_t)best;
            result[3 * t + 1] = bits;
            result[3 * t + 2] = nan ? 1u : 0u;
            if (ids) ids[t] = best < 0 ? 0 : best;
        }
    }
    if (!logits) free(buf);
    return rc;
}
