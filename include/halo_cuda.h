/*
 * halo_cuda.h -- C ABI of the B200 (sm_100a) backend for HALO's quantized weight matmul.
 *
 * This is the boundary a `backends/cuda` adapter binds: plain pointers and sizes, no C++ types,
 * no exceptions.  Every entry point returns 0 on success or a negative status; the statuses map
 * one to one onto halo::ErrorCode (include/halo/core/error.h:15-26 of the reference) as
 * status = -(1 + code), so the adapter can rethrow the error class the CPU backend would throw.
 * halo_cuda_last_error() gives the message of the calling thread's last failure.
 *
 * All validation happens on the host before anything is enqueued (the contract of
 * include/halo/backend/backend.h:7-9): a call that returns non-zero has launched nothing and
 * written nothing.  Work is enqueued on the given stream and runs in stream order; results are
 * readable after halo_cuda_stream_sync().  A context and its streams are driven by one thread.
 *
 * There is no CPU fallback anywhere behind this header: with no usable device every call fails.
 */
#ifndef HALO_CUDA_H
#define HALO_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: -(1 + halo::ErrorCode) ------------------------------------------------ */
#define HALO_CUDA_OK 0
#define HALO_CUDA_E_MODEL (-1)       /* element count not a whole number of blocks */
#define HALO_CUDA_E_MEMORY (-2)      /* allocation failure */
#define HALO_CUDA_E_BACKEND (-3)     /* CUDA runtime failure, stream wait timeout */
#define HALO_CUDA_E_KERNEL (-4)      /* shape / alias / range / alignment problem */
#define HALO_CUDA_E_CONFIG (-5)      /* unknown kernel variant id */
#define HALO_CUDA_E_API (-6)         /* malformed call (null struct, bad op id) */
#define HALO_CUDA_E_DEVICE (-7)      /* no usable device */
#define HALO_CUDA_E_UNSUPPORTED (-8) /* valid request this backend does not implement */

/* ---- weight types: ggml ids, equal to halo::DType (include/halo/tensor/dtype.h:18-32) ------- */
#define HALO_CUDA_T_F32 0
#define HALO_CUDA_T_Q4_0 2
#define HALO_CUDA_T_Q8_0 8
#define HALO_CUDA_T_Q4_K 12
#define HALO_CUDA_T_Q6_K 14

/* ---- operator ids of the variant registry: halo::backend::OpId (backend.h:186-206) ---------- */
#define HALO_CUDA_OP_GET_ROWS 0
#define HALO_CUDA_OP_GEMV 3
#define HALO_CUDA_OP_LM_HEAD 14

/* ---- kernel variants of MATMUL (KernelChoice::variant_id, backend.h:173-176).  Ids are explicit
 * and append-only; 0 selects by shape.  "family" groups variants whose rows are bitwise independent
 * of the batch size among themselves (the batch-invariance contract of backend.h:300-304). -------- */
#define HALO_CUDA_GEMV_DEFAULT 0
#define HALO_CUDA_GEMV_EXACT8 1       /* bit-identical to the CPU backend (8-lane dot order) */
#define HALO_CUDA_GEMV_WARP_F32 2     /* fp32 CUDA-core streaming kernel, warp-shuffle reduce */
#define HALO_CUDA_GEMV_MMA_F16X2 3    /* tensor-core skinny kernel, x split into fp16 hi + lo */
#define HALO_CUDA_GEMM_TCGEN05_F16 4  /* prefill: dequant to fp16 in shared memory + tcgen05 MMA */
#define HALO_CUDA_GEMM_TCGEN05_BF16 5 /* same with bf16 operands */
#define HALO_CUDA_GEMV_MMA_M1 6       /* tensor-core single-row specialist (one launch per x row) */
#define HALO_CUDA_GEMV_MMA_R 7        /* tensor-core skinny kernel over REPACKED Q6_K / Q8_0 / Q4_0 rows (halo_cuda_repack_rows) */
#define HALO_CUDA_GEMV_MMA_I8X2 8     /* tensor-core skinny kernel, x as two signed 8-bit digits per element (16-bit fixed point per
                                         256-element super-block), integer MMA; raw Q4_K rows */
#define HALO_CUDA_GEMV_MMA_I8X2_R 9   /* the same arithmetic over REPACKED Q6_K / Q8_0 / Q4_0 rows (halo_cuda_repack_rows) */
#define HALO_CUDA_GEMM_TCGEN05_F16_R 10  /* the prefill GEMM over REPACKED Q6_K / Q8_0 / Q4_0 rows; also what a call with variant 7 or 9,
                                            HALO_CUDA_GEMV_FLAG_ALLOW_GEMM and n_vec >= 64 runs */
#define HALO_CUDA_GEMM_TCGEN05_BF16_R 11 /* same with bf16 operands */
#define HALO_CUDA_GEMV_VARIANT_MAX 11

#define HALO_CUDA_GEMV_FLAG_ALLOW_GEMM 1u /* GemvArgs::allow_gemm: the caller accepts fp16 GEMM numerics */
#define HALO_CUDA_GEMV_FLAG_NO_SCRATCH 0x80000000u /* never touch context scratch: the tensor-core variants then take their
                                                       statically partitioned kernels (another summation order over K, so the
                                                       last bits differ from the default; batches run slower) */

typedef struct HaloCudaCtx HaloCudaCtx; /* one per device, opaque */
typedef void* HaloCudaStream;           /* a cudaStream_t */
typedef void* HaloCudaEvent;            /* a cudaEvent_t */

typedef struct HaloCudaDeviceInfo {
    char name[128];
    char pci_id[16]; /* "vvvv:dddd" vendor:device, the ProfileKey gpu_device field */
    char arch[16];   /* "sm_100a" */
    int32_t cc_major, cc_minor, sm_count, l2_bytes;
    int32_t driver_version, runtime_version; /* as cudaDriverGetVersion / cudaRuntimeGetVersion */
    uint64_t total_bytes;
    int32_t clock_khz, mem_clock_khz;
} HaloCudaDeviceInfo;

/* One registered kernel variant: halo::backend::VariantInfo (backend.h:210-216). */
typedef struct HaloCudaVariant {
    uint32_t id;
    uint32_t op;
    uint32_t family; /* 0 = fp32 exact order, 1 = fp32 reordered, 2 = tensor-core skinny, 3 = tensor-core single-row, 4 = fp16 GEMM,
                        5 = tensor-core skinny over repacked rows, 6 = int8 tensor-core skinny */
    const char* name;
} HaloCudaVariant;

/* MATMUL / QUANT_GEMV: y[t][n] = sum_i x[t][i] * dequant(W)[n][i].
 * Replaces Backend::gemv(Stream&, const GemvArgs&) (backend.h:283-314, 562) as implemented by
 * CpuBackend::gemv (src/backend/cpu_backend.cpp:338-351).  All pointers are device pointers.
 *   w: `rows` rows of row_bytes(wtype, cols) bytes, w_stride bytes apart (0 = dense), any alignment;
 *   x: n_vec rows of cols fp32, x_stride bytes apart (0 = dense), 4-byte aligned;
 *   y: n_vec rows of rows fp32, y_stride bytes apart (0 = dense), 4-byte aligned; must not overlap x or w.
 * rows == 0 or n_vec == 0 is a no-op. */
typedef struct HaloCudaGemv {
    uint32_t wtype;
    uint32_t variant_id;
    const void* w;
    uint64_t w_stride;
    const float* x;
    uint64_t x_stride;
    float* y;
    uint64_t y_stride;
    uint32_t rows, cols, n_vec;
    uint32_t flags;
} HaloCudaGemv;

/* LM head: gemv over the vocabulary + fused argmax.  Replaces Backend::lm_head(Stream&, const
 * LmHeadArgs&) (backend.h:437-460) as implemented by CpuBackend::lm_head (cpu_backend.cpp:669-770).
 *   gemv.y may be null (logits not wanted); result: n_vec triples {index u32, value bits, nan 0/1}
 *   (12 bytes each, backend.h:430); ids (optional): n_vec int32 winners, 0 for a poisoned vector;
 *   valid_rows: rows at or after it are left out of the argmax (0 = no clamp);
 *   row_offset: added to every winning index (the vocabulary offset of a column-split shard). */
typedef struct HaloCudaLmHead {
    HaloCudaGemv gemv;
    uint32_t* result;
    int32_t* ids;
    uint32_t valid_rows;
    uint32_t row_offset;
} HaloCudaLmHead;

/* GET_ROWS-shaped exact dequantization: out[i] = dequant(table row ids[i]), or row i when ids is null.
 * Replaces Backend::get_rows (backend.h:251-262; cpu_backend.cpp:291-311) for the four block formats;
 * the unpacked values are bit-identical to tensor::dequantize_row (src/tensor/quant.cpp:430-435).
 * An id outside [0, n_rows) sets bit 8 (kStatusBadIndex, backend.h:165) of *status (device word,
 * optional) and writes nothing for that row. */
typedef struct HaloCudaGetRows {
    uint32_t type;
    uint32_t variant_id;
    const void* table;
    uint64_t table_stride;
    const int32_t* ids;
    float* out;
    uint64_t out_stride;
    uint32_t n_rows, cols, n_ids;
    uint32_t* status;
} HaloCudaGetRows;

/* ---- device, context, memory, streams ------------------------------------------------------- */
int halo_cuda_device_count(int* count);
int halo_cuda_ctx_create(int device, HaloCudaCtx** ctx);
int halo_cuda_ctx_destroy(HaloCudaCtx* ctx);
int halo_cuda_device_info(HaloCudaCtx* ctx, HaloCudaDeviceInfo* info);
/* Device memory.  The model allocates every activation buffer of a forward through Backend::allocate
 * (src/models/qwen35.cpp:462-465, 542-579), so this is a sub-allocator: blocks come from a per-context pool that keeps
 * freed memory, and cost microseconds.  flags: HALO_CUDA_MALLOC_ZERO clears the block (Backend::allocate is
 * zero-filled, backend.h:523); HALO_CUDA_MALLOC_SHAREABLE takes the block from the driver instead, which
 * halo_cuda_ipc_export needs.  The pointer is usable on every stream when the call returns.  halo_cuda_free waits
 * for the device first, so a block that queued work still uses is never handed out again early. */
#define HALO_CUDA_MALLOC_ZERO 1
#define HALO_CUDA_MALLOC_SHAREABLE 2
int halo_cuda_malloc(HaloCudaCtx* ctx, uint64_t bytes, int flags, void** ptr);
int halo_cuda_free(HaloCudaCtx* ctx, void* ptr);
int halo_cuda_stream_create(HaloCudaCtx* ctx, HaloCudaStream* stream);
int halo_cuda_stream_destroy(HaloCudaCtx* ctx, HaloCudaStream stream);
/* Stream::wait() (backend.h:497): blocks until the stream drains or timeout_ns passes (0 = no limit).
 * A timeout returns HALO_CUDA_E_BACKEND and marks the context lost (Backend::lost(), backend.h:517-520). */
int halo_cuda_stream_sync(HaloCudaCtx* ctx, HaloCudaStream stream, uint64_t timeout_ns);
int halo_cuda_ctx_lost(HaloCudaCtx* ctx); /* 1 once a wait timed out or the device faulted, else 0 */
/* Bounds the device-side wait of halo_cuda_gemv_reduce's adding kernel: it re-reads a peer's word at most `polls` times (about
 * 0.2 us apart; default 2^22, about a second) before it gives up, raises the context's error word and stores nothing, after which
 * the next halo_cuda_stream_sync returns HALO_CUDA_E_BACKEND and the context is lost (Backend::lost(), backend.h:517-520).  The
 * reference injects its failures on the host (tests/unit/runtime/test_engine_faults.cpp:102-357); this knob is the counterpart for
 * the one wait that lives on the device.  polls == 0 restores the default. */
int halo_cuda_ctx_set_peer_wait_polls(HaloCudaCtx* ctx, uint32_t polls);
/* Streams and scratch: the kernels' on-demand scratch is kept per stream, so calls on different streams of one context may overlap on
 * the device; calls on ONE stream reuse that stream's scratch in stream order.  halo_cuda_stream_destroy releases the stream's scratch.
 * (halo_cuda_lm_head_noalloc is the exception: its fixed array is shared by every call on the GPU.)
 * Bytes of context scratch (staged activations, split-K partials, LM-head logits and argmax partials) the context holds right now:
 * memory the kernels allocated on demand beyond the caller's operands.  Stays 0 for a context that only ever made calls that need
 * none (the exact / fp32 variants, HALO_CUDA_GEMV_FLAG_NO_SCRATCH, halo_cuda_lm_head_noalloc). */
int halo_cuda_ctx_scratch_bytes(HaloCudaCtx* ctx, uint64_t* bytes);
/* Backend::upload / download / copy (backend.h:549-552, 476-481); src of an upload must stay valid until the sync. */
int halo_cuda_memcpy_h2d_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream);
int halo_cuda_memcpy_d2h_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream);
int halo_cuda_memcpy_d2d_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream);
int halo_cuda_memset_async(HaloCudaCtx* ctx, void* dst, int value, uint64_t bytes, HaloCudaStream stream);
/* Pinned host staging memory for uploads and downloads. */
int halo_cuda_host_alloc(HaloCudaCtx* ctx, uint64_t bytes, void** ptr);
int halo_cuda_host_free(HaloCudaCtx* ctx, void* ptr);
/* Device timing for the autotuner's Measurement.device_ns (src/autotune/tuner.cpp:133-138). */
int halo_cuda_event_create(HaloCudaCtx* ctx, HaloCudaEvent* event);
int halo_cuda_event_destroy(HaloCudaCtx* ctx, HaloCudaEvent event);
int halo_cuda_event_record(HaloCudaCtx* ctx, HaloCudaEvent event, HaloCudaStream stream);
int halo_cuda_event_elapsed_ns(HaloCudaCtx* ctx, HaloCudaEvent start, HaloCudaEvent stop, uint64_t* ns);

/* ---- geometry, registry, errors ---------------------------------------------------------------- */
/* tensor::row_bytes (src/tensor/quant.cpp:422-428): E_MODEL if cols is not whole blocks, E_UNSUPPORTED for other types. */
int halo_cuda_row_bytes(uint32_t wtype, uint64_t cols, uint64_t* bytes);
/* Backend::variants(op) (backend.h:556): writes up to cap entries, *count = number registered. */
int halo_cuda_variants(uint32_t op, HaloCudaVariant* out, uint32_t cap, uint32_t* count);
/* The variant id 0 resolves to for this call (what the shape heuristic, or an installed plan, picks). */
int halo_cuda_gemv_resolve(HaloCudaCtx* ctx, const HaloCudaGemv* args, uint32_t* variant_id);
/* Installs the autotuner's choice for one shape bucket: calls with variant_id 0, this wtype, rows, cols and
 * n_vec in [n_vec_lo, n_vec_hi] run `variant_id` (the "KernelPlan" join of ADR-001 5.6).  Variants 7 and 9 are refused (E_CONFIG): they
 * read another weight layout, so they travel with the tensor a loader has repacked, not with a shape. */
int halo_cuda_plan_set(HaloCudaCtx* ctx, uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t n_vec_lo, uint32_t n_vec_hi,
                       uint32_t variant_id);
int halo_cuda_plan_clear(HaloCudaCtx* ctx);
size_t halo_cuda_last_error(char* buf, size_t len);
/* The repacked row layout of the variants HALO_CUDA_GEMV_MMA_R and HALO_CUDA_GEMV_MMA_I8X2_R: a byte permutation (plus padding for Q6_K) of every 256-weight
 * group that makes the rows fetchable by the copy engine, the counterpart of tensor::gemv_repack
 * (include/halo/tensor/repack.h:11-36) and of the kGemvRepacked variant (backend.h:178-183).  cols must be a multiple
 * of 256.  halo_cuda_repacked_row_bytes gives the size of a repacked row (E_UNSUPPORTED for types without one);
 * halo_cuda_repack_rows converts `rows` raw GGUF rows (any alignment) into 16-byte aligned repacked rows on the device. */
int halo_cuda_repacked_row_bytes(uint32_t wtype, uint64_t cols, uint64_t* bytes);
/* The variant id a loader passes with a tensor it has repacked: HALO_CUDA_GEMV_MMA_I8X2_R where the x records of one row of
 * `cols` columns fit in shared memory next to the weight ring, else HALO_CUDA_GEMV_MMA_R.  Under a row split (K cut over
 * ranks) pass the LARGEST local K, so that every rank picks the same family and with it the same reduction. */
int halo_cuda_repacked_variant(uint32_t wtype, uint64_t cols, uint32_t* variant_id);
int halo_cuda_repack_rows(HaloCudaCtx* ctx, uint32_t wtype, const void* src, uint64_t src_stride, void* dst, uint64_t dst_stride,
                          uint32_t rows, uint32_t cols, HaloCudaStream stream);

/* ---- the partition of the balanced skinny kernels, for inspection and tests (halo_cuda_gemv_plan: variants 3 and 7) ----------------------
 * Pure host arithmetic, no device needed: how a rows x cols matmul of `wtype` is cut over a GPU with `sm_count` SMs.
 * A CTA is (16 / slices) row blocks of 16 W rows x `slices` interleaved K slices; a unit is that many row blocks, a
 * column one step of 256 * slices elements of K; CTA c walks columns [start[c], start[c + 1]) of the unit-major
 * sequence (unit u = column / cols_per_unit).  The plan depends on nothing else, in particular not on n_vec. */
#define HALO_CUDA_PLAN_MAX_CTAS 160
typedef struct HaloCudaGemvPlan {
    uint32_t slices, ctas, cols_per_unit, reserved;
    uint32_t start[HALO_CUDA_PLAN_MAX_CTAS + 1];
} HaloCudaGemvPlan;
int halo_cuda_gemv_plan(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, HaloCudaGemvPlan* plan);
/* The same for the int8 family (variants 8 and 9), whose CTAs cut K into 1, 2, 4, 8 or 16 slices: whole units per CTA with the
 * fewest tiles per warp, ceil(units / CTAs) * ceil(cols / 256 / slices), or -- where every x record of a row does not fit in
 * shared memory for a tile of eight rows, or where it walks fewer tiles even with the cross-CTA reduction -- the even split of
 * the columns with one slice.  A function of (wtype, rows, cols, sm_count) alone. */
int halo_cuda_gemv_plan_i8(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, HaloCudaGemvPlan* plan);
/* How the int8 family cuts a call of n_vec x rows into launches (host arithmetic, like the plans above).  A launch holds the x
 * records of its rows in shared memory next to the weight ring: all of them (resident, at most `resident_rows` rows), or -- a
 * batch the resident form cannot hold in one launch, where a CTA walks at least eight columns -- a double buffer of `stretch_cols`
 * columns at a time (streamed).  The records are made in the matmul kernel itself (one row; a batch whose CTAs have few to make)
 * or by ONE conversion launch per call.  Whatever the cut, a row's bits are those of its single-row call. */
typedef struct HaloCudaGemvTiles {
    uint32_t tile_rows;     /* x rows of every matmul launch but the last */
    uint32_t launches;      /* matmul launches: passes over the weights */
    uint32_t conversions;   /* conversion launches ahead of them (0 or 1) */
    uint32_t streamed;      /* 1: launches of two rows and up stream their x records */
    uint32_t stretch_cols;  /* columns per stretch of a streamed launch, else 0 */
    uint32_t resident_rows; /* the most rows the resident form holds for this shape */
    uint32_t reserved[2];
} HaloCudaGemvTiles;
int halo_cuda_gemv_tiles_i8(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* tiles);

/* ---- the operators ------------------------------------------------------------------------------ */
int halo_cuda_gemv(HaloCudaCtx* ctx, const HaloCudaGemv* args, HaloCudaStream stream);
/* MATMUL with the fused input norm of GemvArgs::norm_w / norm_eps (backend.h:292-298): y = W (rms_norm(x) * norm_w), `args->x`
 * being the RAW row and norm_w `cols` fp32 (device, 16-byte aligned like x).  Element i of the normalised row is
 * (x[i] * inv) * norm_w[i] with inv = 1 / sqrt(mean(x^2) + norm_eps), the arithmetic of the CPU backend's rms_norm
 * (backends/cpu/ops_basic.cpp:28-30); the mean is summed in the kernel's own fixed order, so the result differs from
 * rms_norm followed by halo_cuda_gemv only through that order -- the latitude the reference gives its own fused norm.
 * As there: one x row only, and only the kernels that have it (variants 3 and 7 with x resident in shared memory);
 * every other case returns HALO_CUDA_E_UNSUPPORTED, never a product over the raw row. */
int halo_cuda_gemv_normed(HaloCudaCtx* ctx, const HaloCudaGemv* args, const float* norm_w, float norm_eps, HaloCudaStream stream);
/* MATMUL with the GDN gates epilogue of GemvArgs::gates (backend.h:299-313): the matmul over a model's fused beta|alpha rows
 * (rows == 2 * n_v, beta rows first) stores, instead of y, sigmoid(y) for row r < n_v and a[j] * softplus(y + dt_bias[j]) for
 * row n_v + j -- the matmul followed by the CPU backend's gdn_gates on the two row halves (backend.h:316-323), with the
 * device's expf / log1pf (a few ulp from the host's).  dt_bias, a: n_v fp32 (device).  As in the reference: F32 or Q8_0
 * weights only, on the fp32 variants (1, 2); every other case returns HALO_CUDA_E_UNSUPPORTED, never plain y. */
int halo_cuda_gemv_gated(HaloCudaCtx* ctx, const HaloCudaGemv* args, const float* dt_bias, const float* a, uint32_t n_v, HaloCudaStream stream);
int halo_cuda_lm_head(HaloCudaCtx* ctx, const HaloCudaLmHead* args, HaloCudaStream stream);
int halo_cuda_get_rows(HaloCudaCtx* ctx, const HaloCudaGetRows* args, HaloCudaStream stream);

/* ---- row-split tensor parallelism: matmul with a peer-memory all-reduce epilogue ------------------------------------
 * One process per GPU.  Each rank allocates a receive buffer with halo_cuda_malloc (zeroed), exports it
 * (halo_cuda_ipc_export), hands the 64-byte handle to its peers over its own channel, and maps the peers'
 * (halo_cuda_ipc_open).  halo_cuda_gemv_reduce then computes this rank's partial product (a row-split projection: the
 * rank holds some columns of every W row, the call's `cols` and x are the rank's share) and, instead of storing it,
 * its matmul kernel pushes every finished row block into slot `rank` of every peer's receive buffer with plain stores
 * over NVLink, each element as one 8-byte word {value, number of the reduction}; a second small kernel reads the
 * `world` slots until every word carries the current number (bounded; on expiry the context's error word is raised and
 * the next stream wait reports E_BACKEND) and adds them in rank order into y, so every rank gets the same bits.  No
 * counterpart in the reference (its backends are single-device); the single-GPU product of the unsplit projection is
 * the oracle.
 *   slots[p]: rank p's receive buffer as mapped on this rank (own: the local pointer), 2 * world * capacity * 8 bytes
 *   epoch, done: two zeroed words of this rank's own memory
 * rows * n_vec must not exceed capacity; the ranks must issue the same sequence of reductions.  Only the tensor-core
 * skinny variants (3, 7, 8, 9) push; others: E_UNSUPPORTED. */
#define HALO_CUDA_MAX_PEERS 8
typedef struct HaloCudaPeerReduce {
    uint32_t world, rank, capacity, reserved;
    void* slots[HALO_CUDA_MAX_PEERS];
    uint32_t* epoch;
    uint32_t* done;
} HaloCudaPeerReduce;
int halo_cuda_ipc_export(HaloCudaCtx* ctx, void* ptr, uint8_t handle[64]);
int halo_cuda_ipc_open(HaloCudaCtx* ctx, const uint8_t handle[64], void** ptr);
int halo_cuda_ipc_close(HaloCudaCtx* ctx, void* ptr);
int halo_cuda_gemv_reduce(HaloCudaCtx* ctx, const HaloCudaGemv* args, const HaloCudaPeerReduce* peers, HaloCudaStream stream);

/* The LM head for callers that cannot allocate device memory while they run (a serving loop whose buffers were all
 * sized at start-up, an embedder with a fixed memory budget).  No counterpart in the reference: its backends
 * allocate their scratch freely.  Same arguments and results as halo_cuda_lm_head, with three differences: the
 * logits buffer gemv.y is required; the argmax partials live in a fixed 64 KiB array inside the library's device
 * image, so ceil(rows / 8192) * n_vec must not exceed 4096 (E_UNSUPPORTED beyond that); and the matmul runs only
 * variants 0-3, which need no scratch of their own.  The array is shared by all calls on a GPU: calls that overlap
 * on the device race on it, so keep them on one stream.  The first call on each device resolves the array's
 * address and should be made before any stream capture begins.  It calls no cudaMalloc / cudaFree. */
int halo_cuda_lm_head_noalloc(HaloCudaCtx* ctx, const HaloCudaLmHead* args, HaloCudaStream stream);

#ifdef __cplusplus
}
#endif
#endif /* HALO_CUDA_H */
