// Context, memory, streams, registry, operand validation and dispatch of libhalo_cuda.so.
#include <chrono>
#include <cstring>
#include <new>
#include <string>
#include <thread>

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {

namespace {
thread_local std::string g_error;

constexpr HaloCudaVariant kGemvVariants[] = {
    {HALO_CUDA_GEMV_EXACT8, HALO_CUDA_OP_GEMV, 0, "gemv_exact8"},
    {HALO_CUDA_GEMV_WARP_F32, HALO_CUDA_OP_GEMV, 1, "gemv_warp_f32"},
    {HALO_CUDA_GEMV_MMA_F16X2, HALO_CUDA_OP_GEMV, 2, "gemv_mma_f16x2"},
    {HALO_CUDA_GEMM_TCGEN05_F16, HALO_CUDA_OP_GEMV, 4, "gemm_tcgen05_f16"},
    {HALO_CUDA_GEMM_TCGEN05_BF16, HALO_CUDA_OP_GEMV, 4, "gemm_tcgen05_bf16"},
    {HALO_CUDA_GEMV_MMA_M1, HALO_CUDA_OP_GEMV, 3, "gemv_mma_m1"},
    {HALO_CUDA_GEMV_MMA_R, HALO_CUDA_OP_GEMV, 5, "gemv_mma_r"},
    {HALO_CUDA_GEMV_MMA_I8X2, HALO_CUDA_OP_GEMV, 6, "gemv_mma_i8x2"},
    {HALO_CUDA_GEMV_MMA_I8X2_R, HALO_CUDA_OP_GEMV, 6, "gemv_mma_i8x2_r"},
    {HALO_CUDA_GEMM_TCGEN05_F16_R, HALO_CUDA_OP_GEMV, 4, "gemm_tcgen05_f16_r"},
    {HALO_CUDA_GEMM_TCGEN05_BF16_R, HALO_CUDA_OP_GEMV, 4, "gemm_tcgen05_bf16_r"},
};
constexpr HaloCudaVariant kLmHeadVariants[] = {{1, HALO_CUDA_OP_LM_HEAD, 1, "lm_head_gemv_argmax2"}};
constexpr HaloCudaVariant kGetRowsVariants[] = {{1, HALO_CUDA_OP_GET_ROWS, 0, "get_rows_exact"}};

bool ranges_overlap(const void* a, uint64_t a_bytes, const void* b, uint64_t b_bytes) {
    if (a_bytes == 0 || b_bytes == 0) return false;
    const auto lo1 = reinterpret_cast<uintptr_t>(a), lo2 = reinterpret_cast<uintptr_t>(b);
    return lo1 < lo2 + b_bytes && lo2 < lo1 + a_bytes;
}

bool mul_overflows(uint64_t a, uint64_t b) { return b != 0 && a > UINT64_MAX / b; }
}  // namespace

int fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
    return status;
}

bool type_info(uint32_t wtype, TypeInfo* out) {
    switch (wtype) {
        case HALO_CUDA_T_F32: *out = {1, 4}; return true;
        case HALO_CUDA_T_Q4_0: *out = {32, 18}; return true;
        case HALO_CUDA_T_Q8_0: *out = {32, 34}; return true;
        case HALO_CUDA_T_Q4_K: *out = {256, 144}; return true;
        case HALO_CUDA_T_Q6_K: *out = {256, 210}; return true;
        default: return false;
    }
}

int enter(HaloCudaCtx* ctx) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    if (ctx->lost) return fail(HALO_CUDA_E_DEVICE, "device %d is lost (an earlier wait timed out or faulted)", ctx->device);
    HC_CUDA(cudaSetDevice(ctx->device));
    return 0;
}

int workspace(HaloCudaCtx* ctx, int slot, uint64_t bytes, cudaStream_t stream, void** out, bool zeroed) {
    HaloCudaCtx::Scratch& sc = ctx->scratch[stream];  // the calling stream's own set: nothing another stream runs touches it
    if (bytes > sc.bytes[slot]) {
        // Work already enqueued on this stream may still read the old block: drain before releasing it.
        HC_CUDA(cudaStreamSynchronize(stream));
        if (sc.block[slot] != nullptr) HC_CUDA(cudaFree(sc.block[slot]));
        sc.block[slot] = nullptr;
        sc.bytes[slot] = 0;
        const uint64_t want = (bytes + (1u << 20) - 1) & ~uint64_t{(1u << 20) - 1};
        HC_CUDA(cudaMalloc(&sc.block[slot], want));
        sc.bytes[slot] = want;
        if (zeroed) HC_CUDA(cudaMemsetAsync(sc.block[slot], 0, want, stream));
    }
    *out = sc.block[slot];
    return 0;
}

bool reads_repacked_rows(uint32_t variant_id) {
    return variant_id == HALO_CUDA_GEMV_MMA_R || variant_id == HALO_CUDA_GEMV_MMA_I8X2_R || variant_id == HALO_CUDA_GEMM_TCGEN05_F16_R ||
           variant_id == HALO_CUDA_GEMM_TCGEN05_BF16_R;
}

bool gemv_i8_r_supports(const GemvCall& c) {
    switch (c.wtype) {
        case HALO_CUDA_T_Q6_K: return gemv_i8_q6kr_supports(c);
        case HALO_CUDA_T_Q8_0: return gemv_i8_q80r_supports(c);
        case HALO_CUDA_T_Q4_0: return gemv_i8_q40r_supports(c);
        default: return false;
    }
}

uint32_t repacked_variant(uint32_t wtype, uint32_t cols) {
    const bool i8 = wtype == HALO_CUDA_T_Q6_K ? gemv_i8_q6kr_fits(cols) : wtype == HALO_CUDA_T_Q8_0 ? gemv_i8_q80r_fits(cols) : wtype == HALO_CUDA_T_Q4_0 ? gemv_i8_q40r_fits(cols) : false;
    return i8 ? HALO_CUDA_GEMV_MMA_I8X2_R : HALO_CUDA_GEMV_MMA_R;
}

uint32_t gemv_i8_plan(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, mma::SkTable* table) {
    switch (wtype) {
        case HALO_CUDA_T_Q6_K: return gemv_i8_q6kr_plan(rows, cols, sm_count, table);
        case HALO_CUDA_T_Q8_0: return gemv_i8_q80r_plan(rows, cols, sm_count, table);
        case HALO_CUDA_T_Q4_0: return gemv_i8_q40r_plan(rows, cols, sm_count, table);
        default: return gemv_i8_q4k_plan(rows, cols, sm_count, table);
    }
}

bool note_smem_raised(HaloCudaCtx* ctx, const void* kernel) { return ctx->smem_raised.insert(kernel).second; }

int allow_dynamic_smem(HaloCudaCtx* ctx, const void* kernel, uint32_t bytes) {
    if (ctx->smem_raised.count(kernel) != 0) return 0;
    HC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
    note_smem_raised(ctx, kernel);
    return 0;
}

// The checks of the CPU backend's Resolver (src/backend/cpu_backend.cpp:98-162) for raw device pointers:
// presence, stride >= row, overflow-checked extents, fp32 alignment, output disjoint from every input.
int validate_gemv(const HaloCudaGemv* a, const char* op, bool y_optional, GemvCall* c) {
    if (a == nullptr) return fail(HALO_CUDA_E_API, "%s: null argument struct", op);
    TypeInfo ti{};
    if (!type_info(a->wtype, &ti)) return fail(HALO_CUDA_E_UNSUPPORTED, "%s: no dequantization for weight type id %u", op, a->wtype);
    if (a->cols % ti.block_elems != 0)
        return fail(HALO_CUDA_E_MODEL, "%s: %u elements is not a multiple of the block size %u", op, a->cols, ti.block_elems);
    c->wtype = a->wtype;
    c->rows = a->rows;
    c->cols = a->cols;
    c->n_vec = a->n_vec;
    c->flags = a->flags;
    c->row_bytes = uint64_t{a->cols} / ti.block_elems * ti.block_bytes;
    if (reads_repacked_rows(a->variant_id)) {  // the W operand is in the repacked layout: its rows have another size
        if (repacked_row_bytes(a->wtype, 256) == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "%s: variant %u takes repacked Q4_0 / Q8_0 / Q6_K weights", op, a->variant_id);
        if (a->cols % 256u != 0) return fail(HALO_CUDA_E_MODEL, "%s: %u elements is not a multiple of the repacked group size 256", op, a->cols);
        c->row_bytes = repacked_row_bytes(a->wtype, a->cols);
    }
    c->w = static_cast<const uint8_t*>(a->w);
    c->x = a->x;
    c->y = a->y;
    c->w_stride = a->w_stride != 0 ? a->w_stride : c->row_bytes;
    c->x_stride = a->x_stride != 0 ? a->x_stride : uint64_t{a->cols} * 4;
    c->y_stride = a->y_stride != 0 ? a->y_stride : uint64_t{a->rows} * 4;
    struct Op {
        const char* name;
        const void* p;
        uint64_t n, row, stride, align;
        bool optional;
    } ops[3] = {{"w", c->w, a->rows, c->row_bytes, c->w_stride, a->wtype == HALO_CUDA_T_F32 ? 4u : 1u, false},
                {"x", c->x, a->n_vec, uint64_t{a->cols} * 4, c->x_stride, 4, false},
                {"y", c->y, a->n_vec, uint64_t{a->rows} * 4, c->y_stride, 4, y_optional}};
    uint64_t extent[3] = {0, 0, 0};
    for (int i = 0; i < 3; ++i) {
        const Op& o = ops[i];
        if (o.n == 0 || o.row == 0) {
            if (o.p == nullptr) continue;
        }
        if (o.p == nullptr) {
            if (o.optional) continue;
            return fail(HALO_CUDA_E_KERNEL, "%s: operand %s is empty", op, o.name);
        }
        if (o.n > 1 && o.stride < o.row)
            return fail(HALO_CUDA_E_KERNEL, "%s: operand %s row stride %llu < row bytes %llu", op, o.name,
                        (unsigned long long)o.stride, (unsigned long long)o.row);
        if (o.n != 0) {
            if (mul_overflows(o.n - 1, o.stride) || (o.n - 1) * o.stride > UINT64_MAX - o.row)
                return fail(HALO_CUDA_E_KERNEL, "%s: operand %s size overflows", op, o.name);
            extent[i] = (o.n - 1) * o.stride + o.row;
        }
        if (reinterpret_cast<uintptr_t>(o.p) % o.align != 0 || o.stride % o.align != 0)
            return fail(HALO_CUDA_E_KERNEL, "%s: operand %s is not %llu-byte aligned", op, o.name, (unsigned long long)o.align);
    }
    if (c->y != nullptr) {
        if (ranges_overlap(c->y, extent[2], c->x, extent[1])) return fail(HALO_CUDA_E_KERNEL, "%s: output y overlaps operand x", op);
        if (ranges_overlap(c->y, extent[2], c->w, extent[0])) return fail(HALO_CUDA_E_KERNEL, "%s: output y overlaps operand w", op);
    }
    return 0;
}

uint32_t resolve_variant(const HaloCudaCtx* ctx, const GemvCall& c, uint32_t requested) {
    // A repacked tensor travels with its decode variant (7 or 9); a prefill-sized batch whose caller accepts the GEMM's numerics
    // runs the GEMM over the same repacked rows.
    if ((requested == HALO_CUDA_GEMV_MMA_R || requested == HALO_CUDA_GEMV_MMA_I8X2_R) && (c.flags & HALO_CUDA_GEMV_FLAG_ALLOW_GEMM) != 0 &&
        c.n_vec >= 64 && gemm_tcgen05_supports(c, true))
        return HALO_CUDA_GEMM_TCGEN05_F16_R;
    if (requested != HALO_CUDA_GEMV_DEFAULT) return requested;
    if (c.cols == 0) return HALO_CUDA_GEMV_EXACT8;
    const bool gemm_ok = (c.flags & HALO_CUDA_GEMV_FLAG_ALLOW_GEMM) != 0;
    if (ctx != nullptr) {
        for (const PlanEntry& p : ctx->plan) {
            if (p.wtype != c.wtype || p.rows != c.rows || p.cols != c.cols || c.n_vec < p.n_vec_lo || c.n_vec > p.n_vec_hi) continue;
            const bool is_gemm = p.variant_id == HALO_CUDA_GEMM_TCGEN05_F16 || p.variant_id == HALO_CUDA_GEMM_TCGEN05_BF16;
            if (is_gemm && (!gemm_ok || !gemm_tcgen05_supports(c))) continue;
            if ((p.variant_id == HALO_CUDA_GEMV_MMA_F16X2 || p.variant_id == HALO_CUDA_GEMV_MMA_M1) && !gemv_mma_supports(c)) continue;
            if (p.variant_id == HALO_CUDA_GEMV_WARP_F32 && !gemv_warp_f32_supports(c)) continue;
            if (p.variant_id == HALO_CUDA_GEMV_MMA_I8X2 && (!gemv_i8_supports(c) || (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) != 0)) continue;
            return p.variant_id;
        }
    }
    // Without a plan: the tensor-core GEMM only where the caller accepts its numerics and the batch is
    // prefill-sized; otherwise one numerics family for every batch size, so that a row's bits do not depend
    // on how many rows share the call (include/halo/backend/backend.h:300-304).
    if (gemm_ok && c.n_vec >= 64 && gemm_tcgen05_supports(c)) return HALO_CUDA_GEMM_TCGEN05_F16;
    // Q4_K: the int8 tensor-core family at every batch size; calls that may not touch context scratch keep the fp16 family,
    // whose statically partitioned kernels need none
    if ((c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) == 0 && gemv_i8_supports(c)) return HALO_CUDA_GEMV_MMA_I8X2;
    if (gemv_mma_supports(c)) return HALO_CUDA_GEMV_MMA_F16X2;
    if (gemv_warp_f32_supports(c)) return HALO_CUDA_GEMV_WARP_F32;
    return HALO_CUDA_GEMV_EXACT8;
}

/// The outputs of an LM head (result triples, optional ids) must not overlap x, w, the logits or each other
/// (the no_overlap checks of src/backend/cpu_backend.cpp:146-155 for the head's operands, cpu_backend.cpp:669-720).
int lm_head_outputs_disjoint(const GemvCall& c, const void* result, const void* ids, const char* op) {
    const uint64_t res_bytes = uint64_t{c.n_vec} * 12, ids_bytes = ids != nullptr ? uint64_t{c.n_vec} * 4 : 0;
    const uint64_t x_ext = (uint64_t{c.n_vec} - 1) * c.x_stride + uint64_t{c.cols} * 4;
    const uint64_t w_ext = c.rows == 0 ? 0 : (uint64_t{c.rows} - 1) * c.w_stride + c.row_bytes;
    const uint64_t y_ext = c.y == nullptr ? 0 : (uint64_t{c.n_vec} - 1) * c.y_stride + uint64_t{c.rows} * 4;
    struct R { const void* p; uint64_t n; const char* name; };
    const R outs[2] = {{result, res_bytes, "result"}, {ids, ids_bytes, "ids"}};
    const R ins[3] = {{c.x, x_ext, "x"}, {c.w, w_ext, "w"}, {c.y, y_ext, "logits"}};
    for (const R& o : outs)
        for (const R& i : ins)
            if (o.p != nullptr && i.p != nullptr && ranges_overlap(o.p, o.n, i.p, i.n))
                return fail(HALO_CUDA_E_KERNEL, "%s: output %s overlaps operand %s", op, o.name, i.name);
    if (ids != nullptr && ranges_overlap(ids, ids_bytes, result, res_bytes)) return fail(HALO_CUDA_E_KERNEL, "%s: output ids overlaps operand result", op);
    return 0;
}

namespace {
int run_gemv(HaloCudaCtx* ctx, const GemvCall& c, uint32_t requested, cudaStream_t s) {
    const uint32_t v = resolve_variant(ctx, c, requested);
    switch (v) {
        case HALO_CUDA_GEMV_EXACT8: return launch_gemv_exact8(c, s);
        case HALO_CUDA_GEMV_WARP_F32:
            if (!gemv_warp_f32_supports(c)) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_warp_f32 does not take this weight type");
            return launch_gemv_warp_f32(c, s);
        case HALO_CUDA_GEMV_MMA_F16X2:
            if (!gemv_mma_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_f16x2 needs Q4_K weights in dense 16-byte-aligned rows");
            // context scratch holds the balanced kernels' partial sums and staged x; calls that may not touch it
            // take the statically partitioned kernel (same arithmetic per tile, another summation order over K)
            if (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) return launch_gemv_mma(ctx, c, s);
            return launch_gemv_sk_q4k(ctx, c, s);
        case HALO_CUDA_GEMV_MMA_M1:
            if (!gemv_mma_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_m1 needs Q4_K weights in dense 16-byte-aligned rows");
            return launch_gemv_mma_m1(ctx, c, s);
        case HALO_CUDA_GEMV_MMA_I8X2:
            if (!gemv_i8_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_i8x2 needs Q4_K weights in dense 16-byte-aligned rows and 16-byte-aligned x");
            if (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH)
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_i8x2 uses context scratch");
            return launch_gemv_i8(ctx, c, s);
        case HALO_CUDA_GEMV_MMA_I8X2_R:
            if (!gemv_i8_r_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_i8x2_r needs repacked 16-byte-aligned rows whose x records fit in shared memory, and 16-byte-aligned x");
            if (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_i8x2_r uses context scratch");
            switch (c.wtype) {
                case HALO_CUDA_T_Q6_K: return launch_gemv_i8_q6kr(ctx, c, s);
                case HALO_CUDA_T_Q8_0: return launch_gemv_i8_q80r(ctx, c, s);
                default: return launch_gemv_i8_q40r(ctx, c, s);
            }
        case HALO_CUDA_GEMV_MMA_R:
            if (!gemv_mma_r_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemv_mma_r needs repacked 16-byte-aligned rows, cols %% 256 == 0 and 16-byte-aligned x");
            return launch_gemv_mma_r(ctx, c, s);
        case HALO_CUDA_GEMM_TCGEN05_F16:
        case HALO_CUDA_GEMM_TCGEN05_BF16:
            if (!gemm_tcgen05_supports(c))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemm_tcgen05 needs Q4_K weights in 16-byte-aligned rows and cols %% 256 == 0");
            return launch_gemm_tcgen05(ctx, c, v == HALO_CUDA_GEMM_TCGEN05_BF16, false, s);
        case HALO_CUDA_GEMM_TCGEN05_F16_R:
        case HALO_CUDA_GEMM_TCGEN05_BF16_R:
            if (!gemm_tcgen05_supports(c, true))
                return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: gemm_tcgen05_*_r needs repacked Q6_K / Q8_0 / Q4_0 rows, 16-byte aligned, and 16-byte-aligned x");
            return launch_gemm_tcgen05(ctx, c, v == HALO_CUDA_GEMM_TCGEN05_BF16_R, true, s);
        default: return fail(HALO_CUDA_E_CONFIG, "MATMUL: unknown kernel variant id %u on the cuda backend", v);
    }
}
}  // namespace
}  // namespace halo_cuda

using namespace halo_cuda;

extern "C" {

int halo_cuda_device_count(int* count) {
    if (count == nullptr) return fail(HALO_CUDA_E_API, "null count");
    *count = 0;
    const cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        return fail(HALO_CUDA_E_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    return 0;
}

int halo_cuda_ctx_create(int device, HaloCudaCtx** out) {
    if (out == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) return fail(HALO_CUDA_E_DEVICE, "no CUDA device is usable");
    if (device < 0 || device >= n) return fail(HALO_CUDA_E_DEVICE, "device %d outside [0, %d)", device, n);
    HaloCudaCtx* ctx = new (std::nothrow) HaloCudaCtx();
    if (ctx == nullptr) return fail(HALO_CUDA_E_MEMORY, "out of host memory");
    ctx->device = device;
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&ctx->prop, device);
    if (e != cudaSuccess) {
        delete ctx;
        return fail(HALO_CUDA_E_DEVICE, "device %d: %s", device, cudaGetErrorString(e));
    }
    if (ctx->prop.major != 10) {
        // The kernels are built for sm_100a only; there is no other code path.
        const int major = ctx->prop.major, minor = ctx->prop.minor;
        delete ctx;
        return fail(HALO_CUDA_E_DEVICE, "device %d is sm_%d%d; this library holds sm_100a code only", device, major, minor);
    }
    void* host_word = nullptr;
    if (cudaHostAlloc(&host_word, sizeof(uint32_t), cudaHostAllocMapped) == cudaSuccess) {
        ctx->error_word_host = static_cast<uint32_t*>(host_word);
        *ctx->error_word_host = 0;
        void* dev_word = nullptr;
        if (cudaHostGetDevicePointer(&dev_word, host_word, 0) == cudaSuccess) ctx->error_word_dev = static_cast<uint32_t*>(dev_word);
    }
    cudaGetLastError();
    cudaMemPoolProps props{};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    e = cudaMemPoolCreate(&ctx->pool, &props);
    if (e == cudaSuccess) {
        uint64_t keep = UINT64_MAX;  // freed blocks stay with the pool
        e = cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->pool_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        halo_cuda_ctx_destroy(ctx);
        return fail(HALO_CUDA_E_BACKEND, "device %d: cannot set up the allocation pool: %s", device, cudaGetErrorString(e));
    }
    *out = ctx;
    return 0;
}

int halo_cuda_ctx_destroy(HaloCudaCtx* ctx) {
    if (ctx == nullptr) return 0;
    if (cudaSetDevice(ctx->device) == cudaSuccess) {
        if (ctx->pool != nullptr) {
            cudaDeviceSynchronize();
            for (void* p : ctx->pooled) cudaFreeAsync(p, ctx->pool_stream);
            if (ctx->pool_stream != nullptr) {
                cudaStreamSynchronize(ctx->pool_stream);
                cudaStreamDestroy(ctx->pool_stream);
            }
            cudaMemPoolDestroy(ctx->pool);
        }
        for (auto& kv : ctx->scratch)
            for (void* p : kv.second.block)
                if (p != nullptr) cudaFree(p);
        if (ctx->error_word_host != nullptr) cudaFreeHost(ctx->error_word_host);
        for (int i = 0; i < 2; ++i) {
            if (ctx->staging[i] != nullptr) cudaFreeHost(ctx->staging[i]);
            for (cudaEvent_t e : ctx->staging_done[i])
                if (e != nullptr) cudaEventDestroy(e);
        }
    }
    delete ctx;
    return 0;
}

int halo_cuda_device_info(HaloCudaCtx* ctx, HaloCudaDeviceInfo* info) {
    if (ctx == nullptr || info == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    std::memset(info, 0, sizeof *info);
    std::snprintf(info->name, sizeof info->name, "%.127s", ctx->prop.name);
    // cudaDeviceProp carries bus addresses, not the PCI device id: the vendor id is NVIDIA's, and the device id
    // is filled in by NVML-aware callers (0000 marks "not read").
    std::snprintf(info->pci_id, sizeof info->pci_id, "10de:0000");
    std::snprintf(info->arch, sizeof info->arch, "sm_%d%da", ctx->prop.major, ctx->prop.minor);
    info->cc_major = ctx->prop.major;
    info->cc_minor = ctx->prop.minor;
    info->sm_count = ctx->prop.multiProcessorCount;
    info->l2_bytes = ctx->prop.l2CacheSize;
    info->total_bytes = ctx->prop.totalGlobalMem;
    cudaDriverGetVersion(&info->driver_version);
    cudaRuntimeGetVersion(&info->runtime_version);
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, ctx->device) == cudaSuccess) info->clock_khz = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, ctx->device) == cudaSuccess) info->mem_clock_khz = v;
    return 0;
}

int halo_cuda_malloc(HaloCudaCtx* ctx, uint64_t bytes, int flags, void** ptr) {
    if (ptr == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    *ptr = nullptr;
    if (int rc = enter(ctx)) return rc;
    const bool zero = (flags & HALO_CUDA_MALLOC_ZERO) != 0, shareable = (flags & HALO_CUDA_MALLOC_SHAREABLE) != 0;
    const uint64_t size = bytes == 0 ? 1 : bytes;
    const cudaError_t e = shareable ? cudaMalloc(ptr, size) : cudaMallocFromPoolAsync(ptr, size, ctx->pool, ctx->pool_stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *ptr = nullptr;
        return fail(HALO_CUDA_E_MEMORY, "cannot allocate %llu bytes on device %d: %s", (unsigned long long)bytes, ctx->device,
                    cudaGetErrorString(e));
    }
    // The block belongs to the pool's stream until that stream has passed the allocation (and the clear): finish both here,
    // so that the pointer is good on every stream and no later upload can be overtaken by the clear.
    cudaError_t f = cudaSuccess;
    if (zero && bytes != 0) f = cudaMemsetAsync(*ptr, 0, bytes, ctx->pool_stream);
    if (f == cudaSuccess && (!shareable || zero)) f = cudaStreamSynchronize(ctx->pool_stream);
    if (f != cudaSuccess) {
        if (shareable) cudaFree(*ptr);
        else cudaFreeAsync(*ptr, ctx->pool_stream);
        *ptr = nullptr;
        return fail(HALO_CUDA_E_BACKEND, "clearing %llu bytes: %s", (unsigned long long)bytes, cudaGetErrorString(f));
    }
    if (!shareable) ctx->pooled.insert(*ptr);
    return 0;
}

int halo_cuda_free(HaloCudaCtx* ctx, void* ptr) {
    if (ptr == nullptr) return 0;
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    HC_CUDA(cudaSetDevice(ctx->device));
    const auto it = ctx->pooled.find(ptr);
    if (it == ctx->pooled.end()) {
        HC_CUDA(cudaFree(ptr));  // waits for the device, like the pool path below
        return 0;
    }
    // Work that still reads or writes the block may be queued on any stream: wait for the device (a no-op for a caller
    // that frees after its stream wait), then hand the block back to the pool, where the next allocation finds it.
    HC_CUDA(cudaDeviceSynchronize());
    ctx->pooled.erase(it);
    HC_CUDA(cudaFreeAsync(ptr, ctx->pool_stream));
    return 0;
}

int halo_cuda_host_alloc(HaloCudaCtx* ctx, uint64_t bytes, void** ptr) {
    if (ptr == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    *ptr = nullptr;
    if (int rc = enter(ctx)) return rc;
    const cudaError_t e = cudaHostAlloc(ptr, bytes == 0 ? 1 : bytes, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(HALO_CUDA_E_MEMORY, "cannot pin %llu host bytes: %s", (unsigned long long)bytes, cudaGetErrorString(e));
    }
    return 0;
}

int halo_cuda_host_free(HaloCudaCtx* ctx, void* ptr) {
    if (ptr == nullptr) return 0;
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    HC_CUDA(cudaFreeHost(ptr));
    return 0;
}

int halo_cuda_stream_create(HaloCudaCtx* ctx, HaloCudaStream* stream) {
    if (stream == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    if (int rc = enter(ctx)) return rc;
    cudaStream_t s = nullptr;
    HC_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return 0;
}

int halo_cuda_stream_destroy(HaloCudaCtx* ctx, HaloCudaStream stream) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    if (stream == nullptr) return 0;
    HC_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto it = ctx->scratch.find(s);
    if (it != ctx->scratch.end()) {  // the stream's scratch goes with it, once its work has drained
        cudaStreamSynchronize(s);
        for (void* p : it->second.block)
            if (p != nullptr) cudaFree(p);
        ctx->scratch.erase(it);
    }
    HC_CUDA(cudaStreamDestroy(s));
    return 0;
}

int halo_cuda_stream_sync(HaloCudaCtx* ctx, HaloCudaStream stream, uint64_t timeout_ns) {
    if (int rc = enter(ctx)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (timeout_ns == 0) {
        e = cudaStreamSynchronize(s);
    } else {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::nanoseconds(timeout_ns);
        unsigned spins = 0;
        while ((e = cudaStreamQuery(s)) == cudaErrorNotReady) {
            if (std::chrono::steady_clock::now() >= deadline) {
                ctx->lost = true;
                return fail(HALO_CUDA_E_BACKEND, "stream wait exceeded %llu ns; device %d marked lost", (unsigned long long)timeout_ns,
                            ctx->device);
            }
            if (++spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
        }
    }
    if (e != cudaSuccess) {
        ctx->lost = true;
        return fail(HALO_CUDA_E_BACKEND, "stream wait failed on device %d: %s", ctx->device, cudaGetErrorString(e));
    }
    if (ctx->error_word_host != nullptr && *static_cast<volatile uint32_t*>(ctx->error_word_host) != 0) {
        ctx->lost = true;
        return fail(HALO_CUDA_E_BACKEND, "a kernel on device %d gave up a bounded wait (status word 0x%x); device marked lost", ctx->device,
                    *ctx->error_word_host);
    }
    return 0;
}

int halo_cuda_ctx_lost(HaloCudaCtx* ctx) { return ctx != nullptr && ctx->lost ? 1 : 0; }

int halo_cuda_ctx_scratch_bytes(HaloCudaCtx* ctx, uint64_t* bytes) {
    if (ctx == nullptr || bytes == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *bytes = 0;
    for (const auto& kv : ctx->scratch)
        for (uint64_t b : kv.second.bytes) *bytes += b;
    return 0;
}

int halo_cuda_ctx_set_peer_wait_polls(HaloCudaCtx* ctx, uint32_t polls) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    ctx->peer_wait_polls = polls == 0 ? 1u << 22 : polls;
    return 0;
}

int halo_cuda_memcpy_h2d_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (bytes == 0) return 0;
    if (dst == nullptr || src == nullptr) return fail(HALO_CUDA_E_KERNEL, "upload: null pointer");
    HC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return 0;
}

int halo_cuda_memcpy_d2h_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (bytes == 0) return 0;
    if (dst == nullptr || src == nullptr) return fail(HALO_CUDA_E_KERNEL, "download: null pointer");
    HC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
    return 0;
}

int halo_cuda_memcpy_d2d_async(HaloCudaCtx* ctx, void* dst, const void* src, uint64_t bytes, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (bytes == 0) return 0;
    if (dst == nullptr || src == nullptr) return fail(HALO_CUDA_E_KERNEL, "COPY: null pointer");
    const auto d = reinterpret_cast<uintptr_t>(dst), s = reinterpret_cast<uintptr_t>(src);
    if (d < s + bytes && s < d + bytes) return fail(HALO_CUDA_E_KERNEL, "COPY: output dst overlaps operand src");
    HC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return 0;
}

int halo_cuda_memset_async(HaloCudaCtx* ctx, void* dst, int value, uint64_t bytes, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (bytes == 0) return 0;
    if (dst == nullptr) return fail(HALO_CUDA_E_KERNEL, "memset: null pointer");
    HC_CUDA(cudaMemsetAsync(dst, value, bytes, static_cast<cudaStream_t>(stream)));
    return 0;
}

int halo_cuda_event_create(HaloCudaCtx* ctx, HaloCudaEvent* event) {
    if (event == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    if (int rc = enter(ctx)) return rc;
    cudaEvent_t e = nullptr;
    HC_CUDA(cudaEventCreate(&e));
    *event = e;
    return 0;
}

int halo_cuda_event_destroy(HaloCudaCtx* ctx, HaloCudaEvent event) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    if (event == nullptr) return 0;
    HC_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    return 0;
}

int halo_cuda_event_record(HaloCudaCtx* ctx, HaloCudaEvent event, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    HC_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    return 0;
}

int halo_cuda_event_elapsed_ns(HaloCudaCtx* ctx, HaloCudaEvent start, HaloCudaEvent stop, uint64_t* ns) {
    if (ns == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    if (int rc = enter(ctx)) return rc;
    HC_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)));
    float ms = 0.0f;
    HC_CUDA(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
    *ns = static_cast<uint64_t>(static_cast<double>(ms) * 1.0e6);
    return 0;
}

int halo_cuda_row_bytes(uint32_t wtype, uint64_t cols, uint64_t* bytes) {
    if (bytes == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    TypeInfo ti{};
    if (!type_info(wtype, &ti)) return fail(HALO_CUDA_E_UNSUPPORTED, "unknown or unsupported tensor type id %u", wtype);
    if (cols % ti.block_elems != 0)
        return fail(HALO_CUDA_E_MODEL, "%llu elements is not a multiple of the block size %u", (unsigned long long)cols, ti.block_elems);
    const uint64_t nb = cols / ti.block_elems;
    if (nb > uint64_t{INT64_MAX} / ti.block_bytes) return fail(HALO_CUDA_E_MODEL, "byte size overflows");
    *bytes = nb * ti.block_bytes;
    return 0;
}

int halo_cuda_variants(uint32_t op, HaloCudaVariant* out, uint32_t cap, uint32_t* count) {
    if (count == nullptr) return fail(HALO_CUDA_E_API, "null count");
    const HaloCudaVariant* table = nullptr;
    uint32_t n = 0;
    switch (op) {
        case HALO_CUDA_OP_GEMV: table = kGemvVariants; n = sizeof kGemvVariants / sizeof kGemvVariants[0]; break;
        case HALO_CUDA_OP_LM_HEAD: table = kLmHeadVariants; n = 1; break;
        case HALO_CUDA_OP_GET_ROWS: table = kGetRowsVariants; n = 1; break;
        default: *count = 0; return fail(HALO_CUDA_E_UNSUPPORTED, "op id %u is not implemented by the cuda backend", op);
    }
    *count = n;
    for (uint32_t i = 0; i < n && i < cap && out != nullptr; ++i) out[i] = table[i];
    return 0;
}

int halo_cuda_plan_set(HaloCudaCtx* ctx, uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t n_vec_lo, uint32_t n_vec_hi,
                       uint32_t variant_id) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    if (variant_id == 0 || variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "plan: unknown kernel variant id %u", variant_id);
    if (n_vec_lo > n_vec_hi) return fail(HALO_CUDA_E_API, "plan: empty n_vec range");
    if (reads_repacked_rows(variant_id))
        return fail(HALO_CUDA_E_CONFIG, "plan: the repacked variants read another weight layout: the loader that repacks a tensor passes variant id %u with it",
                    variant_id);
    for (PlanEntry& p : ctx->plan) {
        if (p.wtype == wtype && p.rows == rows && p.cols == cols && p.n_vec_lo == n_vec_lo && p.n_vec_hi == n_vec_hi) {
            p.variant_id = variant_id;
            return 0;
        }
    }
    ctx->plan.push_back({wtype, rows, cols, n_vec_lo, n_vec_hi, variant_id});
    return 0;
}

int halo_cuda_plan_clear(HaloCudaCtx* ctx) {
    if (ctx == nullptr) return fail(HALO_CUDA_E_API, "null context");
    ctx->plan.clear();
    return 0;
}

int halo_cuda_repacked_row_bytes(uint32_t wtype, uint64_t cols, uint64_t* bytes) {
    if (bytes == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    if (repacked_row_bytes(wtype, 256) == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "weight type id %u has no repacked layout", wtype);
    if (cols % 256u != 0) return fail(HALO_CUDA_E_MODEL, "%llu elements is not a multiple of the repacked group size 256", (unsigned long long)cols);
    *bytes = repacked_row_bytes(wtype, cols);
    return 0;
}

int halo_cuda_repacked_variant(uint32_t wtype, uint64_t cols, uint32_t* variant_id) {
    if (variant_id == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    uint64_t bytes = 0;
    if (int rc = halo_cuda_repacked_row_bytes(wtype, cols, &bytes)) return rc;
    if (cols > UINT32_MAX) return fail(HALO_CUDA_E_UNSUPPORTED, "%llu columns exceed 32-bit extents", (unsigned long long)cols);
    *variant_id = repacked_variant(wtype, static_cast<uint32_t>(cols));
    return 0;
}

int halo_cuda_repack_rows(HaloCudaCtx* ctx, uint32_t wtype, const void* src, uint64_t src_stride, void* dst, uint64_t dst_stride,
                          uint32_t rows, uint32_t cols, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    uint64_t raw = 0, packed = 0;
    if (int rc = halo_cuda_row_bytes(wtype, cols, &raw)) return rc;
    if (int rc = halo_cuda_repacked_row_bytes(wtype, cols, &packed)) return rc;
    if (rows == 0 || cols == 0) return 0;
    if (src == nullptr || dst == nullptr) return fail(HALO_CUDA_E_KERNEL, "repack: null pointer");
    const uint64_t ss = src_stride != 0 ? src_stride : raw, ds = dst_stride != 0 ? dst_stride : packed;
    if ((rows > 1 && (ss < raw || ds < packed)) || reinterpret_cast<uintptr_t>(dst) % 16 != 0 || ds % 16 != 0)
        return fail(HALO_CUDA_E_KERNEL, "repack: strides below the row size, or a destination that is not 16-byte aligned");
    if (ranges_overlap(dst, (uint64_t{rows} - 1) * ds + packed, src, (uint64_t{rows} - 1) * ss + raw))
        return fail(HALO_CUDA_E_KERNEL, "repack: output dst overlaps operand src");
    return launch_repack(wtype, src, ss, dst, ds, rows, cols, static_cast<cudaStream_t>(stream));
}

size_t halo_cuda_last_error(char* buf, size_t len) {
    if (buf != nullptr && len != 0) std::snprintf(buf, len, "%s", g_error.c_str());
    return g_error.size();
}

int halo_cuda_gemv_resolve(HaloCudaCtx* ctx, const HaloCudaGemv* args, uint32_t* variant_id) {
    if (variant_id == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    GemvCall c{};
    if (int rc = validate_gemv(args, "MATMUL", false, &c)) return rc;
    *variant_id = resolve_variant(ctx, c, args->variant_id);
    return 0;
}

int halo_cuda_gemv(HaloCudaCtx* ctx, const HaloCudaGemv* args, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    GemvCall c{};
    if (int rc = validate_gemv(args, "MATMUL", false, &c)) return rc;
    if (args->variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "MATMUL: unknown kernel variant id %u on the cuda backend", args->variant_id);
    if (c.rows == 0 || c.n_vec == 0) return 0;
    return run_gemv(ctx, c, args->variant_id, static_cast<cudaStream_t>(stream));
}

int halo_cuda_gemv_normed(HaloCudaCtx* ctx, const HaloCudaGemv* args, const float* norm_w, float norm_eps, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    GemvCall c{};
    if (int rc = validate_gemv(args, "MATMUL", false, &c)) return rc;
    if (args->variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "MATMUL: unknown kernel variant id %u on the cuda backend", args->variant_id);
    if (norm_w == nullptr) return fail(HALO_CUDA_E_API, "MATMUL: fused input norm without norm_w");
    if (reinterpret_cast<uintptr_t>(norm_w) % 16 != 0 || reinterpret_cast<uintptr_t>(c.x) % 16 != 0)
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: fused input norm needs 16-byte-aligned x and norm_w");
    if (!(norm_eps >= 0.0f)) return fail(HALO_CUDA_E_KERNEL, "MATMUL: norm_eps must be a non-negative number");
    const uint64_t nbytes = uint64_t{c.cols} * 4;
    if (ranges_overlap(c.y, uint64_t{c.rows} * 4, norm_w, nbytes)) return fail(HALO_CUDA_E_KERNEL, "MATMUL: output y overlaps operand norm_w");
    // the same restrictions as the reference's fused norm (backend.h:292-298): one x row, and only where the kernel has it
    if (c.n_vec != 1) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm takes one x row, not %u", c.n_vec);
    if (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the fused input norm belongs to the kernels that use context scratch");
    const uint32_t v = resolve_variant(ctx, c, args->variant_id);
    const bool has_it = (v == HALO_CUDA_GEMV_MMA_F16X2 && gemv_mma_supports(c)) || (v == HALO_CUDA_GEMV_MMA_R && gemv_mma_r_supports(c)) ||
                        (v == HALO_CUDA_GEMV_MMA_I8X2 && gemv_i8_supports(c)) || (v == HALO_CUDA_GEMV_MMA_I8X2_R && gemv_i8_r_supports(c));
    if (!has_it) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: only the tensor-core skinny variants (3, 7, 8, 9) have the fused input norm");
    if (c.rows == 0) return 0;
    c.norm_w = norm_w;
    c.norm_eps = norm_eps;
    return run_gemv(ctx, c, v, static_cast<cudaStream_t>(stream));
}

int halo_cuda_gemv_gated(HaloCudaCtx* ctx, const HaloCudaGemv* args, const float* dt_bias, const float* a, uint32_t n_v, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    GemvCall c{};
    if (int rc = validate_gemv(args, "MATMUL", false, &c)) return rc;
    if (args->variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "MATMUL: unknown kernel variant id %u on the cuda backend", args->variant_id);
    if (n_v == 0 || dt_bias == nullptr || a == nullptr) return fail(HALO_CUDA_E_API, "MATMUL: gates epilogue without n_v, dt_bias or a");
    if (reinterpret_cast<uintptr_t>(dt_bias) % 4 != 0 || reinterpret_cast<uintptr_t>(a) % 4 != 0)
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: dt_bias and a must be 4-byte aligned");
    if (c.rows != 2ull * n_v) return fail(HALO_CUDA_E_KERNEL, "MATMUL: the gates epilogue needs rows == 2 * n_v (beta rows, then alpha rows), got %u rows for n_v = %u", c.rows, n_v);
    const uint64_t y_bytes = c.n_vec == 0 ? 0 : (uint64_t{c.n_vec} - 1) * c.y_stride + uint64_t{c.rows} * 4;
    if (ranges_overlap(c.y, y_bytes, dt_bias, uint64_t{n_v} * 4) || ranges_overlap(c.y, y_bytes, a, uint64_t{n_v} * 4))
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: output y overlaps operand dt_bias or a");
    // as in the reference (backend.h:304-309): F32 / Q8_0 weights only, and only the kernels that have the epilogue
    if (c.wtype != HALO_CUDA_T_F32 && c.wtype != HALO_CUDA_T_Q8_0)
        return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the gates epilogue takes F32 or Q8_0 weights, not type id %u", c.wtype);
    const uint32_t v = resolve_variant(ctx, c, args->variant_id);
    if (v != HALO_CUDA_GEMV_EXACT8 && !(v == HALO_CUDA_GEMV_WARP_F32 && gemv_warp_f32_supports(c)))
        return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: only the fp32 variants (1, 2) have the gates epilogue");
    if (c.n_vec == 0) return 0;
    c.gate_dt_bias = dt_bias;
    c.gate_a = a;
    c.gate_n_v = n_v;
    return run_gemv(ctx, c, v, static_cast<cudaStream_t>(stream));
}

int halo_cuda_gemv_plan(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, HaloCudaGemvPlan* plan) {
    if (plan == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    const bool grouped = repacked_row_bytes(wtype, 256) != 0;
    if (wtype != HALO_CUDA_T_Q4_K && !grouped) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: no tensor-core skinny kernel for weight type id %u", wtype);
    if (cols == 0 || cols % 256u != 0) return fail(HALO_CUDA_E_MODEL, "MATMUL: %u elements is not a multiple of 256", cols);
    if (rows == 0 || sm_count == 0) return fail(HALO_CUDA_E_KERNEL, "MATMUL: empty matrix or device");
    static_assert(HALO_CUDA_PLAN_MAX_CTAS == mma::kSkMaxCtas, "plan table size of the C ABI");
    mma::SkTable t{};
    std::memset(plan, 0, sizeof *plan);
    plan->slices = mma::plan_partition(rows, cols / 256u, sm_count, mma::format_allows_slices(wtype), &t);
    plan->ctas = t.parts;
    plan->cols_per_unit = t.cols_per_unit;
    for (uint32_t c = 0; c <= t.parts; ++c) plan->start[c] = t.start[c];
    return 0;
}

int halo_cuda_gemv_plan_i8(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t sm_count, HaloCudaGemvPlan* plan) {
    if (plan == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    if (wtype != HALO_CUDA_T_Q4_K && repacked_row_bytes(wtype, 256) == 0)
        return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: no tensor-core skinny kernel for weight type id %u", wtype);
    if (cols == 0 || cols % 256u != 0) return fail(HALO_CUDA_E_MODEL, "MATMUL: %u elements is not a multiple of 256", cols);
    if (rows == 0 || sm_count == 0) return fail(HALO_CUDA_E_KERNEL, "MATMUL: empty matrix or device");
    mma::SkTable t{};
    std::memset(plan, 0, sizeof *plan);
    plan->slices = gemv_i8_plan(wtype, rows, cols, sm_count, &t);
    plan->ctas = t.parts;
    plan->cols_per_unit = t.cols_per_unit;
    for (uint32_t c = 0; c <= t.parts; ++c) plan->start[c] = t.start[c];
    return 0;
}

int halo_cuda_gemv_tiles_i8(uint32_t wtype, uint32_t rows, uint32_t cols, uint32_t n_vec, uint32_t sm_count, HaloCudaGemvTiles* tiles) {
    if (tiles == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    if (wtype != HALO_CUDA_T_Q4_K && repacked_row_bytes(wtype, 256) == 0)
        return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: no tensor-core skinny kernel for weight type id %u", wtype);
    if (cols == 0 || cols % 256u != 0) return fail(HALO_CUDA_E_MODEL, "MATMUL: %u elements is not a multiple of 256", cols);
    if (rows == 0 || sm_count == 0) return fail(HALO_CUDA_E_KERNEL, "MATMUL: empty matrix or device");
    switch (wtype) {
        case HALO_CUDA_T_Q6_K: gemv_i8_q6kr_tiles(rows, cols, n_vec, sm_count, tiles); break;
        case HALO_CUDA_T_Q8_0: gemv_i8_q80r_tiles(rows, cols, n_vec, sm_count, tiles); break;
        case HALO_CUDA_T_Q4_0: gemv_i8_q40r_tiles(rows, cols, n_vec, sm_count, tiles); break;
        default: gemv_i8_q4k_tiles(rows, cols, n_vec, sm_count, tiles); break;
    }
    if (tiles->resident_rows == 0) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the int8 kernels keep x in shared memory; %u columns do not fit", cols);
    return 0;
}

int halo_cuda_gemv_reduce(HaloCudaCtx* ctx, const HaloCudaGemv* args, const HaloCudaPeerReduce* peers, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    GemvCall c{};
    if (int rc = validate_gemv(args, "MATMUL", false, &c)) return rc;
    if (args->variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "MATMUL: unknown kernel variant id %u on the cuda backend", args->variant_id);
    if (peers == nullptr) return fail(HALO_CUDA_E_API, "MATMUL: null peer description");
    if (peers->world == 0 || peers->world > HALO_CUDA_MAX_PEERS || peers->rank >= peers->world)
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: rank %u of %u peers (at most %d)", peers->rank, peers->world, HALO_CUDA_MAX_PEERS);
    if (peers->epoch == nullptr || peers->done == nullptr) return fail(HALO_CUDA_E_KERNEL, "MATMUL: peer reduction without its counters");
    for (uint32_t p = 0; p < peers->world; ++p)
        if (peers->slots[p] == nullptr) return fail(HALO_CUDA_E_KERNEL, "MATMUL: the receive buffer of peer %u is not mapped", p);
    if (uint64_t{c.rows} * c.n_vec > peers->capacity)
        return fail(HALO_CUDA_E_KERNEL, "MATMUL: %u x %u results exceed the peers' slot capacity of %u floats", c.n_vec, c.rows, peers->capacity);
    if (c.rows == 0 || c.n_vec == 0) return 0;  // every rank sees the same shape, so every rank skips
    if (c.flags & HALO_CUDA_GEMV_FLAG_NO_SCRATCH) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: the peer epilogue belongs to the kernels that use context scratch");
    const uint32_t v = resolve_variant(ctx, c, args->variant_id);
    const bool pushes = (v == HALO_CUDA_GEMV_MMA_F16X2 && gemv_mma_supports(c)) || (v == HALO_CUDA_GEMV_MMA_R && gemv_mma_r_supports(c)) ||
                        (v == HALO_CUDA_GEMV_MMA_I8X2 && gemv_i8_supports(c)) || (v == HALO_CUDA_GEMV_MMA_I8X2_R && gemv_i8_r_supports(c));
    if (!pushes) return fail(HALO_CUDA_E_UNSUPPORTED, "MATMUL: only the tensor-core skinny variants (3, 7, 8, 9) have the peer epilogue");
    c.peer = peers;
    const cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (int rc = run_gemv(ctx, c, v, s)) return rc;
    return launch_peer_finish(ctx, *peers, c.y, c.y_stride, c.rows, c.n_vec, s);
}

int halo_cuda_ipc_export(HaloCudaCtx* ctx, void* ptr, uint8_t handle[64]) {
    if (int rc = enter(ctx)) return rc;
    if (ptr == nullptr || handle == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size of the C ABI");
    if (ctx->pooled.count(ptr) != 0)
        return fail(HALO_CUDA_E_KERNEL, "ipc_export: the block comes from the allocation pool; allocate it with HALO_CUDA_MALLOC_SHAREABLE");
    cudaIpcMemHandle_t h;
    HC_CUDA(cudaIpcGetMemHandle(&h, ptr));
    std::memcpy(handle, &h, 64);
    return 0;
}

int halo_cuda_ipc_open(HaloCudaCtx* ctx, const uint8_t handle[64], void** ptr) {
    if (int rc = enter(ctx)) return rc;
    if (ptr == nullptr || handle == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    HC_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}

int halo_cuda_ipc_close(HaloCudaCtx* ctx, void* ptr) {
    if (int rc = enter(ctx)) return rc;
    if (ptr == nullptr) return 0;
    HC_CUDA(cudaIpcCloseMemHandle(ptr));
    return 0;
}

int halo_cuda_lm_head(HaloCudaCtx* ctx, const HaloCudaLmHead* a, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (a == nullptr) return fail(HALO_CUDA_E_API, "LM_HEAD: null argument struct");
    GemvCall c{};
    if (int rc = validate_gemv(&a->gemv, "LM_HEAD", true, &c)) return rc;
    if (a->gemv.variant_id > HALO_CUDA_GEMV_VARIANT_MAX)
        return fail(HALO_CUDA_E_CONFIG, "LM_HEAD: unknown kernel variant id %u on the cuda backend", a->gemv.variant_id);
    if (c.n_vec == 0) return 0;
    if (a->result == nullptr) return fail(HALO_CUDA_E_KERNEL, "LM_HEAD: operand result is empty");
    if (reinterpret_cast<uintptr_t>(a->result) % 4 != 0 || reinterpret_cast<uintptr_t>(a->ids) % 4 != 0)
        return fail(HALO_CUDA_E_KERNEL, "LM_HEAD: result / ids are not 4-byte aligned");
    if (int rc = lm_head_outputs_disjoint(c, a->result, a->ids, "LM_HEAD")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Logits go to the caller's buffer when one is given, else to context scratch; the argmax then runs over
    // exactly the values the gemv stored (cpu_backend.cpp:734-750).
    const uint64_t logits_bytes = c.y == nullptr ? uint64_t{c.n_vec} * c.rows * 4 : 0;
    const uint64_t part_bytes = argmax_scratch_bytes(c.rows, c.n_vec);
    const uint64_t logits_pad = (logits_bytes + 255) & ~uint64_t{255};
    void* ws = nullptr;
    if (int rc = workspace(ctx, 1, logits_pad + part_bytes + 256, s, &ws)) return rc;
    GemvCall g = c;
    if (c.y == nullptr) {
        g.y = static_cast<float*>(ws);
        g.y_stride = uint64_t{c.rows} * 4;
    }
    if (c.rows != 0) {
        if (int rc = run_gemv(ctx, g, a->gemv.variant_id, s)) return rc;
    }
    return launch_argmax(g.y, g.y_stride / 4, c.rows, c.n_vec, a->valid_rows, a->row_offset, a->result, a->ids,
                         static_cast<uint8_t*>(ws) + logits_pad, s);
}

int halo_cuda_get_rows(HaloCudaCtx* ctx, const HaloCudaGetRows* a, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (a == nullptr) return fail(HALO_CUDA_E_API, "GET_ROWS: null argument struct");
    if (a->variant_id > 1) return fail(HALO_CUDA_E_CONFIG, "GET_ROWS: unknown kernel variant id %u on the cuda backend", a->variant_id);
    TypeInfo ti{};
    if (!type_info(a->type, &ti)) return fail(HALO_CUDA_E_UNSUPPORTED, "GET_ROWS: no dequantization for type id %u", a->type);
    if (a->cols % ti.block_elems != 0)
        return fail(HALO_CUDA_E_MODEL, "GET_ROWS: %u elements is not a multiple of the block size %u", a->cols, ti.block_elems);
    const uint64_t rb = uint64_t{a->cols} / ti.block_elems * ti.block_bytes;
    const uint64_t ts = a->table_stride != 0 ? a->table_stride : rb;
    const uint64_t os = a->out_stride != 0 ? a->out_stride : uint64_t{a->cols} * 4;
    if (a->n_ids == 0 || a->cols == 0) return 0;
    if (a->table == nullptr || a->out == nullptr) return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: operand table / out is empty");
    if (a->n_rows > 1 && ts < rb) return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: table row stride %llu < row bytes %llu", (unsigned long long)ts, (unsigned long long)rb);
    if (a->n_ids > 1 && os < uint64_t{a->cols} * 4) return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: out row stride < row bytes");
    if (reinterpret_cast<uintptr_t>(a->out) % 4 != 0 || os % 4 != 0 || reinterpret_cast<uintptr_t>(a->ids) % 4 != 0)
        return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: out / ids are not 4-byte aligned");
    if (a->type == HALO_CUDA_T_F32 && (reinterpret_cast<uintptr_t>(a->table) % 4 != 0 || ts % 4 != 0))
        return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: operand table is not 4-byte aligned");
    if (a->ids == nullptr && a->n_ids > a->n_rows) return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: %u rows requested from a table of %u", a->n_ids, a->n_rows);
    const uint64_t t_ext = a->n_rows == 0 ? 0 : (uint64_t{a->n_rows} - 1) * ts + rb;
    const uint64_t o_ext = (uint64_t{a->n_ids} - 1) * os + uint64_t{a->cols} * 4;
    if (ranges_overlap(a->out, o_ext, a->table, t_ext)) return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: output out overlaps operand table");
    if (a->ids != nullptr && ranges_overlap(a->out, o_ext, a->ids, uint64_t{a->n_ids} * 4))
        return fail(HALO_CUDA_E_KERNEL, "GET_ROWS: output out overlaps operand ids");
    return launch_get_rows(*a, rb, ts, os, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
