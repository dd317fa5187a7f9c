// halo_cuda_lm_head_noalloc: the LM head for callers that must not allocate device memory.
//
// Who needs it: a host that runs the model inside a region where cudaMalloc / cudaFree are off limits -- a
// real-time serving loop that has pre-sized every buffer and treats any allocator call as a latency bug, or an
// embedding application whose memory budget was fixed at start-up.  The regular halo_cuda_lm_head grows a
// per-context scratch block with cudaMalloc the first time a larger vocabulary arrives; this entry point never
// does.  Its only scratch, the per-chunk argmax partials, lives in a fixed array in the library's device image.
//
// Limits and sharing rules:
//   * the caller passes every input and output, including the logits buffer (gemv.y must not be null here);
//   * ceil(rows / 8192) * n_vec partial records must fit kNoAllocMaxParts (4096 records, 64 KiB per GPU, held by
//     every GPU that loads the library until the process exits); larger calls are rejected with E_UNSUPPORTED;
//   * the array is shared by every call on that GPU and keeps the previous call's contents.  Nothing in it has to
//     start at zero: the first stage overwrites each record the second stage reads.  Two calls that overlap on
//     the GPU (different streams) would race on it; issue them on one stream.
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first call
//     before starting any stream capture.
#include <mutex>

#include "internal.h"

namespace halo_cuda {
namespace {

constexpr uint32_t kNoAllocMaxParts = 4096;
constexpr uint32_t kPartBytes = 16;  // one argmax partial: value, index, nan flag, pad
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_noalloc_parts[kNoAllocMaxParts * kPartBytes];

std::mutex g_setup_mutex;
void* g_parts_addr[kMaxDevices] = {};

/// Device address of the static array on ctx's device (which is current).  In host code the symbol's name is only a
/// handle, not an address a kernel could use, so the address is asked for once per device and cached.
int scratch_address(const HaloCudaCtx* ctx, void** out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices) return fail(HALO_CUDA_E_UNSUPPORTED, "LM_HEAD (no-alloc): device ordinal %d", ctx->device);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_parts_addr[ctx->device] == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_parts);
        if (e != cudaSuccess || p == nullptr)
            return fail(HALO_CUDA_E_BACKEND, "LM_HEAD (no-alloc): cudaGetSymbolAddress on device %d: %s", ctx->device, cudaGetErrorString(e));
        g_parts_addr[ctx->device] = p;
    }
    *out = g_parts_addr[ctx->device];
    return 0;
}

}  // namespace
}  // namespace halo_cuda

using namespace halo_cuda;

extern "C" int halo_cuda_lm_head_noalloc(HaloCudaCtx* ctx, const HaloCudaLmHead* a, HaloCudaStream stream) {
    if (int rc = enter(ctx)) return rc;
    if (a == nullptr) return fail(HALO_CUDA_E_API, "LM_HEAD (no-alloc): null argument struct");
    GemvCall c{};
    if (int rc = validate_gemv(&a->gemv, "LM_HEAD (no-alloc)", false, &c)) return rc;
    if (a->gemv.variant_id > HALO_CUDA_GEMV_MMA_F16X2)
        return fail(HALO_CUDA_E_UNSUPPORTED, "LM_HEAD (no-alloc): kernel variant id %u may use context scratch; pass 0, 1, 2 or 3",
                    a->gemv.variant_id);
    if (c.n_vec == 0) return 0;
    if (a->result == nullptr) return fail(HALO_CUDA_E_KERNEL, "LM_HEAD (no-alloc): operand result is empty");
    if (reinterpret_cast<uintptr_t>(a->result) % 4 != 0 || reinterpret_cast<uintptr_t>(a->ids) % 4 != 0)
        return fail(HALO_CUDA_E_KERNEL, "LM_HEAD (no-alloc): result / ids are not 4-byte aligned");
    if (int rc = lm_head_outputs_disjoint(c, a->result, a->ids, "LM_HEAD (no-alloc)")) return rc;
    const uint64_t need = argmax_scratch_bytes(c.rows, c.n_vec);
    if (need > uint64_t{kNoAllocMaxParts} * kPartBytes)
        return fail(HALO_CUDA_E_UNSUPPORTED,
                    "LM_HEAD (no-alloc): %u rows x %u vectors need %llu bytes of argmax partials, the fixed scratch holds %u; "
                    "use halo_cuda_lm_head or split the call",
                    c.rows, c.n_vec, (unsigned long long)need, kNoAllocMaxParts * kPartBytes);
    void* parts = nullptr;
    if (int rc = scratch_address(ctx, &parts)) return rc;
    // The matmul writes the caller's logits buffer; the argmax then runs over exactly those values.  A prefill-only
    // flag is dropped so that the matmul stays inside the variants that take no context scratch.
    HaloCudaGemv g = a->gemv;
    g.flags &= ~HALO_CUDA_GEMV_FLAG_ALLOW_GEMM;
    g.flags |= HALO_CUDA_GEMV_FLAG_NO_SCRATCH;  // batches convert x inside the matmul CTAs instead of in context scratch
    if (c.rows != 0) {
        if (int rc = halo_cuda_gemv(ctx, &g, stream)) return rc;
    }
    return launch_argmax(c.y, c.y_stride / 4, c.rows, c.n_vec, a->valid_rows, a->row_offset, a->result, a->ids, parts,
                         static_cast<cudaStream_t>(stream));
}
