// The second half of halo_cuda_gemv_reduce: add the slots the ranks pushed, in rank order.
// The first half is the push epilogue of the balanced skinny kernels (mma_common.cuh, sk_flush): every element
// arrives as one 8-byte word {value bits, number of the reduction}, so waiting for an element is reading it until
// its tag matches.  Every wait is bounded; on expiry the context's error word is raised and nothing is stored.
#include <cuda_runtime.h>

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {
namespace {

__device__ __forceinline__ unsigned long long ld_relaxed_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) peer_finish_kernel(float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t n_vec,
                                                          const unsigned long long* __restrict__ slots, uint32_t* epoch, uint32_t* blocks_done,
                                                          uint32_t world, uint32_t capacity, uint32_t* error_word,
                                                          uint32_t polls /* reads of one word (~0.2 us apart once sleeping) before its sender is declared lost */) {
    // Launched as a programmatic dependent of the matmul that pushes: resident (and past its launch latency) while that kernel
    // still runs; the kernel behind this one may fill its weight ring meanwhile.  The wait orders this kernel behind everything
    // earlier in the stream: the previous reduction's epoch, earlier readers of y.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t next = *epoch + 1u, set = next & 1u;
    const uint64_t count = uint64_t{rows} * n_vec;
    const unsigned long long* base = slots + uint64_t{set} * world * capacity;
    bool lost = false;
    for (uint64_t i = uint64_t{blockIdx.x} * blockDim.x + threadIdx.x; i < count && !lost; i += uint64_t{gridDim.x} * blockDim.x) {
        // every rank's word of this element is requested before any is looked at: one round trip when they have all arrived
        unsigned long long w[mma::kMaxPeers];
#pragma unroll
        for (uint32_t p = 0; p < mma::kMaxPeers; ++p)
            if (p < world) w[p] = ld_relaxed_sys(base + uint64_t{p} * capacity + i);
        float sum = 0.0f;
#pragma unroll
        for (uint32_t p = 0; p < mma::kMaxPeers; ++p) {
            if (p < world && !lost) {
                const unsigned long long* src = base + uint64_t{p} * capacity + i;
                for (uint32_t n = 0; static_cast<uint32_t>(w[p] >> 32) != next; ++n) {
                    if (n >= polls) {
                        lost = true;
                        break;
                    }
                    if (n > 64) __nanosleep(200);
                    w[p] = ld_relaxed_sys(src);
                }
                const float v = __uint_as_float(static_cast<uint32_t>(w[p]));
                sum = p == 0 ? v : sum + v;  // rank order: every rank adds the same numbers in the same order
            }
        }
        if (lost) break;
        const uint32_t tk = static_cast<uint32_t>(i / rows), n = static_cast<uint32_t>(i - uint64_t{tk} * rows);
        reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{tk} * y_stride)[n] = sum;
    }
    if (lost && error_word != nullptr) atomicOr(error_word, 1u);
    // the last block to finish closes the reduction: the next one uses the other slot set
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(blocks_done, 1u) == gridDim.x - 1u) {
            *blocks_done = 0;
            *epoch = next;
        }
    }
}

}  // namespace

int launch_peer_finish(HaloCudaCtx* ctx, const HaloCudaPeerReduce& p, float* y, uint64_t y_stride, uint32_t rows, uint32_t n_vec, cudaStream_t s) {
    const uint64_t count = uint64_t{rows} * n_vec;
    const uint64_t blocks = (count + 255) / 256;  // one element per thread up to 296 blocks: the reads of an element's words overlap
    const uint32_t grid = static_cast<uint32_t>(blocks < 1 ? 1 : blocks > 296 ? 296 : blocks);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HC_CUDA(cudaLaunchKernelEx(&cfg, peer_finish_kernel, y, y_stride, rows, n_vec, static_cast<const unsigned long long*>(p.slots[p.rank]), p.epoch, p.done,
                               p.world, p.capacity, ctx->error_word_dev, ctx->peer_wait_polls));
    return 0;
}

}  // namespace halo_cuda
