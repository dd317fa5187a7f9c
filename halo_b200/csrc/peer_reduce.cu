// The second half of halo_cuda_gemv_reduce: wait for every rank's arrival flag, add the pushed slots in rank order.
// The first half is the push epilogue of the balanced skinny kernels (mma_common.cuh, sk_flush).
#include <cuda_runtime.h>

#include "internal.h"
#include "mma_common.cuh"

namespace halo_cuda {
namespace {

constexpr uint32_t kFlagPolls = 1u << 20;  // x ~1 us of sleep each: about a second before a peer is declared lost

__global__ void __launch_bounds__(256) peer_finish_kernel(float* __restrict__ y, uint64_t y_stride, uint32_t rows, uint32_t n_vec,
                                                          const float* __restrict__ slots, const uint32_t* __restrict__ flags, uint32_t* epoch,
                                                          uint32_t* blocks_done, uint32_t world, uint32_t capacity, uint32_t* error_word) {
    const uint32_t next = *epoch + 1u, set = next & 1u;
    __shared__ uint32_t ok;
    if (threadIdx.x == 0) {
        uint32_t good = 1;
        for (uint32_t p = 0; p < world && good; ++p) {
            uint32_t n = 0;
            while (mma::ld_acquire_sys(flags + set * world + p) != next) {
                if (++n == kFlagPolls) {
                    good = 0;
                    break;
                }
                __nanosleep(1000);
            }
        }
        if (!good && error_word != nullptr) atomicOr(error_word, 1u);
        ok = good;
    }
    __syncthreads();
    if (ok) {
        const uint64_t count = uint64_t{rows} * n_vec;
        const float* base = slots + uint64_t{set} * world * capacity;
        for (uint64_t i = uint64_t{blockIdx.x} * blockDim.x + threadIdx.x; i < count; i += uint64_t{gridDim.x} * blockDim.x) {
            float sum = __ldcg(base + i);  // the slots were written by other GPUs: read them from L2, not a stale L1 line
            for (uint32_t p = 1; p < world; ++p) sum += __ldcg(base + uint64_t{p} * capacity + i);
            const uint32_t tk = static_cast<uint32_t>(i / rows), n = static_cast<uint32_t>(i - uint64_t{tk} * rows);
            reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(y) + uint64_t{tk} * y_stride)[n] = sum;
        }
    }
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
    const uint32_t grid = static_cast<uint32_t>(count / 2048 < 1 ? 1 : count / 2048 > 64 ? 64 : count / 2048);
    // `done` is free again once the matmul's last row block has raised the flags: it doubles as the block counter here
    peer_finish_kernel<<<grid, 256, 0, s>>>(y, y_stride, rows, n_vec, p.slots[p.rank], p.flags[p.rank], p.epoch, p.done, p.world, p.capacity,
                                            ctx->error_word_dev);
    HC_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace halo_cuda
