#pragma once
/// \file
/// The B200 matmul backend behind HALO's Backend interface (include/halo/backend/backend.h of the reference).
///
/// Scope: MATMUL (gemv), LM_HEAD, GET_ROWS, COPY, upload / download, over libhalo_cuda.so (include/halo_cuda.h).
/// Every other operator of the interface raises Error(Unsupported): this backend never computes on the host and
/// never silently ignores an argument (norm_w, gates, status words and the ids scatter are refused like the CPU
/// backend refuses what it does not implement, src/backend/cpu_backend.cpp:341-342).
///
/// Contracts kept from the CPU backend (src/backend/cpu_backend.cpp:98-162) and the device adapters
/// (include/halo/backend/hip_backend.h:20-46): operands must belong to this backend, outputs must be writable and must
/// not overlap inputs, validation happens before anything is enqueued, allocate() zero-fills, import_host_readonly()
/// copies to the device, import_host() is refused, buffers are not host-addressable, data errors of GET_ROWS surface
/// at the next Stream::wait(), a wait that exceeds its budget raises Error(Backend) and makes lost() true.
///
/// Variant ids (KernelChoice) are those of include/halo_cuda.h; 0 = the shape heuristic or the installed plan.
#include <cstdint>
#include <memory>

#include <string_view>

#include "halo/backend/backend.h"
#include "halo_cuda_gguf.h"

namespace halo::backend {

/// Kind has no CUDA enumerator yet (backend.h:64); the model only special-cases Kind::Vulkan.
inline constexpr Kind kKindCuda = static_cast<Kind>(4);

struct CudaBackendOptions {
    int device_ordinal = 0;
    std::uint32_t default_gemv_variant = 0;  ///< variant run for KernelChoice{}; Error(Config) if not registered
    std::uint64_t wait_timeout_ns = 0;       ///< Stream::wait budget, 0 = unlimited
};

/// One (shape bucket -> variant) decision of the autotuner, installed for KernelChoice{} calls.
struct CudaPlanEntry {
    DType wtype = DType::Q4_K;
    std::uint32_t rows = 0, cols = 0, n_vec_lo = 1, n_vec_hi = 1, variant_id = 0;
};

/// Throws Error(Device) when no sm_100 device is usable, Error(Config) for an unknown default variant.
[[nodiscard]] std::unique_ptr<Backend> make_cuda_backend(const CudaBackendOptions& options = {});

/// The load-time weight repack of the variants gemv_mma_r (id 7) and gemv_mma_i8x2_r (id 9), the counterpart of tensor::gemv_repack for the
/// reference's repacked Vulkan matvecs (include/halo/tensor/repack.h:11-36): `rows` raw GGUF rows of Q6_K / Q8_0 /
/// Q4_0 (cols a multiple of 256) -> a new read-only device buffer in the repacked row layout, to be passed as
/// GemvArgs::w together with KernelChoice{7} or KernelChoice{9}.  Error(Unsupported) for other types, Error(Api) for another backend.
[[nodiscard]] std::unique_ptr<Buffer> cuda_backend_repack(Backend& backend, Stream& stream, DType wtype, const TensorRef& src, std::uint32_t rows,
                                                          std::uint32_t cols);

/// How a matrix is shared out over a tensor-parallel group: Column keeps whole W rows of each rank, Row keeps a K range cut at
/// whole quantization blocks (ranges dealt like ThreadPool::partition_range, include/halo/backends/cpu/thread_pool.h:64-72).
struct CudaSplit {
    enum class Mode : std::uint32_t { None = 0, Column = 1, Row = 2 } mode = Mode::None;
    std::uint32_t rank = 0, world = 1;
    bool repack = false;  ///< store Q6_K / Q8_0 / Q4_0 rows in the repacked layout when the local K is a multiple of 256
};

/// A device-resident matmul operand with what GemvArgs needs beside it: the counterpart of the model's Mat
/// (src/models/qwen35.cpp:52-67).  `kernel` is the repacked variant the loader chose (KernelChoice{9} where the int8 kernels hold the
/// local K in shared memory, else KernelChoice{7}) for repacked rows, else KernelChoice{}.
struct CudaMat {
    std::unique_ptr<Buffer> buf;  ///< null for an empty share
    DType type = DType::F32;
    std::uint32_t rows = 0, cols = 0;  ///< local extents
    std::uint32_t row0 = 0, k0 = 0;    ///< first global row / K element of the share
    std::uint64_t row_stride = 0;
    KernelChoice kernel{};
    [[nodiscard]] TensorRef ref() const { return TensorRef::of(*buf).with_stride(row_stride); }
};

/// Loads tensor `name` of an opened GGUF container (halo_gguf_open / halo_gguf_parse), or one rank's share of it, into device
/// memory of `backend`: what Impl::make_mat + import_host_readonly + try_repack do for the reference's backends
/// (src/models/qwen35.cpp:301-346), with the file read through pinned staging while the previous piece is in flight.
/// Error(Model) for a missing tensor, a tensor that is not a matrix of dense rows; Error(Unsupported) for a type without a kernel.
[[nodiscard]] CudaMat cuda_backend_load_mat(Backend& backend, Stream& stream, const HaloGguf* file, std::string_view name, const CudaSplit& split = {});

/// Installs tuner decisions on a backend made by make_cuda_backend (Error(Api) for any other backend).
void cuda_backend_set_plan(Backend& backend, std::span<const CudaPlanEntry> plan);

}  // namespace halo::backend
