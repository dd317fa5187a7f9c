/*
 * halo_cuda_gguf.h -- C ABI of the weight loader of libhalo_cuda.so: GGUF file -> device-resident matmul operand.
 *
 * This is the step in front of the matmul path: where the reference parses a GGUF container
 * (GgufFile, include/halo/model/gguf.h:133-199; src/model/gguf.cpp:330-470), hands each projection's
 * bytes to Backend::import_host_readonly and optionally repacks them on the way
 * (Impl::make_mat / try_repack, src/models/qwen35.cpp:301-346), this header offers
 *   - an index of the container (metadata scalars and strings, tensor infos, tensor bytes), and
 *   - one call that brings a 2-D tensor, or one rank's tensor-parallel share of it, into device
 *     memory through double-buffered pinned staging, repacked on the device if asked.
 * The file is untrusted input: every count, length, offset and size is checked for overflow and against the bytes
 * that are there before it is used.  Same conventions as halo_cuda.h: int status, 0 = ok, negative = error class;
 * halo_cuda_last_error() has the message.  Malformed file -> HALO_CUDA_E_MODEL; well-formed but not supported
 * (GGUF v1, big-endian) -> HALO_CUDA_E_UNSUPPORTED; a file that cannot be opened or mapped -> HALO_CUDA_E_IO.
 */
#ifndef HALO_CUDA_GGUF_H
#define HALO_CUDA_GGUF_H

#include "halo_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HALO_CUDA_E_IO (-9) /* halo::ErrorCode::Io: the file cannot be opened, read or mapped */

typedef struct HaloGguf HaloGguf; /* an immutable parsed container; concurrent reads are safe */

typedef struct HaloGgufInfo {
    uint32_t version;   /* 2 or 3 */
    uint32_t alignment; /* general.alignment, default 32 */
    uint64_t n_kv, n_tensors;
    uint64_t header_size; /* end of the tensor infos */
    uint64_t data_offset; /* header_size rounded up to the alignment */
    uint64_t file_size;
} HaloGgufInfo;

/* One tensor info (GgufTensorInfo, gguf.h:83-100).  ne[] is in ggml order: ne[0] is the contiguous (input)
 * dimension, so a projection y = W x is stored as ne = {cols, rows}.  `type` is the ggml type id; `supported`
 * is 1 when it is one of the weight types of halo_cuda.h. */
typedef struct HaloGgufTensor {
    char name[64];
    uint32_t n_dims;
    uint32_t type;
    int64_t ne[4];
    uint64_t offset; /* relative to data_offset; a multiple of the alignment */
    uint64_t n_elements;
    uint64_t n_bytes;
    uint32_t supported;
    uint32_t reserved;
} HaloGgufTensor;

/* Opens and maps `path` read-only, or parses `size` bytes the caller keeps alive until halo_gguf_close
 * (GgufFile::open / GgufFile::parse in full mode: every tensor's byte range must lie inside the file). */
int halo_gguf_open(const char* path, HaloGguf** out);
int halo_gguf_parse(const void* bytes, uint64_t size, HaloGguf** out);
int halo_gguf_close(HaloGguf* g);
int halo_gguf_info(const HaloGguf* g, HaloGgufInfo* out);

/* Metadata (GgufFile::get_uint / get_int / get_float / get_string, gguf.h:169-175).  *found = 0 and status 0 when
 * the key is absent; HALO_CUDA_E_MODEL when it is present with a type that cannot represent the request (a
 * string for an integer, a negative value for u64).  halo_gguf_kv_string copies at most cap - 1 bytes plus a
 * terminator and returns the full length in *len. */
int halo_gguf_kv_u64(const HaloGguf* g, const char* key, uint64_t* value, int* found);
int halo_gguf_kv_i64(const HaloGguf* g, const char* key, int64_t* value, int* found);
int halo_gguf_kv_f64(const HaloGguf* g, const char* key, double* value, int* found);
int halo_gguf_kv_string(const HaloGguf* g, const char* key, char* buf, uint64_t cap, uint64_t* len, int* found);

/* Tensors (GgufFile::tensors / find_tensor / tensor_data, gguf.h:178-183).  halo_gguf_find sets *found = 0 for an
 * unknown name.  The data pointer is valid until halo_gguf_close. */
int halo_gguf_tensor(const HaloGguf* g, uint64_t index, HaloGgufTensor* out);
int halo_gguf_find(const HaloGguf* g, const char* name, uint64_t* index, int* found);
int halo_gguf_tensor_data(const HaloGguf* g, uint64_t index, const void** data, uint64_t* bytes);

/* Tensor-parallel share of a matrix.  COLUMN keeps whole W rows [row0, row0 + rows); ROW keeps the K range
 * [k0, k0 + cols) of every row, cut at whole quantization blocks (256 elements for Q4_K / Q6_K, 32 for Q8_0 /
 * Q4_0, 1 for F32).  Items are dealt as contiguous ranges, the first (n mod world) ranks getting one more -- the
 * reference's static partition (include/halo/backends/cpu/thread_pool.h:64-72). */
#define HALO_CUDA_SPLIT_NONE 0
#define HALO_CUDA_SPLIT_COLUMN 1
#define HALO_CUDA_SPLIT_ROW 2

typedef struct HaloCudaUpload {
    uint32_t split;
    uint32_t rank, world; /* world 0 or 1 = the whole matrix */
    uint32_t repack;      /* 1: store the rows in the repacked layout (halo_cuda_repack_rows) when the type and the local K allow it */
    uint64_t staging_bytes; /* size of each of the two pinned staging buffers; 0 = 32 MiB */
} HaloCudaUpload;

/* The device-resident operand: what HaloCudaGemv.w / w_stride / wtype / variant_id / rows / cols take. */
typedef struct HaloCudaMatrix {
    void* w; /* device memory owned by the caller: halo_cuda_free */
    uint64_t w_stride;
    uint64_t bytes;
    uint32_t wtype;
    uint32_t variant_id; /* when repacked: halo_cuda_repacked_variant of the largest local K; else HALO_CUDA_GEMV_DEFAULT */
    uint32_t rows, cols; /* local */
    uint32_t row0, k0;   /* first global row / K element of the share */
} HaloCudaMatrix;

/* The share of a matrix, computed without touching a device (the same arithmetic halo_cuda_upload_matrix uses). */
int halo_cuda_matrix_share(uint32_t wtype, uint32_t rows, uint32_t cols, const HaloCudaUpload* how, HaloCudaMatrix* out);

/* Brings tensor `index` (2-D, a supported type) or this rank's share of it into device memory.  Replaces
 * Impl::make_mat + Backend::import_host_readonly + Impl::try_repack (src/models/qwen35.cpp:301-346).  The bytes go
 * from the mapping into two pinned staging buffers in turn (rows of a ROW share are gathered there) and from
 * each to the device with an asynchronous copy on `stream`, so that the host's reads of the file overlap the
 * transfers; a repack runs as a device kernel behind the last copy.  When the call returns the file is no longer
 * being read; the operand is ready in stream order. */
int halo_cuda_upload_matrix(HaloCudaCtx* ctx, const HaloGguf* g, uint64_t index, const HaloCudaUpload* how, HaloCudaStream stream,
                            HaloCudaMatrix* out);

#ifdef __cplusplus
}
#endif
#endif /* HALO_CUDA_GGUF_H */
