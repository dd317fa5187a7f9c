// halo::backend::Backend over libhalo_cuda.so.  See cuda_backend.h for the contract.
#include "cuda_backend.h"

#include <array>
#include <cstring>
#include <format>
#include <limits>
#include <string>
#include <string_view>
#include <vector>

#include "halo/core/error.h"
#include "halo_cuda.h"

namespace halo::backend {
namespace {

[[noreturn]] void raise(int rc) {
    char buf[768];
    halo_cuda_last_error(buf, sizeof buf);
    const int code = -rc - 1;
    const ErrorCode ec = code >= 0 && code <= static_cast<int>(ErrorCode::Cancelled) ? static_cast<ErrorCode>(code) : ErrorCode::Backend;
    throw Error(ec, buf);
}
void check(int rc) {
    if (rc != 0) raise(rc);
}

class CudaBackend;

class CudaBuffer final : public Buffer {
public:
    CudaBuffer(const CudaBackend* owner, HaloCudaCtx* ctx, void* ptr, std::uint64_t bytes, bool writable)
        : owner_(owner), ctx_(ctx), ptr_(ptr), bytes_(bytes), writable_(writable) {}
    ~CudaBuffer() override { halo_cuda_free(ctx_, ptr_); }
    CudaBuffer(const CudaBuffer&) = delete;
    CudaBuffer& operator=(const CudaBuffer&) = delete;

    [[nodiscard]] std::uint64_t bytes() const noexcept override { return bytes_; }
    [[nodiscard]] Tier tier() const noexcept override { return Tier::Vram; }
    [[nodiscard]] const Backend* backend() const noexcept override;
    [[nodiscard]] bool writable() const noexcept override { return writable_; }
    [[nodiscard]] const std::byte* host_data() const noexcept override { return nullptr; }  // never host-addressable (ADR A-4)
    [[nodiscard]] std::byte* host_ptr() const noexcept override { return nullptr; }
    [[nodiscard]] std::byte* device() const noexcept { return static_cast<std::byte*>(ptr_); }

private:
    const CudaBackend* owner_;
    HaloCudaCtx* ctx_;
    void* ptr_;
    std::uint64_t bytes_;
    bool writable_;
};

class CudaStream final : public Stream {
public:
    CudaStream(const CudaBackend* owner, HaloCudaCtx* ctx, std::uint64_t timeout_ns) : owner_(owner), ctx_(ctx), timeout_ns_(timeout_ns) {
        check(halo_cuda_stream_create(ctx_, &stream_));
        void* p = nullptr;
        check(halo_cuda_malloc(ctx_, 4, 1, &p));
        status_dev_ = static_cast<std::uint32_t*>(p);
    }
    ~CudaStream() override {
        halo_cuda_stream_sync(ctx_, stream_, timeout_ns_);
        halo_cuda_free(ctx_, status_dev_);
        halo_cuda_stream_destroy(ctx_, stream_);
    }
    void submit() override {}
    void wait() override {
        std::uint32_t status = 0;
        int rc = 0;
        if (status_armed_) rc = halo_cuda_memcpy_d2h_async(ctx_, &status, status_dev_, 4, stream_);
        if (rc == 0) rc = halo_cuda_stream_sync(ctx_, stream_, timeout_ns_);
        staged_.clear();
        if (rc != 0) raise(rc);
        if (status_armed_) {
            status_armed_ = false;
            if (status != 0) {
                halo_cuda_memset_async(ctx_, status_dev_, 0, 4, stream_);
                // data errors of device ops surface at the wait (include/halo/backend/hip_backend.h:24-27)
                throw_error(ErrorCode::Kernel, "GET_ROWS: an id lies outside the table (status {:#x})", status);
            }
        }
    }
    void abort() noexcept override {
        halo_cuda_stream_sync(ctx_, stream_, timeout_ns_);
        staged_.clear();
        status_armed_ = false;
    }
    [[nodiscard]] const CudaBackend* owner() const noexcept { return owner_; }
    [[nodiscard]] HaloCudaStream handle() const noexcept { return stream_; }
    [[nodiscard]] std::uint32_t* status_word() noexcept {
        status_armed_ = true;
        return status_dev_;
    }
    /// Keeps a copy of upload bytes alive until wait() (the caller's span only has to live that long too, but the
    /// copy engine reads pageable memory late).
    const std::byte* stage(std::span<const std::byte> src) {
        staged_.emplace_back(src.begin(), src.end());
        return staged_.back().data();
    }

private:
    const CudaBackend* owner_;
    HaloCudaCtx* ctx_;
    std::uint64_t timeout_ns_;
    HaloCudaStream stream_ = nullptr;
    std::uint32_t* status_dev_ = nullptr;
    bool status_armed_ = false;
    std::vector<std::vector<std::byte>> staged_;
};

enum class Access : std::uint8_t { Read, Write };

std::uint64_t mul_u64(std::uint64_t a, std::uint64_t b, const char* op, const char* what) {
    HALO_CHECK(b == 0 || a <= std::numeric_limits<std::uint64_t>::max() / b, ErrorCode::Kernel, "{}: {} size overflows", op, what);
    return a * b;
}

constexpr std::size_t kMaxVariants = 16;

class CudaBackend final : public Backend {
public:
    explicit CudaBackend(const CudaBackendOptions& o) : options_(o) {
        const int rc = halo_cuda_ctx_create(o.device_ordinal, &ctx_);
        if (rc != 0) raise(rc);
        load_variants(HALO_CUDA_OP_GEMV, gemv_variants_, n_gemv_);
        load_variants(HALO_CUDA_OP_LM_HEAD, head_variants_, n_head_);
        load_variants(HALO_CUDA_OP_GET_ROWS, rows_variants_, n_rows_);
        if (o.default_gemv_variant != 0) {
            bool known = false;
            for (std::size_t i = 0; i < n_gemv_; ++i) known = known || gemv_variants_[i].id == o.default_gemv_variant;
            if (!known) {
                halo_cuda_ctx_destroy(ctx_);
                throw_error(ErrorCode::Config, "cuda backend: unknown default MATMUL variant id {}", o.default_gemv_variant);
            }
        }
    }
    ~CudaBackend() override { halo_cuda_ctx_destroy(ctx_); }

    [[nodiscard]] Kind kind() const noexcept override { return kKindCuda; }
    [[nodiscard]] std::string describe() const override {
        HaloCudaDeviceInfo info{};
        halo_cuda_device_info(ctx_, &info);
        return std::format("cuda matmul backend on {} ({}, {} SMs, driver {})", info.name, info.arch, info.sm_count, info.driver_version);
    }
    [[nodiscard]] Limits limits() const noexcept override {
        Limits l{};  // no GDN / attention / rope operators here: their limits stay 0
        l.lm_head_ids = true;
        return l;
    }
    [[nodiscard]] bool lost() const noexcept override { return halo_cuda_ctx_lost(ctx_) != 0; }

    std::unique_ptr<Buffer> allocate(std::uint64_t bytes, Tier /*device memory only*/) override {
        void* p = nullptr;
        check(halo_cuda_malloc(ctx_, bytes, 1, &p));  // zero-filled, as the CPU backend's (backend.h:523)
        return std::make_unique<CudaBuffer>(this, ctx_, p, bytes, true);
    }
    std::unique_ptr<Buffer> import_host(std::span<std::byte>) override {
        throw_error(ErrorCode::Unsupported,
                    "cuda backend: import_host would need a copy, and the caller expects its writes to stay visible in host memory");
    }
    std::unique_ptr<Buffer> import_host_readonly(std::span<const std::byte> bytes) override {
        void* p = nullptr;
        check(halo_cuda_malloc(ctx_, bytes.size(), 0, &p));
        auto buf = std::make_unique<CudaBuffer>(this, ctx_, p, bytes.size(), false);
        if (!bytes.empty()) {
            HaloCudaStream s = nullptr;
            check(halo_cuda_stream_create(ctx_, &s));
            int rc = halo_cuda_memcpy_h2d_async(ctx_, p, bytes.data(), bytes.size(), s);
            if (rc == 0) rc = halo_cuda_stream_sync(ctx_, s, options_.wait_timeout_ns);
            halo_cuda_stream_destroy(ctx_, s);
            check(rc);
        }
        return buf;
    }
    std::unique_ptr<Stream> create_stream() override { return std::make_unique<CudaStream>(this, ctx_, options_.wait_timeout_ns); }

    void upload(Stream& s, TensorRef dst, std::span<const std::byte> src) override {
        CudaStream& cs = stream_of(s, "upload");
        std::byte* d = resolve(dst, src.size(), Access::Write, "upload", "dst");
        if (!src.empty()) check(halo_cuda_memcpy_h2d_async(ctx_, d, cs.stage(src), src.size(), cs.handle()));
    }
    void download(Stream& s, TensorRef src, std::span<std::byte> dst) override {
        CudaStream& cs = stream_of(s, "download");
        const std::byte* p = resolve(src, dst.size(), Access::Read, "download", "src");
        if (!dst.empty()) check(halo_cuda_memcpy_d2h_async(ctx_, dst.data(), p, dst.size(), cs.handle()));
    }

    [[nodiscard]] std::span<const VariantInfo> variants(OpId op, std::string_view /*form*/) const override {
        switch (op) {
            case OpId::Gemv: return {gemv_variants_.data(), n_gemv_};
            case OpId::LmHead: return {head_variants_.data(), n_head_};
            case OpId::GetRows: return {rows_variants_.data(), n_rows_};
            case OpId::Copy: return {&kCopyVariant, 1};
            default: break;
        }
        HALO_CHECK(static_cast<std::size_t>(op) < kOpCount, ErrorCode::Api, "variants: unknown op id {}", static_cast<unsigned>(op));
        throw_error(ErrorCode::Unsupported, "variants: {} is not implemented by the cuda matmul backend", op_name(op));
    }

    // ---- implemented ops -------------------------------------------------------------------------------------------
    void get_rows(Stream& s, const GetRowsArgs& a) override {
        CudaStream& cs = stream_of(s, "GET_ROWS");
        check_status(a.status, OpId::GetRows);
        std::uint64_t rb = 0;
        check(halo_cuda_row_bytes(static_cast<std::uint32_t>(a.type), a.cols, &rb));
        HaloCudaGetRows g{};
        g.type = static_cast<std::uint32_t>(a.type);
        g.variant_id = a.kernel.variant_id;
        g.table = resolve(a.table, extent(a.n_rows, rb, a.table.row_stride, "GET_ROWS", "table"), Access::Read, "GET_ROWS", "table");
        g.table_stride = a.table.row_stride;
        g.ids = reinterpret_cast<const std::int32_t*>(resolve(a.ids, mul_u64(a.n_ids, 4, "GET_ROWS", "ids"), Access::Read, "GET_ROWS", "ids"));
        HALO_CHECK(a.n_ids == 0 || g.ids != nullptr, ErrorCode::Kernel, "GET_ROWS: operand ids is empty");
        g.out = reinterpret_cast<float*>(
            resolve(a.out, extent(a.n_ids, mul_u64(a.cols, 4, "GET_ROWS", "out"), a.out.row_stride, "GET_ROWS", "out"), Access::Write, "GET_ROWS", "out"));
        g.out_stride = a.out.row_stride;
        g.n_rows = a.n_rows;
        g.cols = a.cols;
        g.n_ids = a.n_ids;
        g.status = cs.status_word();
        check(halo_cuda_get_rows(ctx_, &g, cs.handle()));
    }

    void gemv(Stream& s, const GemvArgs& a) override {
        CudaStream& cs = stream_of(s, "MATMUL");
        const HaloCudaGemv g = gemv_struct(a, "MATMUL", false);
        if (a.gates.n_v != 0) {
            // the GDN gates epilogue: the library has it for F32 / Q8_0 weights on the fp32 kernels and refuses the rest
            const std::uint64_t nb = mul_u64(a.gates.n_v, 4, "MATMUL", "gates");
            const auto* db = reinterpret_cast<const float*>(resolve(a.gates.dt_bias, nb, Access::Read, "MATMUL", "gates.dt_bias"));
            const auto* ga = reinterpret_cast<const float*>(resolve(a.gates.a, nb, Access::Read, "MATMUL", "gates.a"));
            check(halo_cuda_gemv_gated(ctx_, &g, db, ga, a.gates.n_v, cs.handle()));
            return;
        }
        if (!a.norm_w.empty()) {
            // the fused input norm: the library has it for one x row on the tensor-core skinny kernels and refuses the rest
            const auto* nw = reinterpret_cast<const float*>(resolve(a.norm_w, mul_u64(a.cols, 4, "MATMUL", "norm_w"), Access::Read, "MATMUL", "norm_w"));
            check(halo_cuda_gemv_normed(ctx_, &g, nw, a.norm_eps, cs.handle()));
            return;
        }
        check(halo_cuda_gemv(ctx_, &g, cs.handle()));
    }

    void lm_head(Stream& s, const LmHeadArgs& a) override {
        CudaStream& cs = stream_of(s, "LM_HEAD");
        check_status(a.status, OpId::LmHead);
        HALO_CHECK(a.kernel.variant_id <= 1, ErrorCode::Config, "LM_HEAD: unknown kernel variant id {} on the cuda backend", a.kernel.variant_id);
        HALO_CHECK(a.ids_slots.empty() == a.ids_scatter.empty() && (a.ids_scatter.empty() || !a.ids.empty()), ErrorCode::Api,
                   "LM_HEAD: ids_slots and ids_scatter go together, and only with ids");
        HALO_CHECK(a.ids_scatter.empty(), ErrorCode::Unsupported, "LM_HEAD: the ids scatter is not implemented by the cuda matmul backend");
        HaloCudaLmHead h{};
        h.gemv = gemv_struct(a.gemv, "LM_HEAD", true);
        const std::uint64_t n = a.gemv.n_vec;
        h.result = reinterpret_cast<std::uint32_t*>(resolve(a.result, mul_u64(n, kArgmaxResultBytes, "LM_HEAD", "result"), Access::Write, "LM_HEAD", "result"));
        h.ids = reinterpret_cast<std::int32_t*>(resolve(a.ids, mul_u64(n, 4, "LM_HEAD", "ids"), Access::Write, "LM_HEAD", "ids"));
        h.valid_rows = a.valid_rows;
        h.row_offset = 0;
        check(halo_cuda_lm_head(ctx_, &h, cs.handle()));
    }

    void copy(Stream& s, const CopyArgs& a) override {
        CudaStream& cs = stream_of(s, "COPY");
        HALO_CHECK(a.kernel.variant_id == 0, ErrorCode::Config, "COPY: unknown kernel variant id {} on the cuda backend", a.kernel.variant_id);
        const std::byte* src = resolve(a.src, a.bytes, Access::Read, "COPY", "src");
        std::byte* dst = resolve(a.dst, a.bytes, Access::Write, "COPY", "dst");
        check(halo_cuda_memcpy_d2d_async(ctx_, dst, src, a.bytes, cs.handle()));
    }

    // ---- everything else: not this backend's, and never a silent host fallback ------------------------------------------------
    void rms_norm(Stream&, const RmsNormArgs&) override { unsupported(OpId::RmsNorm); }
    void add_rms_norm(Stream&, const AddRmsNormArgs&) override { unsupported(OpId::AddRmsNorm); }
    void gdn_gates(Stream&, const GdnGateArgs&) override { unsupported(OpId::GdnGates); }
    void conv1d_silu(Stream&, const Conv1dArgs&) override { unsupported(OpId::Conv1dSilu); }
    void gated_delta_rule(Stream&, const GdnArgs&) override { unsupported(OpId::GatedDeltaRule); }
    void gated_rms_norm(Stream&, const GatedNormArgs&) override { unsupported(OpId::GatedRmsNorm); }
    void partial_rope(Stream&, const RopeArgs&) override { unsupported(OpId::PartialRope); }
    void kv_write(Stream&, const KvWriteArgs&) override { unsupported(OpId::KvWrite); }
    void attention(Stream&, const AttentionArgs&) override { unsupported(OpId::Attention); }
    void swiglu(Stream&, const EltwiseArgs&) override { unsupported(OpId::Swiglu); }
    void mul_sigmoid(Stream&, const EltwiseArgs&) override { unsupported(OpId::MulSigmoid); }
    void add(Stream&, const EltwiseArgs&) override { unsupported(OpId::Add); }
    void argmax(Stream&, const ArgmaxArgs&) override { unsupported(OpId::Argmax); }
    void top_k(Stream&, const TopKArgs&) override { unsupported(OpId::TopK); }

    std::unique_ptr<Buffer> repack(Stream& s, DType wtype, const TensorRef& src, std::uint32_t rows, std::uint32_t cols) {
        CudaStream& cs = stream_of(s, "repack");
        std::uint64_t raw = 0, packed = 0;
        check(halo_cuda_row_bytes(static_cast<std::uint32_t>(wtype), cols, &raw));
        check(halo_cuda_repacked_row_bytes(static_cast<std::uint32_t>(wtype), cols, &packed));
        const std::byte* from = resolve(src, extent(rows, raw, src.row_stride, "repack", "src"), Access::Read, "repack", "src");
        void* p = nullptr;
        check(halo_cuda_malloc(ctx_, std::max<std::uint64_t>(mul_u64(rows, packed, "repack", "dst"), 16), 0, &p));
        auto buf = std::make_unique<CudaBuffer>(this, ctx_, p, mul_u64(rows, packed, "repack", "dst"), false);
        check(halo_cuda_repack_rows(ctx_, static_cast<std::uint32_t>(wtype), from, src.row_stride, p, 0, rows, cols, cs.handle()));
        return buf;
    }

    CudaMat load_mat(Stream& s, const HaloGguf* file, std::string_view name, const CudaSplit& split) {
        CudaStream& cs = stream_of(s, "load_mat");
        HALO_CHECK(file != nullptr, ErrorCode::Api, "load_mat: null container");
        const std::string key(name);
        std::uint64_t index = 0;
        int found = 0;
        check(halo_gguf_find(file, key.c_str(), &index, &found));
        HALO_CHECK(found != 0, ErrorCode::Model, "missing weight matrix {}", name);
        HaloCudaUpload how{};
        how.split = static_cast<std::uint32_t>(split.mode);
        how.rank = split.rank;
        how.world = split.world;
        how.repack = split.repack ? 1 : 0;
        HaloCudaMatrix m{};
        check(halo_cuda_upload_matrix(ctx_, file, index, &how, cs.handle(), &m));
        CudaMat out;
        if (m.w != nullptr) out.buf = std::make_unique<CudaBuffer>(this, ctx_, m.w, m.bytes, false);
        out.type = static_cast<DType>(m.wtype);
        out.rows = m.rows;
        out.cols = m.cols;
        out.row0 = m.row0;
        out.k0 = m.k0;
        out.row_stride = m.w_stride;
        out.kernel = KernelChoice{m.variant_id};
        return out;
    }

    void set_plan(std::span<const CudaPlanEntry> plan) {
        check(halo_cuda_plan_clear(ctx_));
        for (const CudaPlanEntry& p : plan)
            check(halo_cuda_plan_set(ctx_, static_cast<std::uint32_t>(p.wtype), p.rows, p.cols, p.n_vec_lo, p.n_vec_hi, p.variant_id));
    }

private:
    static constexpr VariantInfo kCopyVariant{0, "memcpy_d2d", OpId::Copy, {}};

    [[noreturn]] static void unsupported(OpId op) {
        throw_error(ErrorCode::Unsupported, "{} is not implemented by the cuda matmul backend (and it has no host fallback)", op_name(op));
    }
    static void check_status(const StatusRef& s, OpId op) {
        HALO_CHECK(s.empty(), ErrorCode::Unsupported, "{}: status words are not implemented yet (ADR-001 WS-BI-2)", op_name(op));
    }

    void load_variants(std::uint32_t op, std::array<VariantInfo, kMaxVariants>& out, std::size_t& n) {
        std::array<HaloCudaVariant, kMaxVariants> raw{};
        std::uint32_t count = 0;
        check(halo_cuda_variants(op, raw.data(), kMaxVariants, &count));
        n = count < kMaxVariants ? count : kMaxVariants;
        for (std::size_t i = 0; i < n; ++i) out[i] = VariantInfo{raw[i].id, raw[i].name, static_cast<OpId>(op), {}};
    }

    CudaStream& stream_of(Stream& s, const char* op) const {
        auto* cs = dynamic_cast<CudaStream*>(&s);
        HALO_CHECK(cs != nullptr && cs->owner() == this, ErrorCode::Api, "{}: stream of another backend", op);
        return *cs;
    }

    /// Bytes from the first to one past the last byte of `rows` rows (stride 0 = dense), overflow-checked.
    static std::uint64_t extent(std::uint64_t rows, std::uint64_t row_bytes, std::uint64_t stride, const char* op, const char* name) {
        if (rows == 0) return 0;
        const std::uint64_t st = stride != 0 ? stride : row_bytes;
        const std::uint64_t e = mul_u64(rows - 1, st, op, name) + row_bytes;
        HALO_CHECK(e >= row_bytes, ErrorCode::Kernel, "{}: operand {} size overflows", op, name);
        return e;
    }

    /// Ownership, writability and range checks of the CPU backend's Resolver (src/backend/cpu_backend.cpp:98-142);
    /// stride, alignment and overlap checks follow in the C ABI on the resolved addresses.
    std::byte* resolve(const TensorRef& ref, std::uint64_t need, Access access, const char* op, const char* name) const {
        if (ref.empty()) return nullptr;
        const auto* b = dynamic_cast<const CudaBuffer*>(ref.buffer);
        HALO_CHECK(b != nullptr && b->backend() == this, ErrorCode::Kernel, "{}: operand {} belongs to another backend", op, name);
        HALO_CHECK(access == Access::Read || b->writable(), ErrorCode::Kernel, "{}: output {} is read-only", op, name);
        HALO_CHECK(ref.offset <= b->bytes(), ErrorCode::Kernel, "{}: operand {} offset {} past buffer end {}", op, name, ref.offset, b->bytes());
        const std::uint64_t avail = b->bytes() - ref.offset;
        const std::uint64_t limit = ref.bytes != 0 ? ref.bytes : avail;
        HALO_CHECK(limit <= avail, ErrorCode::Kernel, "{}: operand {} range [{}, +{}) exceeds buffer of {} bytes", op, name, ref.offset, ref.bytes,
                   b->bytes());
        HALO_CHECK(need <= limit, ErrorCode::Kernel, "{}: operand {} needs {} bytes, view has {}", op, name, need, limit);
        return b->device() + ref.offset;
    }

    HaloCudaGemv gemv_struct(const GemvArgs& a, const char* op, bool y_optional) const {
        HALO_CHECK(a.norm_w.empty() || std::string_view(op) == "MATMUL", ErrorCode::Unsupported, "{}: a fused norm (GemvArgs::norm_w) is for MATMUL only", op);
        HALO_CHECK(a.gates.n_v == 0 || (std::string_view(op) == "MATMUL" && a.norm_w.empty()), ErrorCode::Unsupported,
                   "{}: the GDN gates epilogue (GemvArgs::gates) is for MATMUL without a fused norm", op);
        HaloCudaGemv g{};
        g.wtype = static_cast<std::uint32_t>(a.wtype);
        g.variant_id = a.kernel.variant_id != 0 ? a.kernel.variant_id : options_.default_gemv_variant;
        std::uint64_t rb = 0;
        if (g.variant_id == HALO_CUDA_GEMV_MMA_R || g.variant_id == HALO_CUDA_GEMV_MMA_I8X2_R || g.variant_id == HALO_CUDA_GEMM_TCGEN05_F16_R ||
            g.variant_id == HALO_CUDA_GEMM_TCGEN05_BF16_R)
            check(halo_cuda_repacked_row_bytes(g.wtype, a.cols, &rb));  // W is in the variant's layout
        else check(halo_cuda_row_bytes(g.wtype, a.cols, &rb));
        g.w = resolve(a.w, extent(a.rows, rb, a.w.row_stride, op, "w"), Access::Read, op, "w");
        g.w_stride = a.w.row_stride;
        g.x = reinterpret_cast<const float*>(resolve(a.x, extent(a.n_vec, mul_u64(a.cols, 4, op, "x"), a.x.row_stride, op, "x"), Access::Read, op, "x"));
        g.x_stride = a.x.row_stride;
        g.y = reinterpret_cast<float*>(resolve(a.y, extent(a.n_vec, mul_u64(a.rows, 4, op, "y"), a.y.row_stride, op, "y"), Access::Write, op, "y"));
        g.y_stride = a.y.row_stride;
        HALO_CHECK(y_optional || g.y != nullptr || a.n_vec == 0 || a.rows == 0, ErrorCode::Kernel, "{}: operand y is empty", op);
        g.rows = a.rows;
        g.cols = a.cols;
        g.n_vec = a.n_vec;
        g.flags = a.allow_gemm ? HALO_CUDA_GEMV_FLAG_ALLOW_GEMM : 0u;
        return g;
    }

    CudaBackendOptions options_;
    HaloCudaCtx* ctx_ = nullptr;
    std::array<VariantInfo, kMaxVariants> gemv_variants_{}, head_variants_{}, rows_variants_{};
    std::size_t n_gemv_ = 0, n_head_ = 0, n_rows_ = 0;
};

const Backend* CudaBuffer::backend() const noexcept { return owner_; }

}  // namespace

std::unique_ptr<Backend> make_cuda_backend(const CudaBackendOptions& options) { return std::make_unique<CudaBackend>(options); }

std::unique_ptr<Buffer> cuda_backend_repack(Backend& backend, Stream& stream, DType wtype, const TensorRef& src, std::uint32_t rows,
                                            std::uint32_t cols) {
    auto* cb = dynamic_cast<CudaBackend*>(&backend);
    HALO_CHECK(cb != nullptr, ErrorCode::Api, "cuda_backend_repack: not a cuda backend");
    return cb->repack(stream, wtype, src, rows, cols);
}

CudaMat cuda_backend_load_mat(Backend& backend, Stream& stream, const HaloGguf* file, std::string_view name, const CudaSplit& split) {
    auto* cb = dynamic_cast<CudaBackend*>(&backend);
    HALO_CHECK(cb != nullptr, ErrorCode::Api, "cuda_backend_load_mat: not a cuda backend");
    return cb->load_mat(stream, file, name, split);
}

void cuda_backend_set_plan(Backend& backend, std::span<const CudaPlanEntry> plan) {
    auto* cb = dynamic_cast<CudaBackend*>(&backend);
    HALO_CHECK(cb != nullptr, ErrorCode::Api, "cuda_backend_set_plan: not a cuda backend");
    cb->set_plan(plan);
}

}  // namespace halo::backend
