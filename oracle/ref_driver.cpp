// C entry points around the UNMODIFIED reference CPU backend.  TEST INFRASTRUCTURE ONLY.
//
// The Makefile beside this file (target `ref`) compiles it together with the reference's own sources (where they lie
// in the reference tree, never copied) into oracle/_ref/libhalo_ref.so.  The calls below go
// through the reference's public interface exactly as its own tests do:
// halo::backend::make_cpu_backend(&pool) -> import_host* -> Backend::gemv / lm_head
// (tests/unit/backend/test_cpu_backend.cpp:257-284, 479-520).  The library validates the
// plain-C restatement in halo_oracle.c and serves as the "reference" CPU baseline.
//
// Status codes: 0 = ok, otherwise -(1 + halo::ErrorCode) (include/halo/core/error.h:15-26),
// -100 for a non-halo exception.
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <span>
#include <string>

#include "halo/backend/backend.h"
#include "halo/backends/cpu/thread_pool.h"
#include "halo/core/error.h"
#include "halo/tensor/fp16.h"
#include "halo/tensor/quant.h"

namespace hb = halo::backend;

namespace {

thread_local std::string g_last_error;

template <class Fn>
int guarded(Fn&& fn) noexcept {
    try {
        fn();
        return 0;
    } catch (const halo::Error& e) {
        g_last_error = e.what();
        return -(1 + static_cast<int>(e.code()));
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return -100;
    }
}

struct Session {
    halo::cpu::ThreadPool pool;
    std::unique_ptr<hb::Backend> be;
    std::unique_ptr<hb::Stream> st;
    explicit Session(std::size_t threads) : pool(threads), be(hb::make_cpu_backend(&pool)), st(be->create_stream()) {}
};

std::span<const std::byte> cbytes(const void* p, std::uint64_t n) { return {static_cast<const std::byte*>(p), n}; }
std::span<std::byte> wbytes(void* p, std::uint64_t n) { return {static_cast<std::byte*>(p), n}; }

}  // namespace

extern "C" {

const char* halo_ref_last_error() { return g_last_error.c_str(); }

int halo_ref_default_threads() { return static_cast<int>(halo::cpu::ThreadPool::default_threads()); }

float halo_ref_fp16_to_fp32(std::uint16_t h) { return halo::tensor::fp16_to_fp32(h); }
std::uint16_t halo_ref_fp32_to_fp16(float f) { return halo::tensor::fp32_to_fp16(f); }

std::int64_t halo_ref_row_bytes(int type, std::int64_t n) {
    std::int64_t out = 0;
    const int rc = guarded([&] { out = static_cast<std::int64_t>(halo::tensor::row_bytes(static_cast<halo::DType>(type), n)); });
    return rc != 0 ? rc : out;
}

int halo_ref_dequantize_row(int type, const void* src, float* dst, std::int64_t n) {
    return guarded([&] { halo::tensor::dequantize_row(static_cast<halo::DType>(type), static_cast<const std::byte*>(src), dst, n); });
}

void* halo_ref_session_create(int threads) {
    Session* s = nullptr;
    const int rc = guarded([&] { s = new Session(threads < 1 ? 1 : static_cast<std::size_t>(threads)); });
    return rc == 0 ? s : nullptr;
}
void halo_ref_session_destroy(void* s) { delete static_cast<Session*>(s); }

/// Backend::gemv on caller memory.  Spans (w_bytes, x_bytes, y_bytes) are the imported
/// buffers; offsets and strides are in bytes as in TensorRef (0 stride = dense).
int halo_ref_gemv(void* session, int type, const void* w, std::uint64_t w_bytes, std::uint64_t w_off, std::uint64_t w_stride,
                  const void* x, std::uint64_t x_bytes, std::uint64_t x_off, std::uint64_t x_stride, void* y,
                  std::uint64_t y_bytes, std::uint64_t y_off, std::uint64_t y_stride, std::uint32_t rows, std::uint32_t cols,
                  std::uint32_t n_vec, std::uint32_t variant_id) {
    auto* s = static_cast<Session*>(session);
    return guarded([&] {
        const auto wb = s->be->import_host_readonly(cbytes(w, w_bytes));
        // x and y may be the same memory (the overlap-rejection case): import once then.
        const bool same = x == y && x_bytes == y_bytes;
        const auto yb = s->be->import_host(wbytes(y, y_bytes));
        const auto xb = same ? nullptr : s->be->import_host_readonly(cbytes(x, x_bytes));
        hb::GemvArgs a{};
        a.wtype = static_cast<halo::DType>(type);
        a.w = hb::TensorRef{wb.get(), w_off, 0, w_stride};
        a.x = hb::TensorRef{same ? yb.get() : xb.get(), x_off, 0, x_stride};
        a.y = hb::TensorRef{yb.get(), y_off, 0, y_stride};
        a.rows = rows;
        a.cols = cols;
        a.n_vec = n_vec;
        a.kernel = hb::KernelChoice{variant_id};
        s->be->gemv(*s->st, a);
        s->st->wait();
    });
}

/// Backend::lm_head on caller memory.  logits / ids may be null (operand left empty).
int halo_ref_lm_head(void* session, int type, const void* w, std::uint64_t w_bytes, std::uint64_t w_stride, const void* x,
                     std::uint64_t x_bytes, std::uint64_t x_stride, void* logits, std::uint64_t logits_bytes,
                     std::uint64_t logits_stride, void* result, void* ids, std::uint32_t rows, std::uint32_t cols,
                     std::uint32_t n_vec, std::uint32_t valid_rows) {
    auto* s = static_cast<Session*>(session);
    return guarded([&] {
        const auto wb = s->be->import_host_readonly(cbytes(w, w_bytes));
        const auto xb = s->be->import_host_readonly(cbytes(x, x_bytes));
        const auto rb = s->be->import_host(wbytes(result, std::uint64_t{n_vec} * hb::kArgmaxResultBytes));
        std::unique_ptr<hb::Buffer> lb, ib;
        hb::LmHeadArgs a{};
        a.gemv.wtype = static_cast<halo::DType>(type);
        a.gemv.w = hb::TensorRef{wb.get(), 0, 0, w_stride};
        a.gemv.x = hb::TensorRef{xb.get(), 0, 0, x_stride};
        if (logits != nullptr) {
            lb = s->be->import_host(wbytes(logits, logits_bytes));
            a.gemv.y = hb::TensorRef{lb.get(), 0, 0, logits_stride};
        }
        a.gemv.rows = rows;
        a.gemv.cols = cols;
        a.gemv.n_vec = n_vec;
        a.result = hb::TensorRef::of(*rb);
        a.valid_rows = valid_rows;
        if (ids != nullptr) {
            ib = s->be->import_host(wbytes(ids, std::uint64_t{n_vec} * 4));
            a.ids = hb::TensorRef::of(*ib);
        }
        s->be->lm_head(*s->st, a);
        s->st->wait();
    });
}

}  // extern "C"
