// Differential tests THROUGH the reference's Backend interface: the unmodified reference CPU backend (from
// oracle/_ref/libhalo_ref.so) and the cuda adapter run the same calls on the same bytes.  TEST CODE: this file links the
// oracle; the product library does not.  The cases mirror the reference's own adapter tests
// (tests/unit/backend/test_cpu_backend.cpp:257-284, 479-603; tests/unit/backend/test_hip_backend.cpp:363-397, 655-722,
// 925-1040).  pytest loads the library and calls halo_adapter_selftest(); the report names every failed check.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <format>
#include <functional>
#include <random>
#include <string>
#include <vector>

#include "cuda_backend.h"
#include "halo/backend/backend.h"
#include "halo/backends/cpu/thread_pool.h"
#include "halo/core/error.h"
#include "halo/tensor/quant.h"

namespace hb = halo::backend;
using halo::DType;
using halo::ErrorCode;

namespace {

struct Report {
    std::string text;
    int failed = 0, passed = 0;
    void expect(bool ok, const std::string& what) {
        if (ok) {
            ++passed;
        } else {
            ++failed;
            text += "FAILED: " + what + "\n";
        }
    }
};

std::span<const std::byte> cbytes(const void* p, std::size_t n) { return {static_cast<const std::byte*>(p), n}; }
std::span<std::byte> wbytes(void* p, std::size_t n) { return {static_cast<std::byte*>(p), n}; }

int code_of(const std::function<void()>& fn) {
    try {
        fn();
    } catch (const halo::Error& e) {
        return static_cast<int>(e.code());
    } catch (...) {
        return -2;
    }
    return -1;  // no error
}

/// Random block bytes with every fp16 scale field forced to a small finite value.
std::vector<std::byte> random_weights(DType t, std::size_t rows, std::size_t cols, unsigned seed) {
    const std::size_t rb = halo::tensor::row_bytes(t, static_cast<std::int64_t>(cols));
    std::vector<std::byte> w(rows * rb);
    std::mt19937 g(seed);
    for (auto& b : w) b = static_cast<std::byte>(g() & 0xFFu);
    const auto set_f16 = [&](std::size_t off) {  // 0x2C00 = 1/16, low mantissa bits random
        w[off] = static_cast<std::byte>(g() & 0xFFu);
        w[off + 1] = static_cast<std::byte>(0x2C | (g() & 0x03u));
    };
    const std::size_t bb = t == DType::Q4_K ? 144 : t == DType::Q6_K ? 210 : t == DType::Q8_0 ? 34 : 18;
    for (std::size_t blk = 0; blk + bb <= w.size(); blk += bb) {
        if (t == DType::Q6_K) {
            set_f16(blk + 208);
        } else {
            set_f16(blk);
            if (t == DType::Q4_K) set_f16(blk + 2);
        }
    }
    return w;
}

std::vector<float> random_floats(std::size_t n, unsigned seed) {
    std::mt19937 g(seed);
    std::vector<float> v(n);
    for (auto& f : v) f = static_cast<float>(static_cast<int>(g() % 2001) - 1000) / 1000.0f;
    return v;
}

struct Pair {
    halo::cpu::ThreadPool pool{4};
    std::unique_ptr<hb::Backend> cpu = hb::make_cpu_backend(&pool);
    std::unique_ptr<hb::Backend> gpu = hb::make_cuda_backend({});
    std::unique_ptr<hb::Stream> cst = cpu->create_stream();
    std::unique_ptr<hb::Stream> gst = gpu->create_stream();
};

/// y of Backend::gemv on both backends for the same bytes; `variant` goes to the cuda backend only.
void run_gemv_both(Pair& p, DType t, const std::vector<std::byte>& w, const std::vector<float>& x, std::uint32_t rows, std::uint32_t cols,
                   std::uint32_t n_vec, std::uint32_t variant, std::vector<float>& y_cpu, std::vector<float>& y_gpu) {
    y_cpu.assign(std::size_t{n_vec} * rows, 0.0f);
    y_gpu.assign(std::size_t{n_vec} * rows, 0.0f);
    {
        const auto wb = p.cpu->import_host_readonly(w);
        const auto xb = p.cpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
        const auto yb = p.cpu->import_host(wbytes(y_cpu.data(), y_cpu.size() * 4));
        p.cpu->gemv(*p.cst, {t, hb::TensorRef::of(*wb), hb::TensorRef::of(*xb), hb::TensorRef::of(*yb), rows, cols, n_vec, {}});
    }
    {
        const auto wb = p.gpu->import_host_readonly(w);
        const auto xb = p.gpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
        const auto yb = p.gpu->allocate(y_gpu.size() * 4, hb::Tier::Vram);
        p.gpu->gemv(*p.gst, {t, hb::TensorRef::of(*wb), hb::TensorRef::of(*xb), hb::TensorRef::of(*yb), rows, cols, n_vec, {variant}});
        p.gpu->download(*p.gst, hb::TensorRef::of(*yb), wbytes(y_gpu.data(), y_gpu.size() * 4));
        p.gst->wait();
    }
}

bool bitwise(const std::vector<float>& a, const std::vector<float>& b) {
    return a.size() == b.size() && std::memcmp(a.data(), b.data(), a.size() * 4) == 0;
}

void test_registry(Pair& p, Report& r) {
    const auto v = p.gpu->variants(hb::OpId::Gemv);
    const char* names[] = {"gemv_exact8", "gemv_warp_f32", "gemv_mma_f16x2", "gemm_tcgen05_f16", "gemm_tcgen05_bf16", "gemv_mma_m1", "gemv_mma_r",
                           "gemv_mma_i8x2"};
    r.expect(v.size() == 11, "MATMUL has eleven registered variants");
    for (std::size_t i = 0; i < v.size() && i < 8; ++i)
        r.expect(v[i].id == i + 1 && v[i].name == names[i] && v[i].op == hb::OpId::Gemv, std::format("variant id {} is {}", i + 1, names[i]));
    r.expect(code_of([&] { (void)p.gpu->variants(hb::OpId::RmsNorm); }) == static_cast<int>(ErrorCode::Unsupported), "variants(RMS_NORM) is Unsupported");
    r.expect(p.gpu->kind() == hb::kKindCuda && !p.gpu->lost(), "kind and lost()");
    r.expect(p.gpu->describe().find("cuda") != std::string::npos, "describe() names the backend");
}

void test_gemv_bitwise(Pair& p, Report& r) {
    struct Case {
        DType t;
        std::uint32_t n, k, m;
    };
    // the first shape is the reference's own (test_cpu_backend.cpp:257-284); the others are odd row counts and batch sizes
    const Case cases[] = {{DType::Q8_0, 40, 64, 3}, {DType::Q4_K, 37, 512, 1}, {DType::Q6_K, 13, 2560, 3}, {DType::Q4_0, 50, 1024, 17},
                          {DType::Q4_K, 130, 5120, 5}, {DType::F32, 40, 64, 3}};
    for (const Case& c : cases) {
        std::vector<std::byte> w;
        if (c.t == DType::F32) {
            const auto f = random_floats(std::size_t{c.n} * c.k, 9);
            w.assign(reinterpret_cast<const std::byte*>(f.data()), reinterpret_cast<const std::byte*>(f.data() + f.size()));
        } else {
            w = random_weights(c.t, c.n, c.k, 10 + c.n);
        }
        const auto x = random_floats(std::size_t{c.m} * c.k, 8);
        std::vector<float> yc, yg;
        run_gemv_both(p, c.t, w, x, c.n, c.k, c.m, 1 /*gemv_exact8*/, yc, yg);
        r.expect(bitwise(yc, yg), std::format("gemv_exact8 is bitwise the CPU backend (type {}, {}x{}, {} vectors)", static_cast<int>(c.t), c.n, c.k, c.m));
        if (c.t == DType::F32) continue;
        run_gemv_both(p, c.t, w, x, c.n, c.k, c.m, 0 /*default*/, yc, yg);
        float maxref = 0, maxerr = 0;
        for (std::size_t i = 0; i < yc.size(); ++i) {
            maxref = std::max(maxref, std::fabs(yc[i]));
            maxerr = std::max(maxerr, std::fabs(yc[i] - yg[i]));
        }
        r.expect(maxerr <= 1e-3f * maxref, std::format("default variant within 1e-3 of the CPU backend (type {}): {} vs {}", static_cast<int>(c.t), maxerr, maxref));
    }
}

/// The repacked-layout tensor-core variants through the adapter: repack once, KernelChoice{7} (fp16 family) and {9} (int8 family), rows of any batch size.
void test_gemv_repacked(Pair& p, Report& r) {
    struct Case {
        DType t;
        std::uint32_t n, k, m;
    };
    const Case cases[] = {{DType::Q6_K, 37, 2560, 1}, {DType::Q8_0, 130, 512, 5}, {DType::Q4_0, 50, 5120, 16}};
    for (const Case& c : cases) {
        const auto w = random_weights(c.t, c.n, c.k, 20 + c.n);
        const auto x = random_floats(std::size_t{c.m} * c.k, 21);
        std::vector<float> yc, yg;
        run_gemv_both(p, c.t, w, x, c.n, c.k, c.m, 1 /*gemv_exact8*/, yc, yg);  // yc: the CPU backend
        const auto raw = p.gpu->import_host_readonly(w);
        const auto packed = hb::cuda_backend_repack(*p.gpu, *p.gst, c.t, hb::TensorRef::of(*raw), c.n, c.k);
        const auto xb = p.gpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
        const auto yb = p.gpu->allocate(yg.size() * 4, hb::Tier::Vram);
        for (const std::uint32_t variant : {7u, 9u}) {
            p.gpu->gemv(*p.gst, {c.t, hb::TensorRef::of(*packed), hb::TensorRef::of(*xb), hb::TensorRef::of(*yb), c.n, c.k, c.m, {variant}});
            p.gpu->download(*p.gst, hb::TensorRef::of(*yb), wbytes(yg.data(), yg.size() * 4));
            p.gst->wait();
            float maxref = 0, maxerr = 0;
            for (std::size_t i = 0; i < yc.size(); ++i) {
                maxref = std::max(maxref, std::fabs(yc[i]));
                maxerr = std::max(maxerr, std::fabs(yc[i] - yg[i]));
            }
            r.expect(maxerr <= 1e-3f * maxref, std::format("variant {} over repacked rows within 1e-3 of the CPU backend (type {}): {} vs {}", variant, static_cast<int>(c.t), maxerr, maxref));
        }
        // a raw-sized operand must not pass as a repacked one where the layouts differ in size
        if (c.t == DType::Q6_K) {
            bool thrown = false;
            try {
                p.gpu->gemv(*p.gst, {c.t, hb::TensorRef::of(*raw), hb::TensorRef::of(*xb), hb::TensorRef::of(*yb), c.n, c.k, c.m, {7}});
            } catch (const halo::Error& e) {
                thrown = e.code() == halo::ErrorCode::Kernel;
            }
            r.expect(thrown, "raw Q6_K rows are too short for the repacked variant: Error(Kernel)");
        }
    }
    bool refused = false;
    try {
        const auto w = random_weights(DType::Q4_K, 16, 256, 5);
        const auto raw = p.gpu->import_host_readonly(w);
        (void)hb::cuda_backend_repack(*p.gpu, *p.gst, DType::Q4_K, hb::TensorRef::of(*raw), 16, 256);
    } catch (const halo::Error& e) {
        refused = e.code() == halo::ErrorCode::Unsupported;
    }
    r.expect(refused, "Q4_K has no repacked layout: Error(Unsupported)");
}

/// Appends the little-endian bytes of a trivially copyable value.
template <class T>
void put(std::vector<std::byte>& out, T v) {
    const auto* p = reinterpret_cast<const std::byte*>(&v);
    out.insert(out.end(), p, p + sizeof v);
}
void put_string(std::vector<std::byte>& out, std::string_view s) {
    put<std::uint64_t>(out, s.size());
    out.insert(out.end(), reinterpret_cast<const std::byte*>(s.data()), reinterpret_cast<const std::byte*>(s.data()) + s.size());
}

/// Weights loaded from a GGUF image through the adapter: the product over a loaded operand is bitwise the product over the same
/// bytes imported directly, for the whole matrix and for the shares of a tensor-parallel group.
void test_load_mat(Pair& p, Report& r) {
    struct Entry {
        const char* name;
        DType t;
        std::uint32_t n, k;
        std::vector<std::byte> w;
        std::uint64_t offset = 0;
    };
    std::vector<Entry> entries;
    entries.push_back({"blk.0.ffn_up.weight", DType::Q4_K, 45, 1024, {}});
    entries.push_back({"blk.0.ffn_down.weight", DType::Q6_K, 33, 1536, {}});
    entries.push_back({"output.weight", DType::Q4_0, 70, 512, {}});
    std::vector<std::byte> data;
    for (Entry& e : entries) {
        e.w = random_weights(e.t, e.n, e.k, 40 + e.n);
        data.resize((data.size() + 31) / 32 * 32);
        e.offset = data.size();
        data.insert(data.end(), e.w.begin(), e.w.end());
    }
    std::vector<std::byte> img;
    put<std::uint32_t>(img, 0x46554747u);
    put<std::uint32_t>(img, 3);
    put<std::uint64_t>(img, entries.size());
    put<std::uint64_t>(img, 1);
    put_string(img, "general.architecture");
    put<std::uint32_t>(img, 8);
    put_string(img, "qwen35");
    for (const Entry& e : entries) {
        put_string(img, e.name);
        put<std::uint32_t>(img, 2);
        put<std::uint64_t>(img, e.k);
        put<std::uint64_t>(img, e.n);
        put<std::uint32_t>(img, static_cast<std::uint32_t>(e.t));
        put<std::uint64_t>(img, e.offset);
    }
    img.resize((img.size() + 31) / 32 * 32);
    img.insert(img.end(), data.begin(), data.end());

    HaloGguf* file = nullptr;
    r.expect(halo_gguf_parse(img.data(), img.size(), &file) == 0 && file != nullptr, "the GGUF image parses");
    if (file == nullptr) return;
    const std::uint32_t m = 3;
    for (const Entry& e : entries) {
        const auto x = random_floats(std::size_t{m} * e.k, 50);
        std::vector<float> yc, yg;
        run_gemv_both(p, e.t, e.w, x, e.n, e.k, m, 1 /*gemv_exact8*/, yc, yg);
        const auto xb = p.gpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
        const auto run = [&](const hb::CudaMat& mat, const hb::TensorRef& xr, hb::KernelChoice kernel) {
            std::vector<float> y(std::size_t{m} * mat.rows);
            const auto yb = p.gpu->allocate(std::max<std::size_t>(y.size() * 4, 4), hb::Tier::Vram);
            p.gpu->gemv(*p.gst, {mat.type, mat.ref(), xr, hb::TensorRef::of(*yb), mat.rows, mat.cols, m, kernel});
            p.gpu->download(*p.gst, hb::TensorRef::of(*yb), wbytes(y.data(), y.size() * 4));
            p.gst->wait();
            return y;
        };
        const hb::CudaMat whole = hb::cuda_backend_load_mat(*p.gpu, *p.gst, file, e.name);
        r.expect(whole.rows == e.n && whole.cols == e.k && whole.type == e.t && whole.kernel.variant_id == 0, std::format("{}: extents of the loaded operand", e.name));
        r.expect(run(whole, hb::TensorRef::of(*xb), {1}) == yc, std::format("{}: exact-order product over the loaded operand is bitwise the CPU backend's", e.name));
        // column shares: whole rows, bitwise the rows of the CPU backend's product in the exact-order variant
        bool cols_ok = true;
        for (std::uint32_t rank = 0; rank < 3; ++rank) {
            const hb::CudaMat part = hb::cuda_backend_load_mat(*p.gpu, *p.gst, file, e.name, {hb::CudaSplit::Mode::Column, rank, 3, false});
            const auto y = run(part, hb::TensorRef::of(*xb), {1});
            for (std::uint32_t t = 0; t < m; ++t)
                for (std::uint32_t n = 0; n < part.rows; ++n) cols_ok = cols_ok && y[std::size_t{t} * part.rows + n] == yc[std::size_t{t} * e.n + part.row0 + n];
        }
        r.expect(cols_ok, std::format("{}: three column shares give the rows of the whole product bit for bit", e.name));
        // row shares (repacked where the type has the layout): partial products over each rank's K range add up to the whole
        std::vector<double> sum(yc.size(), 0.0);
        for (std::uint32_t rank = 0; rank < 2; ++rank) {
            const hb::CudaMat part = hb::cuda_backend_load_mat(*p.gpu, *p.gst, file, e.name, {hb::CudaSplit::Mode::Row, rank, 2, true});
            r.expect((part.kernel.variant_id == 9) == (e.t != DType::Q4_K), std::format("{}: row share {} repacked (int8 family: its K fits) iff the type has the layout", e.name, rank));
            const auto xr = hb::TensorRef::of(*xb).shifted(std::uint64_t{part.k0} * 4).with_stride(std::uint64_t{e.k} * 4);
            const auto y = run(part, xr, part.kernel);
            for (std::size_t i = 0; i < y.size(); ++i) sum[i] += y[i];
        }
        float maxref = 0, maxerr = 0;
        for (std::size_t i = 0; i < yc.size(); ++i) {
            maxref = std::max(maxref, std::fabs(yc[i]));
            maxerr = std::max(maxerr, std::fabs(yc[i] - static_cast<float>(sum[i])));
        }
        r.expect(maxerr <= 1e-3f * maxref, std::format("{}: two row shares add up to the CPU backend's product: {} vs {}", e.name, maxerr, maxref));
    }
    r.expect(code_of([&] { (void)hb::cuda_backend_load_mat(*p.gpu, *p.gst, file, "blk.7.missing.weight"); }) == static_cast<int>(halo::ErrorCode::Model),
             "a missing tensor: Error(Model)");
    halo_gguf_close(file);
}

/// The fused input norm through the adapter: GemvArgs::norm_w on the cuda backend against the CPU backend's own rms_norm followed by
/// its own gemv (the CPU backend refuses the fused form, src/backend/cpu_backend.cpp:341-342).
void test_fused_norm(Pair& p, Report& r) {
    const std::uint32_t N = 90, K = 2560;
    const auto w = random_weights(DType::Q4_K, N, K, 61);
    auto x = random_floats(K, 62);
    for (float& v : x) v *= 2.5f;
    auto nw = random_floats(K, 63);
    for (float& v : nw) v = 1.0f + 0.1f * v;
    // CPU: rms_norm into a scratch row, then gemv
    const auto cw = p.cpu->import_host_readonly(w);
    const auto cx = p.cpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
    const auto cn = p.cpu->import_host_readonly(cbytes(nw.data(), nw.size() * 4));
    const auto cxn = p.cpu->allocate(K * 4, hb::Tier::Host);
    const auto cy = p.cpu->allocate(N * 4, hb::Tier::Host);
    p.cpu->rms_norm(*p.cst, {hb::TensorRef::of(*cx), hb::TensorRef::of(*cn), hb::TensorRef::of(*cxn), 1, K, 1e-6f, {}});
    p.cpu->gemv(*p.cst, {DType::Q4_K, hb::TensorRef::of(*cw), hb::TensorRef::of(*cxn), hb::TensorRef::of(*cy), N, K, 1, {}});
    std::vector<float> yc(N), yg(N);
    p.cpu->download(*p.cst, hb::TensorRef::of(*cy), wbytes(yc.data(), yc.size() * 4));
    p.cst->wait();
    // cuda: one call
    const auto gw = p.gpu->import_host_readonly(w);
    const auto gx = p.gpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
    const auto gn = p.gpu->import_host_readonly(cbytes(nw.data(), nw.size() * 4));
    const auto gy = p.gpu->allocate(N * 4, hb::Tier::Vram);
    hb::GemvArgs a{DType::Q4_K, hb::TensorRef::of(*gw), hb::TensorRef::of(*gx), hb::TensorRef::of(*gy), N, K, 1, {}};
    a.norm_w = hb::TensorRef::of(*gn);
    a.norm_eps = 1e-6f;
    p.gpu->gemv(*p.gst, a);
    p.gpu->download(*p.gst, hb::TensorRef::of(*gy), wbytes(yg.data(), yg.size() * 4));
    p.gst->wait();
    float maxref = 0, maxerr = 0;
    for (std::size_t i = 0; i < yc.size(); ++i) {
        maxref = std::max(maxref, std::fabs(yc[i]));
        maxerr = std::max(maxerr, std::fabs(yc[i] - yg[i]));
    }
    // the default Q4_K kernel rounds x to 16 bits per super-block: 2e-4 of the largest output is that family's own bar
    r.expect(maxerr <= 2e-4f * maxref, std::format("fused input norm equals the CPU backend's rms_norm + gemv to rounding: {} vs {}", maxerr, maxref));
    a.n_vec = 1;
    a.kernel = {1};
    r.expect(code_of([&] { p.gpu->gemv(*p.gst, a); }) == static_cast<int>(halo::ErrorCode::Unsupported), "fused norm on a kernel without it: Error(Unsupported)");
}

void test_validation_parity(Pair& p, Report& r) {
    const std::uint32_t N = 8, K = 64, T = 2;
    const auto w = random_weights(DType::Q8_0, N, K, 3);
    const auto x = random_floats(T * K, 4);
    std::vector<float> y(T * N);
    // the same rejected call on both backends must raise the same error class (test_hip_backend.cpp:655-722)
    struct Built {
        std::unique_ptr<hb::Buffer> w, x, y, ro;
    };
    const auto build = [&](hb::Backend& be, bool device) {
        Built b;
        b.w = be.import_host_readonly(w);
        b.x = be.import_host_readonly(cbytes(x.data(), x.size() * 4));
        b.y = device ? be.allocate(y.size() * 4, hb::Tier::Vram) : be.import_host(wbytes(y.data(), y.size() * 4));
        b.ro = be.import_host_readonly(cbytes(y.data(), y.size() * 4));
        return b;
    };
    Built c = build(*p.cpu, false), g = build(*p.gpu, true);
    using Mut = std::function<void(hb::GemvArgs&, Built&)>;
    const std::pair<const char*, Mut> cases[] = {
        {"unknown variant id", [](hb::GemvArgs& a, Built&) { a.kernel.variant_id = 99; }},
        {"y overlaps x", [](hb::GemvArgs& a, Built&) { a.y = a.x; }},
        {"read-only output", [](hb::GemvArgs& a, Built& b) { a.y = hb::TensorRef::of(*b.ro); }},
        {"cols not whole blocks", [](hb::GemvArgs& a, Built&) { a.cols = 50; }},
        {"unknown weight type", [](hb::GemvArgs& a, Built&) { a.wtype = static_cast<DType>(5); }},
        {"row stride below row bytes", [](hb::GemvArgs& a, Built&) { a.w = a.w.with_stride(10); }},
        {"view too small", [](hb::GemvArgs& a, Built&) { a.y.bytes = 16; }},
        {"misaligned fp32 operand", [](hb::GemvArgs& a, Built&) { a.x = a.x.shifted(2); a.n_vec = 1; }},
        {"fused norm refused", [](hb::GemvArgs& a, Built&) { a.norm_w = a.x; }},
        {"gates epilogue next to a fused norm refused", [](hb::GemvArgs& a, Built&) { a.gates.n_v = 4; a.norm_w = a.x; }},
        {"empty y", [](hb::GemvArgs& a, Built&) { a.y = {}; }},
    };
    for (const auto& [name, mut] : cases) {
        hb::GemvArgs ac{DType::Q8_0, hb::TensorRef::of(*c.w), hb::TensorRef::of(*c.x), hb::TensorRef::of(*c.y), N, K, T, {}};
        hb::GemvArgs ag{DType::Q8_0, hb::TensorRef::of(*g.w), hb::TensorRef::of(*g.x), hb::TensorRef::of(*g.y), N, K, T, {}};
        mut(ac, c);
        mut(ag, g);
        const int ec = code_of([&] { p.cpu->gemv(*p.cst, ac); });
        const int eg = code_of([&] { p.gpu->gemv(*p.gst, ag); });
        r.expect(ec >= 0 && ec == eg, std::format("{}: cpu raises {}, cuda raises {}", name, ec, eg));
    }
    // foreign buffer / foreign stream
    hb::GemvArgs mixed{DType::Q8_0, hb::TensorRef::of(*g.w), hb::TensorRef::of(*c.x), hb::TensorRef::of(*g.y), N, K, T, {}};
    r.expect(code_of([&] { p.gpu->gemv(*p.gst, mixed); }) == static_cast<int>(ErrorCode::Kernel), "a buffer of another backend is Error(Kernel)");
    hb::GemvArgs ok{DType::Q8_0, hb::TensorRef::of(*g.w), hb::TensorRef::of(*g.x), hb::TensorRef::of(*g.y), N, K, T, {}};
    r.expect(code_of([&] { p.gpu->gemv(*p.cst, ok); }) == static_cast<int>(ErrorCode::Api), "a stream of another backend is Error(Api)");
    // empty calls are no-ops on both
    ok.n_vec = 0;
    r.expect(code_of([&] { p.gpu->gemv(*p.gst, ok); }) == -1, "n_vec == 0 is a no-op");
    // never a host fallback
    r.expect(code_of([&] { p.gpu->rms_norm(*p.gst, {}); }) == static_cast<int>(ErrorCode::Unsupported), "RMS_NORM is Unsupported, not emulated");
    std::vector<std::byte> host(64);
    r.expect(code_of([&] { (void)p.gpu->import_host(host); }) == static_cast<int>(ErrorCode::Unsupported), "import_host is Unsupported on a device backend");
    // run_op dispatches to the typed method
    hb::OpInvocation inv{hb::OpId::Gemv, hb::CopyArgs{}};
    r.expect(code_of([&] { p.gpu->run_op(*p.gst, inv); }) == static_cast<int>(ErrorCode::Api), "run_op with another op's args is Error(Api)");
    p.gst->wait();
}

void test_lm_head(Pair& p, Report& r) {
    const std::uint32_t V = 8192 + 900, E = 256, n = 3;  // across the CPU's 8192-row slab boundary
    const auto w = random_weights(DType::Q4_K, V, E, 28);
    auto x = random_floats(std::size_t{n} * E, 29);
    for (int pass = 0; pass < 2; ++pass) {
        if (pass == 1) x[1 * E] = std::nanf("");  // poisons batch row 1 only
        std::vector<std::byte> res_c(n * hb::kArgmaxResultBytes), res_g(n * hb::kArgmaxResultBytes);
        std::vector<float> log_c(std::size_t{n} * V), log_g(std::size_t{n} * V);
        std::vector<std::int32_t> ids_c(n), ids_g(n);
        {
            const auto wb = p.cpu->import_host_readonly(w);
            const auto xb = p.cpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
            const auto lb = p.cpu->import_host(wbytes(log_c.data(), log_c.size() * 4));
            const auto rb = p.cpu->import_host(res_c);
            const auto ib = p.cpu->import_host(wbytes(ids_c.data(), n * 4));
            hb::LmHeadArgs a{};
            a.gemv = {DType::Q4_K, hb::TensorRef::of(*wb), hb::TensorRef::of(*xb), hb::TensorRef::of(*lb), V, E, n, {}};
            a.result = hb::TensorRef::of(*rb);
            a.ids = hb::TensorRef::of(*ib);
            a.valid_rows = 9000;
            p.cpu->lm_head(*p.cst, a);
        }
        {
            const auto wb = p.gpu->import_host_readonly(w);
            const auto xb = p.gpu->import_host_readonly(cbytes(x.data(), x.size() * 4));
            const auto lb = p.gpu->allocate(log_g.size() * 4, hb::Tier::Vram);
            const auto rb = p.gpu->allocate(res_g.size(), hb::Tier::Vram);
            const auto ib = p.gpu->allocate(n * 4, hb::Tier::Vram);
            hb::LmHeadArgs a{};
            a.gemv = {DType::Q4_K, hb::TensorRef::of(*wb), hb::TensorRef::of(*xb), hb::TensorRef::of(*lb), V, E, n, {1}};
            a.result = hb::TensorRef::of(*rb);
            a.ids = hb::TensorRef::of(*ib);
            a.valid_rows = 9000;
            p.gpu->lm_head(*p.gst, a);
            p.gpu->download(*p.gst, hb::TensorRef::of(*lb), wbytes(log_g.data(), log_g.size() * 4));
            p.gpu->download(*p.gst, hb::TensorRef::of(*rb), res_g);
            p.gpu->download(*p.gst, hb::TensorRef::of(*ib), wbytes(ids_g.data(), n * 4));
            p.gst->wait();
        }
        r.expect(res_c == res_g, std::format("LM_HEAD result words equal the CPU backend's (pass {})", pass));
        r.expect(ids_c == ids_g, std::format("LM_HEAD dense ids equal the CPU backend's (pass {})", pass));
        bool same = true;  // bit for bit, except that a NaN only has to be a NaN (payload and sign bits are not part of the contract)
        for (std::size_t i = 0; i < log_c.size() && same; ++i)
            same = std::isnan(log_c[i]) ? std::isnan(log_g[i]) : std::memcmp(&log_c[i], &log_g[i], 4) == 0;
        r.expect(same, std::format("LM_HEAD logits are bitwise the CPU backend's (pass {})", pass));
        const auto dec = hb::decode_argmax(res_g);
        if (pass == 1) r.expect(dec[1].index == -1 && std::isnan(dec[1].value) && dec[0].index >= 0, "a NaN poisons only its own vector");
    }
}

void test_get_rows_and_memory(Pair& p, Report& r) {
    const std::uint32_t rows = 10, cols = 512;
    const auto w = random_weights(DType::Q6_K, rows, cols, 30);
    const std::vector<std::int32_t> ids{3, 0, 9, 3};
    std::vector<float> out_c(ids.size() * cols), out_g(ids.size() * cols);
    {
        const auto tb = p.cpu->import_host_readonly(w);
        const auto ib = p.cpu->import_host_readonly(cbytes(ids.data(), ids.size() * 4));
        const auto ob = p.cpu->import_host(wbytes(out_c.data(), out_c.size() * 4));
        p.cpu->get_rows(*p.cst, {DType::Q6_K, hb::TensorRef::of(*tb), hb::TensorRef::of(*ib), hb::TensorRef::of(*ob), rows, cols, 4, {}, {}});
    }
    const auto tb = p.gpu->import_host_readonly(w);
    const auto ib = p.gpu->import_host_readonly(cbytes(ids.data(), ids.size() * 4));
    const auto ob = p.gpu->allocate(out_g.size() * 4, hb::Tier::Vram);
    p.gpu->get_rows(*p.gst, {DType::Q6_K, hb::TensorRef::of(*tb), hb::TensorRef::of(*ib), hb::TensorRef::of(*ob), rows, cols, 4, {}, {}});
    p.gpu->download(*p.gst, hb::TensorRef::of(*ob), wbytes(out_g.data(), out_g.size() * 4));
    p.gst->wait();
    r.expect(bitwise(out_c, out_g), "GET_ROWS is bit-identical to tensor::dequantize_row");
    const std::vector<std::int32_t> bad{1, 10};
    const auto bb = p.gpu->import_host_readonly(cbytes(bad.data(), 8));
    p.gpu->get_rows(*p.gst, {DType::Q6_K, hb::TensorRef::of(*tb), hb::TensorRef::of(*bb), hb::TensorRef::of(*ob), rows, cols, 2, {}, {}});
    r.expect(code_of([&] { p.gst->wait(); }) == static_cast<int>(ErrorCode::Kernel), "an id outside the table raises Error(Kernel) at the wait");
    r.expect(code_of([&] { p.gst->wait(); }) == -1, "the stream is usable again after the data error");
    // allocate is zero-filled; upload / copy / download round trip
    const auto a = p.gpu->allocate(1024, hb::Tier::Vram);
    std::vector<std::byte> got(1024, std::byte{0x55});
    p.gpu->download(*p.gst, hb::TensorRef::of(*a), got);
    p.gst->wait();
    bool zero = true;
    for (auto b : got) zero = zero && b == std::byte{0};
    r.expect(zero, "allocate() zero-fills");
    std::vector<std::byte> src(512);
    for (std::size_t i = 0; i < src.size(); ++i) src[i] = static_cast<std::byte>(i & 0xFF);
    const auto b2 = p.gpu->allocate(512, hb::Tier::Vram);
    p.gpu->upload(*p.gst, hb::TensorRef{a.get(), 0, 512, 0}, src);
    p.gpu->copy(*p.gst, {hb::TensorRef{a.get(), 0, 512, 0}, hb::TensorRef::of(*b2), 512, {}});
    std::vector<std::byte> back(512);
    p.gpu->download(*p.gst, hb::TensorRef::of(*b2), back);
    p.gst->wait();
    r.expect(back == src, "upload -> copy -> download round trip");
    r.expect(code_of([&] { p.gpu->copy(*p.gst, {hb::TensorRef{a.get(), 0, 512, 0}, hb::TensorRef{a.get(), 256, 512, 0}, 512, {}}); }) ==
                 static_cast<int>(ErrorCode::Kernel),
             "COPY rejects overlapping ranges");
}

void test_plan(Pair& p, Report& r) {
    const std::uint32_t N = 64, K = 1024;
    const auto w = random_weights(DType::Q4_K, N, K, 40);
    const auto x = random_floats(K, 41);
    std::vector<float> yc, y_default, y_planned;
    run_gemv_both(p, DType::Q4_K, w, x, N, K, 1, 0, yc, y_default);
    const hb::CudaPlanEntry e{DType::Q4_K, N, K, 1, 16, 1 /*gemv_exact8*/};
    hb::cuda_backend_set_plan(*p.gpu, std::span<const hb::CudaPlanEntry>(&e, 1));
    run_gemv_both(p, DType::Q4_K, w, x, N, K, 1, 0, yc, y_planned);
    r.expect(bitwise(yc, y_planned), "an installed plan routes KernelChoice{} to the tuned variant");
    hb::cuda_backend_set_plan(*p.gpu, {});
    r.expect(code_of([&] { hb::cuda_backend_set_plan(*p.cpu, {}); }) == static_cast<int>(ErrorCode::Api), "set_plan on another backend is Error(Api)");
}

}  // namespace

extern "C" int halo_adapter_selftest(char* report, std::size_t len) {
    Report r;
    try {
        Pair p;
        test_registry(p, r);
        test_gemv_repacked(p, r);
        test_load_mat(p, r);
        test_fused_norm(p, r);
        test_gemv_bitwise(p, r);
        test_validation_parity(p, r);
        test_lm_head(p, r);
        test_get_rows_and_memory(p, r);
        test_plan(p, r);
    } catch (const std::exception& e) {
        r.expect(false, std::string("uncaught exception: ") + e.what());
    }
    r.text += std::format("{} checks passed, {} failed\n", r.passed, r.failed);
    if (report != nullptr && len != 0) std::snprintf(report, len, "%s", r.text.c_str());
    return r.failed;
}
