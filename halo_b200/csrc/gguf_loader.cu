// GGUF container index and the file -> device upload of one matmul operand (halo_cuda_gguf.h).
//
// The parser follows the published GGUF v2/v3 layout (little-endian): magic, version, tensor count, metadata count,
// the metadata pairs, the tensor infos, then the data section at the next multiple of general.alignment.  It keeps
// what the reference's parser checks (src/model/gguf.cpp:330-470): magic and version, limits on counts, string and
// array lengths and nesting, duplicate keys and names, 1..4 dimensions, element and byte counts without overflow,
// ne[0] a whole number of blocks, offsets aligned, ranges disjoint and inside the file.  Unlike the reference it
// stores no metadata values: a key is remembered with the position of its value and decoded on request, and arrays
// are only walked, so a header costs memory in proportion to its number of keys and tensors, not to its bytes.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <string>
#include <string_view>
#include <thread>
#include <unordered_map>
#include <vector>

#include "halo_cuda_gguf.h"
#include "internal.h"

using namespace halo_cuda;

namespace {

// Parser limits (GgufLimits, include/halo/model/gguf.h:107-118).
constexpr uint64_t kMaxKv = 1u << 16, kMaxTensors = 1u << 20, kMaxStringBytes = 16u << 20, kMaxArrayElems = 1u << 26;
constexpr int kMaxArrayDepth = 8;
constexpr uint64_t kMaxNameBytes = 63, kMaxAlignment = 1u << 20;

enum : uint32_t { kU8, kI8, kU16, kI16, kU32, kI32, kF32, kBool, kString, kArray, kU64, kI64, kF64, kTypeEnd };

// {elements per block, bytes per block} of every ggml tensor type id; {0, 0} marks an id ggml never assigned or
// has retired.  A tensor of a type this backend has no kernel for stays in the index (a real model file carries
// F16 / Q5_K / ... tensors next to the projections); only its upload is refused.
struct Geometry {
    uint32_t elems, bytes;
};
constexpr Geometry kGgmlTypes[] = {
    {1, 4},     {1, 2},     {32, 18},   {32, 20},   {0, 0},    {0, 0},     {32, 22},   {32, 24},  // F32 F16 Q4_0 Q4_1 - - Q5_0 Q5_1
    {32, 34},   {32, 36},   {256, 84},  {256, 110}, {256, 144}, {256, 176}, {256, 210}, {256, 292},  // Q8_0 Q8_1 Q2_K..Q6_K Q8_K
    {256, 66},  {256, 74},  {256, 98},  {256, 50},  {32, 18},  {256, 110}, {256, 82},  {256, 136},  // IQ2_XXS IQ2_XS IQ3_XXS IQ1_S IQ4_NL IQ3_S IQ2_S IQ4_XS
    {1, 1},     {1, 2},     {1, 4},     {1, 8},     {1, 8},    {256, 56},  {1, 2},  // I8 I16 I32 I64 F64 IQ1_M BF16
};

bool mul_ok(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_mul_overflow(a, b, out); }
bool add_ok(uint64_t a, uint64_t b, uint64_t* out) { return !__builtin_add_overflow(a, b, out); }

struct KvEntry {
    uint32_t type;
    uint64_t pos;  // of the value
};

struct Reader {
    const uint8_t* p;
    uint64_t size, pos = 0;
    const char* src;
    int status = 0;

    bool need(uint64_t n, const char* what) {
        if (status != 0) return false;
        if (n > size - pos) {
            status = fail(HALO_CUDA_E_MODEL, "%s: truncated at offset %llu reading %s (%llu bytes needed, %llu left)", src,
                          (unsigned long long)pos, what, (unsigned long long)n, (unsigned long long)(size - pos));
            return false;
        }
        return true;
    }
    template <class T>
    T scalar(const char* what) {
        T v{};
        if (need(sizeof(T), what)) {
            std::memcpy(&v, p + pos, sizeof(T));
            pos += sizeof(T);
        }
        return v;
    }
    std::string_view string(const char* what, uint64_t cap) {
        const uint64_t len = scalar<uint64_t>(what);
        if (status != 0) return {};
        if (len > cap) {
            status = fail(HALO_CUDA_E_MODEL, "%s: %s length %llu at offset %llu exceeds limit %llu", src, what, (unsigned long long)len,
                          (unsigned long long)(pos - 8), (unsigned long long)cap);
            return {};
        }
        if (!need(len, what)) return {};
        std::string_view s(reinterpret_cast<const char*>(p + pos), len);
        pos += len;
        return s;
    }
    /// A count of items of at least `min_bytes` each: bounded by `cap` and by what is left of the file.
    uint64_t count(const char* what, uint64_t cap, uint64_t min_bytes) {
        const uint64_t n = scalar<uint64_t>(what);
        if (status != 0) return 0;
        if (n > cap) {
            status = fail(HALO_CUDA_E_MODEL, "%s: %s count %llu exceeds limit %llu", src, what, (unsigned long long)n, (unsigned long long)cap);
            return 0;
        }
        if (min_bytes != 0 && n > (size - pos) / min_bytes) {
            status = fail(HALO_CUDA_E_MODEL, "%s: %s count %llu cannot fit in the %llu remaining bytes", src, what, (unsigned long long)n,
                          (unsigned long long)(size - pos));
            return 0;
        }
        return n;
    }
};

uint32_t scalar_bytes(uint32_t type) {
    switch (type) {
        case kU8: case kI8: case kBool: return 1;
        case kU16: case kI16: return 2;
        case kU32: case kI32: case kF32: return 4;
        case kU64: case kI64: case kF64: return 8;
        default: return 0;
    }
}

/// Walks over one metadata value without storing it.
void skip_value(Reader& r, uint32_t type, int depth) {
    if (r.status != 0) return;
    if (type >= kTypeEnd) {
        r.status = fail(HALO_CUDA_E_MODEL, "%s: invalid GGUF value type %u at offset %llu", r.src, type, (unsigned long long)r.pos);
        return;
    }
    if (const uint32_t n = scalar_bytes(type)) {
        if (!r.need(n, "value")) return;
        if (type == kBool && r.p[r.pos] > 1) {
            r.status = fail(HALO_CUDA_E_MODEL, "%s: invalid bool value %u at offset %llu", r.src, r.p[r.pos], (unsigned long long)r.pos);
            return;
        }
        r.pos += n;
        return;
    }
    if (type == kString) {
        r.string("string value", kMaxStringBytes);
        return;
    }
    if (depth >= kMaxArrayDepth) {
        r.status = fail(HALO_CUDA_E_MODEL, "%s: array nesting deeper than %d at offset %llu", r.src, kMaxArrayDepth, (unsigned long long)r.pos);
        return;
    }
    const uint32_t elem = r.scalar<uint32_t>("array element type");
    if (r.status == 0 && elem >= kTypeEnd) {
        r.status = fail(HALO_CUDA_E_MODEL, "%s: invalid GGUF value type %u for array elements at offset %llu", r.src, elem,
                        (unsigned long long)(r.pos - 4));
        return;
    }
    const uint32_t eb = scalar_bytes(elem);
    const uint64_t n = r.count("array element", kMaxArrayElems, eb != 0 ? eb : (elem == kString ? 8 : 12));
    if (r.status != 0) return;
    if (eb != 0 && elem != kBool) {
        if (r.need(n * eb, "array")) r.pos += n * eb;
        return;
    }
    for (uint64_t i = 0; i < n && r.status == 0; ++i) skip_value(r, elem, depth + 1);
}

}  // namespace

struct HaloGguf {
    std::string source;
    const uint8_t* bytes = nullptr;
    uint64_t size = 0;
    void* mapping = nullptr;  // non-null when this object owns an mmap of `size` bytes
    HaloGgufInfo info{};
    std::vector<HaloGgufTensor> tensors;
    std::unordered_map<std::string, uint64_t> tensor_index;
    std::unordered_map<std::string, KvEntry> kv;
};

namespace {

int parse_all(HaloGguf& g) {
    Reader r{g.bytes, g.size, 0, g.source.c_str()};
    const char* src = r.src;
    const uint32_t magic = r.scalar<uint32_t>("magic");
    if (r.status != 0) return r.status;
    if (magic != 0x46554747u) return fail(HALO_CUDA_E_MODEL, "%s: not a GGUF file (bad magic)", src);
    const uint32_t version = r.scalar<uint32_t>("version");
    if (r.status != 0) return r.status;
    if (version != 2 && version != 3) {
        if (version == 1) return fail(HALO_CUDA_E_UNSUPPORTED, "%s: GGUF v1 is not supported", src);
        const uint32_t swapped = __builtin_bswap32(version);
        if (swapped == 2 || swapped == 3) return fail(HALO_CUDA_E_UNSUPPORTED, "%s: big-endian GGUF is not supported", src);
        return fail(HALO_CUDA_E_MODEL, "%s: unknown GGUF version %u", src, version);
    }
    // a tensor info is at least 8 (name length) + 4 (dims) + 4 (type) + 8 (offset) bytes, a pair 8 + 4 + 1
    const uint64_t n_tensors = r.count("tensor", kMaxTensors, 0);
    const uint64_t n_kv = r.count("metadata", kMaxKv, 13);
    if (r.status != 0) return r.status;

    g.kv.reserve(n_kv);
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string_view key = r.string("metadata key", kMaxStringBytes);
        const uint32_t type = r.scalar<uint32_t>("value type");
        if (r.status != 0) return r.status;
        const uint64_t at = r.pos;
        skip_value(r, type, 0);
        if (r.status != 0) return r.status;
        if (!g.kv.emplace(std::string(key), KvEntry{type, at}).second)
            return fail(HALO_CUDA_E_MODEL, "%s: duplicate metadata key '%.*s'", src, (int)std::min<size_t>(key.size(), 200), key.data());
    }

    uint64_t alignment = 32;
    if (auto it = g.kv.find("general.alignment"); it != g.kv.end()) {
        if (it->second.type != kU32) return fail(HALO_CUDA_E_MODEL, "%s: general.alignment has value type %u, expected UINT32", src, it->second.type);
        uint32_t a = 0;
        std::memcpy(&a, g.bytes + it->second.pos, 4);
        if (a == 0 || (a & (a - 1)) != 0 || a > kMaxAlignment) return fail(HALO_CUDA_E_MODEL, "%s: invalid general.alignment %u", src, a);
        alignment = a;
    }

    if (n_tensors > (r.size - r.pos) / 24)
        return fail(HALO_CUDA_E_MODEL, "%s: tensor count %llu cannot fit in the %llu remaining bytes", src, (unsigned long long)n_tensors,
                    (unsigned long long)(r.size - r.pos));
    g.tensors.reserve(n_tensors);
    g.tensor_index.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        HaloGgufTensor t{};
        const std::string_view name = r.string("tensor name", kMaxNameBytes);
        if (r.status != 0) return r.status;
        std::memcpy(t.name, name.data(), name.size());
        t.n_dims = r.scalar<uint32_t>("tensor dims");
        if (r.status != 0) return r.status;
        if (t.n_dims < 1 || t.n_dims > 4) return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' has %u dims (expected 1..4)", src, t.name, t.n_dims);
        uint64_t n_el = 1;
        for (int d = 0; d < 4; ++d) t.ne[d] = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            const uint64_t e = r.scalar<uint64_t>("tensor extent");
            if (r.status != 0) return r.status;
            if (e > uint64_t(INT64_MAX) || !mul_ok(n_el, e, &n_el) || n_el > uint64_t(INT64_MAX))
                return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' element count overflows", src, t.name);
            t.ne[d] = int64_t(e);
        }
        t.n_elements = n_el;
        t.type = r.scalar<uint32_t>("tensor type");
        t.offset = r.scalar<uint64_t>("tensor offset");
        if (r.status != 0) return r.status;
        const Geometry geo = t.type < sizeof kGgmlTypes / sizeof kGgmlTypes[0] ? kGgmlTypes[t.type] : Geometry{0, 0};
        if (geo.elems == 0) return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' has invalid type id %u", src, t.name, t.type);
        if (uint64_t(t.ne[0]) % geo.elems != 0)
            return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' ne[0]=%lld is not a multiple of the block size %u", src, t.name, (long long)t.ne[0], geo.elems);
        if (!mul_ok(n_el / geo.elems, geo.bytes, &t.n_bytes)) return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' byte size overflows", src, t.name);
        if (t.offset % alignment != 0)
            return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' offset %llu is not a multiple of the alignment %llu", src, t.name,
                        (unsigned long long)t.offset, (unsigned long long)alignment);
        uint64_t end = 0;
        if (!add_ok(t.offset, t.n_bytes, &end)) return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' data range overflows", src, t.name);
        TypeInfo ti;
        t.supported = type_info(t.type, &ti) ? 1 : 0;
        if (!g.tensor_index.emplace(t.name, i).second) return fail(HALO_CUDA_E_MODEL, "%s: duplicate tensor name '%s'", src, t.name);
        g.tensors.push_back(t);
    }

    g.info.version = version;
    g.info.alignment = uint32_t(alignment);
    g.info.n_kv = n_kv;
    g.info.n_tensors = n_tensors;
    g.info.header_size = r.pos;
    g.info.file_size = g.size;
    uint64_t padded = 0;
    if (!add_ok(r.pos, alignment - 1, &padded)) return fail(HALO_CUDA_E_MODEL, "%s: offset overflow", src);
    g.info.data_offset = padded / alignment * alignment;

    // data ranges: disjoint, and inside the file
    std::vector<uint64_t> order(g.tensors.size());
    for (uint64_t k = 0; k < order.size(); ++k) order[k] = k;
    std::sort(order.begin(), order.end(), [&](uint64_t a, uint64_t b) { return g.tensors[a].offset < g.tensors[b].offset; });
    for (uint64_t k = 1; k < order.size(); ++k) {
        const HaloGgufTensor &prev = g.tensors[order[k - 1]], &cur = g.tensors[order[k]];
        if (prev.offset + prev.n_bytes > cur.offset)
            return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' [%llu, %llu) overlaps '%s' starting at %llu", src, prev.name, (unsigned long long)prev.offset,
                        (unsigned long long)(prev.offset + prev.n_bytes), cur.name, (unsigned long long)cur.offset);
    }
    if (!g.tensors.empty() && g.info.data_offset > g.size)
        return fail(HALO_CUDA_E_MODEL, "%s: data section starts at %llu, past end of file (%llu bytes)", src, (unsigned long long)g.info.data_offset,
                    (unsigned long long)g.size);
    for (const HaloGgufTensor& t : g.tensors) {
        uint64_t end = 0;
        if (!add_ok(g.info.data_offset, t.offset + t.n_bytes, &end) || end > g.size)
            return fail(HALO_CUDA_E_MODEL, "%s: tensor '%s' data [%llu, %llu) extends past end of file (%llu bytes)", src, t.name,
                        (unsigned long long)(g.info.data_offset + t.offset), (unsigned long long)(g.info.data_offset + t.offset + t.n_bytes),
                        (unsigned long long)g.size);
    }
    return 0;
}

void destroy(HaloGguf* g) {
    if (g == nullptr) return;
    if (g->mapping != nullptr) munmap(g->mapping, g->size);
    delete g;
}

const KvEntry* find_kv(const HaloGguf* g, const char* key) {
    auto it = g->kv.find(key);
    return it == g->kv.end() ? nullptr : &it->second;
}

/// Reads an integer-typed value widened to 64 bits; `negative` tells whether a signed value was below zero.
bool read_integer(const HaloGguf* g, const KvEntry& e, uint64_t* mag, int64_t* as_signed, bool* is_signed) {
    const uint8_t* p = g->bytes + e.pos;
    *is_signed = false;
    switch (e.type) {
        case kU8: *mag = p[0]; return true;
        case kU16: { uint16_t v; std::memcpy(&v, p, 2); *mag = v; return true; }
        case kU32: { uint32_t v; std::memcpy(&v, p, 4); *mag = v; return true; }
        case kU64: { uint64_t v; std::memcpy(&v, p, 8); *mag = v; return true; }
        case kI8: { int8_t v; std::memcpy(&v, p, 1); *as_signed = v; *is_signed = true; return true; }
        case kI16: { int16_t v; std::memcpy(&v, p, 2); *as_signed = v; *is_signed = true; return true; }
        case kI32: { int32_t v; std::memcpy(&v, p, 4); *as_signed = v; *is_signed = true; return true; }
        case kI64: { int64_t v; std::memcpy(&v, p, 8); *as_signed = v; *is_signed = true; return true; }
        default: return false;
    }
}

}  // namespace

extern "C" {

int halo_gguf_parse(const void* bytes, uint64_t size, HaloGguf** out) {
    if (out == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    *out = nullptr;
    if (bytes == nullptr && size != 0) return fail(HALO_CUDA_E_API, "null image");
    HaloGguf* g = new HaloGguf;
    g->source = "<memory>";
    g->bytes = static_cast<const uint8_t*>(bytes);
    g->size = size;
    if (int rc = parse_all(*g)) {
        destroy(g);
        return rc;
    }
    *out = g;
    return 0;
}

int halo_gguf_open(const char* path, HaloGguf** out) {
    if (out == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    *out = nullptr;
    if (path == nullptr) return fail(HALO_CUDA_E_API, "null path");
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(HALO_CUDA_E_IO, "%s: cannot open: %s", path, std::strerror(errno));
    struct stat st {};
    if (fstat(fd, &st) != 0 || !S_ISREG(st.st_mode)) {
        const int e = errno;
        close(fd);
        return fail(HALO_CUDA_E_IO, "%s: not a readable regular file: %s", path, std::strerror(e));
    }
    HaloGguf* g = new HaloGguf;
    g->source = path;
    g->size = uint64_t(st.st_size);
    if (g->size != 0) {
        void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, fd, 0);
        if (m == MAP_FAILED) {
            const int e = errno;
            close(fd);
            delete g;
            return fail(HALO_CUDA_E_IO, "%s: cannot map %llu bytes: %s", path, (unsigned long long)st.st_size, std::strerror(e));
        }
        g->mapping = m;
        g->bytes = static_cast<const uint8_t*>(m);
    }
    close(fd);
    if (int rc = parse_all(*g)) {
        destroy(g);
        return rc;
    }
    *out = g;
    return 0;
}

int halo_gguf_close(HaloGguf* g) {
    destroy(g);
    return 0;
}

int halo_gguf_info(const HaloGguf* g, HaloGgufInfo* out) {
    if (g == nullptr || out == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *out = g->info;
    return 0;
}

int halo_gguf_kv_u64(const HaloGguf* g, const char* key, uint64_t* value, int* found) {
    if (g == nullptr || key == nullptr || value == nullptr || found == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *found = 0;
    const KvEntry* e = find_kv(g, key);
    if (e == nullptr) return 0;
    uint64_t mag = 0;
    int64_t sv = 0;
    bool is_signed = false;
    if (!read_integer(g, *e, &mag, &sv, &is_signed)) return fail(HALO_CUDA_E_MODEL, "%s: key %s has value type %u, expected an integer", g->source.c_str(), key, e->type);
    if (is_signed) {
        if (sv < 0) return fail(HALO_CUDA_E_MODEL, "%s: key %s = %lld must be non-negative", g->source.c_str(), key, (long long)sv);
        mag = uint64_t(sv);
    }
    *value = mag;
    *found = 1;
    return 0;
}

int halo_gguf_kv_i64(const HaloGguf* g, const char* key, int64_t* value, int* found) {
    if (g == nullptr || key == nullptr || value == nullptr || found == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *found = 0;
    const KvEntry* e = find_kv(g, key);
    if (e == nullptr) return 0;
    uint64_t mag = 0;
    int64_t sv = 0;
    bool is_signed = false;
    if (!read_integer(g, *e, &mag, &sv, &is_signed)) return fail(HALO_CUDA_E_MODEL, "%s: key %s has value type %u, expected an integer", g->source.c_str(), key, e->type);
    if (!is_signed) {
        if (mag > uint64_t(INT64_MAX)) return fail(HALO_CUDA_E_MODEL, "%s: key %s = %llu overflows int64", g->source.c_str(), key, (unsigned long long)mag);
        sv = int64_t(mag);
    }
    *value = sv;
    *found = 1;
    return 0;
}

int halo_gguf_kv_f64(const HaloGguf* g, const char* key, double* value, int* found) {
    if (g == nullptr || key == nullptr || value == nullptr || found == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *found = 0;
    const KvEntry* e = find_kv(g, key);
    if (e == nullptr) return 0;
    if (e->type == kF32) {
        float v;
        std::memcpy(&v, g->bytes + e->pos, 4);
        *value = v;
    } else if (e->type == kF64) {
        std::memcpy(value, g->bytes + e->pos, 8);
    } else {
        return fail(HALO_CUDA_E_MODEL, "%s: key %s has value type %u, expected a float", g->source.c_str(), key, e->type);
    }
    *found = 1;
    return 0;
}

int halo_gguf_kv_string(const HaloGguf* g, const char* key, char* buf, uint64_t cap, uint64_t* len, int* found) {
    if (g == nullptr || key == nullptr || found == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    *found = 0;
    const KvEntry* e = find_kv(g, key);
    if (e == nullptr) return 0;
    if (e->type != kString) return fail(HALO_CUDA_E_MODEL, "%s: key %s has value type %u, expected STRING", g->source.c_str(), key, e->type);
    uint64_t n = 0;
    std::memcpy(&n, g->bytes + e->pos, 8);  // validated while parsing
    if (len != nullptr) *len = n;
    if (buf != nullptr && cap != 0) {
        const uint64_t c = std::min<uint64_t>(n, cap - 1);
        std::memcpy(buf, g->bytes + e->pos + 8, c);
        buf[c] = 0;
    }
    *found = 1;
    return 0;
}

int halo_gguf_tensor(const HaloGguf* g, uint64_t index, HaloGgufTensor* out) {
    if (g == nullptr || out == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    if (index >= g->tensors.size()) return fail(HALO_CUDA_E_API, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    *out = g->tensors[index];
    return 0;
}

int halo_gguf_find(const HaloGguf* g, const char* name, uint64_t* index, int* found) {
    if (g == nullptr || name == nullptr || index == nullptr || found == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    auto it = g->tensor_index.find(name);
    *found = it != g->tensor_index.end();
    if (*found) *index = it->second;
    return 0;
}

int halo_gguf_tensor_data(const HaloGguf* g, uint64_t index, const void** data, uint64_t* bytes) {
    if (g == nullptr || data == nullptr || bytes == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    if (index >= g->tensors.size()) return fail(HALO_CUDA_E_API, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    const HaloGgufTensor& t = g->tensors[index];
    *data = g->bytes + g->info.data_offset + t.offset;
    *bytes = t.n_bytes;
    return 0;
}

}  // extern "C"

// ---- file -> device ---------------------------------------------------------------------------------------------------

namespace {

/// [begin, end) of part `i` when n items are dealt to `parts` contiguous parts, the first n % parts one longer.
void even_part(uint64_t n, uint32_t parts, uint32_t i, uint64_t* begin, uint64_t* end) {
    const uint64_t base = n / parts, extra = n % parts;
    *begin = i * base + std::min<uint64_t>(i, extra);
    *end = *begin + base + (i < extra ? 1 : 0);
}

struct Share {
    uint64_t max_cols;  // the largest local K over the ranks (decides the variant of a repacked tensor alike on every rank)
    uint64_t row0, rows, k0, cols;
    uint64_t byte0, row_bytes;  // of the share inside a source row
    uint64_t src_row_bytes;
    bool repack;
};

int plan_share(uint32_t wtype, uint64_t rows, uint64_t cols, const HaloCudaUpload* how, Share* s) {
    TypeInfo ti;
    if (!type_info(wtype, &ti)) return fail(HALO_CUDA_E_UNSUPPORTED, "upload: ggml type %u has no matmul kernel in this backend", wtype);
    if (cols % ti.block_elems != 0) return fail(HALO_CUDA_E_MODEL, "upload: %llu columns is not a whole number of %u-element blocks", (unsigned long long)cols, ti.block_elems);
    if (rows > UINT32_MAX || cols > UINT32_MAX) return fail(HALO_CUDA_E_UNSUPPORTED, "upload: %llu x %llu exceeds 32-bit extents", (unsigned long long)rows, (unsigned long long)cols);
    const uint32_t split = how != nullptr ? how->split : HALO_CUDA_SPLIT_NONE;
    const uint32_t world = how != nullptr && how->world > 1 ? how->world : 1;
    const uint32_t rank = how != nullptr && world > 1 ? how->rank : 0;
    if (split > HALO_CUDA_SPLIT_ROW) return fail(HALO_CUDA_E_API, "upload: unknown split mode %u", split);
    if (rank >= world) return fail(HALO_CUDA_E_API, "upload: rank %u of %u", rank, world);
    *s = Share{cols, 0, rows, 0, cols, 0, 0, cols / ti.block_elems * ti.block_bytes, false};
    if (split == HALO_CUDA_SPLIT_COLUMN && world > 1) {
        uint64_t b, e;
        even_part(rows, world, rank, &b, &e);
        s->row0 = b;
        s->rows = e - b;
    } else if (split == HALO_CUDA_SPLIT_ROW && world > 1) {
        uint64_t b, e;
        even_part(cols / ti.block_elems, world, rank, &b, &e);
        s->k0 = b * ti.block_elems;
        s->cols = (e - b) * ti.block_elems;
        s->byte0 = b * ti.block_bytes;
        even_part(cols / ti.block_elems, world, 0, &b, &e);  // rank 0 holds a largest share
        s->max_cols = (e - b) * ti.block_elems;
    }
    s->row_bytes = s->cols / ti.block_elems * ti.block_bytes;
    // The repacked layout selects the kernel variant, and with it whether a row split reduces through the peer epilogue or a
    // collective: every rank of a row split must decide alike, so the decision looks at EVERY rank's share, not at this one.
    bool groups = s->cols != 0 && s->cols % 256 == 0;
    if (split == HALO_CUDA_SPLIT_ROW && world > 1) {
        for (uint32_t r = 0; r < world && groups; ++r) {
            uint64_t b, e;
            even_part(cols / ti.block_elems, world, r, &b, &e);
            groups = e > b && (e - b) * ti.block_elems % 256 == 0;
        }
    }
    s->repack = how != nullptr && how->repack != 0 && s->rows != 0 && groups && repacked_row_bytes(wtype, s->cols) != 0;
    return 0;
}

void fill_matrix(uint32_t wtype, const Share& s, HaloCudaMatrix* out) {
    std::memset(out, 0, sizeof *out);
    out->wtype = wtype;
    out->rows = uint32_t(s.rows);
    out->cols = uint32_t(s.cols);
    out->row0 = uint32_t(s.row0);
    out->k0 = uint32_t(s.k0);
    out->variant_id = s.repack ? repacked_variant(wtype, uint32_t(s.max_cols)) : HALO_CUDA_GEMV_DEFAULT;
    out->w_stride = s.repack ? repacked_row_bytes(wtype, s.cols) : s.row_bytes;
    out->bytes = s.rows * out->w_stride;
}

constexpr uint32_t kMaxLanes = 8;  // HaloCudaCtx::staging_done holds two events per lane

/// The context's two pinned staging buffers of at least `bytes` each (grown on demand) and the events of their lanes.
int staging(HaloCudaCtx* ctx, uint64_t bytes) {
    for (int i = 0; i < 2; ++i)
        for (uint32_t l = 0; l < kMaxLanes; ++l)
            if (ctx->staging_done[i][l] == nullptr) HC_CUDA(cudaEventCreateWithFlags(&ctx->staging_done[i][l], cudaEventDisableTiming));
    // The last copies of an earlier upload may still be reading the buffers, cut into lanes of another size: let them drain
    // (a fraction of a millisecond) before this upload's lanes write there.
    for (int i = 0; i < 2; ++i)
        for (uint32_t l = 0; l < kMaxLanes; ++l) HC_CUDA(cudaEventSynchronize(ctx->staging_done[i][l]));
    if (ctx->staging_bytes >= bytes) return 0;
    for (int i = 0; i < 2; ++i) {
        if (ctx->staging[i] != nullptr) {
            HC_CUDA(cudaFreeHost(ctx->staging[i]));
            ctx->staging[i] = nullptr;
        }
    }
    ctx->staging_bytes = 0;
    for (int i = 0; i < 2; ++i) {
        const cudaError_t e = cudaHostAlloc(&ctx->staging[i], bytes, cudaHostAllocDefault);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(HALO_CUDA_E_MEMORY, "cannot pin %llu host bytes for staging: %s", (unsigned long long)bytes, cudaGetErrorString(e));
        }
    }
    ctx->staging_bytes = bytes;
    return 0;
}

/// One lane of the upload: rows [row_begin, row_end) of the share go, `lane_rows` at a time, from the mapping into this lane's
/// part of the two staging buffers in turn and from there to the device.  Lanes run on host threads of their own -- one core's
/// memcpy out of the page cache carries a fraction of what the link to the device does -- and share nothing but the stream.
struct Lane {
    HaloCudaCtx* ctx;
    cudaStream_t stream;
    uint32_t index;
    const uint8_t* src;  // first byte of the share's row 0
    uint8_t* dst;        // device, dense rows
    uint64_t row_begin, row_end, lane_rows, row_bytes, src_row_bytes;
    cudaError_t status = cudaSuccess;

    void run() {
        status = cudaSetDevice(ctx->device);
        uint32_t turn = 0;
        for (uint64_t r0 = row_begin; r0 < row_end && status == cudaSuccess; r0 += lane_rows, turn ^= 1) {
            const uint64_t n = std::min(lane_rows, row_end - r0);
            uint8_t* stage = static_cast<uint8_t*>(ctx->staging[turn]) + uint64_t{index} * lane_rows * row_bytes;
            // the copy that last read this part of the buffer must have drained before the host overwrites it
            status = cudaEventSynchronize(ctx->staging_done[turn][index]);
            if (status != cudaSuccess) break;
            if (row_bytes == src_row_bytes) {
                std::memcpy(stage, src + r0 * src_row_bytes, n * row_bytes);
            } else {
                for (uint64_t r = 0; r < n; ++r) std::memcpy(stage + r * row_bytes, src + (r0 + r) * src_row_bytes, row_bytes);
            }
            status = cudaMemcpyAsync(dst + r0 * row_bytes, stage, n * row_bytes, cudaMemcpyHostToDevice, stream);
            if (status == cudaSuccess) status = cudaEventRecord(ctx->staging_done[turn][index], stream);
        }
    }
};

}  // namespace

extern "C" {

int halo_cuda_matrix_share(uint32_t wtype, uint32_t rows, uint32_t cols, const HaloCudaUpload* how, HaloCudaMatrix* out) {
    if (out == nullptr) return fail(HALO_CUDA_E_API, "null out pointer");
    Share s;
    if (int rc = plan_share(wtype, rows, cols, how, &s)) return rc;
    fill_matrix(wtype, s, out);
    return 0;
}

int halo_cuda_upload_matrix(HaloCudaCtx* ctx, const HaloGguf* g, uint64_t index, const HaloCudaUpload* how, HaloCudaStream stream,
                            HaloCudaMatrix* out) {
    if (out == nullptr || g == nullptr) return fail(HALO_CUDA_E_API, "null argument");
    std::memset(out, 0, sizeof *out);
    if (int rc = enter(ctx)) return rc;
    if (index >= g->tensors.size()) return fail(HALO_CUDA_E_API, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    const HaloGgufTensor& t = g->tensors[index];
    if (t.n_dims > 2 && (t.ne[2] != 1 || t.ne[3] != 1)) return fail(HALO_CUDA_E_MODEL, "tensor '%s' is not a matrix (%u dims)", t.name, t.n_dims);
    Share s;
    if (int rc = plan_share(t.type, uint64_t(t.ne[1]), uint64_t(t.ne[0]), how, &s)) return rc;
    if (t.n_bytes != uint64_t(t.ne[1]) * s.src_row_bytes) return fail(HALO_CUDA_E_MODEL, "tensor '%s': %llu bytes are not dense rows", t.name, (unsigned long long)t.n_bytes);
    fill_matrix(t.type, s, out);
    const uint64_t raw_bytes = s.rows * s.row_bytes;
    if (raw_bytes == 0) return 0;  // an empty share: nothing to hold

    const cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const uint64_t want = how != nullptr && how->staging_bytes != 0 ? how->staging_bytes : (32ull << 20);
    // one lane per 8 MiB of the share, each with room for whole rows (at least one) in both staging buffers
    const uint32_t lanes = uint32_t(std::min<uint64_t>({kMaxLanes, std::max(1u, std::thread::hardware_concurrency()), std::max<uint64_t>(1, raw_bytes >> 23), s.rows}));
    const uint64_t lane_rows = std::min(std::max<uint64_t>(1, want / lanes / s.row_bytes), (s.rows + lanes - 1) / lanes);
    if (int rc = staging(ctx, lanes * lane_rows * s.row_bytes)) return rc;

    void* raw = nullptr;
    if (int rc = halo_cuda_malloc(ctx, raw_bytes, 0, &raw)) return rc;
    const uint8_t* src = g->bytes + g->info.data_offset + t.offset + s.row0 * s.src_row_bytes + s.byte0;
    std::vector<Lane> work(lanes);
    for (uint32_t l = 0; l < lanes; ++l) {
        uint64_t b, e;
        even_part(s.rows, lanes, l, &b, &e);
        work[l] = Lane{ctx, cs, l, src, static_cast<uint8_t*>(raw), b, e, lane_rows, s.row_bytes, s.src_row_bytes};
    }
    {
        std::vector<std::thread> helpers;
        helpers.reserve(lanes - 1);
        for (uint32_t l = 1; l < lanes; ++l) helpers.emplace_back(&Lane::run, &work[l]);
        work[0].run();
        for (std::thread& th : helpers) th.join();
    }
    int rc = 0;
    for (const Lane& l : work)
        if (l.status != cudaSuccess && rc == 0) rc = fail(HALO_CUDA_E_BACKEND, "upload of '%s': %s", t.name, cudaGetErrorString(l.status));
    void* packed = nullptr;
    if (rc == 0 && s.repack) {
        rc = halo_cuda_malloc(ctx, out->bytes, 0, &packed);
        if (rc == 0) rc = launch_repack(t.type, raw, s.row_bytes, packed, out->w_stride, out->rows, out->cols, cs);
        // the raw copy is only the repack's source: wait for the kernel, then give the memory back
        if (rc == 0) {
            const cudaError_t e = cudaStreamSynchronize(cs);
            if (e != cudaSuccess) rc = fail(HALO_CUDA_E_BACKEND, "repack of '%s': %s", t.name, cudaGetErrorString(e));
        }
    }
    if (rc != 0) {
        cudaStreamSynchronize(cs);
        halo_cuda_free(ctx, raw);
        if (packed != nullptr) halo_cuda_free(ctx, packed);
        std::memset(out, 0, sizeof *out);
        return rc;
    }
    if (s.repack) {
        halo_cuda_free(ctx, raw);
        out->w = packed;
    } else {
        out->w = raw;
    }
    return 0;
}

}  // extern "C"
