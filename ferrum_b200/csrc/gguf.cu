// GGUF v2 / v3 index and tensor reads, and the loader that hands a tensor's packed blocks to the device:
// the counterpart of `GgufReader` (src/loader/gguf.rs:162-530: bounds-checked header, metadata and tensor
// descriptors, alignment, range and overlap checks, streaming tensor reads), of `gguf_matrix`
// (src/hybrid/weights.rs:671-736: geometry and payload checks, Q3_K stored as Q6_K) with `q3k_to_q6k`
// (:761-805), and of the host-side Q8_0 row quantiser (:1397-1415).  Host code only.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "internal.h"

namespace {

constexpr uint64_t MAX_TENSORS = 1000000, MAX_METADATA = 1000000, MAX_ARRAY_ITEMS = 4000000, MAX_STRING_BYTES = 16ull << 20;
constexpr uint64_t MAX_TENSOR_NAME_BYTES = 64, MAX_UNTAGGED_TENSOR_NAME_BYTES = 256;

enum MetaType : uint32_t { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 };

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0; // unsigned integers and bool
    int64_t i = 0;  // signed integers
    double f = 0;   // floats
    std::string s;
    uint32_t element_type = 0; // arrays
    uint64_t count = 0;        // arrays: elements in the file (kept or skipped)
    std::vector<MetaValue> values;
};

struct TensorEntry {
    std::string name;
    std::vector<uint64_t> dims; // GGUF order: dimension zero is the contiguous one
    uint32_t type_id = 0;
    uint64_t offset = 0, byte_len = 0;
};

struct Fail {
    std::string message;
};
[[noreturn]] void fail(const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw Fail{buf};
}

// Physical GGML block layouts (src/loader/gguf.rs:87-121).
bool block_layout(uint32_t type_id, uint32_t &elements, uint32_t &bytes) {
    static const struct { uint32_t id, el, by; } table[] = {
        {0, 1, 4}, {1, 1, 2}, {2, 32, 18}, {3, 32, 20}, {6, 32, 22}, {7, 32, 24}, {8, 32, 34}, {9, 32, 36}, {10, 256, 84},
        {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292}, {18, 256, 98}, {20, 32, 18},
        {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {30, 1, 2}, {42, 64, 18}};
    for (const auto &t : table)
        if (t.id == type_id) {
            elements = t.el;
            bytes = t.by;
            return true;
        }
    return false;
}

struct Reader {
    FILE *f;
    uint64_t file_len;
    void bytes(void *dst, size_t n, const char *what) {
        if (n && fread(dst, 1, n, f) != n) fail("read %s: unexpected end of file", what);
    }
    template <typename T> T le(const char *what) {
        uint8_t b[sizeof(T)];
        bytes(b, sizeof(T), what);
        uint64_t v = 0;
        for (size_t i = 0; i < sizeof(T); i++) v |= (uint64_t)b[i] << (8 * i);
        T out;
        memcpy(&out, &v, sizeof(T)); // little-endian host
        return out;
    }
    void skip(uint64_t n) {
        char scratch[4096];
        while (n) {
            const size_t k = (size_t)std::min<uint64_t>(n, sizeof scratch);
            if (fread(scratch, 1, k, f) != k) fail("metadata array is truncated");
            n -= k;
        }
    }
    std::string string(const char *what) {
        const uint64_t len = le<uint64_t>("string length");
        if (len > MAX_STRING_BYTES || len > file_len) fail("unreasonable %s length %llu", what, (unsigned long long)len);
        std::string s((size_t)len, '\0');
        bytes(&s[0], (size_t)len, what);
        // UTF-8 validity, as String::from_utf8 demands
        for (size_t i = 0; i < s.size();) {
            const uint8_t c = (uint8_t)s[i];
            const int extra = c < 0x80 ? 0 : (c >> 5) == 6 ? 1 : (c >> 4) == 14 ? 2 : (c >> 3) == 30 ? 3 : -1;
            if (extra < 0 || i + extra >= s.size() + (extra == 0)) fail("invalid UTF-8 in %s", what);
            for (int k = 1; k <= extra; k++)
                if (((uint8_t)s[i + k] >> 6) != 2) fail("invalid UTF-8 in %s", what);
            i += extra + 1;
        }
        return s;
    }
};

MetaValue read_value(Reader &r, uint32_t type, uint64_t max_items) {
    MetaValue v;
    v.type = type;
    switch (type) {
    case U8: v.u = r.le<uint8_t>("uint8 metadata"); break;
    case I8: v.i = r.le<int8_t>("int8 metadata"); break;
    case U16: v.u = r.le<uint16_t>("uint16 metadata"); break;
    case I16: v.i = r.le<int16_t>("int16 metadata"); break;
    case U32: v.u = r.le<uint32_t>("uint32 metadata"); break;
    case I32: v.i = r.le<int32_t>("int32 metadata"); break;
    case F32: v.f = r.le<float>("float32 metadata"); break;
    case BOOL: {
        const int8_t b = r.le<int8_t>("bool metadata");
        if (b != 0 && b != 1) fail("invalid bool value %d", (int)b);
        v.u = (uint64_t)b;
        break;
    }
    case STRING: v.s = r.string("string metadata"); break;
    case ARRAY: {
        const uint32_t et = r.le<uint32_t>("array element type");
        if (et > F64) fail("unsupported metadata type %u", et);
        if (et == ARRAY) fail("nested metadata arrays are unsupported");
        const uint64_t count = r.le<uint64_t>("array element count");
        if (count > MAX_ARRAY_ITEMS || count > r.file_len) fail("unreasonable metadata array length %llu", (unsigned long long)count);
        v.element_type = et;
        v.count = count;
        if (count > max_items) { // skipped, read back empty
            const int width = (et == U8 || et == I8 || et == BOOL) ? 1 : (et == U16 || et == I16) ? 2 : (et == U32 || et == I32 || et == F32) ? 4
                              : (et == STRING) ? 0 : 8;
            if (width) r.skip(count * width);
            else
                for (uint64_t k = 0; k < count; k++) {
                    const uint64_t len = r.le<uint64_t>("string length");
                    if (len > MAX_STRING_BYTES || len > r.file_len) fail("unreasonable string length %llu", (unsigned long long)len);
                    r.skip(len);
                }
            break;
        }
        v.values.reserve((size_t)count);
        for (uint64_t k = 0; k < count; k++) v.values.push_back(read_value(r, et, ~0ull));
        break;
    }
    case U64: v.u = r.le<uint64_t>("uint64 metadata"); break;
    case I64: v.i = r.le<int64_t>("int64 metadata"); break;
    case F64: v.f = r.le<double>("float64 metadata"); break;
    default: fail("unsupported metadata type %u", type);
    }
    return v;
}

} // namespace

struct fq_gguf {
    FILE *f = nullptr;
    uint64_t file_len = 0, tensor_data_offset = 0;
    uint32_t version = 0, alignment = 32;
    std::map<std::string, MetaValue> metadata;
    std::map<std::string, TensorEntry> tensors; // ordered by name, as the reference's BTreeMap
    std::string error;
};

namespace {

int gguf_fail(fq_gguf *g, int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (g) g->error = buf;
    return status;
}

void parse(fq_gguf *g, bool require_architecture, uint64_t max_items) {
    Reader r{g->f, g->file_len};
    char magic[4];
    r.bytes(magic, 4, "magic");
    if (memcmp(magic, "GGUF", 4)) fail("invalid magic; expected GGUF");
    g->version = r.le<uint32_t>("version");
    if (g->version != 2 && g->version != 3) fail("unsupported version %u", g->version);
    const uint64_t tensor_count = r.le<uint64_t>("tensor count"), metadata_count = r.le<uint64_t>("metadata count");
    if (tensor_count > MAX_TENSORS || metadata_count > MAX_METADATA)
        fail("unreasonable descriptor counts: %llu tensors, %llu metadata entries", (unsigned long long)tensor_count, (unsigned long long)metadata_count);
    for (uint64_t k = 0; k < metadata_count; k++) {
        const std::string key = r.string("metadata key");
        const uint32_t type = r.le<uint32_t>("metadata value type");
        if (type > F64) fail("unsupported metadata type %u", type);
        MetaValue v = read_value(r, type, max_items);
        if (!g->metadata.emplace(key, std::move(v)).second) fail("duplicate metadata key %s", key.c_str());
    }
    auto it = g->metadata.find("general.alignment");
    if (it != g->metadata.end()) {
        if (it->second.type != U32) fail("general.alignment must have uint32 type");
        g->alignment = (uint32_t)it->second.u;
    }
    if (g->alignment < 8 || g->alignment % 8) fail("general.alignment must be a positive multiple of 8, got %u", g->alignment);
    if (require_architecture) {
        auto a = g->metadata.find("general.architecture");
        if (a == g->metadata.end() || a->second.type != STRING) fail("missing or invalid general.architecture metadata");
    }
    bool contains_quantized = false;
    for (uint64_t k = 0; k < tensor_count; k++) {
        TensorEntry t;
        t.name = r.string("tensor name");
        const uint64_t max_name = require_architecture ? MAX_TENSOR_NAME_BYTES : MAX_UNTAGGED_TENSOR_NAME_BYTES;
        if (t.name.size() > max_name) fail("tensor name exceeds %llu bytes", (unsigned long long)max_name);
        const uint32_t rank = r.le<uint32_t>("tensor rank");
        if (rank < 1 || rank > 4) fail("tensor %s has unsupported rank %u", t.name.c_str(), rank);
        for (uint32_t d = 0; d < rank; d++) {
            const uint64_t dim = r.le<uint64_t>("tensor dimension");
            if (dim == 0) fail("tensor %s has an empty dimension", t.name.c_str());
            t.dims.push_back(dim);
        }
        t.type_id = r.le<uint32_t>("tensor type");
        t.offset = r.le<uint64_t>("tensor data offset");
        uint32_t el = 0, by = 0;
        if (!block_layout(t.type_id, el, by)) fail("tensor %s: unsupported GGML tensor type %u", t.name.c_str(), t.type_id);
        uint64_t elements = 1;
        for (uint64_t d : t.dims) {
            if (d && elements > ~0ull / d) fail("tensor %s element count overflow", t.name.c_str());
            elements *= d;
        }
        if (t.dims[0] % el) fail("tensor %s fastest dimension %llu is not divisible by block size %u for type %u", t.name.c_str(),
                                 (unsigned long long)t.dims[0], el, t.type_id);
        const uint64_t blocks = elements / el;
        if (blocks > ~0ull / by) fail("tensor %s byte size overflow", t.name.c_str());
        t.byte_len = blocks * by;
        if (t.offset % g->alignment) fail("tensor %s offset %llu is not aligned to %u", t.name.c_str(), (unsigned long long)t.offset, g->alignment);
        contains_quantized |= !(t.type_id == 0 || t.type_id == 1 || t.type_id == 30);
        const std::string name = t.name;
        if (!g->tensors.emplace(name, std::move(t)).second) fail("duplicate tensor name %s", name.c_str());
    }
    const long pos = ftell(g->f);
    if (pos < 0) fail("read tensor descriptors: position unknown");
    const uint64_t end = (uint64_t)pos, rem = end % g->alignment;
    g->tensor_data_offset = rem ? end + (g->alignment - rem) : end;
    // Ranges relative to the data section, overlap rejected even if entries are listed out of file order.
    std::vector<std::pair<uint64_t, std::pair<uint64_t, const TensorEntry *>>> ranges;
    for (const auto &kv : g->tensors) {
        const TensorEntry &t = kv.second;
        if (t.offset > ~0ull - g->tensor_data_offset) fail("tensor %s offset overflow", t.name.c_str());
        const uint64_t start = g->tensor_data_offset + t.offset;
        if (t.byte_len > ~0ull - start) fail("tensor %s end overflow", t.name.c_str());
        const uint64_t stop = start + t.byte_len;
        if (stop > g->file_len)
            fail("tensor %s range %llu..%llu exceeds file length %llu", t.name.c_str(), (unsigned long long)start, (unsigned long long)stop,
                 (unsigned long long)g->file_len);
        ranges.push_back({start, {stop, &t}});
    }
    std::sort(ranges.begin(), ranges.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
    for (size_t k = 1; k < ranges.size(); k++)
        if (ranges[k - 1].second.first > ranges[k].first)
            fail("tensor ranges overlap: %s and %s", ranges[k - 1].second.second->name.c_str(), ranges[k].second.second->name.c_str());
    if (require_architecture && contains_quantized) {
        auto q = g->metadata.find("general.quantization_version");
        if (q == g->metadata.end() || q->second.type != U32) fail("quantized tensor file is missing uint32 general.quantization_version");
    }
}

const MetaValue *meta(const fq_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->metadata.find(key);
    return it == g->metadata.end() ? nullptr : &it->second;
}

void fill(const TensorEntry &t, fq_gguf_tensor *out) {
    memset(out, 0, sizeof *out);
    snprintf(out->name, sizeof out->name, "%s", t.name.c_str());
    out->n_dims = (uint32_t)t.dims.size();
    for (size_t d = 0; d < t.dims.size(); d++) out->dims[d] = t.dims[d];
    out->type_id = t.type_id;
    out->offset = t.offset;
    out->byte_len = t.byte_len;
}

} // namespace

extern "C" int fq_block_layout(uint32_t type_id, uint32_t *elements, uint32_t *bytes) {
    uint32_t el = 0, by = 0;
    if (!elements || !bytes) return FQ_ERR_PARAM;
    if (!block_layout(type_id, el, by)) return FQ_ERR_GGUF;
    *elements = el;
    *bytes = by;
    return FQ_OK;
}

extern "C" int fq_gguf_open(const char *path, int require_architecture, uint64_t skip_arrays_over, fq_gguf **out, char *err, size_t err_len) {
    auto report = [&](const std::string &m) {
        if (err && err_len) snprintf(err, err_len, "%s", m.c_str());
        return FQ_ERR_GGUF;
    };
    if (!path || !out) return FQ_ERR_PARAM;
    *out = nullptr;
    FILE *f = fopen(path, "rb");
    if (!f) return report(std::string(path) + ": cannot open");
    setvbuf(f, nullptr, _IOFBF, 1 << 20); // the header is millions of small values
    fq_gguf *g = new fq_gguf();
    g->f = f;
    if (fseek(f, 0, SEEK_END) != 0) {
        fclose(f);
        delete g;
        return report("seek to end failed");
    }
    g->file_len = (uint64_t)ftell(f);
    fseek(f, 0, SEEK_SET);
    try {
        parse(g, require_architecture != 0, skip_arrays_over ? skip_arrays_over : ~0ull);
    } catch (const Fail &e) {
        fclose(f);
        delete g;
        return report(e.message);
    }
    *out = g;
    return FQ_OK;
}

extern "C" int fq_gguf_close(fq_gguf *g) {
    if (!g) return FQ_ERR_PARAM;
    if (g->f) fclose(g->f);
    delete g;
    return FQ_OK;
}

extern "C" const char *fq_gguf_last_error(const fq_gguf *g) { return g ? g->error.c_str() : "null file handle"; }

extern "C" int fq_gguf_info(const fq_gguf *g, fq_gguf_info_t *out) {
    if (!g || !out) return FQ_ERR_PARAM;
    out->version = g->version;
    out->alignment = g->alignment;
    out->file_len = g->file_len;
    out->tensor_data_offset = g->tensor_data_offset;
    out->tensor_count = g->tensors.size();
    out->metadata_count = g->metadata.size();
    return FQ_OK;
}

extern "C" int fq_gguf_tensor_by_name(fq_gguf *g, const char *name, fq_gguf_tensor *out) {
    if (!g || !name || !out) return FQ_ERR_PARAM;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return gguf_fail(g, FQ_ERR_GGUF, "missing tensor %s", name);
    fill(it->second, out);
    return FQ_OK;
}

extern "C" int fq_gguf_tensor_by_index(fq_gguf *g, uint64_t index, fq_gguf_tensor *out) {
    if (!g || !out) return FQ_ERR_PARAM;
    if (index >= g->tensors.size()) return gguf_fail(g, FQ_ERR_GGUF, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    auto it = g->tensors.begin();
    std::advance(it, (long)index);
    fill(it->second, out);
    return FQ_OK;
}

// `read_tensor_into`: the destination is exactly the tensor's bytes.
extern "C" int fq_gguf_read_tensor(fq_gguf *g, const char *name, void *dst, size_t len) {
    if (!g || !name || !dst) return FQ_ERR_PARAM;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return gguf_fail(g, FQ_ERR_GGUF, "missing tensor %s", name);
    const TensorEntry &t = it->second;
    if (len != t.byte_len) return gguf_fail(g, FQ_ERR_GGUF, "tensor %s has %llu bytes, destination has %zu", name, (unsigned long long)t.byte_len, len);
    if (fseek(g->f, (long)(g->tensor_data_offset + t.offset), SEEK_SET) != 0) return gguf_fail(g, FQ_ERR_GGUF, "seek to tensor %s failed", name);
    if (fread(dst, 1, len, g->f) != len) return gguf_fail(g, FQ_ERR_GGUF, "read tensor %s: unexpected end of file", name);
    return FQ_OK;
}

extern "C" int fq_gguf_metadata_u64(fq_gguf *g, const char *key, uint64_t *out) {
    const MetaValue *v = meta(g, key);
    if (!v || !out) return gguf_fail(g, FQ_ERR_GGUF, "missing metadata %s", key ? key : "(null)");
    switch (v->type) {
    case U8: case U16: case U32: case U64: case BOOL: *out = v->u; return FQ_OK;
    case I8: case I16: case I32: case I64:
        if (v->i < 0) return gguf_fail(g, FQ_ERR_GGUF, "metadata %s is negative", key);
        *out = (uint64_t)v->i;
        return FQ_OK;
    default: return gguf_fail(g, FQ_ERR_GGUF, "metadata %s is not an integer", key);
    }
}

extern "C" int fq_gguf_metadata_f64(fq_gguf *g, const char *key, double *out) {
    const MetaValue *v = meta(g, key);
    if (!v || !out) return gguf_fail(g, FQ_ERR_GGUF, "missing metadata %s", key ? key : "(null)");
    if (v->type != F32 && v->type != F64) return gguf_fail(g, FQ_ERR_GGUF, "metadata %s is not a float", key);
    *out = v->f;
    return FQ_OK;
}

extern "C" int fq_gguf_metadata_string(fq_gguf *g, const char *key, char *out, size_t len) {
    const MetaValue *v = meta(g, key);
    if (!v || !out || !len) return gguf_fail(g, FQ_ERR_GGUF, "missing metadata %s", key ? key : "(null)");
    if (v->type != STRING) return gguf_fail(g, FQ_ERR_GGUF, "metadata %s is not a string", key);
    if (v->s.size() + 1 > len) return gguf_fail(g, FQ_ERR_GGUF, "metadata %s needs %zu bytes", key, v->s.size() + 1);
    memcpy(out, v->s.c_str(), v->s.size() + 1);
    return FQ_OK;
}

// Element count of an array in the file and how many of them were kept (0 when it was skipped at open).
extern "C" int fq_gguf_metadata_array(fq_gguf *g, const char *key, uint32_t *element_type, uint64_t *count, uint64_t *kept) {
    const MetaValue *v = meta(g, key);
    if (!v) return gguf_fail(g, FQ_ERR_GGUF, "missing metadata %s", key ? key : "(null)");
    if (v->type != ARRAY) return gguf_fail(g, FQ_ERR_GGUF, "metadata %s is not an array", key);
    if (element_type) *element_type = v->element_type;
    if (count) *count = v->count;
    if (kept) *kept = v->values.size();
    return FQ_OK;
}

// Q3_K blocks (hmask[32], qs[64], scales[12] = sixteen 6-bit values, d) as Q6_K blocks holding the same values:
// both formats weigh 16 groups of 16 as d x scale x q; Q3_K's scales (-32..31) fit Q6_K's 8-bit ones and its
// 3-bit weights (-4..3) the 6-bit ones (stored + 32), and d carries over (src/hybrid/weights.rs:761-805).
extern "C" int fq_q3k_to_q6k(const void *src, size_t blocks, void *dst) {
    if (!src || !dst) return FQ_ERR_PARAM;
    const uint8_t *x = (const uint8_t *)src;
    uint8_t *y = (uint8_t *)dst;
    for (size_t b = 0; b < blocks; b++, x += 110, y += 210) {
        const uint8_t *hmask = x, *qs = x + 32, *packed = x + 96;
        uint8_t q[256];
        for (int i = 0; i < 256; i++) {
            const int half = i / 128, rest = i % 128, shift = rest / 32, l = rest % 32;
            const int low = (qs[32 * half + l] >> (2 * shift)) & 3, high = (hmask[l] >> (4 * half + shift)) & 1;
            q[i] = (uint8_t)(low + 4 * high + 28); // the value low - 4 + 4 high, plus Q6_K's 32
        }
        uint8_t *ql = y, *qh = y + 128, *sc = y + 192;
        for (int half = 0; half < 2; half++)
            for (int l = 0; l < 32; l++) {
                const uint8_t a0 = q[128 * half + l], a1 = q[128 * half + l + 32], a2 = q[128 * half + l + 64], a3 = q[128 * half + l + 96];
                ql[64 * half + l] = (uint8_t)((a0 & 0xF) | ((a2 & 0xF) << 4));
                ql[64 * half + l + 32] = (uint8_t)((a1 & 0xF) | ((a3 & 0xF) << 4));
                qh[32 * half + l] = (uint8_t)((a0 >> 4) | ((a1 >> 4) << 2) | ((a2 >> 4) << 4) | ((a3 >> 4) << 6));
            }
        for (int j = 0; j < 16; j++) {
            const int low = j < 8 ? (packed[j] & 0xF) : (packed[j - 8] >> 4), high = (packed[8 + j % 4] >> (2 * (j / 4))) & 3;
            sc[j] = (uint8_t)(int8_t)((low | (high << 4)) - 32);
        }
        y[208] = x[108];
        y[209] = x[109];
    }
    return FQ_OK;
}

namespace {
uint16_t f32_to_f16_bits(float v) { // round to nearest even, as half::f16::from_f32
    uint32_t x;
    memcpy(&x, &v, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u | (man >> 13) : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const int shift = 14 - exp;
        uint32_t half = man >> shift;
        const uint32_t rest = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
        if (rest > mid || (rest == mid && (half & 1))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rest = man & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1))) half++;
    return (uint16_t)(sign | half);
}
} // namespace

// ggml's reference Q8_0 row quantisation (src/hybrid/weights.rs:1397-1415): per 32 values d = amax / 127,
// q = round(v / d) (ties away from zero, as f32::round), d stored as f16.  `n` must be a multiple of 32.
extern "C" int fq_quantize_q8_0(const float *x, size_t n, void *out) {
    if (!x || !out || n % 32) return FQ_ERR_PARAM;
    uint8_t *o = (uint8_t *)out;
    for (size_t b = 0; b < n / 32; b++, x += 32, o += 34) {
        float amax = 0.f;
        for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(x[i]));
        const float d = amax / 127.f, id = d != 0.f ? 1.f / d : 0.f;
        const uint16_t h = f32_to_f16_bits(d);
        o[0] = (uint8_t)(h & 0xFF);
        o[1] = (uint8_t)(h >> 8);
        for (int i = 0; i < 32; i++) o[2 + i] = (uint8_t)(int8_t)std::round(x[i] * id);
    }
    return FQ_OK;
}

// `gguf_matrix`: tensor `name` as `experts` stacked [rows, cols] slices (GGUF dims [cols, rows] or
// [cols, rows, experts]) in its stored encoding, or Q3_K as Q6_K with `q3k_as_q6k`.
extern "C" int fq_matrix_from_gguf(fq_device *dev, fq_gguf *g, const char *name, uint64_t experts, uint64_t rows, uint64_t cols, int q3k_as_q6k,
                                   fq_matrix **out) {
    if (!dev || !g || !name || !out) return FQ_ERR_PARAM;
    *out = nullptr;
    auto it = g->tensors.find(name);
    if (it == g->tensors.end()) return fq_fail(dev, FQ_ERR_GGUF, "missing tensor %s", name);
    const TensorEntry &t = it->second;
    const bool dims_ok = experts == 1 ? (t.dims.size() == 2 && t.dims[0] == cols && t.dims[1] == rows)
                                      : (t.dims.size() == 3 && t.dims[0] == cols && t.dims[1] == rows && t.dims[2] == experts);
    if (!dims_ok) {
        std::string found;
        for (uint64_t d : t.dims) found += (found.empty() ? "" : ", ") + std::to_string(d);
        return fq_fail(dev, FQ_ERR_WEIGHT, "%s: expected GGUF dims [%llu, %llu%s], found [%s]", name, (unsigned long long)cols, (unsigned long long)rows,
                       experts == 1 ? "" : (", " + std::to_string(experts)).c_str(), found.c_str());
    }
    const bool q3k = q3k_as_q6k && t.type_id == 11;
    const uint32_t stored = q3k ? 14u : t.type_id;
    if (stored != FQ_Q8_0 && stored != FQ_Q4_K && stored != FQ_Q5_K && stored != FQ_Q6_K && stored != FQ_IQ4_NL && stored != FQ_IQ4_XS)
        return fq_fail(dev, FQ_ERR_WEIGHT, "%s: GGML type %u has no kernel", name, t.type_id);
    uint32_t el = 0, by = 0;
    block_layout(t.type_id, el, by);
    if (cols % el || cols % 64) return fq_fail(dev, FQ_ERR_WEIGHT, "%s: row width is not a whole number of blocks", name);
    if (cols / el * by * rows * experts != t.byte_len) return fq_fail(dev, FQ_ERR_WEIGHT, "%s: byte length differs from geometry", name);
    std::vector<uint8_t> bytes((size_t)t.byte_len);
    if (int rc = fq_gguf_read_tensor(g, name, bytes.data(), bytes.size())) return fq_fail(dev, rc, "%s", g->error.c_str());
    if (q3k) {
        std::vector<uint8_t> q6(bytes.size() / 110 * 210);
        fq_q3k_to_q6k(bytes.data(), bytes.size() / 110, q6.data());
        bytes.swap(q6);
    }
    return fq_matrix_create(dev, (int)stored, rows, cols, experts, bytes.data(), bytes.size(), out);
}
