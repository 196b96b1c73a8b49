// GGUF tensor reader (host code): walks the header the way the reference's bounded inspector does
// (inference/crates/icn-models/src/gguf.rs:75-149: magic, version 2..3, counts with bounds, the
// metadata key/value table, the tensor-info loop at :110-136 and the alignment rule at :138-149)
// and hands the packed blocks of a named tensor to the weight upload, whole or as one rank's shard.
// Every read is checked against the file length; nothing here touches the GPU except the final
// upload call.
#include <errno.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/b200q.h"

namespace {

constexpr uint64_t kMaxMetadataEntries = 1000000;       // bounds of the reference inspector (gguf.rs:9-14)
constexpr uint64_t kMaxTensors = 10000000;
constexpr uint64_t kMaxStringBytes = 16ull << 20;
constexpr uint64_t kMaxStringArrayBytes = 64ull << 20;
constexpr uint32_t kMaxDims = 8;

// weights per block and bytes per block of the ggml tensor types a GGUF file may carry
struct TypeSize { int id, elems, bytes; };
const TypeSize kTypeSizes[] = {
    {0, 1, 4},     {1, 1, 2},     {2, 32, 18},   {3, 32, 20},   {6, 32, 22},    {7, 32, 24},    {8, 32, 34},
    {9, 32, 40},   {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210}, {15, 256, 292},
    {16, 256, 66}, {17, 256, 74}, {18, 256, 98}, {19, 256, 50}, {20, 32, 18},   {21, 256, 110}, {22, 256, 82},
    {23, 256, 136}, {24, 1, 1},   {25, 1, 2},    {26, 1, 4},    {27, 1, 8},     {28, 1, 8},     {29, 256, 56},
    {30, 1, 2},    {34, 256, 54}, {35, 256, 66}, {39, 32, 17},   {40, 64, 36},   {41, 128, 18},
};
const TypeSize *type_size(uint32_t id) {
    for (const TypeSize &t : kTypeSizes)
        if ((uint32_t)t.id == id) return &t;
    return nullptr;
}

struct MetaValue {
    enum Kind { U32, I32, U64, I64, STRING, STRING_ARRAY, OTHER } kind = OTHER;
    uint64_t u = 0;
    int64_t i = 0;
    std::string s;
    std::vector<std::string> arr;
};

struct TensorInfo {
    std::string name;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[kMaxDims] = {0};
    uint64_t elements = 0, bytes = 0;
    uint64_t rel_offset = 0;        // as stored: relative to the start of the data section
};

}  // namespace

struct b200q_gguf {
    FILE *f = nullptr;
    std::string path;
    uint64_t file_len = 0, pos = 0;
    uint32_t version = 0;
    uint64_t tensor_count = 0, metadata_count = 0;
    uint64_t alignment = 32, header_bytes = 0, tensor_storage_bytes = 0, parameter_count = 0;
    std::map<std::string, MetaValue> meta;
    std::vector<TensorInfo> tensors;
    std::map<std::string, uint64_t> by_name;
    std::string err;
};

namespace {

struct ParseError {
    b200q_status code;
    std::string text;
};

void invalid(const char *what) { throw ParseError{B200Q_ERR_INVALID_CONFIG, std::string("GGUF header is structurally invalid: ") + what}; }

struct Reader {
    b200q_gguf *g;
    void need(uint64_t n) {
        if (g->pos + n < g->pos || g->pos + n > g->file_len) invalid("header extends beyond end of file");
    }
    void read(void *dst, uint64_t n) {
        need(n);
        if (n && fread(dst, 1, (size_t)n, g->f) != (size_t)n) throw ParseError{B200Q_ERR_BACKEND, "failed to read GGUF: short read"};
        g->pos += n;
    }
    void skip(uint64_t n) {
        need(n);
        if (fseeko(g->f, (off_t)n, SEEK_CUR) != 0) throw ParseError{B200Q_ERR_BACKEND, "failed to read GGUF: seek"};
        g->pos += n;
    }
    template <typename T> T le() {
        unsigned char b[sizeof(T)];
        read(b, sizeof(T));
        T v = 0;
        for (size_t i = 0; i < sizeof(T); ++i) v |= (T)((T)b[i] << (8 * i));
        return v;
    }
    std::string str() {
        const uint64_t n = le<uint64_t>();
        if (n > kMaxStringBytes) invalid("metadata string exceeds inspection bound");
        std::string s((size_t)n, '\0');
        read(&s[0], n);
        return s;
    }
    MetaValue value(uint32_t type) {
        MetaValue v;
        switch (type) {
        case 0: v.kind = MetaValue::U32, v.u = le<uint8_t>(); break;
        case 1: v.kind = MetaValue::I32, v.i = (int8_t)le<uint8_t>(); break;
        case 2: v.kind = MetaValue::U32, v.u = le<uint16_t>(); break;
        case 3: v.kind = MetaValue::I32, v.i = (int16_t)le<uint16_t>(); break;
        case 4: v.kind = MetaValue::U32, v.u = le<uint32_t>(); break;
        case 5: v.kind = MetaValue::I32, v.i = (int32_t)le<uint32_t>(); break;
        case 6: skip(4); break;                                   // f32
        case 7: (void)le<uint8_t>(); break;                       // bool
        case 8: v.kind = MetaValue::STRING, v.s = str(); break;
        case 9: {
            const uint32_t et = le<uint32_t>();
            const uint64_t count = le<uint64_t>();
            if (count > kMaxMetadataEntries) invalid("metadata array exceeds inspection bound");
            if (et == 8) {
                v.kind = MetaValue::STRING_ARRAY;
                uint64_t total = 0;
                for (uint64_t i = 0; i < count; ++i) {
                    v.arr.push_back(str());
                    total += v.arr.back().size();
                    if (total > kMaxStringArrayBytes) invalid("metadata string array exceeds inspection bound");
                }
            } else {
                for (uint64_t i = 0; i < count; ++i) (void)value(et);
            }
            break;
        }
        case 10: v.kind = MetaValue::U64, v.u = le<uint64_t>(); break;
        case 11: v.kind = MetaValue::I64, v.i = (int64_t)le<uint64_t>(); break;
        case 12: skip(8); break;                                  // f64
        default: invalid("unknown metadata value type");
        }
        return v;
    }
};

bool meta_u64(const b200q_gguf *g, const char *key, uint64_t *out) {
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return false;
    const MetaValue &v = it->second;
    if (v.kind == MetaValue::U32 || v.kind == MetaValue::U64) {
        *out = v.u;
        return true;
    }
    if ((v.kind == MetaValue::I32 || v.kind == MetaValue::I64) && v.i >= 0) {
        *out = (uint64_t)v.i;
        return true;
    }
    return false;
}

bool mul_overflow(uint64_t a, uint64_t b, uint64_t *out) { return __builtin_mul_overflow(a, b, out); }

void parse(b200q_gguf *g) {
    Reader r{g};
    char magic[4];
    if (g->file_len < 4) throw ParseError{B200Q_ERR_INVALID_CONFIG, "file is not GGUF"};
    r.read(magic, 4);
    if (memcmp(magic, "GGUF", 4) != 0) throw ParseError{B200Q_ERR_INVALID_CONFIG, "file is not GGUF"};
    g->version = r.le<uint32_t>();
    if (g->version < 2 || g->version > 3) {
        char buf[64];
        snprintf(buf, sizeof(buf), "unsupported GGUF version %u", g->version);
        throw ParseError{B200Q_ERR_INVALID_CONFIG, buf};
    }
    g->tensor_count = r.le<uint64_t>();
    g->metadata_count = r.le<uint64_t>();
    if (g->tensor_count > kMaxTensors) invalid("tensor count exceeds inspection bound");
    if (g->metadata_count > kMaxMetadataEntries) invalid("metadata count exceeds inspection bound");
    for (uint64_t i = 0; i < g->metadata_count; ++i) {
        std::string key = r.str();
        const uint32_t type = r.le<uint32_t>();
        g->meta[key] = r.value(type);
    }
    uint64_t params = 0;
    for (uint64_t i = 0; i < g->tensor_count; ++i) {
        TensorInfo t;
        t.name = r.str();
        t.n_dims = r.le<uint32_t>();
        if (t.n_dims == 0 || t.n_dims > kMaxDims) invalid("tensor dimension count is invalid");
        t.elements = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            t.dims[d] = r.le<uint64_t>();
            if (mul_overflow(t.elements, t.dims[d], &t.elements)) invalid("tensor element count overflow");
        }
        if (__builtin_add_overflow(params, t.elements, &params)) invalid("model parameter count overflow");
        t.type = r.le<uint32_t>();
        const TypeSize *ts = type_size(t.type);
        if (!ts || t.dims[0] % (uint64_t)ts->elems) invalid("tensor storage shape or type is invalid");
        uint64_t rows = 1;
        for (uint32_t d = 1; d < t.n_dims; ++d)
            if (mul_overflow(rows, t.dims[d], &rows)) invalid("tensor storage shape or type is invalid");
        uint64_t row_bytes;
        if (mul_overflow(t.dims[0] / (uint64_t)ts->elems, (uint64_t)ts->bytes, &row_bytes) || mul_overflow(row_bytes, rows, &t.bytes))
            invalid("tensor storage shape or type is invalid");
        if (__builtin_add_overflow(g->tensor_storage_bytes, t.bytes, &g->tensor_storage_bytes)) invalid("tensor storage bytes overflow");
        t.rel_offset = r.le<uint64_t>();
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    uint64_t al = 32;
    if (meta_u64(g, "general.alignment", &al) && al > 0xFFFFFFFFull) al = 0;
    if (al == 0 || (al & (al - 1))) invalid("GGUF alignment is invalid");
    g->alignment = al;
    if (g->pos + (al - 1) < g->pos) invalid("GGUF header alignment overflow");
    g->header_bytes = (g->pos + al - 1) & ~(al - 1);
    if (g->header_bytes > g->file_len) invalid("GGUF header extends beyond end of file");
    if (!meta_u64(g, "general.parameter_count", &g->parameter_count)) g->parameter_count = params;
}

b200q_status set_err(b200q_gguf *g, b200q_status code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    if (g) g->err = buf;
    return code;
}

}  // namespace

extern "C" {

int64_t b200q_tensor_storage_bytes_shape(int32_t type, int32_t n_dims, const int64_t *dims) {
    if (n_dims < 1 || n_dims > (int32_t)kMaxDims || !dims) return -1;
    const TypeSize *ts = type_size((uint32_t)type);
    if (!ts || dims[0] < 0 || dims[0] % ts->elems) return -1;
    uint64_t total = (uint64_t)dims[0] / (uint64_t)ts->elems;
    if (mul_overflow(total, (uint64_t)ts->bytes, &total)) return -1;
    for (int32_t d = 1; d < n_dims; ++d) {
        if (dims[d] < 0 || mul_overflow(total, (uint64_t)dims[d], &total)) return -1;
    }
    return total > 0x7FFFFFFFFFFFFFFFull ? -1 : (int64_t)total;
}

b200q_status b200q_gguf_open(const char *path, b200q_gguf **out, char *err, size_t err_n) {
    if (err && err_n) err[0] = 0;
    if (!out) return B200Q_ERR_INVALID_CONFIG;
    *out = nullptr;
    auto report = [&](b200q_status code, const std::string &text) {
        if (err && err_n) snprintf(err, err_n, "%s", text.c_str());
        return code;
    };
    if (!path) return report(B200Q_ERR_INVALID_CONFIG, "null path");
    b200q_gguf *g = new (std::nothrow) b200q_gguf();
    if (!g) return report(B200Q_ERR_OVERLOADED, "out of host memory");
    g->path = path;
    g->f = fopen(path, "rb");
    if (!g->f) {
        const std::string text = std::string("failed to read GGUF: ") + strerror(errno);
        delete g;
        return report(B200Q_ERR_BACKEND, text);
    }
    if (fseeko(g->f, 0, SEEK_END) != 0) {
        fclose(g->f);
        delete g;
        return report(B200Q_ERR_BACKEND, "failed to read GGUF: seek");
    }
    g->file_len = (uint64_t)ftello(g->f);
    fseeko(g->f, 0, SEEK_SET);
    try {
        parse(g);
    } catch (const ParseError &e) {
        fclose(g->f);
        delete g;
        return report(e.code, e.text);
    } catch (const std::bad_alloc &) {
        fclose(g->f);
        delete g;
        return report(B200Q_ERR_OVERLOADED, "out of host memory reading the GGUF header");
    } catch (...) {
        fclose(g->f);
        delete g;
        return report(B200Q_ERR_BACKEND, "failed to read GGUF");
    }
    *out = g;
    return B200Q_OK;
}

void b200q_gguf_close(b200q_gguf *g) {
    if (!g) return;
    if (g->f) fclose(g->f);
    delete g;
}

b200q_status b200q_gguf_last_error(const b200q_gguf *g, char *buf, size_t n) {
    if (!g || !buf || n == 0) return B200Q_ERR_INVALID_CONFIG;
    snprintf(buf, n, "%s", g->err.c_str());
    return B200Q_OK;
}

b200q_status b200q_gguf_summary(const b200q_gguf *g, b200q_gguf_summary_t *out) {
    if (!g || !out) return B200Q_ERR_INVALID_CONFIG;
    out->version = g->version;
    out->alignment = (uint32_t)g->alignment;
    out->tensor_count = g->tensor_count;
    out->metadata_count = g->metadata_count;
    out->tensor_storage_bytes = g->tensor_storage_bytes;
    out->header_bytes = g->header_bytes;
    out->parameter_count = g->parameter_count;
    out->file_bytes = g->file_len;
    return B200Q_OK;
}

const char *b200q_gguf_metadata_string(const b200q_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.kind != MetaValue::STRING) return nullptr;
    return it->second.s.c_str();
}

b200q_status b200q_gguf_metadata_u64(const b200q_gguf *g, const char *key, uint64_t *out) {
    if (!g || !key || !out) return B200Q_ERR_INVALID_CONFIG;
    return meta_u64(g, key, out) ? B200Q_OK : B200Q_ERR_INVALID_CONFIG;
}

b200q_status b200q_gguf_tensor_info(const b200q_gguf *g, uint64_t index, b200q_gguf_tensor_t *out) {
    if (!g || !out || index >= g->tensors.size()) return B200Q_ERR_INVALID_CONFIG;
    const TensorInfo &t = g->tensors[(size_t)index];
    out->name = t.name.c_str();
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (uint32_t d = 0; d < kMaxDims; ++d) out->dims[d] = d < t.n_dims ? t.dims[d] : 1;
    out->elements = t.elements;
    out->bytes = t.bytes;
    out->file_offset = g->header_bytes + t.rel_offset;
    return B200Q_OK;
}

b200q_status b200q_gguf_find(const b200q_gguf *g, const char *name, uint64_t *index) {
    if (!g || !name || !index) return B200Q_ERR_INVALID_CONFIG;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return B200Q_ERR_INVALID_CONFIG;
    *index = it->second;
    return B200Q_OK;
}

b200q_status b200q_gguf_read_tensor(b200q_gguf *g, uint64_t index, void *dst, size_t dst_bytes) {
    if (!g || index >= g->tensors.size()) return B200Q_ERR_INVALID_CONFIG;
    const TensorInfo &t = g->tensors[(size_t)index];
    if (t.rel_offset % g->alignment) return set_err(g, B200Q_ERR_INVALID_CONFIG, "tensor '%s': data offset %llu is not a multiple of the alignment %llu", t.name.c_str(), (unsigned long long)t.rel_offset, (unsigned long long)g->alignment);
    uint64_t begin, end;
    if (__builtin_add_overflow(g->header_bytes, t.rel_offset, &begin) || __builtin_add_overflow(begin, t.bytes, &end) || end > g->file_len)
        return set_err(g, B200Q_ERR_INVALID_CONFIG, "tensor '%s': data extends beyond end of file", t.name.c_str());
    if (dst_bytes != t.bytes || (t.bytes && !dst)) return set_err(g, B200Q_ERR_INVALID_CONFIG, "tensor '%s': buffer of %zu bytes for %llu bytes of data", t.name.c_str(), dst_bytes, (unsigned long long)t.bytes);
    if (t.bytes == 0) return B200Q_OK;
    if (fseeko(g->f, (off_t)begin, SEEK_SET) != 0 || fread(dst, 1, (size_t)t.bytes, g->f) != (size_t)t.bytes)
        return set_err(g, B200Q_ERR_BACKEND, "tensor '%s': failed to read %llu bytes", t.name.c_str(), (unsigned long long)t.bytes);
    return B200Q_OK;
}

b200q_status b200q_gguf_upload(b200q_ctx *ctx, b200q_gguf *g, uint64_t index, int32_t split, int32_t rank, int32_t world,
                               int64_t align_rows, b200q_weight **out) {
    if (!g || !out || index >= g->tensors.size()) return B200Q_ERR_INVALID_CONFIG;
    *out = nullptr;
    const TensorInfo &t = g->tensors[(size_t)index];
    if (t.type != B200Q_TYPE_Q8_0 && t.type != B200Q_TYPE_Q4_K && t.type != B200Q_TYPE_Q6_K)
        return set_err(g, B200Q_ERR_INVALID_CONFIG, "tensor '%s': ggml type %u is not one of Q8_0 (8), Q4_K (12), Q6_K (14)", t.name.c_str(), t.type);
    if (t.n_dims > 2) {
        for (uint32_t d = 2; d < t.n_dims; ++d)
            if (t.dims[d] != 1) return set_err(g, B200Q_ERR_INVALID_CONFIG, "tensor '%s': only matrices can be uploaded as projection weights", t.name.c_str());
    }
    const int64_t K = (int64_t)t.dims[0], N = t.n_dims > 1 ? (int64_t)t.dims[1] : 1;     // GGUF: dims[0] is the row length
    std::vector<unsigned char> buf;
    try {
        buf.resize((size_t)t.bytes);
    } catch (...) {
        return set_err(g, B200Q_ERR_OVERLOADED, "tensor '%s': out of host memory staging %llu bytes", t.name.c_str(), (unsigned long long)t.bytes);
    }
    b200q_status s = b200q_gguf_read_tensor(g, index, buf.data(), buf.size());
    if (s != B200Q_OK) return s;
    s = b200q_weight_upload_shard(ctx, (int32_t)t.type, N, K, buf.data(), buf.size(), split, rank, world, align_rows, out);
    if (s != B200Q_OK) {
        char text[400] = {0};
        if (ctx) b200q_last_error(ctx, text, sizeof(text));
        set_err(g, s, "tensor '%s': %s", t.name.c_str(), text);
    }
    return s;
}

}  // extern "C"
