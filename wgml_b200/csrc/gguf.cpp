// GGUF parser: header, metadata key/values, tensor infos; tensor bytes are used in place from a
// read-only mapping of the file.  Follows Gguf::from_bytes of crates/wgml/src/gguf.rs:452-623:
// same magic numbers, value types, alignment rule and set of tensor types whose data is read.
#include "common.cuh"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

constexpr uint32_t GGUF_FILE_MAGIC_LE = 0x46554747;  // gguf.rs:19
constexpr uint32_t GGUF_FILE_MAGIC_BE = 0x47475546;  // gguf.rs:20

struct MetaValue {
    std::string key;
    int type = 0;
    int elem_type = -1;
    uint64_t len = 0;           // array length or string length
    const uint8_t *ptr = nullptr;  // scalar bytes, string bytes or first array element
    std::vector<std::pair<const char *, uint64_t>> strings;  // elements of a string array
};

struct TensorInfo {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = { 1, 1, 1, 1 };
    uint32_t type = 0;
    uint64_t offset = 0;
    uint64_t n_bytes = 0;
    const void *data = nullptr;
};

int scalar_size(int type)
{
    switch (type) {
    case WGB_META_U8: case WGB_META_I8: case WGB_META_BOOL: return 1;
    case WGB_META_U16: case WGB_META_I16: return 2;
    case WGB_META_U32: case WGB_META_I32: case WGB_META_F32: return 4;
    case WGB_META_U64: case WGB_META_I64: case WGB_META_F64: return 8;
    default: return 0;
    }
}

}  // namespace

struct wgb_gguf {
    const uint8_t *bytes = nullptr;
    size_t len = 0;
    void *mapping = nullptr;
    size_t mapping_len = 0;
    uint32_t version = 0;
    uint64_t tensor_count = 0, metadata_count = 0;
    uint32_t alignment = 32;
    std::vector<MetaValue> meta;
    std::vector<TensorInfo> tensors;
    std::unordered_map<std::string, size_t> meta_index, tensor_index;
};

namespace {

struct Reader {
    const uint8_t *b;
    size_t len, off = 0;
    bool ok = true;
    bool need(size_t n)
    {
        if (!ok || n > len - off) { ok = false; return false; }
        return true;
    }
    template <typename T>
    T pod()
    {
        T v{};
        if (need(sizeof(T))) { memcpy(&v, b + off, sizeof(T)); off += sizeof(T); }
        return v;
    }
    // read_string, gguf.rs:658-662
    bool str(const char **p, uint64_t *n)
    {
        uint64_t l = pod<uint64_t>();
        if (!need(l)) return false;
        *p = (const char *)(b + off);
        *n = l;
        off += l;
        return true;
    }
};

// MetadataValueType::read_array, gguf.rs:411-448.  Nested arrays are walked (to find their end)
// but their elements are not recorded.
bool skip_array(Reader &r, int elem_type, uint64_t len, MetaValue *rec, int *err_type)
{
    if (elem_type == WGB_META_STRING) {
        for (uint64_t i = 0; i < len; i++) {
            const char *p; uint64_t n;
            if (!r.str(&p, &n)) return false;
            if (rec) rec->strings.emplace_back(p, n);
        }
        return true;
    }
    if (elem_type == WGB_META_ARRAY) {
        for (uint64_t i = 0; i < len; i++) {
            uint32_t ty = r.pod<uint32_t>();
            uint64_t l = r.pod<uint64_t>();
            if (!r.ok) return false;
            if (ty > WGB_META_F64) { *err_type = (int)ty; return false; }
            if (!skip_array(r, (int)ty, l, nullptr, err_type)) return false;
        }
        return true;
    }
    const int sz = scalar_size(elem_type);
    if (len > (r.len - r.off) / (size_t)sz) { r.ok = false; return false; }
    r.off += len * sz;
    return true;
}

// Bytes of a tensor whose data the reference reads (gguf.rs:548-619); 0 for the others.
uint64_t tensor_bytes(uint32_t type, uint64_t n_elems)
{
    const int bb = wgb::block_bytes((int)type), bl = wgb::block_len((int)type);
    if (!bb) return 0;
    return n_elems / (uint64_t)bl * (uint64_t)bb;
}

int parse(wgb_gguf *g)
{
    Reader r{ g->bytes, g->len };
    // load_header, gguf.rs:474-490
    const uint32_t magic = r.pod<uint32_t>();
    if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "file shorter than a GGUF header");
    if (magic != GGUF_FILE_MAGIC_LE && magic != GGUF_FILE_MAGIC_BE)
        return wgb::fail(WGB_ERR_PARSE, "the input file isn't a gguf binary file. Got a magic number of %#x", magic);
    g->version = r.pod<uint32_t>();
    g->tensor_count = r.pod<uint64_t>();
    g->metadata_count = r.pod<uint64_t>();
    if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "file shorter than a GGUF header");
    if (g->metadata_count > g->len || g->tensor_count > g->len)
        return wgb::fail(WGB_ERR_PARSE, "implausible header counts (%llu key/values, %llu tensors)",
                         (unsigned long long)g->metadata_count, (unsigned long long)g->tensor_count);

    // load_metadata, gguf.rs:492-505
    for (uint64_t i = 0; i < g->metadata_count; i++) {
        const char *kp; uint64_t kn;
        if (!r.str(&kp, &kn)) return wgb::fail(WGB_ERR_PARSE, "truncated metadata key %llu", (unsigned long long)i);
        MetaValue v;
        v.key.assign(kp, kn);
        const uint32_t ty = r.pod<uint32_t>();
        if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "truncated metadata value of '%s'", v.key.c_str());
        if (ty > WGB_META_F64)
            return wgb::fail(WGB_ERR_UNSUPPORTED, "metadata value of type %u is not part of the supported gguf version", ty);
        v.type = (int)ty;
        if (ty == WGB_META_STRING) {
            const char *p; uint64_t n;
            if (!r.str(&p, &n)) return wgb::fail(WGB_ERR_PARSE, "truncated string value of '%s'", v.key.c_str());
            v.ptr = (const uint8_t *)p;
            v.len = n;
        } else if (ty == WGB_META_ARRAY) {
            const uint32_t et = r.pod<uint32_t>();
            const uint64_t n = r.pod<uint64_t>();
            if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "truncated array header of '%s'", v.key.c_str());
            if (et > WGB_META_F64)
                return wgb::fail(WGB_ERR_UNSUPPORTED, "metadata value of type %u is not part of the supported gguf version", et);
            v.elem_type = (int)et;
            v.len = n;
            v.ptr = r.b + r.off;
            int bad = -1;
            if (!skip_array(r, (int)et, n, &v, &bad)) {
                if (bad >= 0)
                    return wgb::fail(WGB_ERR_UNSUPPORTED, "metadata value of type %d is not part of the supported gguf version", bad);
                return wgb::fail(WGB_ERR_PARSE, "truncated array value of '%s'", v.key.c_str());
            }
        } else {
            const int sz = scalar_size((int)ty);
            if (!r.need(sz)) return wgb::fail(WGB_ERR_PARSE, "truncated value of '%s'", v.key.c_str());
            v.ptr = r.b + r.off;
            r.off += sz;
        }
        g->meta_index[v.key] = g->meta.size();  // a repeated key keeps the last value, as HashMap::insert does
        g->meta.push_back(std::move(v));
    }

    // general.alignment, gguf.rs:456-464: honoured only when stored as u32
    auto it = g->meta_index.find("general.alignment");
    if (it != g->meta_index.end() && g->meta[it->second].type == WGB_META_U32) {
        uint32_t al;
        memcpy(&al, g->meta[it->second].ptr, 4);
        if (al == 0) return wgb::fail(WGB_ERR_PARSE, "general.alignment is zero");
        g->alignment = al;
    }

    // load_tensors, gguf.rs:507-537
    for (uint64_t i = 0; i < g->tensor_count; i++) {
        const char *np; uint64_t nn;
        if (!r.str(&np, &nn)) return wgb::fail(WGB_ERR_PARSE, "truncated tensor name %llu", (unsigned long long)i);
        TensorInfo t;
        t.name.assign(np, nn);
        t.n_dims = r.pod<uint32_t>();
        if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "truncated tensor info of '%s'", t.name.c_str());
        if (t.n_dims > 4)
            return wgb::fail(WGB_ERR_UNSUPPORTED, "Tensors of dimensions larger than 4 are not supported yet.");
        for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = r.pod<uint64_t>();
        t.type = r.pod<uint32_t>();
        t.offset = r.pod<uint64_t>();
        if (!r.ok) return wgb::fail(WGB_ERR_PARSE, "truncated tensor info of '%s'", t.name.c_str());
        if (t.type > 29) return wgb::fail(WGB_ERR_UNSUPPORTED, "tensor of type %u is not part of the supported gguf version", t.type);
        g->tensor_index[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }

    // align_offset, gguf.rs:540,707-709
    const uint64_t al = g->alignment;
    const uint64_t data_start = r.off + (al - (r.off % al)) % al;
    for (TensorInfo &t : g->tensors) {
        t.offset += data_start;
        uint64_t n_elems = 1;
        for (int d = 0; d < 4; d++) {
            if (t.dims[d] != 0 && n_elems > UINT64_MAX / t.dims[d])
                return wgb::fail(WGB_ERR_PARSE, "tensor '%s' has an overflowing element count", t.name.c_str());
            n_elems *= t.dims[d];
        }
        t.n_bytes = tensor_bytes(t.type, n_elems);
        if (t.n_bytes) {
            if (t.offset > g->len || t.n_bytes > g->len - t.offset)
                return wgb::fail(WGB_ERR_PARSE, "tensor '%s' extends past the end of the file", t.name.c_str());
            t.data = g->bytes + t.offset;
        }
    }
    return WGB_OK;
}

const MetaValue *meta_at(const wgb_gguf *g, uint64_t index)
{
    if (!g || index >= g->meta.size()) {
        wgb::fail(WGB_ERR_NOT_FOUND, "metadata index %llu out of range", (unsigned long long)index);
        return nullptr;
    }
    return &g->meta[index];
}

template <typename T>
T rd(const uint8_t *p)
{
    T v;
    memcpy(&v, p, sizeof(T));
    return v;
}

// Integer-like scalar at p widened to 64 bits.  Returns false for float / string / array types.
bool as_i64(int type, const uint8_t *p, int64_t *s, uint64_t *u)
{
    switch (type) {
    case WGB_META_U8: *u = rd<uint8_t>(p); *s = (int64_t)*u; return true;
    case WGB_META_BOOL: *u = rd<uint8_t>(p) != 0; *s = (int64_t)*u; return true;  // gguf.rs:399
    case WGB_META_I8: *s = rd<int8_t>(p); *u = (uint64_t)*s; return true;
    case WGB_META_U16: *u = rd<uint16_t>(p); *s = (int64_t)*u; return true;
    case WGB_META_I16: *s = rd<int16_t>(p); *u = (uint64_t)*s; return true;
    case WGB_META_U32: *u = rd<uint32_t>(p); *s = (int64_t)*u; return true;
    case WGB_META_I32: *s = rd<int32_t>(p); *u = (uint64_t)*s; return true;
    case WGB_META_U64: *u = rd<uint64_t>(p); *s = (int64_t)*u; return true;
    case WGB_META_I64: *s = rd<int64_t>(p); *u = (uint64_t)*s; return true;
    default: return false;
    }
}

bool as_f64(int type, const uint8_t *p, double *out)
{
    if (type == WGB_META_F32) { *out = rd<float>(p); return true; }
    if (type == WGB_META_F64) { *out = rd<double>(p); return true; }
    return false;
}

}  // namespace

WGB_EXPORT int wgb_gguf_from_bytes(const void *bytes, size_t len, wgb_gguf **out)
{
    WGB_REQUIRE(bytes && out, "null argument");
    wgb_gguf *g = new wgb_gguf();
    g->bytes = (const uint8_t *)bytes;
    g->len = len;
    const int rc = parse(g);
    if (rc != WGB_OK) { delete g; return rc; }
    *out = g;
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_open(const char *path, wgb_gguf **out)
{
    WGB_REQUIRE(path && out, "null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return wgb::fail(WGB_ERR_NOT_FOUND, "cannot open '%s'", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); return wgb::fail(WGB_ERR_PARSE, "cannot stat '%s' or empty file", path); }
    void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return wgb::fail(WGB_ERR_PARSE, "cannot map '%s'", path);
    wgb_gguf *g = new wgb_gguf();
    g->bytes = (const uint8_t *)map;
    g->len = (size_t)st.st_size;
    g->mapping = map;
    g->mapping_len = (size_t)st.st_size;
    const int rc = parse(g);
    if (rc != WGB_OK) { munmap(map, g->mapping_len); delete g; return rc; }
    *out = g;
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_close(wgb_gguf *g)
{
    if (!g) return WGB_OK;
    if (g->mapping) munmap(g->mapping, g->mapping_len);
    delete g;
    return WGB_OK;
}

WGB_EXPORT uint32_t wgb_gguf_version(const wgb_gguf *g) { return g ? g->version : 0; }
WGB_EXPORT uint64_t wgb_gguf_tensor_count(const wgb_gguf *g) { return g ? g->tensors.size() : 0; }
WGB_EXPORT uint64_t wgb_gguf_metadata_count(const wgb_gguf *g) { return g ? g->meta.size() : 0; }
WGB_EXPORT uint32_t wgb_gguf_alignment(const wgb_gguf *g) { return g ? g->alignment : 0; }

WGB_EXPORT int64_t wgb_gguf_meta_find(const wgb_gguf *g, const char *key)
{
    if (!g || !key) return -1;
    auto it = g->meta_index.find(key);
    return it == g->meta_index.end() ? -1 : (int64_t)it->second;
}

WGB_EXPORT const char *wgb_gguf_meta_key(const wgb_gguf *g, uint64_t index)
{
    const MetaValue *v = meta_at(g, index);
    return v ? v->key.c_str() : nullptr;
}

WGB_EXPORT int wgb_gguf_meta_type(const wgb_gguf *g, uint64_t index, int *type, int *elem_type, uint64_t *len)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return WGB_ERR_NOT_FOUND;
    if (type) *type = v->type;
    if (elem_type) *elem_type = v->elem_type;
    if (len) *len = v->len;
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_u64(const wgb_gguf *g, uint64_t index, uint64_t *out)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return WGB_ERR_NOT_FOUND;
    int64_t s;
    if (!out || !as_i64(v->type, v->ptr, &s, out)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_i64(const wgb_gguf *g, uint64_t index, int64_t *out)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return WGB_ERR_NOT_FOUND;
    uint64_t u;
    if (!out || !as_i64(v->type, v->ptr, out, &u)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_f64(const wgb_gguf *g, uint64_t index, double *out)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return WGB_ERR_NOT_FOUND;
    if (!out || !as_f64(v->type, v->ptr, out)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_str(const wgb_gguf *g, uint64_t index, const char **ptr, uint64_t *len)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return WGB_ERR_NOT_FOUND;
    if (v->type != WGB_META_STRING || !ptr || !len) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    *ptr = (const char *)v->ptr;
    *len = v->len;
    return WGB_OK;
}

static const MetaValue *array_at(const wgb_gguf *g, uint64_t index, uint64_t i)
{
    const MetaValue *v = meta_at(g, index);
    if (!v) return nullptr;
    if (v->type != WGB_META_ARRAY || i >= v->len) {
        wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type or element index.");
        return nullptr;
    }
    return v;
}

WGB_EXPORT int wgb_gguf_meta_arr_u64(const wgb_gguf *g, uint64_t index, uint64_t i, uint64_t *out)
{
    const MetaValue *v = array_at(g, index, i);
    if (!v) return WGB_ERR_INVALID;
    int64_t s;
    const int sz = scalar_size(v->elem_type);
    if (!out || !sz || !as_i64(v->elem_type, v->ptr + i * sz, &s, out)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_arr_i64(const wgb_gguf *g, uint64_t index, uint64_t i, int64_t *out)
{
    const MetaValue *v = array_at(g, index, i);
    if (!v) return WGB_ERR_INVALID;
    uint64_t u;
    const int sz = scalar_size(v->elem_type);
    if (!out || !sz || !as_i64(v->elem_type, v->ptr + i * sz, out, &u)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_arr_f64(const wgb_gguf *g, uint64_t index, uint64_t i, double *out)
{
    const MetaValue *v = array_at(g, index, i);
    if (!v) return WGB_ERR_INVALID;
    const int sz = scalar_size(v->elem_type);
    if (!out || !sz || !as_f64(v->elem_type, v->ptr + i * sz, out)) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    return WGB_OK;
}

WGB_EXPORT int wgb_gguf_meta_arr_str(const wgb_gguf *g, uint64_t index, uint64_t i, const char **ptr, uint64_t *len)
{
    const MetaValue *v = array_at(g, index, i);
    if (!v) return WGB_ERR_INVALID;
    if (v->elem_type != WGB_META_STRING || !ptr || !len) return wgb::fail(WGB_ERR_INVALID, "unwrap: unexpected GGUF attribute type.");
    *ptr = v->strings[i].first;
    *len = v->strings[i].second;
    return WGB_OK;
}

WGB_EXPORT int64_t wgb_gguf_tensor_find(const wgb_gguf *g, const char *name)
{
    if (!g || !name) return -1;
    auto it = g->tensor_index.find(name);
    return it == g->tensor_index.end() ? -1 : (int64_t)it->second;
}

WGB_EXPORT int wgb_gguf_tensor_info(const wgb_gguf *g, uint64_t index, wgb_gguf_tensor *out)
{
    WGB_REQUIRE(g && out, "null argument");
    if (index >= g->tensors.size()) return wgb::fail(WGB_ERR_NOT_FOUND, "tensor index %llu out of range", (unsigned long long)index);
    const TensorInfo &t = g->tensors[index];
    out->name = t.name.c_str();
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->dims[d] = t.dims[d];
    out->type = t.type;
    out->offset = t.offset;
    out->n_bytes = t.n_bytes;
    out->data = t.data;
    return WGB_OK;
}
