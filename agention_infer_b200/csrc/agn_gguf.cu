// GGUF container glue: header, metadata and tensor directory of a GGUF v2/v3 file, and the
// upload of one tensor's bytes to the device (the quantised embedding table that
// agn_get_rows_* reads, or a norm weight).  Host code only.
//
// Reference: `parser::parse` (src/parser.rs:9-66, value decoding :158-186), `loader::load`
// (src/loader.rs:14-19, memory-mapped), `GgufFile` accessors and `MetadataValue::as_*`
// (src/types.rs), tensor addressing `data_offset + byte_offset` with dims[0] the contiguous
// dimension (src/quant/mod.rs:97-135), weight pre-upload (src/model/llama/gpu_resident.rs:112-152).
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>
#include <string>
#include <vector>

#include "agn_common.cuh"

namespace {

struct MetaValue {
    uint32_t type = 0;       // GGUF value type id, 9 = array
    uint64_t u = 0;          // unsigned / bool payload
    int64_t i = 0;           // signed payload
    double f = 0.0;          // float payload
    std::string s;           // string payload
    uint32_t elem_type = 0;  // arrays: element type and count; string / float elements are skipped,
    uint64_t count = 0;      // integer elements are kept (as i64, `MetadataValue::as_i64`) in ints
    std::vector<int64_t> ints;
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t ggml_type = 0;
    uint64_t byte_offset = 0;
};

struct Cursor {
    const uint8_t *data;
    size_t len, pos;
    bool ok;
    size_t err_pos;
    bool need(size_t n) {
        if (!ok) return false;
        if (len - pos < n) {
            ok = false;
            err_pos = pos;
            return false;
        }
        return true;
    }
    template <typename T> T read() {
        T v{};
        if (need(sizeof(T))) {
            memcpy(&v, data + pos, sizeof(T));
            pos += sizeof(T);
        }
        return v;
    }
    std::string read_string() {
        const uint64_t n = read<uint64_t>();
        if (!ok) return std::string();
        if (n > len - pos) {
            ok = false;
            err_pos = pos;
            return std::string();
        }
        std::string s(reinterpret_cast<const char *>(data + pos), (size_t)n);
        pos += (size_t)n;
        return s;
    }
};

int32_t gfail(char *err, size_t err_len, int32_t status, const char *fmt, ...) {
    if (err && err_len) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, err_len, fmt, ap);
        va_end(ap);
    }
    return status;
}

// the GgmlType ids the reference knows (src/types.rs:9-46); 4 and 5 were removed from ggml
bool known_ggml_type(uint32_t t) { return t <= 33 && t != 4 && t != 5; }

}  // namespace

struct agn_gguf {
    uint32_t version = 0;
    uint64_t tensor_count = 0, data_offset = 0;
    std::map<std::string, MetaValue> meta;
    std::vector<Tensor> tensors;
    const uint8_t *data = nullptr;  // whole file (mapping or caller's memory)
    size_t len = 0;
    void *mapping = nullptr;        // non-null when this object owns an mmap
    size_t map_len = 0;
    // further files of a split model (`MultiFileMmap`, src/loader.rs:44-90): only the first file
    // holds the header; tensor offsets run on through the files as if they were concatenated
    struct Part {
        void *mapping;
        size_t len;
        uint64_t start;  // offset of this file's first byte in the concatenated byte space
    };
    std::vector<Part> parts;

    // `MultiFileMmap::slice`: the bytes [offset, offset + n) if they lie inside one file, else null
    // (offsets and sizes come from the file: every comparison is written so that it cannot wrap)
    const uint8_t *slice(uint64_t offset, uint64_t n) const {
        if (n <= len && offset <= len - n) return data + offset;
        for (const Part &p : parts)
            if (p.start <= offset && n <= p.len && offset - p.start <= p.len - n)
                return static_cast<const uint8_t *>(p.mapping) + (offset - p.start);
        return nullptr;
    }
};

namespace {

// src/parser.rs:158-186.  Returns false on an unknown type id.
bool read_value(Cursor &c, uint32_t type, MetaValue &v, bool keep) {
    v.type = type;
    switch (type) {
    case 0: v.u = c.read<uint8_t>(); break;
    case 1: v.i = c.read<int8_t>(); break;
    case 2: v.u = c.read<uint16_t>(); break;
    case 3: v.i = c.read<int16_t>(); break;
    case 4: v.u = c.read<uint32_t>(); break;
    case 5: v.i = c.read<int32_t>(); break;
    case 6: v.f = c.read<float>(); break;
    case 7: v.u = c.read<uint8_t>() != 0; break;
    case 8: { std::string s = c.read_string(); if (keep) v.s.swap(s); break; }
    case 9: {
        v.elem_type = c.read<uint32_t>();
        if (c.ok && (v.elem_type > 12 || v.elem_type == 9)) return false;  // MetadataArrayType::from_u32
        v.count = c.read<uint64_t>();
        // integer arrays (token types, a per-layer head_count_kv) keep their values; types 0-5, 10, 11
        const bool ints = v.elem_type <= 5 || v.elem_type == 10 || v.elem_type == 11;
        const bool is_signed = v.elem_type == 1 || v.elem_type == 3 || v.elem_type == 5 || v.elem_type == 11;
        for (uint64_t k = 0; k < v.count && c.ok; k++) {
            MetaValue e;
            if (!read_value(c, v.elem_type, e, false)) return false;
            if (keep && ints && c.ok) v.ints.push_back(is_signed ? e.i : (int64_t)e.u);
        }
        break;
    }
    case 10: v.u = c.read<uint64_t>(); break;
    case 11: v.i = c.read<int64_t>(); break;
    case 12: v.f = c.read<double>(); break;
    default: return false;
    }
    return true;
}

int32_t parse_into(agn_gguf *g, char *err, size_t err_len) {
    Cursor c{g->data, g->len, 0, true, 0};
    // src/parser.rs:12-24
    uint8_t magic[4] = {0, 0, 0, 0};
    if (c.need(4)) { memcpy(magic, c.data, 4); c.pos = 4; }
    if (!c.ok) return gfail(err, err_len, AGN_EFORMAT, "unexpected end of data at offset %zu", c.err_pos);
    if (memcmp(magic, "GGUF", 4) != 0) return gfail(err, err_len, AGN_EFORMAT, "invalid GGUF magic");
    g->version = c.read<uint32_t>();
    if (c.ok && (g->version < 2 || g->version > 3))
        return gfail(err, err_len, AGN_EFORMAT, "unsupported GGUF version %u", g->version);
    g->tensor_count = c.read<uint64_t>();
    const uint64_t kv_count = c.read<uint64_t>();
    for (uint64_t k = 0; k < kv_count && c.ok; k++) {  // :27-33
        std::string key = c.read_string();
        const uint32_t type = c.read<uint32_t>();
        MetaValue v;
        if (c.ok && !read_value(c, type, v, true))
            return gfail(err, err_len, AGN_EFORMAT, "unknown metadata type %u", c.ok ? (type == 9 ? v.elem_type : type) : type);
        if (c.ok) g->meta[key] = v;
    }
    for (uint64_t k = 0; k < g->tensor_count && c.ok; k++) {  // :36-55
        Tensor t;
        t.name = c.read_string();
        t.n_dims = c.read<uint32_t>();
        if (c.ok && t.n_dims > 4) return gfail(err, err_len, AGN_EFORMAT, "tensor '%s' has %u dimensions", t.name.c_str(), t.n_dims);
        for (uint32_t d = 0; d < t.n_dims && c.ok; d++) t.dims[d] = c.read<uint64_t>();
        t.ggml_type = c.read<uint32_t>();
        if (c.ok && !known_ggml_type(t.ggml_type)) return gfail(err, err_len, AGN_EFORMAT, "unknown ggml type %u", t.ggml_type);
        t.byte_offset = c.read<uint64_t>();
        if (c.ok) g->tensors.push_back(t);
    }
    if (!c.ok) return gfail(err, err_len, AGN_EFORMAT, "unexpected end of data at offset %zu", c.err_pos);
    g->data_offset = ((uint64_t)c.pos + 31) & ~(uint64_t)31;  // :58, 32-byte alignment
    return AGN_OK;
}

const MetaValue *find_meta(const agn_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

int32_t agn_gguf_parse(const void *data, size_t len, agn_gguf **out, char *err, size_t err_len) {
    if (err && err_len) err[0] = '\0';
    if (!out || (!data && len)) return gfail(err, err_len, AGN_EINVAL, "agn_gguf_parse: null argument");
    *out = nullptr;
    agn_gguf *g = new agn_gguf();
    g->data = static_cast<const uint8_t *>(data);
    g->len = len;
    const int32_t rc = parse_into(g, err, err_len);
    if (rc != AGN_OK) {
        delete g;
        return rc;
    }
    *out = g;
    return AGN_OK;
}

// `parse_split_index` (src/loader.rs:25-38): "name-00001-of-00004.gguf" -> (1, 4).
int32_t agn_gguf_split_index(const char *name, uint64_t *index, uint64_t *total) {
    if (!name) return AGN_EINVAL;
    std::string s(name);
    const std::string suffix = ".gguf";
    if (s.size() < suffix.size() || s.compare(s.size() - suffix.size(), suffix.size(), suffix) != 0) return AGN_ENOTFOUND;
    s.erase(s.size() - suffix.size());
    const size_t of_pos = s.rfind("-of-");
    if (of_pos == std::string::npos) return AGN_ENOTFOUND;
    const std::string total_str = s.substr(of_pos + 4), before = s.substr(0, of_pos);
    const size_t dash = before.rfind('-');
    if (dash == std::string::npos) return AGN_ENOTFOUND;
    const std::string index_str = before.substr(dash + 1);
    auto parse = [](const std::string &t, uint64_t *v) {  // str::parse::<usize>: digits only (a leading '+' is allowed)
        size_t i = (!t.empty() && t[0] == '+') ? 1 : 0;
        if (i >= t.size()) return false;
        uint64_t acc = 0;
        for (; i < t.size(); i++) {
            if (t[i] < '0' || t[i] > '9') return false;
            if (acc > (UINT64_MAX - (uint64_t)(t[i] - '0')) / 10) return false;
            acc = acc * 10 + (uint64_t)(t[i] - '0');
        }
        *v = acc;
        return true;
    };
    uint64_t i = 0, n = 0;
    if (!parse(index_str, &i) || !parse(total_str, &n)) return AGN_ENOTFOUND;
    if (index) *index = i;
    if (total) *total = n;
    return AGN_OK;
}

namespace {
int32_t map_file(const char *path, void **m, size_t *len, char *err, size_t err_len) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return gfail(err, err_len, AGN_EIO, "cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        return gfail(err, err_len, AGN_EIO, "cannot stat %s or the file is empty", path);
    }
    void *p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) return gfail(err, err_len, AGN_EIO, "cannot map %s: %s", path, strerror(errno));
    *m = p;
    *len = (size_t)st.st_size;
    return AGN_OK;
}
}  // namespace

int32_t agn_gguf_open(const char *path, agn_gguf **out, char *err, size_t err_len) {
    if (err && err_len) err[0] = '\0';
    if (!path || !out) return gfail(err, err_len, AGN_EINVAL, "agn_gguf_open: null argument");
    *out = nullptr;
    void *m = nullptr;
    size_t len = 0;
    int32_t rc = map_file(path, &m, &len, err, err_len);
    if (rc != AGN_OK) return rc;
    agn_gguf *g = new agn_gguf();
    g->data = static_cast<const uint8_t *>(m);
    g->len = len;
    g->mapping = m;
    g->map_len = len;
    rc = parse_into(g, err, err_len);
    // a split model: file 1 of N names its siblings (`MultiFileMmap::load`, `sibling_path`, src/loader.rs:49-103)
    const std::string full(path);
    const size_t slash = full.rfind('/');
    const std::string dir = slash == std::string::npos ? std::string() : full.substr(0, slash + 1);
    const std::string base = slash == std::string::npos ? full : full.substr(slash + 1);
    uint64_t index = 1, total = 1;
    if (rc == AGN_OK && agn_gguf_split_index(base.c_str(), &index, &total) == AGN_OK && total > 1 && total <= 99999) {
        char pat[32];
        snprintf(pat, sizeof pat, "-00001-of-%05llu", (unsigned long long)total);
        const size_t at = base.find(pat);
        uint64_t cumulative = len;
        for (uint64_t i = 2; at != std::string::npos && i <= total && rc == AGN_OK; i++) {
            char rep[32];
            snprintf(rep, sizeof rep, "-%05llu-of-%05llu", (unsigned long long)i, (unsigned long long)total);
            std::string sib = base;
            sib.replace(at, strlen(pat), rep);
            void *pm = nullptr;
            size_t pl = 0;
            rc = map_file((dir + sib).c_str(), &pm, &pl, err, err_len);
            if (rc == AGN_OK) {
                g->parts.push_back({pm, pl, cumulative});
                cumulative += pl;
            }
        }
    }
    if (rc != AGN_OK) {
        agn_gguf_close(g);
        return rc;
    }
    *out = g;
    return AGN_OK;
}

int32_t agn_gguf_close(agn_gguf *g) {
    if (!g) return AGN_OK;
    if (g->mapping) munmap(g->mapping, g->map_len);
    for (const agn_gguf::Part &p : g->parts) munmap(p.mapping, p.len);
    delete g;
    return AGN_OK;
}

uint32_t agn_gguf_version(const agn_gguf *g) { return g ? g->version : 0; }
uint64_t agn_gguf_tensor_count(const agn_gguf *g) { return g ? g->tensor_count : 0; }
uint64_t agn_gguf_data_offset(const agn_gguf *g) { return g ? g->data_offset : 0; }
uint64_t agn_gguf_metadata_count(const agn_gguf *g) { return g ? g->meta.size() : 0; }

// `GgufFile::get_u64` -> `MetadataValue::as_u64` (unsigned types only), src/types.rs
int32_t agn_gguf_get_u64(const agn_gguf *g, const char *key, uint64_t *out) {
    const MetaValue *v = find_meta(g, key);
    if (!v || !out) return AGN_ENOTFOUND;
    if (v->type == 0 || v->type == 2 || v->type == 4 || v->type == 10) {
        *out = v->u;
        return AGN_OK;
    }
    return AGN_ENOTFOUND;
}

// `MetadataValue::as_f32`: Float32, or Float64 narrowed
int32_t agn_gguf_get_f32(const agn_gguf *g, const char *key, float *out) {
    const MetaValue *v = find_meta(g, key);
    if (!v || !out || (v->type != 6 && v->type != 12)) return AGN_ENOTFOUND;
    *out = (float)v->f;
    return AGN_OK;
}

// `GgufFile::get_string`; the pointer lives as long as the agn_gguf
int32_t agn_gguf_get_string(const agn_gguf *g, const char *key, const char **out) {
    const MetaValue *v = find_meta(g, key);
    if (!v || !out || v->type != 8) return AGN_ENOTFOUND;
    *out = v->s.c_str();
    return AGN_OK;
}

// arrays are indexed, not kept: element type id and length
int32_t agn_gguf_get_array_info(const agn_gguf *g, const char *key, uint32_t *elem_type, uint64_t *count) {
    const MetaValue *v = find_meta(g, key);
    if (!v || v->type != 9) return AGN_ENOTFOUND;
    if (elem_type) *elem_type = v->elem_type;
    if (count) *count = v->count;
    return AGN_OK;
}

// `GgufFile::get_i64_array` (src/types.rs:451-454): an array of integers of any width as i64.
// *count receives the array length; up to cap values are copied to out (out may be NULL to ask
// for the length only).  AGN_ENOTFOUND: no such key, not an array, or not an array of integers.
int32_t agn_gguf_get_array_i64(const agn_gguf *g, const char *key, int64_t *out, uint64_t cap, uint64_t *count) {
    const MetaValue *v = find_meta(g, key);
    if (!v || v->type != 9) return AGN_ENOTFOUND;
    const bool ints = v->elem_type <= 5 || v->elem_type == 10 || v->elem_type == 11;
    if (!ints || v->ints.size() != v->count) return AGN_ENOTFOUND;
    if (count) *count = v->count;
    if (out)
        for (uint64_t k = 0; k < v->count && k < cap; k++) out[k] = v->ints[(size_t)k];
    return AGN_OK;
}

int32_t agn_gguf_tensor_at(const agn_gguf *g, uint64_t index, agn_tensor_info *out) {
    if (!g || !out || index >= g->tensors.size()) return AGN_ENOTFOUND;
    const Tensor &t = g->tensors[(size_t)index];
    memset(out, 0, sizeof(*out));
    out->name = t.name.c_str();
    out->ggml_type = (int32_t)t.ggml_type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->dims[d] = t.dims[d];
    out->byte_offset = t.byte_offset;
    // dims and offsets are whatever the file says: a product or sum that does not fit 64 bits is a
    // malformed file (the reference's checked slices reject it, src/quant/mod.rs:124-131), never
    // a wrapped-around small number
    if (t.byte_offset > UINT64_MAX - g->data_offset) return AGN_EFORMAT;
    out->file_offset = g->data_offset + t.byte_offset;
    uint64_t rows = 1;
    for (uint32_t d = 1; d < t.n_dims; d++) {
        if (t.dims[d] != 0 && rows > UINT64_MAX / t.dims[d]) return AGN_EFORMAT;
        rows *= t.dims[d];
    }
    out->n_rows = t.n_dims <= 1 ? 1 : rows;
    out->row_len = t.n_dims >= 1 ? t.dims[0] : 0;
    if (out->row_len > (UINT64_MAX >> 4)) return AGN_EFORMAT;  // type_size rounds up to blocks of at most 256 bytes per value group
    out->row_bytes = agn_type_size((int32_t)t.ggml_type, (size_t)out->row_len);  // 0: no codec for this type
    if (out->n_rows != 0 && out->row_bytes > UINT64_MAX / out->n_rows) return AGN_EFORMAT;
    out->n_bytes = out->row_bytes * out->n_rows;
    return AGN_OK;
}

int32_t agn_gguf_find_tensor(const agn_gguf *g, const char *name, agn_tensor_info *out) {
    if (!g || !name || !out) return AGN_ENOTFOUND;
    for (size_t k = 0; k < g->tensors.size(); k++)
        if (g->tensors[k].name == name) return agn_gguf_tensor_at(g, k, out);
    return AGN_ENOTFOUND;
}

// Copies one tensor's bytes into a new device allocation (freed with agn_free).  The copy is
// stream-ordered on the context's stream and complete when the call returns.
int32_t agn_gguf_upload_tensor(agn_ctx *ctx, const agn_gguf *g, const char *name, void **dptr, agn_tensor_info *info) {
    AGN_CHECK_CTX(ctx);
    if (!g || !name || !dptr) return agn_fail(ctx, AGN_EINVAL, "agn_gguf_upload_tensor: null argument");
    *dptr = nullptr;
    agn_tensor_info ti;
    const int32_t frc = agn_gguf_find_tensor(g, name, &ti);
    if (frc == AGN_EFORMAT) return agn_fail(ctx, AGN_EFORMAT, "tensor '%s': dimensions or offset overflow 64 bits", name);
    if (frc != AGN_OK) return agn_fail(ctx, AGN_ENOTFOUND, "tensor '%s' not found", name);
    if (ti.row_bytes == 0)
        return agn_fail(ctx, AGN_EUNSUPPORTED_DTYPE, "tensor '%s' has ggml type %d, which has no codec here", name, ti.ggml_type);
    // "tensor row .. extends beyond data section", src/quant/mod.rs:124-131; in a split model the
    // bytes must lie inside one of the files (`MultiFileMmap::slice`, src/loader.rs:79-89)
    const uint8_t *src = g->slice(ti.file_offset, ti.n_bytes);
    if (!src)
        return agn_fail(ctx, AGN_EFORMAT, "tensor '%s' extends beyond the file or straddles two files (offset %llu + %llu bytes)",
                        name, (unsigned long long)ti.file_offset, (unsigned long long)ti.n_bytes);
    void *d = nullptr;
    int32_t rc = agn_malloc(ctx, (size_t)ti.n_bytes, &d);
    if (rc != AGN_OK) return rc;
    rc = agn_memcpy_h2d(ctx, d, src, (size_t)ti.n_bytes);
    if (rc == AGN_OK) rc = agn_sync(ctx);
    if (rc != AGN_OK) {
        agn_free(ctx, d);
        return rc;
    }
    *dptr = d;
    if (info) *info = ti;
    return AGN_OK;
}

// The tensor's bytes where they lie in the mapping (or in the caller's buffer): the slice
// `&raw_data[byte_offset .. byte_offset + byte_size]` the reference hands to its codecs
// (src/quant/mod.rs:97-135).  Valid until agn_gguf_close.
int32_t agn_gguf_tensor_data(const agn_gguf *g, const char *name, const void **data, uint64_t *n_bytes) {
    if (!g || !name || !data) return AGN_EINVAL;
    *data = nullptr;
    agn_tensor_info ti;
    const int32_t rc = agn_gguf_find_tensor(g, name, &ti);
    if (rc != AGN_OK) return rc;
    if (ti.row_bytes == 0) return AGN_EUNSUPPORTED_DTYPE;
    const uint8_t *src = g->slice(ti.file_offset, ti.n_bytes);
    if (!src) return AGN_EFORMAT;  // beyond the file, or astride two files of a split model
    *data = src;
    if (n_bytes) *n_bytes = ti.n_bytes;
    return AGN_OK;
}

// `release_mmap_prefix` (src/model/llama/gpu_resident.rs:29-49): drop the page-cache pages that lie
// wholly inside the file bytes [from, to) (start rounded up, end rounded down to page boundaries)
// with madvise(MADV_DONTNEED).  The mappings are read-only and file-backed, so a later access
// re-faults the page from disk: slower, never wrong.  *mark (may be null) receives the offset up to
// which pages are gone — the rounded-down end, what the reference returns for its next call — or
// `from` when no whole page lay inside the range.
static uint64_t release_range(const agn_gguf *g, uint64_t from, uint64_t to, uint64_t *mark) {
    if (mark) *mark = from;
    if (to <= from) return 0;
    long ps = sysconf(_SC_PAGESIZE);
    const uint64_t page = ps > 0 ? (uint64_t)ps : 4096u;
    uint64_t total = 0;
    auto release_in = [&](void *mapping, size_t len, uint64_t start) {  // one mapped file covering [start, start + len)
        if (!mapping) return;
        const uint64_t lo = from > start ? from : start, hi = to < start + len ? to : start + len;
        if (hi <= lo) return;
        // mmap returns page-aligned addresses: round the offsets inside the file
        const uint64_t o0 = (lo - start + page - 1) / page * page, o1 = (hi - start) / page * page;
        if (o1 > o0 && madvise(static_cast<uint8_t *>(mapping) + o0, (size_t)(o1 - o0), MADV_DONTNEED) == 0) {
            total += o1 - o0;
            if (mark && start + o1 > *mark) *mark = start + o1;
        }
    };
    release_in(g->mapping, g->map_len, 0);
    for (const agn_gguf::Part &p : g->parts) release_in(p.mapping, p.len, p.start);
    return total;
}

int32_t agn_gguf_release_pages(const agn_gguf *g, uint64_t from, uint64_t to, uint64_t *released_bytes) {
    if (released_bytes) *released_bytes = 0;
    if (!g) return AGN_EINVAL;
    const uint64_t got = release_range(g, from, to, nullptr);
    if (released_bytes) *released_bytes = got;
    return AGN_OK;
}

// The upload loop of `pre_upload_gpu` (src/model/llama/gpu_resident.rs:112-152): the named tensors
// are copied in ascending file-offset order, not in the order given, and — with release_pages — the
// part of the mapping that lies below the tensor just uploaded is dropped from the page cache, so
// that a file of about the size of host memory does not sit in the page cache next to its growing
// copy on the device.  Results are returned in the caller's order.
int32_t agn_gguf_upload_tensors(agn_ctx *ctx, const agn_gguf *g, const char *const *names, uint64_t n, void **dptrs,
                                agn_tensor_info *infos, int32_t release_pages, uint64_t *released_bytes) {
    AGN_CHECK_CTX(ctx);
    if (released_bytes) *released_bytes = 0;
    if (!g || (n && (!names || !dptrs))) return agn_fail(ctx, AGN_EINVAL, "agn_gguf_upload_tensors: null argument");
    std::vector<agn_tensor_info> ti(n);
    std::vector<uint64_t> order(n);
    for (uint64_t i = 0; i < n; i++) {
        dptrs[i] = nullptr;
        order[i] = i;
    }
    for (uint64_t i = 0; i < n; i++) {
        if (!names[i]) return agn_fail(ctx, AGN_EINVAL, "agn_gguf_upload_tensors: names[%llu] is null", (unsigned long long)i);
        const int32_t frc = agn_gguf_find_tensor(g, names[i], &ti[i]);
        if (frc == AGN_EFORMAT) return agn_fail(ctx, AGN_EFORMAT, "tensor '%s': dimensions or offset overflow 64 bits", names[i]);
        if (frc != AGN_OK) return agn_fail(ctx, AGN_ENOTFOUND, "tensor '%s' not found", names[i]);
    }
    for (uint64_t i = 1; i < n; i++)  // insertion sort by file offset (a few hundred names at most)
        for (uint64_t j = i; j > 0 && ti[order[j]].file_offset < ti[order[j - 1]].file_offset; j--) std::swap(order[j], order[j - 1]);
    uint64_t released_up_to = g->data_offset, total = 0;  // the header pages stay
    for (uint64_t k = 0; k < n; k++) {
        const uint64_t i = order[k];
        const int32_t rc = agn_gguf_upload_tensor(ctx, g, names[i], &dptrs[i], nullptr);
        if (rc != AGN_OK) {
            for (uint64_t j = 0; j < n; j++) {
                if (dptrs[j]) agn_free(ctx, dptrs[j]);
                dptrs[j] = nullptr;
            }
            return rc;
        }
        const uint64_t end = ti[i].file_offset + ti[i].n_bytes;
        if (release_pages && end > released_up_to) total += release_range(g, released_up_to, end, &released_up_to);
    }
    if (infos)
        for (uint64_t i = 0; i < n; i++) infos[i] = ti[i];
    if (released_bytes) *released_bytes = total;
    return AGN_OK;
}

}  // extern "C"
