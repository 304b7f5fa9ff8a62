// Torch-free, Python-free reader of the .rwkvq container (host code only).
//
// The container is a safetensors file: 8 bytes of little-endian header length, a JSON header
// {"<key>::<field>": {"dtype", "shape", "data_offsets"}, ..., "__metadata__": {"rwkvq": "<manifest
// JSON as a string>"}}, then the buffers.  The manifest names the model dimensions and, per
// tensor, kind / shape / bits / gw_gs / gw_sb / transposed / fields (formats/writer.py:111-139);
// reading rules as formats/codec.py:462-511 and formats/reader.py:42-93: a foreign container, a
// file without manifest and a format_version newer than 2 are refused.
//
// rwkvq_file_open maps the file read-only and indexes it; rwkvq_file_tensor hands out a
// rwkvq_qtensor whose pointers look into the mapping (host memory); rwkvq_file_upload copies
// one tensor's buffers into one device allocation and returns the descriptor the kernels take.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdlib>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "rwkvq_common.cuh"

namespace rwkvq {
namespace {

// ---- a small JSON reader (objects keep insertion order) -----------------------------------
struct JVal {
    enum Type { Null, Bool, Num, Str, Arr, Obj } t = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;
    const JVal* get(const char* key) const {
        if (t != Obj) return nullptr;
        for (const auto& kv : obj)
            if (kv.first == key) return &kv.second;
        return nullptr;
    }
    long long as_int(long long dflt = 0) const { return t == Num ? static_cast<long long>(num) : t == Bool ? b : dflt; }
};

struct JParser {
    const char* p;
    const char* end;
    bool ok = true;
    int depth = 0;
    void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
    bool lit(const char* s) {
        const size_t n = strlen(s);
        if (static_cast<size_t>(end - p) >= n && memcmp(p, s, n) == 0) { p += n; return true; }
        return false;
    }
    static void utf8(std::string& out, unsigned cp) {
        if (cp < 0x80) out += static_cast<char>(cp);
        else if (cp < 0x800) { out += static_cast<char>(0xC0 | (cp >> 6)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
        else if (cp < 0x10000) {
            out += static_cast<char>(0xE0 | (cp >> 12)); out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
            out += static_cast<char>(0x80 | (cp & 0x3F));
        } else {
            out += static_cast<char>(0xF0 | (cp >> 18)); out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
            out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); out += static_cast<char>(0x80 | (cp & 0x3F));
        }
    }
    bool hex4(unsigned& v) {
        if (end - p < 4) return false;
        v = 0;
        for (int i = 0; i < 4; ++i) {
            const char c = p[i];
            v <<= 4;
            if (c >= '0' && c <= '9') v |= c - '0';
            else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
            else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
            else return false;
        }
        p += 4;
        return true;
    }
    bool string(std::string& out) {
        if (p >= end || *p != '"') return ok = false;
        ++p;
        while (p < end && *p != '"') {
            if (*p != '\\') { out += *p++; continue; }
            if (++p >= end) return ok = false;
            const char c = *p++;
            switch (c) {
                case '"': out += '"'; break;
                case '\\': out += '\\'; break;
                case '/': out += '/'; break;
                case 'b': out += '\b'; break;
                case 'f': out += '\f'; break;
                case 'n': out += '\n'; break;
                case 'r': out += '\r'; break;
                case 't': out += '\t'; break;
                case 'u': {
                    unsigned cp;
                    if (!hex4(cp)) return ok = false;
                    if (cp >= 0xD800 && cp < 0xDC00 && end - p >= 6 && p[0] == '\\' && p[1] == 'u') {
                        p += 2;
                        unsigned lo;
                        if (!hex4(lo)) return ok = false;
                        cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
                    }
                    utf8(out, cp);
                    break;
                }
                default: return ok = false;
            }
        }
        if (p >= end) return ok = false;
        ++p;
        return true;
    }
    bool value(JVal& v) {
        if (++depth > 64) return ok = false;
        ws();
        if (p >= end) return ok = false;
        bool good = true;
        if (*p == '{') {
            v.t = JVal::Obj;
            ++p;
            ws();
            if (p < end && *p == '}') ++p;
            else
                for (;;) {
                    ws();
                    std::string k;
                    if (!string(k)) { good = false; break; }
                    ws();
                    if (p >= end || *p++ != ':') { good = false; break; }
                    v.obj.emplace_back(std::move(k), JVal());
                    if (!value(v.obj.back().second)) { good = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == '}') { ++p; break; }
                    good = false;
                    break;
                }
        } else if (*p == '[') {
            v.t = JVal::Arr;
            ++p;
            ws();
            if (p < end && *p == ']') ++p;
            else
                for (;;) {
                    v.arr.emplace_back();
                    if (!value(v.arr.back())) { good = false; break; }
                    ws();
                    if (p < end && *p == ',') { ++p; continue; }
                    if (p < end && *p == ']') { ++p; break; }
                    good = false;
                    break;
                }
        } else if (*p == '"') {
            v.t = JVal::Str;
            good = string(v.str);
        } else if (lit("true")) { v.t = JVal::Bool; v.b = true; }
        else if (lit("false")) { v.t = JVal::Bool; v.b = false; }
        else if (lit("null")) { v.t = JVal::Null; }
        else if (lit("NaN") || lit("Infinity") || lit("-Infinity")) { v.t = JVal::Num; v.num = 0; }   // Python's json emits these
        else {
            char* e = nullptr;
            std::string tmp(p, static_cast<size_t>(std::min<ptrdiff_t>(end - p, 64)));
            v.num = strtod(tmp.c_str(), &e);
            if (e == tmp.c_str()) good = false;
            else { v.t = JVal::Num; p += e - tmp.c_str(); }
        }
        --depth;
        if (!good) ok = false;
        return good;
    }
};

bool parse_json(const char* s, size_t n, JVal& out) {
    JParser ps{s, s + n};
    if (!ps.value(out)) return false;
    ps.ws();
    return ps.ok && ps.p == ps.end;
}


// ---- the indexed file ------------------------------------------------------------------------
struct Buffer {
    const unsigned char* ptr = nullptr;
    size_t bytes = 0;
    std::string dtype;
    std::vector<long long> shape;
};

struct TensorEntry {
    std::string key;
    int kind = 0, bits = 16, gs = 0, sb = 0;
    long long rows = 1, cols = 1;
    bool transposed = false;
    std::map<std::string, Buffer> fields;
    const Buffer* field(const char* name) const {
        auto it = fields.find(name);
        return it == fields.end() ? nullptr : &it->second;
    }
};

size_t dtype_size(const std::string& d) {
    if (d == "U8" || d == "I8" || d == "BOOL") return 1;
    if (d == "F16" || d == "BF16" || d == "I16" || d == "U16") return 2;
    if (d == "F32" || d == "I32" || d == "U32") return 4;
    if (d == "F64" || d == "I64" || d == "U64") return 8;
    return 0;
}

int kind_of(const std::string& k) {
    if (k == "dense") return RWKVQ_KIND_DENSE;
    if (k == "sb6") return RWKVQ_KIND_SB6;
    if (k == "sym") return RWKVQ_KIND_SYM;
    if (k == "asym") return RWKVQ_KIND_ASYM;
    if (k == "rtn") return RWKVQ_KIND_RTN;
    return -1;
}

}  // namespace
}  // namespace rwkvq

struct rwkvq_file {
    int fd = -1;
    unsigned char* map = nullptr;
    size_t size = 0;
    rwkvq_file_info info{};
    std::vector<rwkvq::TensorEntry> tensors;
    std::map<std::string, int> index;
};

namespace rwkvq {
namespace {

void release(rwkvq_file* f) {
    if (!f) return;
    if (f->map) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

// Host-pointer descriptor of one tensor; the codec's rule for which code buffer is present
// decides the branch, not `bits` (formats/codec.py:234-237).
int fill_view(const TensorEntry& t, rwkvq_qtensor* v) {
    memset(v, 0, sizeof(*v));
    v->kind = t.kind; v->bits = t.bits; v->gs = t.gs; v->sb = t.sb;
    v->rows = static_cast<int32_t>(t.rows); v->cols = static_cast<int32_t>(t.cols);
    auto ptr = [&](const char* name) -> const void* {
        const Buffer* b = t.field(name);
        return b ? b->ptr : nullptr;
    };
    switch (t.kind) {
        case RWKVQ_KIND_DENSE: v->codes = ptr("dense"); break;
        case RWKVQ_KIND_SB6:
            v->codes = ptr("codes_packed"); v->qh = ptr("gw_qh"); v->qh2 = ptr("gw_qh2");
            v->qsqm = ptr("gw_qsqm"); v->d = ptr("gw_d"); v->dm = ptr("gw_dm");
            break;
        case RWKVQ_KIND_SYM:
            v->codes = ptr("codes") ? ptr("codes") : ptr("codes_packed");
            v->qh = ptr("gw_qh"); v->qh2 = ptr("gw_qh2"); v->qs = ptr("gw_qs"); v->d = ptr("gw_d");
            break;
        case RWKVQ_KIND_ASYM: v->codes = ptr("codes"); v->scale = ptr("gw_scale"); v->mn = ptr("gw_min"); break;
        case RWKVQ_KIND_RTN:
            v->codes = ptr("codes") ? ptr("codes") : ptr("codes_packed");
            v->scale = ptr("scale");
            break;
        default: return fail(RWKVQ_E_DTYPE, "%s: unknown layout kind %d", t.key.c_str(), t.kind);
    }
    if (!v->codes) return fail(RWKVQ_E_FORMAT, "%s: the code buffer of its layout is missing", t.key.c_str());
    // The descriptor carries no buffer sizes, so every buffer the kernels will index is checked here
    // against the byte count its layout, bit width and manifest shape imply (formats/writer.py:236-337).
    const unsigned long long R = static_cast<unsigned long long>(t.rows), Cc = static_cast<unsigned long long>(t.cols);
    const unsigned long long n = R * Cc;
    int rc = RWKVQ_OK;
    auto need = [&](const char* name, unsigned long long bytes, bool required) {
        if (rc) return;
        const Buffer* b = t.field(name);
        if (!b) {
            if (required) rc = fail(RWKVQ_E_FORMAT, "%s: buffer %s of its layout is missing", t.key.c_str(), name);
            return;
        }
        if (b->bytes != bytes)
            rc = fail(RWKVQ_E_FORMAT, "%s: buffer %s holds %zu bytes, shape [%lld, %lld] at %d bits needs %llu",
                      t.key.c_str(), name, b->bytes, t.rows, t.cols, t.bits, bytes);
    };
    switch (t.kind) {
        case RWKVQ_KIND_DENSE: need("dense", n * 2, true); break;
        case RWKVQ_KIND_SB6: {
            if (t.gs <= 0 || t.sb <= 0 || Cc % (static_cast<unsigned long long>(t.gs) * t.sb))
                return fail(RWKVQ_E_FORMAT, "%s: %lld columns do not divide into groups of %d x %d", t.key.c_str(), t.cols, t.gs, t.sb);
            const unsigned long long nsb = Cc / (static_cast<unsigned long long>(t.gs) * t.sb);
            need("codes_packed", n / 2, true);
            need("gw_qh", n / 8, t.bits >= 5);
            need("gw_qh2", n / 8, t.bits >= 6);
            need("gw_qsqm", R * nsb * (static_cast<unsigned long long>(t.sb) * 12 / 8), true);
            need("gw_d", R * nsb * 2, true);
            need("gw_dm", R * nsb * 2, true);
            break;
        }
        case RWKVQ_KIND_SYM: {
            if (t.gs <= 0 || t.sb <= 0 || Cc % (static_cast<unsigned long long>(t.gs) * t.sb))
                return fail(RWKVQ_E_FORMAT, "%s: %lld columns do not divide into groups of %d x %d", t.key.c_str(), t.cols, t.gs, t.sb);
            if (t.field("codes")) need("codes", n, true);
            else {
                need("codes_packed", n / 2, true);
                need("gw_qh", n / 8, t.bits >= 5);
                need("gw_qh2", n / 8, t.bits >= 6);
            }
            need("gw_qs", R * (Cc / t.gs), true);
            need("gw_d", R * (Cc / (static_cast<unsigned long long>(t.gs) * t.sb)) * 2, true);
            break;
        }
        case RWKVQ_KIND_ASYM: {
            if (t.gs <= 0) return fail(RWKVQ_E_FORMAT, "%s: group size %d", t.key.c_str(), t.gs);
            const unsigned long long nb = (Cc + t.gs - 1) / t.gs;
            need("codes", n, true);
            need("gw_scale", R * nb * 4, true);
            need("gw_min", R * nb * 4, true);
            break;
        }
        default:   // per-row
            if (t.field("codes")) need("codes", n, true);
            else need("codes_packed", R * ((Cc + 1) / 2), true);
            need("scale", R * 2, true);
            break;
    }
    return rc;
}

}  // namespace
}  // namespace rwkvq

using namespace rwkvq;

extern "C" {

int rwkvq_file_open(const char* path, rwkvq_file** out) {
    RWKVQ_REQUIRE(path && out, RWKVQ_E_NULL, "rwkvq_file_open: null pointer");
    *out = nullptr;
    rwkvq_file* f = new rwkvq_file();
    auto bail = [&](int code, const char* what) {
        release(f);
        return fail(code, "%s: %s", path, what);
    };
    f->fd = open(path, O_RDONLY);
    if (f->fd < 0) return bail(RWKVQ_E_FORMAT, "cannot open");
    struct stat st;
    if (fstat(f->fd, &st) != 0 || st.st_size < 8) return bail(RWKVQ_E_FORMAT, "truncated file");
    f->size = static_cast<size_t>(st.st_size);
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { f->map = nullptr; return bail(RWKVQ_E_FORMAT, "mmap failed"); }
    f->map = static_cast<unsigned char*>(m);
    if (memcmp(f->map, "PK\x03\x04", 4) == 0)
        return bail(RWKVQ_E_FORMAT, "legacy pickle (torch.save) container; only the safetensors container is supported");
    unsigned long long n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | f->map[i];
    if (n > f->size - 8) return bail(RWKVQ_E_FORMAT, "unreadable safetensors header (length beyond the file)");
    JVal header;
    if (!parse_json(reinterpret_cast<const char*>(f->map + 8), static_cast<size_t>(n), header) || header.t != JVal::Obj)
        return bail(RWKVQ_E_FORMAT, "unreadable safetensors header");
    const JVal* meta = header.get("__metadata__");
    const JVal* mj = meta ? meta->get("rwkvq") : nullptr;
    if (!mj || mj->t != JVal::Str) return bail(RWKVQ_E_FORMAT, "not a .rwkvq file (no rwkvq manifest)");
    JVal man;
    if (!parse_json(mj->str.data(), mj->str.size(), man) || man.t != JVal::Obj) return bail(RWKVQ_E_FORMAT, "unreadable manifest");
    const JVal* fmt = man.get("format");
    if (!fmt || fmt->t != JVal::Str || fmt->str != "rwkvq") return bail(RWKVQ_E_FORMAT, "manifest format is not 'rwkvq'");
    const JVal* ver = man.get("format_version");
    f->info.format_version = ver ? static_cast<int32_t>(ver->as_int()) : 0;
    if (f->info.format_version > 2) return bail(RWKVQ_E_FORMAT, "format_version is newer than this reader understands (2)");
    const JVal* naming = man.get("naming");
    f->info.naming = naming && naming->t == JVal::Str && naming->str == "custom" ? 1 : 0;
    auto geti = [&](const char* k) { const JVal* v = man.get(k); return v ? static_cast<int32_t>(v->as_int()) : 0; };
    f->info.n_layer = geti("n_layer"); f->info.n_embd = geti("n_embd");
    f->info.head_size = geti("head_size"); f->info.vocab_size = geti("vocab_size");
    const JVal* tensors = man.get("tensors");
    if (!tensors || tensors->t != JVal::Obj) return bail(RWKVQ_E_FORMAT, "manifest has no tensor table");
    const unsigned char* data = f->map + 8 + n;
    const size_t data_bytes = f->size - 8 - static_cast<size_t>(n);
    for (const auto& kv : tensors->obj) {
        TensorEntry t;
        t.key = kv.first;
        const JVal& e = kv.second;
        const JVal* kind = e.get("kind");
        t.kind = kind && kind->t == JVal::Str ? kind_of(kind->str) : -1;
        if (t.kind < 0) return bail(RWKVQ_E_FORMAT, "a tensor has an unknown layout kind");
        const JVal* v;
        t.bits = (v = e.get("bits")) ? static_cast<int>(v->as_int()) : 16;
        t.gs = (v = e.get("gw_gs")) ? static_cast<int>(v->as_int()) : 0;
        t.sb = (v = e.get("gw_sb")) ? static_cast<int>(v->as_int()) : 0;
        if ((v = e.get("transposed"))) t.transposed = v->as_int() != 0;
        else {
            // version-1 manifests: world checkpoints keep blocks.N.att.{w,a,v,g}{1,2} as [in, out]
            const size_t dot = t.key.rfind('.');
            const std::string last = dot == std::string::npos ? t.key : t.key.substr(dot + 1);
            t.transposed = f->info.naming == 0 && t.key.find(".att.") != std::string::npos && last.size() == 2 &&
                           strchr("wavg", last[0]) && (last[1] == '1' || last[1] == '2');
        }
        const JVal* shape = e.get("shape");
        if (shape && shape->t == JVal::Arr && !shape->arr.empty()) {
            t.cols = shape->arr.back().as_int(1);
            for (size_t i = 0; i + 1 < shape->arr.size(); ++i) t.rows *= shape->arr[i].as_int(1);
        }
        if (t.rows < 1 || t.cols < 1 || t.rows > INT32_MAX || t.cols > INT32_MAX) return bail(RWKVQ_E_FORMAT, "a tensor has an unusable shape");
        const JVal* fields = e.get("fields");
        if (!fields || fields->t != JVal::Arr) return bail(RWKVQ_E_FORMAT, "a tensor lists no fields");
        for (const JVal& fn : fields->arr) {
            if (fn.t != JVal::Str) return bail(RWKVQ_E_FORMAT, "a field name is not a string");
            const std::string name = t.key + "::" + fn.str;
            const JVal* h = header.get(name.c_str());
            const JVal* off = h ? h->get("data_offsets") : nullptr;
            const JVal* dt = h ? h->get("dtype") : nullptr;
            const JVal* shp = h ? h->get("shape") : nullptr;
            if (!off || off->t != JVal::Arr || off->arr.size() != 2 || !dt || dt->t != JVal::Str || !shp || shp->t != JVal::Arr)
                return bail(RWKVQ_E_FORMAT, "a buffer named by the manifest is missing from the safetensors header");
            const long long b = off->arr[0].as_int(-1), en = off->arr[1].as_int(-1);
            if (b < 0 || en < b || static_cast<size_t>(en) > data_bytes) return bail(RWKVQ_E_FORMAT, "a buffer lies outside the file");
            Buffer buf;
            buf.ptr = data + b;
            buf.bytes = static_cast<size_t>(en - b);
            buf.dtype = dt->str;
            size_t count = 1;
            for (const JVal& d : shp->arr) { buf.shape.push_back(d.as_int()); count *= static_cast<size_t>(d.as_int()); }
            if (dtype_size(buf.dtype) == 0 || count * dtype_size(buf.dtype) != buf.bytes)
                return bail(RWKVQ_E_FORMAT, "a buffer's dtype and shape do not match its size");
            t.fields.emplace(fn.str, std::move(buf));
        }
        f->index[t.key] = static_cast<int>(f->tensors.size());
        f->tensors.push_back(std::move(t));
    }
    f->info.n_tensors = static_cast<int32_t>(f->tensors.size());
    *out = f;
    return RWKVQ_OK;
}

void rwkvq_file_close(rwkvq_file* f) { release(f); }

int rwkvq_file_get_info(const rwkvq_file* f, rwkvq_file_info* out) {
    RWKVQ_REQUIRE(f && out, RWKVQ_E_NULL, "rwkvq_file_get_info: null pointer");
    *out = f->info;
    return RWKVQ_OK;
}

const char* rwkvq_file_tensor_key(const rwkvq_file* f, int index) {
    if (!f || index < 0 || index >= static_cast<int>(f->tensors.size())) return nullptr;
    return f->tensors[index].key.c_str();
}

int rwkvq_file_tensor(const rwkvq_file* f, const char* key, rwkvq_qtensor* host_view, int32_t* transposed,
                      const void** outlier_indices, const void** outlier_values, int64_t* n_outliers) {
    RWKVQ_REQUIRE(f && key && host_view, RWKVQ_E_NULL, "rwkvq_file_tensor: null pointer");
    auto it = f->index.find(key);
    RWKVQ_REQUIRE(it != f->index.end(), RWKVQ_E_FORMAT, "rwkvq_file_tensor: no tensor named %s", key);
    const TensorEntry& t = f->tensors[it->second];
    const int rc = fill_view(t, host_view);
    if (rc) return rc;
    if (transposed) *transposed = t.transposed ? 1 : 0;
    const Buffer* oi = t.field("outlier_indices");
    const Buffer* ov = t.field("outlier_values");
    const bool has = oi && ov && oi->bytes > 0;
    if (has) {
        RWKVQ_REQUIRE(oi->dtype == "I32" && ov->dtype == "BF16" && oi->bytes == 4 * ov->bytes, RWKVQ_E_FORMAT,
                      "%s: outlier buffers are not int32 [n, 2] + bf16 [n]", key);
        const int32_t* rc2 = reinterpret_cast<const int32_t*>(oi->ptr);      // an override outside the tensor would
        for (size_t i = 0; i < ov->bytes / 2; ++i)                           // become a stray device write
            RWKVQ_REQUIRE(rc2[2 * i] >= 0 && rc2[2 * i] < t.rows && rc2[2 * i + 1] >= 0 && rc2[2 * i + 1] < t.cols,
                          RWKVQ_E_FORMAT, "%s: outlier %zu at (%d, %d) lies outside the [%lld, %lld] tensor", key, i,
                          rc2[2 * i], rc2[2 * i + 1], t.rows, t.cols);
    }
    if (outlier_indices) *outlier_indices = has ? oi->ptr : nullptr;
    if (outlier_values) *outlier_values = has ? ov->ptr : nullptr;
    if (n_outliers) *n_outliers = has ? static_cast<int64_t>(ov->bytes / 2) : 0;
    return RWKVQ_OK;
}

int rwkvq_file_upload(const rwkvq_file* f, const char* key, rwkvq_qtensor* dev_view, void** slab, void* stream) {
    RWKVQ_REQUIRE(f && key && dev_view && slab, RWKVQ_E_NULL, "rwkvq_file_upload: null pointer");
    *slab = nullptr;
    auto it = f->index.find(key);
    RWKVQ_REQUIRE(it != f->index.end(), RWKVQ_E_FORMAT, "rwkvq_file_upload: no tensor named %s", key);
    const TensorEntry& t = f->tensors[it->second];
    rwkvq_qtensor host;
    int rc = fill_view(t, &host);
    if (rc) return rc;
    // which file buffer backs each pointer of the descriptor
    struct Slot { const void* rwkvq_qtensor::*member; const void* host_ptr; size_t bytes; size_t off; };
    std::vector<Slot> slots;
    size_t total = 0;
    auto add = [&](const void* rwkvq_qtensor::*member) {
        const void* hp = host.*member;
        if (!hp) return;
        for (const auto& kv : t.fields)
            if (kv.second.ptr == hp) {
                slots.push_back({member, hp, kv.second.bytes, total});
                total += (kv.second.bytes + 255) / 256 * 256;
                return;
            }
    };
    add(&rwkvq_qtensor::codes); add(&rwkvq_qtensor::qh); add(&rwkvq_qtensor::qh2); add(&rwkvq_qtensor::qsqm);
    add(&rwkvq_qtensor::qs); add(&rwkvq_qtensor::d); add(&rwkvq_qtensor::dm); add(&rwkvq_qtensor::scale);
    add(&rwkvq_qtensor::mn);
    RWKVQ_REQUIRE(total > 0, RWKVQ_E_FORMAT, "rwkvq_file_upload: %s has no bytes", key);
    void* dev = nullptr;
    cudaError_t e = cudaMalloc(&dev, total);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_file_upload(%s, %zu bytes): %s", key, total, cudaGetErrorString(e));
    *dev_view = host;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (const Slot& sl : slots) {
        char* dst = static_cast<char*>(dev) + sl.off;
        if (sl.bytes) e = cudaMemcpyAsync(dst, sl.host_ptr, sl.bytes, cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) {
            cudaFree(dev);
            return fail(RWKVQ_E_LAUNCH, "rwkvq_file_upload(%s): %s", key, cudaGetErrorString(e));
        }
        dev_view->*(sl.member) = dst;
    }
    *slab = dev;
    return RWKVQ_OK;
}

int rwkvq_file_free_slab(void* slab) {
    cudaError_t e = cudaFree(slab);
    if (e != cudaSuccess) return fail(RWKVQ_E_LAUNCH, "rwkvq_file_free_slab: %s", cudaGetErrorString(e));
    return RWKVQ_OK;
}

}  // extern "C"
