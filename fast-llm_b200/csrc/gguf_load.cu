// GGUF model files -> decoder. The reader mirrors what class Gguf gives the
// reference's decoder (src/model/gguf.h:28-79, src/model/gguf.cpp:133-266):
// versions 2 and 3, every metadata scalar kept as int64 or double, strings and
// string arrays kept, other arrays skipped, per-file alignment, split models.
// Where the reference aborts on a malformed file this reader returns a status;
// it also refuses payloads that run past the end of their file.
//
// The loader half creates the Llama-shape decoder from a file: each tensor is
// copied once from the mapping to device memory (the tensor-parallel slices are
// cut by the copy itself), so nothing is staged on the host.
#include "capi_internal.h"

#include <cctype>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <fcntl.h>
#include <map>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

using namespace flb;

namespace {

constexpr uint32_t kMagic = 0x46554747u;   // "GGUF", little endian
// value type ids of the metadata section
enum : uint32_t { V_U8 = 0, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STR, V_ARR, V_U64, V_I64, V_F64 };

struct Mapping {
    int fd = -1;
    const uint8_t *base = nullptr;
    size_t size = 0;
    uint64_t data_off = 0;
};

struct TensorRec {
    std::string name;
    uint32_t type = 0, n_dims = 0, shard = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0, nbytes = 0;
};

struct Truncated {};   // thrown by the reader below, caught in map_file

// Bounds-checked little-endian reader over one mapping.
struct Reader {
    const uint8_t *p, *end;
    void need(uint64_t n) const { if ((uint64_t)(end - p) < n) throw Truncated(); }
    template <typename T> T get() {
        need(sizeof(T));
        T v;
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        need(n);
        std::string s((const char *)p, (size_t)n);
        p += n;
        return s;
    }
    void skip(uint64_t n) { need(n); p += n; }
};

uint32_t scalar_bytes(uint32_t t) {
    switch (t) {
    case V_U8: case V_I8: case V_BOOL: return 1;
    case V_U16: case V_I16: return 2;
    case V_U32: case V_I32: case V_F32: return 4;
    case V_U64: case V_I64: case V_F64: return 8;
    default: return 0;
    }
}

// Skips one array value (element type and count follow); arrays may nest, up to kMaxArrayDepth levels (a nested
// level costs 12 bytes of input, so an unbounded depth would let a small file exhaust the stack).
constexpr int kMaxArrayDepth = 4;
bool skip_array(Reader &r, std::vector<std::string> *keep_strings, int depth = 0) {
    if (depth >= kMaxArrayDepth) return false;
    const uint32_t et = r.get<uint32_t>();
    const uint64_t n = r.get<uint64_t>();
    if (et == V_STR) {
        if (keep_strings) keep_strings->reserve((size_t)std::min<uint64_t>(n, 1u << 20));
        for (uint64_t i = 0; i < n; ++i) {
            std::string s = r.str();
            if (keep_strings) keep_strings->push_back(std::move(s));
        }
        return true;
    }
    if (et == V_ARR) {
        for (uint64_t i = 0; i < n; ++i)
            if (!skip_array(r, nullptr, depth + 1)) return false;
        return true;
    }
    const uint32_t sz = scalar_bytes(et);
    if (!sz) return false;
    if (n > (uint64_t)(r.end - r.p) / sz) throw Truncated();
    r.skip(n * sz);
    return true;
}

int fmt_of_ggml(uint32_t t) {
    switch (t) {
    case FL_B200_GGML_F32: return FL_B200_F32;
    case FL_B200_GGML_Q8_0: return FL_B200_Q8_0;
    case FL_B200_GGML_Q5_0: return FL_B200_Q5_0;
    case FL_B200_GGML_Q4_K: return FL_B200_Q4_K;
    case FL_B200_GGML_Q6_K: return FL_B200_Q6_K;
    case FL_B200_GGML_IQ2_XXS: return 5;
    case FL_B200_GGML_IQ3_XXS: return 6;
    default: return -1;
    }
}

// Bytes of one row in any format the reference knows (fl_row_bytes, src/runtime/quants.h:97-99); the two
// IQ formats have 256-weight blocks of 66 and 98 bytes.
uint64_t any_row_bytes(int fmt, uint64_t cols) {
    if (fmt == 5) return cols / 256 * 66;
    if (fmt == 6) return cols / 256 * 98;
    return row_bytes(fmt, (uint32_t)cols);
}

} // namespace

struct fl_b200_gguf {
    std::vector<Mapping> shards;
    std::vector<TensorRec> tensors;
    std::map<std::string, int64_t> ints;
    std::map<std::string, double> floats;
    std::map<std::string, std::string> strings;
    std::map<std::string, std::vector<std::string>> string_arrays;
    uint32_t alignment = 32;
    ~fl_b200_gguf() {
        for (Mapping &m : shards) {
            if (m.base) munmap((void *)m.base, m.size);
            if (m.fd >= 0) close(m.fd);
        }
    }
};

namespace {

// "<stem>-NNNNN-of-MMMMM.gguf": the number of parts and a printf pattern for the siblings; 0 = not split.
int split_pattern(const std::string &path, std::string *pattern) {
    static const char kExt[] = ".gguf";
    const size_t ext = sizeof(kExt) - 1, tag = 15;   // "-NNNNN-of-MMMMM"
    if (path.size() < ext + tag || path.compare(path.size() - ext, ext, kExt) != 0) return 0;
    const size_t at = path.size() - ext - tag;
    const char *t = path.c_str() + at;
    if (t[0] != '-' || strncmp(t + 6, "-of-", 4) != 0) return 0;
    for (int i = 1; i <= 5; ++i)
        if (!isdigit((unsigned char)t[i]) || !isdigit((unsigned char)t[9 + i])) return 0;
    const int total = atoi(t + 10);
    if (total < 1 || total > 999) return 0;
    *pattern = path.substr(0, at) + "-%05d-of-" + path.substr(at + 10, 5) + kExt;
    return total;
}

// Maps one file and appends its tensors; only the file the caller named contributes metadata.
int map_file(fl_b200_gguf *g, const std::string &path, bool keep_meta) {
    Mapping m;
    m.fd = open(path.c_str(), O_RDONLY);
    if (m.fd < 0) return set_err(FL_B200_ERR_IO, "gguf: cannot open %s", path.c_str());
    struct stat st {};
    if (fstat(m.fd, &st) != 0 || st.st_size <= 0) {
        close(m.fd);
        return set_err(FL_B200_ERR_IO, "gguf: cannot stat %s", path.c_str());
    }
    m.size = (size_t)st.st_size;
    void *mem = mmap(nullptr, m.size, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (mem == MAP_FAILED) {
        close(m.fd);
        return set_err(FL_B200_ERR_IO, "gguf: cannot map %s", path.c_str());
    }
    m.base = (const uint8_t *)mem;
    const uint32_t shard = (uint32_t)g->shards.size();
    g->shards.push_back(m);   // owned from here on: closed by the destructor on every path

    fl_b200_gguf scratch;     // metadata of the other shards is parsed and dropped
    fl_b200_gguf *meta = keep_meta ? g : &scratch;
    uint32_t align = 32;
    try {
        Reader r{m.base, m.base + m.size};
        if (r.get<uint32_t>() != kMagic) return set_err(FL_B200_ERR_FORMAT, "gguf: %s: bad magic", path.c_str());
        const uint32_t version = r.get<uint32_t>();
        if (version < 2 || version > 3) return set_err(FL_B200_ERR_FORMAT, "gguf: %s: unsupported version %u", path.c_str(), version);
        const uint64_t n_tensors = r.get<uint64_t>();
        const uint64_t n_kv = r.get<uint64_t>();
        for (uint64_t i = 0; i < n_kv; ++i) {
            const std::string key = r.str();
            const uint32_t t = r.get<uint32_t>();
            switch (t) {
            case V_U8: meta->ints[key] = r.get<uint8_t>(); break;
            case V_I8: meta->ints[key] = r.get<int8_t>(); break;
            case V_BOOL: meta->ints[key] = r.get<uint8_t>() != 0; break;
            case V_U16: meta->ints[key] = r.get<uint16_t>(); break;
            case V_I16: meta->ints[key] = r.get<int16_t>(); break;
            case V_U32: meta->ints[key] = r.get<uint32_t>(); break;
            case V_I32: meta->ints[key] = r.get<int32_t>(); break;
            case V_U64: meta->ints[key] = (int64_t)r.get<uint64_t>(); break;
            case V_I64: meta->ints[key] = r.get<int64_t>(); break;
            case V_F32: meta->floats[key] = r.get<float>(); break;
            case V_F64: meta->floats[key] = r.get<double>(); break;
            case V_STR: meta->strings[key] = r.str(); break;
            case V_ARR: {
                // peek at the element type: only string arrays are kept
                Reader look = r;
                const bool strings = look.get<uint32_t>() == V_STR;
                if (!skip_array(r, strings ? &meta->string_arrays[key] : nullptr))
                    return set_err(FL_B200_ERR_FORMAT, "gguf: %s: bad element type or more than %d nested levels in array '%s'",
                                   path.c_str(), kMaxArrayDepth, key.c_str());
                break;
            }
            default:
                return set_err(FL_B200_ERR_FORMAT, "gguf: %s: bad value type %u for '%s'", path.c_str(), t, key.c_str());
            }
            if (key == "general.alignment") {   // a per-file property: each shard pads with its own
                auto it = meta->ints.find(key);
                if (it != meta->ints.end() && it->second > 0) align = (uint32_t)it->second;
            }
        }
        if (align & (align - 1)) return set_err(FL_B200_ERR_FORMAT, "gguf: %s: alignment %u is not a power of two", path.c_str(), align);
        if (keep_meta) g->alignment = align;
        if (n_tensors > m.size / 24) throw Truncated();   // an info record is longer than that
        const size_t first = g->tensors.size();
        g->tensors.reserve(first + (size_t)n_tensors);
        for (uint64_t i = 0; i < n_tensors; ++i) {
            TensorRec t;
            t.name = r.str();
            t.n_dims = r.get<uint32_t>();
            if (t.n_dims < 1 || t.n_dims > 4) return set_err(FL_B200_ERR_FORMAT, "gguf: %s: tensor '%s' has %u dimensions", path.c_str(), t.name.c_str(), t.n_dims);
            for (uint32_t d = 0; d < t.n_dims; ++d) t.ne[d] = r.get<uint64_t>();
            t.type = r.get<uint32_t>();
            t.offset = r.get<uint64_t>();
            const int fmt = fmt_of_ggml(t.type);
            // sizes with checked arithmetic: a wrapped product could pass the runs-past-the-end check below
            uint64_t outer = 0, row = 0;
            bool bad = t.ne[0] > UINT32_MAX;   // row_bytes takes 32-bit column counts
            bad = bad || __builtin_mul_overflow(t.ne[1], t.ne[2], &outer) || __builtin_mul_overflow(outer, t.ne[3], &outer);
            if (!bad) {
                if (fmt >= 0) row = any_row_bytes(fmt, t.ne[0]);
                else if (t.type == FL_B200_GGML_F16) row = 2 * t.ne[0];
                // any other type has no kernels: visible in the listing with nbytes 0, payload unusable
                bad = __builtin_mul_overflow(row, outer, &t.nbytes);
            }
            if (bad)
                return set_err(FL_B200_ERR_FORMAT, "gguf: %s: tensor '%s' has dimensions whose size does not fit 64 bits",
                               path.c_str(), t.name.c_str());
            t.shard = shard;
            g->tensors.push_back(std::move(t));
        }
        const uint64_t meta_end = (uint64_t)(r.p - m.base);
        g->shards[shard].data_off = (meta_end + align - 1) & ~(uint64_t)(align - 1);
        const uint64_t room = g->shards[shard].data_off <= m.size ? m.size - g->shards[shard].data_off : 0;
        for (size_t i = first; i < g->tensors.size(); ++i) {
            const TensorRec &t = g->tensors[i];
            if (t.offset > room || t.nbytes > room - t.offset)
                return set_err(FL_B200_ERR_FORMAT, "gguf: %s: tensor '%s' runs past the end of the file", path.c_str(), t.name.c_str());
        }
    } catch (const Truncated &) {
        return set_err(FL_B200_ERR_FORMAT, "gguf: %s: truncated file", path.c_str());
    } catch (const std::exception &e) {   // bad_alloc / length_error from a string or vector a hostile count asked for
        return set_err(FL_B200_ERR_FORMAT, "gguf: %s: %s while reading the metadata", path.c_str(), e.what());
    }
    return FL_B200_OK;
}

void fill_info(const fl_b200_gguf *g, const TensorRec &t, fl_b200_gguf_tensor *o) {
    o->fmt = fmt_of_ggml(t.type);
    o->ggml_type = t.type;
    o->n_dims = t.n_dims;
    o->shard = t.shard;
    for (int d = 0; d < 4; ++d) o->ne[d] = t.ne[d];
    o->offset = t.offset;
    o->nbytes = t.nbytes;
    const Mapping &m = g->shards[t.shard];
    o->data = m.base + m.data_off + t.offset;
}

const TensorRec *find_rec(const fl_b200_gguf *g, const char *name) {
    for (const TensorRec &t : g->tensors)
        if (t.name == name) return &t;
    return nullptr;
}

int copy_string(const std::string &s, char *out, size_t cap, size_t *len_out) {
    if (len_out) *len_out = s.size();
    if (out && cap) {
        const size_t n = std::min(cap - 1, s.size());
        memcpy(out, s.data(), n);
        out[n] = 0;
    }
    return FL_B200_OK;
}

} // namespace

extern "C" {

int fl_b200_gguf_open(const char *path, fl_b200_gguf **out) {
    if (!path || !out) return set_err(FL_B200_ERR_ARG, "gguf_open: null pointer");
    *out = nullptr;
    fl_b200_gguf *g = nullptr;
    int rc = FL_B200_OK;
    try {
    g = new fl_b200_gguf();
    std::string pattern;
    const int parts = split_pattern(path, &pattern);
    if (parts <= 1) {
        rc = map_file(g, path, true);
    } else {
        char name[1024];
        for (int i = 1; i <= parts && rc == FL_B200_OK; ++i) {
            snprintf(name, sizeof name, pattern.c_str(), i);
            rc = map_file(g, name, strcmp(name, path) == 0);
        }
        const auto want = g->ints.find("split.tensors.count");
        if (rc == FL_B200_OK && want != g->ints.end() && want->second > 0 && (int64_t)g->tensors.size() != want->second)
            rc = set_err(FL_B200_ERR_FORMAT, "gguf: split.tensors.count = %lld but the shards hold %zu tensors",
                         (long long)want->second, g->tensors.size());
    }
    } catch (const std::exception &e) {   // nothing may cross the C boundary
        rc = set_err(FL_B200_ERR_IO, "gguf_open: %s", e.what());
    }
    if (rc != FL_B200_OK) {
        delete g;
        return rc;
    }
    *out = g;
    return FL_B200_OK;
}

void fl_b200_gguf_close(fl_b200_gguf *g) { delete g; }

int fl_b200_gguf_counts(const fl_b200_gguf *g, uint32_t *n_tensors, uint32_t *n_shards, uint32_t *alignment) {
    if (!g) return set_err(FL_B200_ERR_ARG, "gguf_counts: null");
    if (n_tensors) *n_tensors = (uint32_t)g->tensors.size();
    if (n_shards) *n_shards = (uint32_t)g->shards.size();
    if (alignment) *alignment = g->alignment;
    return FL_B200_OK;
}

int fl_b200_gguf_tensor_at(const fl_b200_gguf *g, uint32_t index, char *name_out, size_t cap, fl_b200_gguf_tensor *info) {
    if (!g || index >= g->tensors.size()) return set_err(FL_B200_ERR_ARG, "gguf_tensor_at: index out of range");
    const TensorRec &t = g->tensors[index];
    copy_string(t.name, name_out, cap, nullptr);
    if (info) fill_info(g, t, info);
    return FL_B200_OK;
}

int fl_b200_gguf_find(const fl_b200_gguf *g, const char *name, fl_b200_gguf_tensor *info) {
    if (!g || !name) return set_err(FL_B200_ERR_ARG, "gguf_find: null");
    const TensorRec *t = find_rec(g, name);
    if (!t) return set_err(FL_B200_ERR_ARG, "gguf: no tensor '%s'", name);
    if (info) fill_info(g, *t, info);
    return FL_B200_OK;
}

int fl_b200_gguf_has(const fl_b200_gguf *g, const char *key) {
    if (!g || !key) return 0;
    return (g->ints.count(key) || g->floats.count(key) || g->strings.count(key) || g->string_arrays.count(key)) ? 1 : 0;
}

int64_t fl_b200_gguf_kv_i(const fl_b200_gguf *g, const char *key, int64_t dflt) {
    if (!g || !key) return dflt;
    const auto i = g->ints.find(key);
    if (i != g->ints.end()) return i->second;
    const auto f = g->floats.find(key);
    return f != g->floats.end() ? (int64_t)f->second : dflt;
}

double fl_b200_gguf_kv_f(const fl_b200_gguf *g, const char *key, double dflt) {
    if (!g || !key) return dflt;
    const auto f = g->floats.find(key);
    if (f != g->floats.end()) return f->second;
    const auto i = g->ints.find(key);
    return i != g->ints.end() ? (double)i->second : dflt;
}

int fl_b200_gguf_kv_s(const fl_b200_gguf *g, const char *key, const char *dflt, char *out, size_t cap, size_t *len_out) {
    if (!g || !key) return set_err(FL_B200_ERR_ARG, "gguf_kv_s: null");
    const auto s = g->strings.find(key);
    return copy_string(s != g->strings.end() ? s->second : std::string(dflt ? dflt : ""), out, cap, len_out);
}

int64_t fl_b200_gguf_kv_sarr_count(const fl_b200_gguf *g, const char *key) {
    if (!g || !key) return -1;
    const auto a = g->string_arrays.find(key);
    return a == g->string_arrays.end() ? -1 : (int64_t)a->second.size();
}

int fl_b200_gguf_kv_sarr_at(const fl_b200_gguf *g, const char *key, uint64_t i, char *out, size_t cap, size_t *len_out) {
    if (!g || !key) return set_err(FL_B200_ERR_ARG, "gguf_kv_sarr_at: null");
    const auto a = g->string_arrays.find(key);
    if (a == g->string_arrays.end() || i >= a->second.size()) return set_err(FL_B200_ERR_ARG, "gguf_kv_sarr_at: '%s'[%llu] does not exist", key, (unsigned long long)i);
    return copy_string(a->second[(size_t)i], out, cap, len_out);
}

int fl_b200_gguf_llama_cfg(const fl_b200_gguf *g, uint32_t max_kv, fl_b200_llama_cfg *cfg) {
    if (!g || !cfg) return set_err(FL_B200_ERR_ARG, "gguf_llama_cfg: null");
    const auto arch = g->strings.find("general.architecture");
    if (arch == g->strings.end() || arch->second != "llama")
        return set_err(FL_B200_ERR_FORMAT, "gguf: architecture '%s' (the decoder runs 'llama' files)",
                       arch == g->strings.end() ? "" : arch->second.c_str());
    auto I = [&](const char *k, int64_t d) { return fl_b200_gguf_kv_i(g, (std::string("llama.") + k).c_str(), d); };
    auto F = [&](const char *k, double d) { return fl_b200_gguf_kv_f(g, (std::string("llama.") + k).c_str(), d); };
    fl_b200_llama_cfg c{};
    c.n_embd = (uint32_t)I("embedding_length", 0);
    c.n_layer = (uint32_t)I("block_count", 0);
    c.n_head = (uint32_t)I("attention.head_count", 0);
    c.n_kv_head = (uint32_t)I("attention.head_count_kv", c.n_head);
    c.n_ff = (uint32_t)I("feed_forward_length", 0);
    c.eps = (float)F("attention.layer_norm_rms_epsilon", 1e-5);
    c.rope_base = (float)F("rope.freq_base", 10000.0);
    if (!c.n_embd || !c.n_layer || !c.n_head || !c.n_ff)
        return set_err(FL_B200_ERR_FORMAT, "gguf: llama.embedding_length / block_count / attention.head_count / feed_forward_length missing");
    c.head_dim = (uint32_t)I("attention.key_length", c.n_embd / c.n_head);
    if ((uint32_t)I("attention.value_length", c.head_dim) != c.head_dim || (uint32_t)I("rope.dimension_count", c.head_dim) != c.head_dim)
        return set_err(FL_B200_ERR_FORMAT, "gguf: key, value and rotary sizes differ (one head size is built)");
    const auto scaling = g->strings.find("llama.rope.scaling.type");
    if ((scaling != g->strings.end() && scaling->second != "none") || find_rec(g, "rope_freqs.weight"))
        return set_err(FL_B200_ERR_FORMAT, "gguf: the file asks for RoPE scaling, which the decoder does not apply");
    const TensorRec *emb = find_rec(g, "token_embd.weight");
    if (!emb) return set_err(FL_B200_ERR_FORMAT, "gguf: no token_embd.weight");
    c.n_vocab = (uint32_t)emb->ne[1];
    c.max_kv = max_kv;
    *cfg = c;
    return FL_B200_OK;
}

} // extern "C"

namespace {

// One tensor of the file, checked against the shape the decoder expects.
struct Wanted {
    const TensorRec *t = nullptr;
    int fmt = -1;
    const uint8_t *host = nullptr;
};

int want_tensor(const fl_b200_gguf *g, const std::string &name, uint64_t cols, uint64_t rows, bool matrix, Wanted *w) {
    const TensorRec *t = find_rec(g, name.c_str());
    if (!t) return set_err(FL_B200_ERR_FORMAT, "gguf: missing %s", name.c_str());
    const int fmt = fmt_of_ggml(t->type);
    if (matrix ? (fmt != FL_B200_Q4_K && fmt != FL_B200_Q6_K && fmt != FL_B200_Q8_0) : fmt != FL_B200_F32)
        return set_err(FL_B200_ERR_FORMAT, "gguf: %s has ggml type %u (matrices: Q4_K, Q6_K or Q8_0; norms: F32)", name.c_str(), t->type);
    if (t->ne[0] != cols || t->ne[1] != rows || t->ne[2] != 1 || t->ne[3] != 1)
        return set_err(FL_B200_ERR_FORMAT, "gguf: %s is %llu x %llu, expected %llu x %llu", name.c_str(),
                       (unsigned long long)t->ne[1], (unsigned long long)t->ne[0], (unsigned long long)rows, (unsigned long long)cols);
    const Mapping &m = g->shards[t->shard];
    *w = {t, fmt, m.base + m.data_off + t->offset};
    return FL_B200_OK;
}

// Rows [row0, row0 + rows) and columns [col0, col0 + cols) of a packed tensor with `full_cols` columns, copied
// to fresh device memory the decoder owns. A column range becomes rows zero-padded to a multiple of 16 bytes.
int upload_slice(fl_b200_decoder *d, const Wanted &w, uint64_t full_cols, uint64_t row0, uint64_t rows,
                 uint64_t col0, uint64_t cols, void **dev_out) {
    const uint64_t rb = row_bytes(w.fmt, (uint32_t)full_cols);
    const uint8_t *src = w.host + row0 * rb;
    void *dev = nullptr;
    if (col0 == 0 && cols == full_cols) {
        if (cudaError_t e = cudaMalloc(&dev, rows * rb)) return cuda_err(e, "cudaMalloc (weights)");
        decoder_adopt(d, dev);
        if (cudaError_t e = cudaMemcpy(dev, src, rows * rb, cudaMemcpyHostToDevice)) return cuda_err(e, "weight upload");
    } else {
        const uint32_t be = blk_elems(w.fmt), bb = blk_bytes(w.fmt);
        const uint64_t width = cols / be * bb, pitch = (width + 15) & ~(uint64_t)15;
        if (cudaError_t e = cudaMalloc(&dev, rows * pitch)) return cuda_err(e, "cudaMalloc (weights)");
        decoder_adopt(d, dev);
        if (cudaError_t e = cudaMemset(dev, 0, rows * pitch)) return cuda_err(e, "cudaMemset (weights)");
        if (cudaError_t e = cudaMemcpy2D(dev, pitch, src + col0 / be * bb, rb, width, rows, cudaMemcpyHostToDevice))
            return cuda_err(e, "weight upload (column slice)");
    }
    *dev_out = dev;
    return FL_B200_OK;
}

} // namespace

extern "C" int fl_b200_decoder_create_gguf(fl_b200_ctx *ctx, const fl_b200_gguf *g, uint32_t max_kv, uint32_t rank,
                                           uint32_t world, fl_b200_decoder **out) {
    if (!ctx || !g || !out) return set_err(FL_B200_ERR_ARG, "decoder_create_gguf: null pointer");
    *out = nullptr;
    fl_b200_llama_cfg c{};
    if (int rc = fl_b200_gguf_llama_cfg(g, max_kv, &c)) return rc;
    fl_b200_decoder *d = nullptr;
    if (int rc = fl_b200_decoder_create_tp(ctx, &c, rank, world, &d)) return rc;
    auto fail = [&](int rc) { fl_b200_decoder_destroy(d); return rc; };
    if (cudaError_t e = cudaSetDevice(ctx->device)) return fail(cuda_err(e, "cudaSetDevice"));

    const uint64_t E = c.n_embd, D = c.head_dim, QD = (uint64_t)c.n_head * D, KD = (uint64_t)c.n_kv_head * D;
    const uint64_t F = c.n_ff, V = c.n_vocab;
    // this rank's share: whole KV heads with their query heads, FFN rows, vocabulary rows
    const uint64_t qd = QD / world, kd = KD / world, f = F / world, v = V / world;
    struct Spec { const char *name; int which; uint64_t cols, rows, row0, nrows, col0, ncols; };
    const Spec specs[7] = {
        {"attn_q", FL_B200_T_WQ, E, QD, rank * qd, qd, 0, E},
        {"attn_k", FL_B200_T_WK, E, KD, rank * kd, kd, 0, E},
        {"attn_v", FL_B200_T_WV, E, KD, rank * kd, kd, 0, E},
        {"attn_output", FL_B200_T_WO, QD, E, 0, E, rank * qd, qd},
        {"ffn_gate", FL_B200_T_GATE, E, F, rank * f, f, 0, E},
        {"ffn_up", FL_B200_T_UP, E, F, rank * f, f, 0, E},
        {"ffn_down", FL_B200_T_DOWN, F, E, 0, E, rank * f, f},
    };
    char name[96];
    Wanted w;
    void *dev = nullptr;
    auto upload_norm = [&](const char *nm, const float **dev_norm) -> int {
        if (int rc = want_tensor(g, nm, E, 1, false, &w)) return rc;
        if (int rc = upload_slice(d, w, E, 0, 1, 0, E, &dev)) return rc;
        *dev_norm = (const float *)dev;
        return FL_B200_OK;
    };
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        for (const Spec &s : specs) {
            snprintf(name, sizeof name, "blk.%u.%s.weight", l, s.name);
            if (int rc = want_tensor(g, name, s.cols, s.rows, true, &w)) return fail(rc);
            if (int rc = upload_slice(d, w, s.cols, s.row0, s.nrows, s.col0, s.ncols, &dev)) return fail(rc);
            if (int rc = fl_b200_decoder_set_layer_tensor(d, l, s.which, w.fmt, dev)) return fail(rc);
        }
        const float *an = nullptr, *fn = nullptr;
        snprintf(name, sizeof name, "blk.%u.attn_norm.weight", l);
        if (int rc = upload_norm(name, &an)) return fail(rc);
        snprintf(name, sizeof name, "blk.%u.ffn_norm.weight", l);
        if (int rc = upload_norm(name, &fn)) return fail(rc);
        if (int rc = fl_b200_decoder_set_layer_norms(d, l, an, fn)) return fail(rc);
    }
    const float *on = nullptr;
    if (int rc = upload_norm("output_norm.weight", &on)) return fail(rc);
    if (int rc = fl_b200_decoder_set_out_norm(d, on)) return fail(rc);
    // the embedding table is whole on every rank; the head is split by rows (and is the embedding table again
    // when the file ties them)
    if (int rc = want_tensor(g, "token_embd.weight", E, V, true, &w)) return fail(rc);
    if (int rc = upload_slice(d, w, E, 0, V, 0, E, &dev)) return fail(rc);
    if (int rc = fl_b200_decoder_set_global(d, FL_B200_G_TOK_EMBD, w.fmt, dev)) return fail(rc);
    const bool tied = find_rec(g, "output.weight") == nullptr;
    if (!tied)
        if (int rc = want_tensor(g, "output.weight", E, V, true, &w)) return fail(rc);
    if (!tied || world > 1)
        if (int rc = upload_slice(d, w, E, rank * v, v, 0, E, &dev)) return fail(rc);
    if (int rc = fl_b200_decoder_set_global(d, FL_B200_G_OUTPUT, w.fmt, dev)) return fail(rc);
    *out = d;
    return FL_B200_OK;
}
