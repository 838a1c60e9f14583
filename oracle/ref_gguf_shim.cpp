// Test infrastructure, not product code.
//
// Re-exports the reference's own GGUF reader (class Gguf, src/model/gguf.h:28-79,
// compiled from src/model/gguf.cpp where the reference checkout lies) through a
// C ABI, so that the CPU tests can hold the library's reader against it on the
// same files. Nothing from the reference is copied here.
#include "model/gguf.h"

#include <cstring>

using fastllm::Gguf;
using fastllm::GgufTensor;

extern "C" {

// Null when the file does not exist (Gguf::open returns false). Malformed files abort
// inside the reference, so the tests hand this only well-formed ones.
void *flref_gguf_open(const char *path) {
    Gguf *g = new Gguf();
    if (!g->open(path)) {
        delete g;
        return nullptr;
    }
    return g;
}

void flref_gguf_close(void *h) { delete (Gguf *)h; }

void flref_gguf_counts(void *h, uint32_t *n_tensors, uint32_t *n_shards, uint32_t *alignment) {
    const Gguf *g = (const Gguf *)h;
    *n_tensors = (uint32_t)g->tensors().size();
    *n_shards = (uint32_t)g->n_shards();
    *alignment = g->alignment();
}

// Tensor i in the reader's order. fmt = the Fmt value Gguf::fmt_of gives, -1 when it has none.
void flref_gguf_tensor(void *h, uint32_t i, char *name, size_t cap, uint32_t *type, int32_t *n_dims, uint64_t *ne,
                       uint64_t *offset, uint64_t *nbytes, int32_t *shard, int32_t *fmt, const uint8_t **data) {
    const Gguf *g = (const Gguf *)h;
    const GgufTensor &t = g->tensors()[i];
    strncpy(name, t.name.c_str(), cap - 1);
    name[cap - 1] = 0;
    *type = t.type;
    *n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) ne[d] = t.ne[d];
    *offset = t.offset;
    *nbytes = t.nbytes;
    *shard = t.shard;
    fastllm::Fmt f;
    *fmt = Gguf::fmt_of(t.type, &f) ? (int32_t)f : -1;
    *data = g->data(t);
}

// Index of the tensor Gguf::find returns for `name`, -1 when there is none.
int64_t flref_gguf_find(void *h, const char *name) {
    const Gguf *g = (const Gguf *)h;
    const GgufTensor *t = g->find(name);
    return t ? (int64_t)(t - g->tensors().data()) : -1;
}

int flref_gguf_has(void *h, const char *k) { return ((const Gguf *)h)->has(k) ? 1 : 0; }
int64_t flref_gguf_kv_i(void *h, const char *k, int64_t d) { return ((const Gguf *)h)->kv_i(k, d); }
double flref_gguf_kv_f(void *h, const char *k, double d) { return ((const Gguf *)h)->kv_f(k, d); }

size_t flref_gguf_kv_s(void *h, const char *k, const char *d, char *out, size_t cap) {
    const std::string s = ((const Gguf *)h)->kv_s(k, d);
    if (cap) {
        const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        memcpy(out, s.data(), n);
        out[n] = 0;
    }
    return s.size();
}

int64_t flref_gguf_kv_sarr_count(void *h, const char *k) {
    const auto *v = ((const Gguf *)h)->kv_sarr(k);
    return v ? (int64_t)v->size() : -1;
}

size_t flref_gguf_kv_sarr_at(void *h, const char *k, uint64_t i, char *out, size_t cap) {
    const std::string &s = (*((const Gguf *)h)->kv_sarr(k))[i];
    if (cap) {
        const size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
        memcpy(out, s.data(), n);
        out[n] = 0;
    }
    return s.size();
}

} // extern "C"
