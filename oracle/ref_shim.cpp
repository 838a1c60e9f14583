// Test infrastructure, not product code.
//
// Re-exports the reference's own CPU implementation of the decode hot path
// through a C ABI, so that the parity tests and the CPU-baseline leg of the
// benchmark can call it from Python. Nothing from the reference is copied
// here: its headers are included from where the reference checkout lies
// (-I<reference>/include -I<reference>/src -I<reference>/src/runtime) and its
// graph.cpp / arena.cpp / runtime.cpp / shadow.cpp are compiled next to this
// file by oracle/Makefile with the reference's own flags
// (-O2 -ffp-contract=off, CMakeLists.txt:13, src/runtime/CMakeLists.txt:14).
//
// What is exported, and the reference symbol each one calls:
//   ops table (flref_ops)     fl_half2float / fl_float2half (quants.h:40,:333),
//                             dequant_chunk (kernels.h:162), a STREAM_DOT Task
//                             through exec_task_scalar_host (graph.cpp:13),
//                             fl_op_* (decode_params.h:101-295)
//   flref_stream_dot_tasks    Graph/run_serial (graph.cpp:116) or the CPU worker
//                             pool Runtime with gpu_enabled=false
//                             (runtime.cpp:178-292), tiles of `rowsz` rows as
//                             the reference's builder emits (decoder.cpp:610-635)
//   flref_dot_row_fast        dot_row_fast_dequant (kernels.h:244-254)
#include "fastllm/fastllm.h"
#include "runtime_internal.h"
#include "kernels.h"
#include "flo_ops.h"

#include <cstdio>
#include <cstring>
#include <memory>
#include <vector>

using namespace fastllm;

namespace {

float r_h2f(uint16_t h) { return fl_half2float(h); }
uint16_t r_f2h(float f) { return fl_float2half(f); }

void r_dequant(int fmt, const uint8_t *row, uint32_t elem0, uint32_t n, float *out) {
    dequant_chunk((Fmt)fmt, row, elem0, n, out);
}

void r_stream_dot(int fmt, const uint8_t *w, uint32_t rows, uint32_t cols,
                  const float *x, uint32_t nx, uint32_t xstride,
                  float *y, uint32_t ystride) {
    Task t{};
    t.kind = TaskKind::STREAM_DOT;
    t.fmt = (Fmt)fmt;
    t.w = w;
    t.w_bytes = (uint64_t)rows * fl_row_bytes((Fmt)fmt, cols);
    t.x = x;
    t.y = y;
    t.rows = rows;
    t.cols = cols;
    t.nx = nx ? nx : 1;
    t.xstride = xstride;
    t.ystride = ystride;
    exec_task_scalar_host(t);
}

void r_rmsnorm(const float *wnorm, const float *x, float *y, float eps, uint32_t n) {
    RmsNormP p{wnorm, x, y, eps, n};
    Task t{};
    t.kind = TaskKind::RMSNORM;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_add2(const float *a, const float *b, float *y, uint32_t n) {
    Add2P p{a, b, y, n};
    Task t{};
    t.kind = TaskKind::ADD2;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_rope(float *buf, int32_t pos, uint32_t n_head, uint32_t head_stride,
            uint32_t rot_off, uint32_t n_rot, float freq_base) {
    RopeP p{};
    p.buf = buf;
    p.pos = &pos;
    p.n_head = n_head;
    p.head_stride = head_stride;
    p.rot_off = rot_off;
    p.n_rot = n_rot;
    p.freq_base = freq_base;
    p.freq_scale = 1.0f;
    p.ext_factor = 0.0f;
    p.attn_factor = 1.0f;
    p.beta_fast = 32.0f;
    p.beta_slow = 1.0f;
    p.n_ctx_orig = 8192;
    Task t{};
    t.kind = TaskKind::ROPE_DS2;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_kv_append(const float *kvb, float *kcache, float *vcache, int32_t pos,
                 uint32_t n_head, uint32_t d_k, uint32_t d_v, uint32_t max_kv) {
    KvAppendP p{};
    p.kvb = kvb;
    p.kpe = nullptr;
    p.kcache = kcache;
    p.vcache = vcache;
    p.pos = &pos;
    p.n_head = n_head;
    p.d_nope = d_k;
    p.d_rope = 0;
    p.d_v = d_v;
    p.max_kv = max_kv;
    Task t{};
    t.kind = TaskKind::KV_APPEND;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_attn_head(const float *q, const float *kcache, const float *vcache,
                 float *scratch, float *out, int32_t pos, float scale,
                 uint32_t head, uint32_t n_head, uint32_t dk, uint32_t dv,
                 uint32_t max_kv) {
    AttnHeadP p{};
    p.q = q;
    p.kcache = kcache;
    p.vcache = vcache;
    p.scratch = scratch;
    p.out = out;
    p.pos = &pos;
    p.scale = scale;
    p.head = head;
    p.n_head = n_head;
    p.dk = dk;
    p.dv = dv;
    p.max_kv = max_kv;
    Task t{};
    t.kind = TaskKind::ATTN_HEAD;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_silu_mul(const float *gate, const float *up, float *h, uint32_t n) {
    SiluMulP p{gate, up, h, n};
    Task t{};
    t.kind = TaskKind::SILU_MUL;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_router_sel(const float *logits, uint32_t *ids, float *gates,
                  uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale) {
    RouterP p{logits, ids, gates, n_expert, top_k, norm, scale};
    Task t{};
    t.kind = TaskKind::ROUTER_SEL;
    t.aux = &p;
    exec_task_scalar_host(t);
}

void r_wmerge(const float *parts, const float *gates, const float *add1,
              const float *add2, float *y, float scale, uint32_t n_parts, uint32_t n) {
    WmergeP p{};
    p.parts = parts;
    p.gates = gates;
    p.add1 = add1;
    p.add2 = add2;
    p.y = y;
    p.scale = scale;
    p.n_parts = n_parts;
    p.n = n;
    p.n_full = 0;
    Task t{};
    t.kind = TaskKind::WMERGE;
    t.aux = &p;
    exec_task_scalar_host(t);
}

const flo_ops_t kOps = {
    "reference", r_h2f, r_f2h, r_dequant, r_stream_dot, r_rmsnorm, r_add2, r_rope,
    r_kv_append, r_attn_head, r_silu_mul, r_router_sel, r_wmerge,
};

// One worker pool per thread count, kept alive between calls like the
// reference's decoder keeps its Runtime (decoder.cpp:668-671).
struct Pool {
    std::unique_ptr<Arena> arena;
    std::unique_ptr<Runtime> rt;
    int threads = 0;
    bool fast = false;
};
Pool g_pool;

Runtime *pool_for(int threads, bool fast) {
    if (g_pool.rt && g_pool.threads == threads && g_pool.fast == fast)
        return g_pool.rt.get();
    g_pool.rt.reset();
    g_pool.arena = Arena::create((size_t)64 << 20);
    RuntimeConfig cfg;
    cfg.cpu_threads = threads;
    cfg.gpu_enabled = false;
    cfg.fast_kernels = fast;
    cfg.collect_handoff = false;
    g_pool.rt = Runtime::create(*g_pool.arena, cfg);
    g_pool.rt->start();
    g_pool.threads = threads;
    g_pool.fast = fast;
    return g_pool.rt.get();
}

} // namespace

extern "C" {

const flo_ops_t *flref_ops(void) { return &kOps; }

// The f32 fast path the reference's CPU pool runs with fast_kernels=true.
float flref_dot_row_fast(int fmt, const uint8_t *row, const float *x, uint32_t cols) {
    return dot_row_fast_dequant((Fmt)fmt, row, x, cols);
}

float flref_dot_row(int fmt, const uint8_t *row, const float *x, uint32_t cols) {
    return fl_dot_row_any((Fmt)fmt, row, x, cols);
}

// y[p*ystride + r] += W[r] . x[p] through the reference's task graph:
// row tiles of `rowsz` rows, one SIGNAL sink. threads <= 0: run_serial;
// threads >= 1: the CPU worker pool (Runtime, gpu_enabled=false).
// Returns the wall time of the run in nanoseconds (RunMetrics::wall_ns).
uint64_t flref_stream_dot_tasks(int fmt, const uint8_t *w, uint32_t rows, uint32_t cols,
                                const float *x, uint32_t nx, uint32_t xstride,
                                float *y, uint32_t ystride,
                                uint32_t rowsz, int threads, int fast) {
    if (rowsz == 0) rowsz = 192;
    const uint32_t n_tiles = (rows + rowsz - 1) / rowsz;
    auto arena = Arena::create(sizeof(Task) * (size_t)(n_tiles + 2) + 4096);
    auto g = Graph::create(*arena, n_tiles + 1);
    const uint64_t rb = fl_row_bytes((Fmt)fmt, cols);
    Task sig{};
    sig.kind = TaskKind::SIGNAL;
    std::vector<uint32_t> ids;
    for (uint32_t r0 = 0; r0 < rows; r0 += rowsz) {
        const uint32_t nr = rows - r0 < rowsz ? rows - r0 : rowsz;
        Task t{};
        t.kind = TaskKind::STREAM_DOT;
        t.affinity = Engine::CPU;
        t.fmt = (Fmt)fmt;
        t.w = w + (size_t)r0 * rb;
        t.w_bytes = (uint64_t)nr * rb;
        t.x = x;
        t.y = y + r0;
        t.rows = nr;
        t.cols = cols;
        t.nx = nx ? nx : 1;
        t.xstride = xstride;
        t.ystride = ystride;
        ids.push_back(g->add(t));
    }
    const uint32_t s = g->add(sig);
    for (uint32_t id : ids) g->edge(id, s);
    g->freeze();
    RunMetrics m;
    if (threads <= 0) m = run_serial(*g);
    else m = pool_for(threads, fast != 0)->run(*g);
    return m.wall_ns;
}

void flref_pool_shutdown(void) {
    g_pool.rt.reset();
    g_pool.arena.reset();
    g_pool.threads = 0;
}

} // extern "C"
