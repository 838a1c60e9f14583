// Mixture-of-experts feed-forward block of the decode graph, single GPU or expert
// parallel over the GPUs of one box. Per token: router logits (f32 matvec),
// ROUTER_SEL (fl_op_router_sel, src/runtime/decode_params.h:234-265), the chosen
// experts' gate / up / down through the expert-indexed matvec (STREAM_DOT_IDX,
// src/runtime/runtime_internal.h:149-152) with the SiLU product between them, and
// WMERGE (fl_op_wmerge, :274-295); the reference builds the same chain as tasks
// (src/model/decoder.cpp:925-1045) and has no multi-GPU form.
//
// The tokens of a block are grouped by expert on the device (a stable counting sort of the (token, slot)
// pairs), and each of this rank's experts is walked ONCE per block: gate, up and down run as multi-column
// matmuls (matvec_tc_nx.cu) over the tokens that chose the expert, up to 8 per pass, with the token list
// and its length read on the device (an expert nobody chose costs launches that return at entry, no
// weight traffic). The reference describes the same grouping for its task graph ("one tile set per
// DISTINCT expert serving every position that routed to it", src/model/decoder.cpp:927-930).
//
// Expert parallel: rank r of w holds experts [r * n / w, (r + 1) * n / w). The hidden states are
// replicated, so the dispatch half of the all-to-all moves nothing: every rank routes every token, runs
// only its own experts, merges with the other slots' gates set to zero, and the ranks' partial outputs
// are summed through peer memory by the exchange kernel of the tensor-parallel decoder (rank order, so
// every rank ends with identical bits). That sum is the combine half.
#include "capi_internal.h"

#include <cstdlib>

using namespace flb;

struct fl_b200_moe {
    fl_b200_ctx *ctx = nullptr;
    fl_b200_moe_cfg c{};
    uint32_t rank = 0, world = 1, n_local = 0, base = 0;
    const float *router = nullptr;
    const uint8_t *wg = nullptr, *wu = nullptr, *wd = nullptr;
    float *logits = nullptr, *gates = nullptr, *mgates = nullptr, *g = nullptr, *u = nullptr, *part = nullptr, *partial = nullptr;
    uint32_t *ids = nullptr, *lids = nullptr;
    uint32_t *cnt = nullptr, *tok_list = nullptr, *pair_list = nullptr;   // the pairs grouped by local expert (launch_group_by_expert)
    uint8_t *comm = nullptr;
    uint8_t *peers[kCommMaxRanks] = {};
    bool peers_set = false;
    uint32_t *comm_state = nullptr;
    // The launches of one forward call, recorded as a CUDA graph the second time a call repeats the
    // (x, y, n_tok) of the one before it, and replayed from then on (about 10 launches per token otherwise
    // cost more host time than the kernels take).
    struct { const float *x = nullptr; float *y = nullptr; uint32_t n_tok = 0; cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr; } rec;
};

namespace {

// Router logits of all tokens in one launch: logits[t][e] = dot(router[e], x[t]); one block per (expert, token).
// wnorm != nullptr: x is the raw hidden state and the logits are those of RMSNorm(x) * wnorm (fl_op_rmsnorm,
// src/runtime/decode_params.h:101-106, fused: every block norms the token itself).
__global__ void __launch_bounds__(128) router_logits_kernel(const float *__restrict__ router, const float *__restrict__ x,
                                                            float *__restrict__ logits, uint32_t n_embd, uint32_t n_expert,
                                                            const float *__restrict__ wnorm = nullptr, float eps = 0.f) {
    __shared__ float red[4];
    const uint32_t e = blockIdx.x, t = blockIdx.y;
    const float4 *w = reinterpret_cast<const float4 *>(router + (size_t)e * n_embd);
    const float4 *v = reinterpret_cast<const float4 *>(x + (size_t)t * n_embd);
    float inv_rms = 1.f;
    if (wnorm) {
        float ss = 0.f;
        for (uint32_t i = threadIdx.x; i < n_embd / 4; i += 128) {
            const float4 b = v[i];
            ss += (b.x * b.x + b.y * b.y) + (b.z * b.z + b.w * b.w);
        }
        ss = warp_sum(ss);
        if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        inv_rms = 1.0f / sqrtf(((red[0] + red[1]) + (red[2] + red[3])) / (float)n_embd + eps);
        __syncthreads();
    }
    float acc = 0.f;
    for (uint32_t i = threadIdx.x; i < n_embd / 4; i += 128) {
        const float4 a = w[i];
        float4 b = v[i];
        if (wnorm) {
            const float4 g = reinterpret_cast<const float4 *>(wnorm)[i];
            b.x = b.x * inv_rms * g.x; b.y = b.y * inv_rms * g.y; b.z = b.z * inv_rms * g.z; b.w = b.w * inv_rms * g.w;
        }
        acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) logits[(size_t)t * n_expert + e] = (red[0] + red[1]) + (red[2] + red[3]);
}

#define CKM(call)                                                      \
    do {                                                               \
        cudaError_t e_ = (call);                                       \
        if (e_ != cudaSuccess) return cuda_err(e_, #call);             \
    } while (0)

} // namespace

extern "C" {

int fl_b200_moe_create(fl_b200_ctx *ctx, const fl_b200_moe_cfg *cfg, uint32_t rank, uint32_t world, fl_b200_moe **out) {
    if (!ctx || !cfg || !out) return set_err(FL_B200_ERR_ARG, "moe_create: null pointer");
    const fl_b200_moe_cfg &c = *cfg;
    if (world == 0 || world > kCommMaxRanks || rank >= world) return set_err(FL_B200_ERR_ARG, "moe_create: rank %u of %u", rank, world);
    if (c.n_expert == 0 || c.n_expert > 256 || c.top_k == 0 || c.top_k > c.n_expert || c.n_expert % world)
        return set_err(FL_B200_ERR_ARG, "moe_create: %u experts, top %u, %u ranks", c.n_expert, c.top_k, world);
    if (c.n_embd % 256 || c.n_ff % 256 || c.n_embd < 512 || c.n_ff < 512 || c.max_tokens == 0)
        return set_err(FL_B200_ERR_ARG, "moe_create: n_embd and n_ff must be multiples of 256 (>= 512), max_tokens > 0");
    if (c.n_embd > 18432 || c.n_ff > 18432)
        return set_err(FL_B200_ERR_ARG, "moe_create: n_embd / n_ff above 18432 (the streaming matvec's column limit)");
    if (world > 1 && (c.n_embd > kCommMaxVec || c.n_embd % (4 * kCommChunks)))
        return set_err(FL_B200_ERR_ARG, "moe_create: n_embd %u does not fit the exchange buffer", c.n_embd);
    for (int fmt : {c.fmt_gate_up, c.fmt_down})
        if (fmt != FL_B200_Q4_K && fmt != FL_B200_Q6_K) return set_err(FL_B200_ERR_ARG, "moe_create: expert format %d (Q4_K or Q6_K)", fmt);
    CKM(cudaSetDevice(ctx->device));
    fl_b200_moe *m = new fl_b200_moe();
    m->ctx = ctx; m->c = c; m->rank = rank; m->world = world;
    m->n_local = c.n_expert / world;
    m->base = rank * m->n_local;
    const size_t T = c.max_tokens, K = c.top_k, E = c.n_embd, F = c.n_ff;
    auto fail = [&](int rc) { fl_b200_moe_destroy(m); return rc; };
    auto alloc = [&](void **p, size_t bytes) -> int {
        if (cudaError_t e = cudaMalloc(p, bytes)) return cuda_err(e, "cudaMalloc (moe)");
        if (cudaError_t e = cudaMemsetAsync(*p, 0, bytes, ctx->stream)) return cuda_err(e, "cudaMemsetAsync (moe)");
        return FL_B200_OK;
    };
    // zero-filled: a slot that is skipped leaves its buffer as it was, and what is there is then multiplied by gate 0
    if (int rc = alloc((void **)&m->logits, T * c.n_expert * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->gates, T * K * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->mgates, T * K * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->ids, T * K * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->lids, T * K * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->g, T * K * F * 4)) return fail(rc);   // gate / up outputs, one row per (token, slot) pair
    if (int rc = alloc((void **)&m->u, T * K * F * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->cnt, (size_t)m->n_local * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->tok_list, (size_t)m->n_local * T * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->pair_list, (size_t)m->n_local * T * 4)) return fail(rc);
    if (int rc = alloc((void **)&m->part, T * K * E * 4)) return fail(rc);
    if (world > 1) {
        if (int rc = alloc((void **)&m->partial, T * E * 4)) return fail(rc);
        if (int rc = alloc((void **)&m->comm, comm_buffer_bytes())) return fail(rc);
        if (int rc = alloc((void **)&m->comm_state, 64)) return fail(rc);
    }
    CKM(cudaStreamSynchronize(ctx->stream));
    *out = m;
    return FL_B200_OK;
}

void fl_b200_moe_destroy(fl_b200_moe *m) {
    if (!m) return;
    cudaSetDevice(m->ctx->device);
    cudaStreamSynchronize(m->ctx->stream);
    cudaFree(m->logits); cudaFree(m->gates); cudaFree(m->mgates); cudaFree(m->ids); cudaFree(m->lids); cudaFree(m->g);
    cudaFree(m->cnt); cudaFree(m->tok_list); cudaFree(m->pair_list);
    cudaFree(m->u); cudaFree(m->part); cudaFree(m->partial); cudaFree(m->comm); cudaFree(m->comm_state);
    if (m->rec.exec) cudaGraphExecDestroy(m->rec.exec);
    if (m->rec.graph) cudaGraphDestroy(m->rec.graph);
    delete m;
}

int fl_b200_moe_set_weights(fl_b200_moe *m, const float *router, const void *gate, const void *up, const void *down) {
    if (!m || !router || !gate || !up || !down) return set_err(FL_B200_ERR_ARG, "moe_set_weights: null pointer");
    if (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)down | (uintptr_t)router) & 15u)
        return set_err(FL_B200_ERR_ARG, "moe_set_weights: tensors must be 16-byte aligned");
    m->router = router;
    m->wg = (const uint8_t *)gate; m->wu = (const uint8_t *)up; m->wd = (const uint8_t *)down;
    return FL_B200_OK;
}

int fl_b200_moe_comm(fl_b200_moe *m, void **buf, size_t *bytes) {
    if (!m || !buf || !bytes) return set_err(FL_B200_ERR_ARG, "moe_comm: null");
    *buf = m->comm;
    *bytes = m->comm ? comm_buffer_bytes() : 0;
    return FL_B200_OK;
}

int fl_b200_moe_set_peers(fl_b200_moe *m, void *const *bufs, uint32_t n) {
    if (!m || !bufs) return set_err(FL_B200_ERR_ARG, "moe_set_peers: null");
    if (n != m->world) return set_err(FL_B200_ERR_ARG, "moe_set_peers: %u buffers for %u ranks", n, m->world);
    for (uint32_t p = 0; p < n; ++p) {
        if (!bufs[p]) return set_err(FL_B200_ERR_ARG, "moe_set_peers: buffer of rank %u is null", p);
        m->peers[p] = (uint8_t *)bufs[p];
    }
    if (m->world > 1 && m->peers[m->rank] != m->comm) return set_err(FL_B200_ERR_ARG, "moe_set_peers: entry %u must be this rank's own buffer", m->rank);
    m->peers_set = true;
    return FL_B200_OK;
}

static int moe_enqueue(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y);

int fl_b200_moe_forward(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y) {
    if (!m || !x || !y) return set_err(FL_B200_ERR_ARG, "moe_forward: null pointer");
    if (!m->router) return set_err(FL_B200_ERR_STATE, "moe_forward: set the weights first");
    if (m->world > 1 && !m->peers_set) return set_err(FL_B200_ERR_STATE, "moe_forward: set the peers' exchange buffers first");
    if (n_tok == 0 || n_tok > m->c.max_tokens) return set_err(FL_B200_ERR_ARG, "moe_forward: %u tokens outside 1..%u", n_tok, m->c.max_tokens);
    cudaStream_t s = m->ctx->stream;
    CKM(cudaSetDevice(m->ctx->device));
    auto &rec = m->rec;
    const bool same = rec.x == x && rec.y == y && rec.n_tok == n_tok;
    if (same && rec.exec) {
        CKM(cudaGraphLaunch(rec.exec, s));
        return FL_B200_OK;
    }
    if (rec.exec) { cudaGraphExecDestroy(rec.exec); rec.exec = nullptr; }
    if (rec.graph) { cudaGraphDestroy(rec.graph); rec.graph = nullptr; }
    if (!same) {   // first sight of this call: run it directly
        rec.x = x; rec.y = y; rec.n_tok = n_tok;
        return moe_enqueue(m, x, n_tok, y);
    }
    CKM(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    const int rc = moe_enqueue(m, x, n_tok, y);
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(s, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    CKM(e);
    rec.graph = g;
    CKM(cudaGraphInstantiate(&rec.exec, g, 0));
    CKM(cudaGraphLaunch(rec.exec, s));
    return FL_B200_OK;
}

} // extern "C"

// One gate | up launch and one down launch per (token, slot) through the expert-indexed one-column matvec: the form
// for shapes the multi-column matmul does not take (rows that are not 16-byte pitched, e.g. Q6_K with 1024 columns).
// wnorm / resid (one token, inside a decoder step): x is the raw hidden state, normed on the fly by the router kernel
// and by the gate | up launch's prologue, and y = resid + the block's output (the merge's add1 term).
static int moe_enqueue_per_slot(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y, const float *wnorm = nullptr,
                                float eps = 0.f, const float *resid = nullptr) {
    fl_b200_ctx *ctx = m->ctx;
    cudaStream_t s = ctx->stream;
    const fl_b200_moe_cfg &c = m->c;
    const uint32_t E = c.n_embd, F = c.n_ff, K = c.top_k, NE = c.n_expert;
    const uint64_t stride_gu = (uint64_t)F * row_bytes(c.fmt_gate_up, E), stride_d = (uint64_t)E * row_bytes(c.fmt_down, F);
    router_logits_kernel<<<dim3(NE, n_tok), 128, 0, s>>>(m->router, x, m->logits, E, NE, wnorm, eps);
    CKM(cudaGetLastError());
    CKM(launch_router_sel(m->logits, m->ids, m->gates, n_tok, NE, K, c.norm, c.scale, s, m->lids, m->mgates, m->base, m->n_local));
    const uint32_t rows_gu = (uint32_t)(stride_gu / row_bytes(c.fmt_gate_up, E)), rows_d = (uint32_t)(stride_d / row_bytes(c.fmt_down, F));
    static const int kMoePdl = getenv("FLB_MOE_PDL") ? atoi(getenv("FLB_MOE_PDL")) : 1;
    bool first_launch = true;
    const bool down_streams = matvec_is_streaming(c.fmt_down, F) && row_bytes(c.fmt_down, F) % 16 == 0;
    for (uint32_t t = 0; t < n_tok; ++t) {
        const float *xt = x + (size_t)t * E;
        for (uint32_t k = 0; k < K; ++k) {
            const uint32_t *lid = m->lids + (size_t)t * K + k;
            {   // gate and up of the slot's expert in one launch (both tensors carry the same id)
                MatvecArgs a{};
                a.n_tensors = 2;
                a.t[0] = {m->wg, m->g, nullptr, F, c.fmt_gate_up, 0, lid, rows_gu};
                a.t[1] = {m->wu, m->u, nullptr, F, c.fmt_gate_up, 0, lid, rows_gu};
                a.x = xt; a.cols = E; a.x_mode = MV_X_PLAIN; a.status = ctx->status;
                if (wnorm) { a.x_mode = MV_X_RMSNORM; a.wnorm = wnorm; a.eps = eps; }
                // Programmatic dependent launch from the second matvec launch on: the first one is an ordinary
                // dependent of the kernel that wrote the expert ids, and every later launch starts after it did,
                // so the ids (read at kernel entry, before the dependency wait) are in place for all of them.
                a.pdl = first_launch ? 0 : kMoePdl;
                a.expert_ids_ready = first_launch ? 0 : 1;
                first_launch = false;
                CKM(launch_matvec(a, ctx->sms, s));
            }
            {   // down, with silu(g) * u built while the activation is loaded (the streaming kernel's prologue;
                // rows that are not 16-byte pitched go through the generic kernel after a separate SiLU launch)
                MatvecArgs a{};
                a.n_tensors = 1;
                a.t[0] = {m->wd, m->part + ((size_t)t * K + k) * E, nullptr, E, c.fmt_down, 0, lid, rows_d};
                a.x = m->g; a.x2 = m->u; a.cols = F; a.x_mode = MV_X_SILU_MUL; a.status = ctx->status;
                a.pdl = kMoePdl;
                a.expert_ids_ready = 1;
                if (!down_streams) {
                    CKM(launch_silu_mul(m->g, m->u, m->g, F, s));
                    a.x2 = nullptr; a.x_mode = MV_X_PLAIN; a.pdl = 0;
                }
                CKM(launch_matvec(a, ctx->sms, s));
            }
        }
        float *dst = (m->world > 1 ? m->partial : y) + (size_t)t * E;
        CKM(launch_wmerge(m->part + (size_t)t * K * E, m->mgates + (size_t)t * K, m->world > 1 ? nullptr : resid, nullptr, dst, 1.0f, K, E, K, s));
    }
    if (m->world > 1) {
        for (uint32_t t = 0; t < n_tok; ++t) {   // the combine: sum of the ranks' partial outputs, rank order
            AllReduceArgs r{};
            for (uint32_t p = 0; p < m->world; ++p) r.peers[p] = m->peers[p];
            r.in = m->partial + (size_t)t * E; r.resid = nullptr; r.out = y + (size_t)t * E; r.n = E;
            r.rank = m->rank; r.world = m->world; r.st = CommState{m->comm_state}; r.status = ctx->status; r.wait_ns = ctx->wait_limit_ns;
            CKM(launch_allreduce_resid(r, s, false));
        }
    }
    return FL_B200_OK;
}

// the multi-column launches of the block as programmatic dependents of one another (FLB_MOE_PDL=0: plain launches)
static const int kMoePdlNx = getenv("FLB_MOE_PDL") ? atoi(getenv("FLB_MOE_PDL")) : 1;

static int moe_enqueue(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y) {
    fl_b200_ctx *ctx = m->ctx;
    cudaStream_t s = ctx->stream;
    const fl_b200_moe_cfg &c = m->c;
    const uint32_t E = c.n_embd, F = c.n_ff, K = c.top_k, NE = c.n_expert, T = c.max_tokens;
    const uint64_t stride_gu = (uint64_t)F * row_bytes(c.fmt_gate_up, E), stride_d = (uint64_t)E * row_bytes(c.fmt_down, F);
    if (row_bytes(c.fmt_gate_up, E) % 16 != 0 || row_bytes(c.fmt_down, F) % 16 != 0)
        return moe_enqueue_per_slot(m, x, n_tok, y);
    router_logits_kernel<<<dim3(NE, n_tok), 128, 0, s>>>(m->router, x, m->logits, E, NE);
    CKM(cudaGetLastError());
    CKM(launch_router_sel(m->logits, m->ids, m->gates, n_tok, NE, K, c.norm, c.scale, s, m->lids, m->mgates, m->base, m->n_local));
    CKM(launch_group_by_expert(m->lids, n_tok * K, K, m->n_local, T, m->cnt, m->tok_list, m->pair_list, s));
    // Every local expert once: the tokens that chose it, 8 columns per pass. The lists live on the device, so the
    // launch sequence is the same for every routing (and can be replayed as a graph); a pass without columns
    // returns at entry.
    for (uint32_t e = 0; e < m->n_local; ++e) {
        const uint32_t *cnt = m->cnt + e, *toks = m->tok_list + (size_t)e * T, *pairs = m->pair_list + (size_t)e * T;
        for (uint32_t off = 0; off < n_tok; off += 8) {
            const uint32_t P = n_tok - off < 8 ? n_tok - off : 8;
            NxCall g{};
            g.fmt = c.fmt_gate_up; g.w = m->wg + (uint64_t)e * stride_gu; g.rows = F; g.cols = E;
            g.x = x; g.P = P; g.xstride = E; g.y = m->g; g.ystride = F;
            g.cnt = cnt; g.col_idx = toks; g.out_idx = pairs; g.col_off = off;
            g.pdl = kMoePdlNx;
            cudaError_t er = launch_matmul_tc_nx(g, ctx->xq, ctx->status, ctx->sms, s);
            if (er == cudaErrorNotSupported) return set_err(FL_B200_ERR_ARG, "moe_forward: shape not taken by the multi-column matmul");
            CKM(er);
            NxCall u = g;
            u.w = m->wu + (uint64_t)e * stride_gu; u.y = m->u; u.skip_convert = 1;   // the same columns, already converted
            CKM(launch_matmul_tc_nx(u, ctx->xq, ctx->status, ctx->sms, s));
            NxCall d{};   // down: the column of pair p is silu(g[p]) * u[p], built while it is converted
            d.fmt = c.fmt_down; d.w = m->wd + (uint64_t)e * stride_d; d.rows = E; d.cols = F;
            d.x = m->g; d.x2 = m->u; d.P = P; d.xstride = F; d.y = m->part; d.ystride = E;
            d.cnt = cnt; d.col_idx = pairs; d.out_idx = pairs; d.col_off = off;
            d.pdl = kMoePdlNx;
            er = launch_matmul_tc_nx(d, ctx->xq, ctx->status, ctx->sms, s);
            if (er == cudaErrorNotSupported) return set_err(FL_B200_ERR_ARG, "moe_forward: shape not taken by the multi-column matmul");
            CKM(er);
        }
    }
    // WMERGE of every token: y[t] = sum_k gate[t][k] * part[t][k] (slots of experts held elsewhere carry gate 0)
    CKM(launch_wmerge_tokens(m->part, m->mgates, m->world > 1 ? m->partial : y, K, E, n_tok, s));
    if (m->world > 1) {
        for (uint32_t t = 0; t < n_tok; ++t) {   // the combine: sum of the ranks' partial outputs, rank order
            AllReduceArgs r{};
            for (uint32_t p = 0; p < m->world; ++p) r.peers[p] = m->peers[p];
            r.in = m->partial + (size_t)t * E; r.resid = nullptr; r.out = y + (size_t)t * E; r.n = E;
            r.rank = m->rank; r.world = m->world; r.st = CommState{m->comm_state}; r.status = ctx->status; r.wait_ns = ctx->wait_limit_ns;
            CKM(launch_allreduce_resid(r, s, false));
        }
    }
    return FL_B200_OK;
}

int flb::moe_enqueue_tokens(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y, uint32_t *n_launch, const float *wnorm,
                            float eps, const float *resid) {
    if (!m || !m->router || !m->wg) return set_err(FL_B200_ERR_STATE, "moe: weights not set");
    if (n_tok == 0 || n_tok > m->c.max_tokens) return set_err(FL_B200_ERR_ARG, "moe: %u tokens outside 1..%u", n_tok, m->c.max_tokens);
    const fl_b200_moe_cfg &c = m->c;
    if (n_tok == 1) {
        const bool down_streams = matvec_is_streaming(c.fmt_down, c.n_ff) && row_bytes(c.fmt_down, c.n_ff) % 16 == 0;
        if (n_launch) *n_launch = 2 + c.top_k * (down_streams ? 2u : 3u) + 1 + (m->world > 1 ? 1u : 0u);
        if (m->world > 1 && (wnorm || resid)) return set_err(FL_B200_ERR_ARG, "moe: the fused norm / residual form is for one GPU");
        return moe_enqueue_per_slot(m, x, 1, y, wnorm, eps, resid);
    }
    if (wnorm || resid) return set_err(FL_B200_ERR_ARG, "moe: the fused norm / residual form takes one token");
    if (n_launch) *n_launch = 0;   // not counted: the batch pass does not report launches
    return moe_enqueue(m, x, n_tok, y);
}
fl_b200_ctx *flb::moe_ctx(const fl_b200_moe *m) { return m->ctx; }
const fl_b200_moe_cfg *flb::moe_cfg(const fl_b200_moe *m) { return &m->c; }
uint32_t flb::moe_world(const fl_b200_moe *m) { return m->world; }
uint64_t flb::moe_bytes_per_token(const fl_b200_moe *m) {
    const fl_b200_moe_cfg &c = m->c;
    return (uint64_t)c.n_expert * c.n_embd * 4 +
           (uint64_t)c.top_k * (2ull * c.n_ff * row_bytes(c.fmt_gate_up, c.n_embd) + (uint64_t)c.n_embd * row_bytes(c.fmt_down, c.n_ff));
}

extern "C" {

int fl_b200_moe_routing(fl_b200_moe *m, uint32_t n_tok, uint32_t *ids_host, float *gates_host) {
    if (!m || n_tok == 0 || n_tok > m->c.max_tokens) return set_err(FL_B200_ERR_ARG, "moe_routing: bad argument");
    const size_t n = (size_t)n_tok * m->c.top_k;
    if (ids_host) if (int rc = fl_b200_download(m->ctx, ids_host, m->ids, n * 4)) return rc;
    if (gates_host) if (int rc = fl_b200_download(m->ctx, gates_host, m->gates, n * 4)) return rc;
    return FL_B200_OK;
}

} // extern "C"
