// Llama-shape greedy decoder on one B200: the per-token launch sequence of the
// decode hot path, recorded once as a CUDA graph and replayed per token. It
// plays the role of the reference's Decoder (src/model/decoder.h:52-81): build
// once (src/model/decoder.cpp:639-672), then per token embed -> run -> argmax
// (src/model/decoder.cpp:1176-1264). The reference's persistent task executor
// is replaced by a static launch plan: the graph is frozen and identical every
// token, and the position is read from a device scalar, so one recording serves
// every position.
//
// Per layer (5 launches): [RMSNorm + Q/K/V matvec] ->
// [RoPE + f16 KV append + split-KV GQA attention + combine] -> [O matvec + residual] ->
// [RMSNorm + gate/up matvec] -> [SiLU*up + down matvec + residual];
// then [RMSNorm + head matvec] -> [argmax] -> [advance].
#include "capi_internal.h"

#include <cmath>
#include <cstdlib>
#include <vector>

using namespace flb;

#define CK(call)                                                       \
    do {                                                               \
        cudaError_t e_ = (call);                                       \
        if (e_ != cudaSuccess) return cuda_err(e_, #call);             \
    } while (0)

namespace {

struct Tensor { int fmt = -1; const uint8_t *w = nullptr; uint32_t pitch = 0; };

// Timeline records start as {~0, ~0, 0, 0} (two minima, two maxima).
__global__ void trace_init_kernel(unsigned long long *t, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * 4) t[i] = (i & 2u) ? 0ull : ~0ull;
}

// After a step: history[count++] <- argmax, pos += 1, and the next input token: the argmax (greedy
// decoding) or, while a draft is being verified (*use_forced != 0), the draft's token forced[count].
__global__ void advance_kernel(int32_t *token, const int32_t *next, int32_t *pos, int32_t *hist,
                               uint32_t *hist_n, uint32_t hist_cap, const uint32_t *use_forced, const int32_t *forced,
                               const float *margin, float *margin_hist) {
    griddep_launch_dependents();
    griddep_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const int32_t t = *next;
        const uint32_t k = *hist_n;
        if (k < hist_cap) { hist[k] = t; margin_hist[k] = *margin; }
        *token = (*use_forced && k < hist_cap) ? forced[k] : t;
        *hist_n = k + 1;
        *pos = *pos + 1;
    }
}

} // namespace

struct fl_b200_decoder {
    fl_b200_ctx *ctx = nullptr;
    fl_b200_llama_cfg c{};                  // the whole model
    // Tensor parallelism: this rank's share. Q/K/V, gate/up and the head are split
    // by output rows (whole KV heads with their 4 query heads), O and down by
    // input columns; the hidden state is replicated.
    uint32_t tp_rank = 0, tp_size = 1;
    uint32_t Hq = 0, Hkv = 0, F = 0, V = 0;  // local query heads, KV heads, FFN rows, vocabulary rows
    uint8_t *comm = nullptr;                // this rank's exchange buffer (mapped by the peers)
    uint8_t *peers[kCommMaxRanks] = {};     // all ranks' buffers as mapped here
    bool peers_set = false;
    uint32_t *comm_state = nullptr;         // epoch counters of the exchange kernels
    float *partial = nullptr, *top3 = nullptr;
    float2 *rope_table = nullptr;           // (cos, sin) of this step's position, shared by all layers
    std::vector<Tensor> lw;                 // n_layer * 7
    std::vector<const float *> attn_norm, ffn_norm;
    std::vector<fl_b200_moe *> moe;         // per layer: a mixture-of-experts block in place of gate / up / down (or nullptr)
    Tensor tok_embd, output;
    const float *out_norm = nullptr;
    std::vector<__half *> kc, vc;
    // device state
    int32_t *d_token = nullptr, *d_next = nullptr, *d_pos = nullptr, *d_hist = nullptr, *d_forced = nullptr;
    float *d_margin_hist = nullptr;         // top1 - top2 margin of every step since the last host call, beside d_hist
    uint32_t *d_use_forced = nullptr;
    uint32_t *d_hist_n = nullptr;
    float *d_margin = nullptr;
    uint32_t hist_cap = 4096;
    float *xa = nullptr, *xb = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr;
    float *g = nullptr, *u = nullptr, *logits = nullptr, *xn_final = nullptr, *part = nullptr;
    uint32_t *tickets = nullptr;
    bool fused_swiglu = false;              // the gate/up launch writes silu(gate)*up into g
    unsigned long long *trace = nullptr;    // FLB_TRACE=1: 4 device timestamps per launch of the step
    uint32_t trace_n = 0;
    uint32_t n_splits = 1;
    int32_t *h_pin = nullptr;               // pinned: [0] token, [1] pos, [2] next
    int32_t n_past = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint32_t launches = 0;
    bool finalized = false;
    std::vector<void *> owned;              // device memory the decoder frees (tensors uploaded from a model file)
    // Batch pass (Decoder::step_batch): m <= kMaxBatch tokens at consecutive positions through the model in one
    // pass; buffers are [kMaxBatch][...] and one CUDA graph per m, all made at the first call.
    struct Batch {
        float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *g = nullptr, *u = nullptr;
        float *logits = nullptr, *margin = nullptr, *part = nullptr;
        float *partial = nullptr, *top3 = nullptr;   // tensor parallel: this rank's partial O / down outputs, argmax records
        int32_t *io = nullptr;              // [0..8) tokens, [8..16) positions, [16..24) greedy next tokens
        uint32_t *tickets = nullptr;
        int32_t *h_io = nullptr;            // pinned image of io, then the 8 margins
        cudaGraph_t graph[FL_B200_MAX_BATCH + 1] = {};
        cudaGraphExec_t exec[FL_B200_MAX_BATCH + 1] = {};
        uint32_t last_m = 0;
        bool ready = false;
    } b;
    // Independent sequences decoded in lock step (fl_b200_decoder_seqs_*): per layer one cache [n_seq][n_kv_head][max_kv][128]
    // for K and one for V, a position per sequence, and one CUDA graph of the pass (the batch pass's buffers serve it).
    struct Seqs {
        uint32_t n = 0;
        std::vector<__half *> kc, vc;
        int32_t pos[FL_B200_MAX_BATCH] = {};
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
    } sq;
};

void flb::decoder_adopt(fl_b200_decoder *d, void *dev) { d->owned.push_back(dev); }

// Every kernel of the step after the embedding lookup is launched with
// programmatic dependent launch: its preamble (barrier set-up, weight prefetch
// into shared memory) overlaps the tail of the kernel before it.
static int kPdl = 1;
// Which matvec launches request their first weight stages after the activation loads (bit 0 Q/K/V, 1 gate|up,
// 2 down, 3 head, 4 O). Measured on the 8B-shape step: gate|up alone +2 % (457 -> 467 tokens/s), the others within noise.
static int issue_late() { static const int v = getenv("FLB_ISSUE_LATE") ? atoi(getenv("FLB_ISSUE_LATE")) : 2; return v; }

// Kernel classes, for timing one class of the step in isolation.
enum : uint32_t { K_MATVEC = 1u, K_ATTN = 2u, K_OTHER = 4u, K_COMM = 8u, K_ALL = 15u };

static int enqueue_step(fl_b200_decoder *d, cudaStream_t s, uint32_t *n_launch, uint32_t mask = K_ALL) {
    uint32_t n = 0;   // launches so far
    auto do_matvec = [&](MatvecArgs &a) -> int {
        // Q8_0 streams only in launches of its own: a group that mixes it with the K-quants goes out one
        // tensor per launch (each with the group's prologue). The caller counts the last launch.
        bool q8 = false, kq = false;
        for (int i = 0; i < a.n_tensors; ++i) (a.t[i].fmt == FL_B200_Q8_0 ? q8 : kq) = true;
        if (q8 && kq && !a.swiglu) {
            for (int i = 0; i < a.n_tensors; ++i) {
                MatvecArgs one = a;
                one.n_tensors = 1;
                one.t[0] = a.t[i];
                if (d->trace && mask == K_ALL) one.trace = d->trace + 4 * (size_t)n;
                if (int rc = cuda_err(launch_matvec(one, d->ctx->sms, s), "matvec launch")) return rc;
                if (i + 1 < a.n_tensors) ++n;
            }
            return FL_B200_OK;
        }
        if (d->trace && mask == K_ALL) a.trace = d->trace + 4 * (size_t)n;
        return cuda_err(launch_matvec(a, d->ctx->sms, s), "matvec launch");
    };
    const fl_b200_llama_cfg &c = d->c;
    fl_b200_ctx *ctx = d->ctx;
    const uint32_t E = c.n_embd, D = c.head_dim, QD = d->Hq * D, KD = d->Hkv * D;
    const bool tp = d->tp_size > 1;
    const CommState cst{d->comm_state};
    // sum of the ranks' partial vectors + residual (the exchange step after O and after down)
    // Two forms: one kernel that pushes, waits and adds (the default), or (FLB_TP_FUSED=1) a push-only
    // kernel whose sum is taken by the prologue of the matvec that consumes it (one launch and one pass
    // through memory less; the consumer's CTAs start while the pushes are still crossing NVLink).
    static const bool fused = getenv("FLB_TP_FUSED") && getenv("FLB_TP_FUSED")[0] == '1';
    struct { const float *resid; float *out; bool on; } pend = {nullptr, nullptr, false};
    auto do_allreduce = [&](const float *resid, float *out) -> int {
        AllReduceArgs r{};
        for (uint32_t p = 0; p < d->tp_size; ++p) r.peers[p] = d->peers[p];
        r.in = d->partial; r.resid = resid; r.out = out; r.n = E; r.rank = d->tp_rank; r.world = d->tp_size;
        r.st = cst; r.status = ctx->status; r.wait_ns = ctx->wait_limit_ns;
        if (!fused) return cuda_err(launch_allreduce_resid(r, s, kPdl != 0), "all-reduce launch");
        pend.resid = resid; pend.out = out; pend.on = true;
        return cuda_err(launch_allreduce_push(r, s, kPdl != 0), "all-reduce push launch");
    };
    auto take_pending = [&](MatvecArgs &a) {   // the matvec whose activation is the pending sum
        if (!pend.on) return;
        a.xr_buf = d->peers[d->tp_rank]; a.xr_epoch = d->comm_state; a.xr_resid = pend.resid; a.xr_out = pend.out;
        a.xr_world = d->tp_size; a.x = pend.out;
        pend.on = false;
    };
    const float theta_scale = powf(c.rope_base, -2.0f / (float)D);
    if (mask & K_OTHER) { CK(launch_rope_table(d->d_pos, theta_scale, D, d->rope_table, s)); ++n; }
    if (mask & K_OTHER) { CK(launch_embed(d->tok_embd.fmt, d->tok_embd.w, d->d_token, E, d->xa, s, false)); ++n; }
    // The matvec launches of the step, by builder (the launch order is below).
    auto mk_qkv = [&](uint32_t l) {   // RMSNorm + Q/K/V
        const Tensor *w = &d->lw[(size_t)l * 7];
        MatvecArgs a{};
        a.n_tensors = 3;
        a.t[0] = {w[FL_B200_T_WQ].w, d->q, nullptr, QD, w[FL_B200_T_WQ].fmt, 0};
        a.t[1] = {w[FL_B200_T_WK].w, d->k, nullptr, KD, w[FL_B200_T_WK].fmt, 0};
        a.t[2] = {w[FL_B200_T_WV].w, d->v, nullptr, KD, w[FL_B200_T_WV].fmt, 0};
        a.x = d->xa; a.wnorm = d->attn_norm[l]; a.eps = c.eps; a.cols = E;
        a.x_mode = MV_X_RMSNORM; a.status = ctx->status; a.pdl = kPdl; a.issue_late = issue_late() & 1;
        return a;
    };
    auto mk_o = [&](uint32_t l) {     // O projection + residual: xb = xa + Wo att (tensor parallel: partial sums over this
        const Tensor *w = &d->lw[(size_t)l * 7];   // rank's columns, then the exchange adds the ranks' partials and the residual)
        MatvecArgs a{};
        a.n_tensors = 1;
        a.t[0] = {w[FL_B200_T_WO].w, tp ? d->partial : d->xb, tp ? nullptr : d->xa, E, w[FL_B200_T_WO].fmt, w[FL_B200_T_WO].pitch};
        a.x = d->att; a.cols = QD; a.x_mode = MV_X_PLAIN; a.status = ctx->status; a.pdl = kPdl;
        a.issue_late = (issue_late() >> 4) & 1;
        return a;
    };
    auto mk_gate_up = [&](uint32_t l) {   // RMSNorm + gate / up with the SwiGLU product in the epilogue: g <- silu(gate x) * (up x)
        const Tensor *w = &d->lw[(size_t)l * 7];
        MatvecArgs a{};
        a.n_tensors = 2;
        a.t[0] = {w[FL_B200_T_GATE].w, d->g, nullptr, d->F, w[FL_B200_T_GATE].fmt, 0};
        a.t[1] = {w[FL_B200_T_UP].w, d->u, nullptr, d->F, w[FL_B200_T_UP].fmt, 0};
        a.x = d->xb; a.wnorm = d->ffn_norm[l]; a.eps = c.eps; a.cols = E;
        a.x_mode = MV_X_RMSNORM; a.status = ctx->status; a.pdl = kPdl;
        // (Q8_0 streams without the fused product: the down projection then takes silu(g) * u on load)
        a.swiglu = (w[FL_B200_T_GATE].fmt == w[FL_B200_T_UP].fmt && w[FL_B200_T_GATE].fmt != FL_B200_Q8_0) ? 1 : 0;
        a.issue_late = (issue_late() >> 1) & 1;
        return a;
    };
    auto mk_down = [&](uint32_t l, bool fused_swiglu) {   // down projection + residual: xa = xb + Wdown h
        const Tensor *w = &d->lw[(size_t)l * 7];
        MatvecArgs a{};
        a.n_tensors = 1;
        a.t[0] = {w[FL_B200_T_DOWN].w, tp ? d->partial : d->xa, tp ? nullptr : d->xb, E, w[FL_B200_T_DOWN].fmt, w[FL_B200_T_DOWN].pitch};
        a.x = d->g; a.x2 = d->u; a.cols = d->F; a.status = ctx->status; a.pdl = kPdl;
        a.x_mode = fused_swiglu ? MV_X_PLAIN : MV_X_SILU_MUL;
        a.issue_late = (issue_late() >> 2) & 1;
        return a;
    };
    auto mk_head = [&]() {   // output norm + head
        MatvecArgs a{};
        a.n_tensors = 1;
        a.t[0] = {d->output.w, d->logits, nullptr, d->V, d->output.fmt, 0};
        a.x = d->xa; a.wnorm = d->out_norm; a.eps = c.eps; a.cols = E;
        a.x_mode = MV_X_RMSNORM; a.status = ctx->status; a.pdl = kPdl;   // the normed vector itself: computed when the tap is read
        a.issue_late = (issue_late() >> 3) & 1;
        return a;
    };
    // One GPU: the four matvecs between two attention launches, O -> gate|up -> down -> the next layer's Q/K/V (or the
    // head), go out as ONE launch with grid-wide barriers between them (launch_matvec_tc_chain): the weights of the next
    // matvec stream into shared memory while the current one drains and the next activation is built. Off by default
    // (FLB_CHAIN=1 switches it on): measured on the 8B-shape step it is SLOWER than one launch per matvec with
    // programmatic dependent launch (391 against 441 tokens/s): a phase boundary inside the kernel costs about 3 us
    // more than a kernel boundary. A tensor-parallel decoder (its exchange launches sit between the matvecs) and shapes
    // the chain does not take always go out as one launch per matvec.
    static const bool chain_on = getenv("FLB_CHAIN") && getenv("FLB_CHAIN")[0] == '1';
    bool qkv_done = false;   // the Q/K/V of the coming layer already went out with the previous layer's chain
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        if (!qkv_done) {
            MatvecArgs a = mk_qkv(l);
            take_pending(a);
            if (mask & K_MATVEC) { if (int rc = do_matvec(a)) return rc; ++n; }
        }
        qkv_done = false;
        {   // RoPE on q and k, the f16 append of k and v, and the attention itself: one kernel
            AttnArgs a{};
            a.rope_k = d->k; a.rope_v = d->v; a.k_append = d->kc[l]; a.v_append = d->vc[l];
            a.theta_scale = theta_scale; a.rope_table = d->rope_table;
            a.q = d->q; a.k = d->kc[l]; a.v = d->vc[l]; a.out = d->att; a.part = d->part; a.tickets = d->tickets;
            a.pos = d->d_pos; a.kv_len = 0; a.kv_stride = c.max_kv;
            a.batch_stride = (uint64_t)d->Hkv * c.max_kv * D;
            a.n_q_head = d->Hq; a.n_kv_head = d->Hkv; a.batch = 1; a.n_splits = d->n_splits;
            a.scale = 1.0f / sqrtf((float)D); a.status = ctx->status; a.pdl = kPdl;
            if (d->trace && mask == K_ALL) a.trace = d->trace + 4 * (size_t)n;
            if (mask & K_ATTN) { CK(attn_make_maps(a)); CK(launch_attn_decode(a, s)); ++n; }
        }
        if (d->moe[l]) {
            // Mixture-of-experts layer: xb = xa + Wo att as usual, then xa = xb + MoE(RMSNorm(xb)). The block's own launches
            // (router, selection, the selected experts through the expert-indexed matvec, merge) are part of the captured
            // step; the norm is taken inside the router kernel and the gate | up launches, the residual inside the merge.
            MatvecArgs ao = mk_o(l);
            if (mask & K_MATVEC) { if (int rc = do_matvec(ao)) return rc; ++n; }
            if (mask & K_MATVEC) {
                uint32_t nl = 0;
                if (int rc = moe_enqueue_tokens(d->moe[l], d->xb, 1, d->xa, &nl, d->ffn_norm[l], c.eps, d->xb)) return rc;
                n += nl;
            }
            continue;
        }
        MatvecArgs ao = mk_o(l), ag = mk_gate_up(l);
        d->fused_swiglu = ag.swiglu != 0;
        MatvecArgs ad = mk_down(l, d->fused_swiglu);
        if (chain_on && !tp && (mask & K_MATVEC)) {
            MatvecArgs ch[4] = {ao, ag, ad, l + 1 < c.n_layer ? mk_qkv(l + 1) : mk_head()};
            if (d->trace && mask == K_ALL) ch[0].trace = d->trace + 4 * (size_t)n;
            ch[0].grid_bar = ctx->grid_bar;
            const cudaError_t e = launch_matvec_tc_chain(ch, 4, ctx->sms, s);
            if (e == cudaSuccess) { ++n; qkv_done = true; continue; }
            if (e != cudaErrorNotSupported) return cuda_err(e, "matvec chain launch");
        }
        if (mask & K_MATVEC) { if (int rc = do_matvec(ao)) return rc; ++n; }
        if (tp && (mask & K_COMM)) { if (int rc = do_allreduce(d->xa, d->xb)) return rc; ++n; }
        take_pending(ag);
        if (mask & K_MATVEC) { if (int rc = do_matvec(ag)) return rc; ++n; }
        if (mask & K_MATVEC) { if (int rc = do_matvec(ad)) return rc; ++n; }
        if (tp && (mask & K_COMM)) { if (int rc = do_allreduce(d->xb, d->xa)) return rc; ++n; }
    }
    if (!qkv_done) {
        MatvecArgs a = mk_head();
        take_pending(a);
        if (mask & K_MATVEC) { if (int rc = do_matvec(a)) return rc; ++n; }
    }
    if (mask & K_OTHER) {
        CK(launch_argmax(d->logits, d->V, d->d_next, d->d_margin, ctx->argmax_scratch, ctx->argmax_ticket,
                         ctx->sms, s, kPdl != 0, d->top3)); ++n;
    }
    if (tp && (mask & K_COMM)) {   // merge the ranks' (best, index, runner-up): the same token on every rank
        TopExchangeArgs x{};
        for (uint32_t p = 0; p < d->tp_size; ++p) x.peers[p] = d->peers[p];
        x.top3 = d->top3; x.index_base = d->tp_rank * d->V; x.out_idx = d->d_next; x.out_margin = d->d_margin;
        x.rank = d->tp_rank; x.world = d->tp_size; x.st = cst; x.status = ctx->status; x.wait_ns = ctx->wait_limit_ns;
        CK(launch_argmax_exchange(x, s, kPdl != 0)); ++n;
    }
    if (mask == K_ALL) {   // state only advances in the real step
        CK(launch_kernel(advance_kernel, dim3(1), dim3(32), 0, s, kPdl != 0, d->d_token, d->d_next, d->d_pos, d->d_hist,
                         d->d_hist_n, d->hist_cap, (const uint32_t *)d->d_use_forced, (const int32_t *)d->d_forced,
                         (const float *)d->d_margin, d->d_margin_hist)); ++n;
    }
    if (n_launch) *n_launch = n;
    return FL_B200_OK;
}

extern "C" {

int fl_b200_decoder_create(fl_b200_ctx *ctx, const fl_b200_llama_cfg *cfg, fl_b200_decoder **out) {
    return fl_b200_decoder_create_tp(ctx, cfg, 0, 1, out);
}

int fl_b200_decoder_create_tp(fl_b200_ctx *ctx, const fl_b200_llama_cfg *cfg, uint32_t rank, uint32_t world,
                              fl_b200_decoder **out) {
    if (!ctx || !cfg || !out) return set_err(FL_B200_ERR_ARG, "decoder_create: null pointer");
    const fl_b200_llama_cfg &c = *cfg;
    if (world == 0 || world > kCommMaxRanks || rank >= world)
        return set_err(FL_B200_ERR_ARG, "decoder_create: rank %u of %u (at most %u ranks)", rank, world, kCommMaxRanks);
    if (world > 1) {
        if (c.n_kv_head % world || c.n_ff % (256 * world) || c.n_vocab % world)
            return set_err(FL_B200_ERR_ARG, "decoder_create: %u ranks do not divide n_kv_head %u, n_ff %u / 256 and n_vocab %u",
                           world, c.n_kv_head, c.n_ff, c.n_vocab);
        if (c.n_embd > kCommMaxVec || c.n_embd % (4 * kCommChunks) || (c.n_ff / world) < 512 ||
            (c.n_head / world) * c.head_dim < 512)
            return set_err(FL_B200_ERR_ARG, "decoder_create: shape too small or too large for %u ranks", world);
    }
    if (c.head_dim != 128) return set_err(FL_B200_ERR_ARG, "decoder_create: head_dim %u (only 128 is built)", c.head_dim);
    if (c.n_kv_head == 0 || c.n_head != 4 * c.n_kv_head)
        return set_err(FL_B200_ERR_ARG, "decoder_create: %u heads over %u KV heads (only groups of 4 are built)", c.n_head, c.n_kv_head);
    if (c.n_layer == 0 || c.n_embd == 0 || c.n_ff == 0 || c.n_vocab == 0 || c.max_kv == 0)
        return set_err(FL_B200_ERR_ARG, "decoder_create: zero-sized dimension");
    if (c.n_embd % 256 || c.n_ff % 256 || c.n_embd < 512 || c.n_ff < 512)
        return set_err(FL_B200_ERR_ARG, "decoder_create: n_embd and n_ff must be multiples of 256 (>= 512)");
    fl_b200_decoder *d = new fl_b200_decoder();
    d->ctx = ctx;
    d->c = c;
    d->tp_rank = rank;
    d->tp_size = world;
    d->Hq = c.n_head / world;
    d->Hkv = c.n_kv_head / world;
    d->F = c.n_ff / world;
    d->V = c.n_vocab / world;
    d->lw.resize((size_t)c.n_layer * 7);
    d->attn_norm.assign(c.n_layer, nullptr);
    d->ffn_norm.assign(c.n_layer, nullptr);
    d->moe.assign(c.n_layer, nullptr);
    d->kc.assign(c.n_layer, nullptr);
    d->vc.assign(c.n_layer, nullptr);
    // every failure from here on destroys d (the KV caches already allocated would otherwise stay for the life of the process)
    auto alloc = [&]() -> int {
    CK(cudaSetDevice(ctx->device));
    const size_t kvb = (size_t)d->Hkv * c.max_kv * c.head_dim * sizeof(__half);
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        CK(cudaMalloc(&d->kc[l], kvb));
        CK(cudaMalloc(&d->vc[l], kvb));
        CK(cudaMemsetAsync(d->kc[l], 0, kvb, ctx->stream));
        CK(cudaMemsetAsync(d->vc[l], 0, kvb, ctx->stream));
    }
    const uint32_t QD = d->Hq * c.head_dim, KD = d->Hkv * c.head_dim;
    CK(cudaMalloc(&d->d_token, 64));
    d->d_next = d->d_token + 1;
    d->d_pos = d->d_token + 2;
    d->d_hist_n = (uint32_t *)(d->d_token + 3);
    d->d_margin = (float *)(d->d_token + 4);
    d->d_use_forced = (uint32_t *)(d->d_token + 5);
    CK(cudaMemsetAsync(d->d_token, 0, 64, ctx->stream));
    CK(cudaMalloc(&d->d_hist, d->hist_cap * sizeof(int32_t)));
    CK(cudaMalloc(&d->d_margin_hist, d->hist_cap * sizeof(float)));
    CK(cudaMalloc(&d->d_forced, d->hist_cap * sizeof(int32_t)));
    CK(cudaMalloc(&d->xa, c.n_embd * 4));
    CK(cudaMalloc(&d->xb, c.n_embd * 4));
    CK(cudaMalloc(&d->q, QD * 4));
    CK(cudaMalloc(&d->k, KD * 4));
    CK(cudaMalloc(&d->v, KD * 4));
    CK(cudaMalloc(&d->att, QD * 4));
    CK(cudaMalloc(&d->g, d->F * 4));
    CK(cudaMalloc(&d->u, d->F * 4));
    CK(cudaMalloc(&d->logits, (size_t)d->V * 4));
    CK(cudaMalloc(&d->top3, 16));
    CK(cudaMalloc(&d->rope_table, (c.head_dim / 2) * sizeof(float2)));
    if (world > 1) {
        CK(cudaMalloc(&d->comm, comm_buffer_bytes()));
        CK(cudaMemsetAsync(d->comm, 0, comm_buffer_bytes(), ctx->stream));
        CK(cudaMalloc(&d->comm_state, 64));
        CK(cudaMemsetAsync(d->comm_state, 0, 64, ctx->stream));
        CK(cudaMalloc(&d->partial, c.n_embd * 4));
    }
    CK(cudaMalloc(&d->xn_final, c.n_embd * 4));
    d->n_splits = attn_pick_splits(d->Hkv, 1, c.max_kv, ctx->sms);
    CK(cudaMalloc(&d->part, attn_part_floats(d->Hq, 1, d->n_splits) * sizeof(float)));
    CK(cudaMalloc(&d->tickets, 256 * sizeof(uint32_t)));
    CK(cudaMemsetAsync(d->tickets, 0, 256 * sizeof(uint32_t), ctx->stream));
    CK(cudaMallocHost(&d->h_pin, 64));
    CK(cudaStreamSynchronize(ctx->stream));
    return FL_B200_OK;
    };
    const int rc = alloc();
    if (rc != FL_B200_OK) {
        fl_b200_decoder_destroy(d);
        return rc;
    }
    *out = d;
    return FL_B200_OK;
}

void fl_b200_decoder_destroy(fl_b200_decoder *d) {
    if (!d) return;
    cudaSetDevice(d->ctx->device);
    cudaStreamSynchronize(d->ctx->stream);
    if (d->exec) cudaGraphExecDestroy(d->exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    for (auto p : d->kc) cudaFree(p);
    for (auto p : d->vc) cudaFree(p);
    for (auto p : d->sq.kc) cudaFree(p);
    for (auto p : d->sq.vc) cudaFree(p);
    if (d->sq.exec) cudaGraphExecDestroy(d->sq.exec);
    if (d->sq.graph) cudaGraphDestroy(d->sq.graph);
    cudaFree(d->d_token); cudaFree(d->d_hist); cudaFree(d->d_margin_hist); cudaFree(d->d_forced); cudaFree(d->xa); cudaFree(d->xb); cudaFree(d->q);
    cudaFree(d->k); cudaFree(d->v); cudaFree(d->att); cudaFree(d->g); cudaFree(d->u); cudaFree(d->logits);
    cudaFree(d->xn_final); cudaFree(d->part); cudaFree(d->tickets);
    cudaFree(d->top3); cudaFree(d->rope_table); cudaFree(d->comm); cudaFree(d->comm_state); cudaFree(d->partial);
    cudaFree(d->trace);
    for (void *p : d->owned) cudaFree(p);
    for (uint32_t m = 0; m <= FL_B200_MAX_BATCH; ++m) {
        if (d->b.exec[m]) cudaGraphExecDestroy(d->b.exec[m]);
        if (d->b.graph[m]) cudaGraphDestroy(d->b.graph[m]);
    }
    cudaFree(d->b.x); cudaFree(d->b.xn); cudaFree(d->b.q); cudaFree(d->b.k); cudaFree(d->b.v); cudaFree(d->b.att);
    cudaFree(d->b.g); cudaFree(d->b.u); cudaFree(d->b.logits); cudaFree(d->b.margin); cudaFree(d->b.part);
    cudaFree(d->b.io); cudaFree(d->b.tickets); cudaFree(d->b.partial); cudaFree(d->b.top3);
    cudaFreeHost(d->b.h_io);
    cudaFreeHost(d->h_pin);
    delete d;
}

static int check_weight(const fl_b200_decoder *d, int fmt, const void *w, uint32_t cols) {
    (void)d;
    if (!w) return set_err(FL_B200_ERR_ARG, "decoder: null weight pointer");
    if (fmt != FL_B200_Q4_K && fmt != FL_B200_Q6_K && fmt != FL_B200_Q8_0)
        return set_err(FL_B200_ERR_ARG, "decoder: weight format %d (the decoder streams Q4_K, Q6_K and Q8_0)", fmt);
    if (((uintptr_t)w & 15u) != 0) return set_err(FL_B200_ERR_ARG, "decoder: weights must be 16-byte aligned");
    if (cols % 256 || cols < 512) return set_err(FL_B200_ERR_ARG, "decoder: cols %u not a multiple of 256 (>= 512)", cols);
    return FL_B200_OK;
}

int fl_b200_decoder_set_layer_tensor(fl_b200_decoder *d, uint32_t layer, int which, int fmt, const void *w) {
    if (!d || layer >= d->c.n_layer || which < 0 || which > FL_B200_T_DOWN)
        return set_err(FL_B200_ERR_ARG, "decoder_set_layer_tensor: bad layer / tensor id");
    if (d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_set_layer_tensor: after finalize");
    const uint32_t cols = which == FL_B200_T_DOWN ? d->F : which == FL_B200_T_WO ? d->Hq * d->c.head_dim : d->c.n_embd;
    if (int rc = check_weight(d, fmt, w, cols)) return rc;
    // Column slices (O, down) are stored with their rows zero-padded to a multiple of 16 bytes.
    const uint32_t pitch = (uint32_t)((row_bytes(fmt, cols) + 15u) & ~(uint64_t)15u);
    d->lw[(size_t)layer * 7 + which] = {fmt, (const uint8_t *)w, pitch};
    return FL_B200_OK;
}

int fl_b200_decoder_set_layer_norms(fl_b200_decoder *d, uint32_t layer, const float *an, const float *fn) {
    if (!d || layer >= d->c.n_layer || !an || !fn) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_norms: bad argument");
    if (d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_set_layer_norms: after finalize");
    d->attn_norm[layer] = an;
    d->ffn_norm[layer] = fn;
    return FL_B200_OK;
}

int fl_b200_decoder_set_global(fl_b200_decoder *d, int which, int fmt, const void *w) {
    if (!d || (which != FL_B200_G_TOK_EMBD && which != FL_B200_G_OUTPUT))
        return set_err(FL_B200_ERR_ARG, "decoder_set_global: bad tensor id");
    if (d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_set_global: after finalize");
    if (int rc = check_weight(d, fmt, w, d->c.n_embd)) return rc;
    (which == FL_B200_G_TOK_EMBD ? d->tok_embd : d->output) = {fmt, (const uint8_t *)w, 0};
    return FL_B200_OK;
}

int fl_b200_decoder_set_out_norm(fl_b200_decoder *d, const float *w) {
    if (!d || !w) return set_err(FL_B200_ERR_ARG, "decoder_set_out_norm: null");
    d->out_norm = w;
    return FL_B200_OK;
}

int fl_b200_decoder_kv(fl_b200_decoder *d, uint32_t layer, uint16_t **k, uint16_t **v) {
    if (!d || layer >= d->c.n_layer) return set_err(FL_B200_ERR_ARG, "decoder_kv: bad layer");
    if (k) *k = (uint16_t *)d->kc[layer];
    if (v) *v = (uint16_t *)d->vc[layer];
    return FL_B200_OK;
}

int fl_b200_decoder_comm(fl_b200_decoder *d, void **buf, size_t *bytes) {
    if (!d || !buf || !bytes) return set_err(FL_B200_ERR_ARG, "decoder_comm: null");
    *buf = d->comm;
    *bytes = d->comm ? comm_buffer_bytes() : 0;
    return FL_B200_OK;
}

int fl_b200_decoder_set_peers(fl_b200_decoder *d, void *const *bufs, uint32_t n) {
    if (!d || !bufs) return set_err(FL_B200_ERR_ARG, "decoder_set_peers: null");
    if (d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_set_peers: after finalize");
    if (n != d->tp_size) return set_err(FL_B200_ERR_ARG, "decoder_set_peers: %u buffers for %u ranks", n, d->tp_size);
    for (uint32_t p = 0; p < n; ++p) {
        if (!bufs[p]) return set_err(FL_B200_ERR_ARG, "decoder_set_peers: buffer of rank %u is null", p);
        d->peers[p] = (uint8_t *)bufs[p];
    }
    if (d->tp_size > 1 && d->peers[d->tp_rank] != d->comm)
        return set_err(FL_B200_ERR_ARG, "decoder_set_peers: entry %u must be this rank's own buffer", d->tp_rank);
    d->peers_set = true;
    return FL_B200_OK;
}

int fl_b200_decoder_set_layer_moe(fl_b200_decoder *d, uint32_t layer, fl_b200_moe *moe) {
    if (!d || !moe) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: null");
    if (d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_set_layer_moe: the decoder is finalized");
    if (layer >= d->c.n_layer) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: layer %u of %u", layer, d->c.n_layer);
    if (d->tp_size > 1 || moe_world(moe) > 1) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: one GPU only");
    if (moe_ctx(moe) != d->ctx) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: the block belongs to another context");
    const fl_b200_moe_cfg *mc = moe_cfg(moe);
    if (mc->n_embd != d->c.n_embd) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: block n_embd %u, model %u", mc->n_embd, d->c.n_embd);
    if (d->c.n_head * d->c.head_dim < d->c.n_embd) return set_err(FL_B200_ERR_ARG, "decoder_set_layer_moe: the query buffer is narrower than n_embd");
    d->moe[layer] = moe;
    return FL_B200_OK;
}

int fl_b200_decoder_finalize(fl_b200_decoder *d) {
    if (!d) return set_err(FL_B200_ERR_ARG, "decoder_finalize: null");
    if (d->finalized) return FL_B200_OK;
    for (size_t i = 0; i < d->lw.size(); ++i)
        if (!d->lw[i].w && !(d->moe[i / 7] && i % 7 >= FL_B200_T_GATE))   // a MoE layer has no gate / up / down of its own
            return set_err(FL_B200_ERR_STATE, "decoder_finalize: layer %zu tensor %zu not set", i / 7, i % 7);
    for (uint32_t l = 0; l < d->c.n_layer; ++l)
        if (!d->attn_norm[l] || !d->ffn_norm[l]) return set_err(FL_B200_ERR_STATE, "decoder_finalize: norms of layer %u not set", l);
    if (!d->tok_embd.w || !d->output.w || !d->out_norm) return set_err(FL_B200_ERR_STATE, "decoder_finalize: embedding / head / output norm not set");
    if (d->tp_size > 1 && !d->peers_set) return set_err(FL_B200_ERR_STATE, "decoder_finalize: set the peers' exchange buffers first");
    cudaStream_t s = d->ctx->stream;
    CK(cudaSetDevice(d->ctx->device));
    CK(cudaStreamSynchronize(s));
    if (const char *e = getenv("FLB_TRACE")) {
        if (e[0] == '1' && !d->trace) {
            d->trace_n = 8 + 16 * d->c.n_layer;   // room for groups that go out one tensor per launch
            CK(cudaMalloc(&d->trace, (size_t)d->trace_n * 4 * sizeof(unsigned long long)));
        }
    }
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    uint32_t n = 0;
    int rc = enqueue_step(d, s, &n);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(s, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    CK(e);
    d->graph = g;
    CK(cudaGraphInstantiate(&d->exec, g, 0));
    CK(cudaGraphUpload(d->exec, s));
    d->launches = n;
    d->finalized = true;
    return FL_B200_OK;
}

int fl_b200_decoder_set_n_past(fl_b200_decoder *d, int32_t n_past) {
    if (!d || n_past < 0 || (uint32_t)n_past > d->c.max_kv) return set_err(FL_B200_ERR_ARG, "decoder_set_n_past: out of range");
    d->n_past = n_past;
    return FL_B200_OK;
}

int fl_b200_decoder_n_past(fl_b200_decoder *d, int32_t *out) {
    if (!d || !out) return set_err(FL_B200_ERR_ARG, "decoder_n_past: null");
    *out = d->n_past;
    return FL_B200_OK;
}

static int check_dev_status(fl_b200_decoder *d) {
    uint32_t st = 0;
    if (int rc = fl_b200_device_status(d->ctx, &st)) return rc;
    if (st != 0) {
        // a kernel that gave up may have left its arrival counters non-zero: clear them, so that a caller who
        // carries on does not get a combine that fires with splits missing
        cudaMemsetAsync(d->tickets, 0, 256 * sizeof(uint32_t), d->ctx->stream);
        if (d->b.tickets) cudaMemsetAsync(d->b.tickets, 0, (size_t)d->Hkv * FL_B200_MAX_BATCH * sizeof(uint32_t), d->ctx->stream);
        cudaMemsetAsync(d->ctx->attn_tickets, 0, d->ctx->attn_tickets_cap * sizeof(uint32_t), d->ctx->stream);
        return set_err(FL_B200_ERR_DEVICE, "decoder: a kernel reported status %u (bounded wait gave up)", st);
    }
    return FL_B200_OK;
}

int fl_b200_decoder_step(fl_b200_decoder *d, int32_t token, int32_t *next_out) {
    if (!d || !next_out) return set_err(FL_B200_ERR_ARG, "decoder_step: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_step: finalize first");
    if ((uint32_t)d->n_past >= d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_step: kv full (%d of %u)", d->n_past, d->c.max_kv);
    if (token < 0 || (uint32_t)token >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_step: token %d outside the vocabulary", token);
    cudaStream_t s = d->ctx->stream;
    d->h_pin[0] = token;
    d->h_pin[1] = 0;            // next (unused on the way in)
    d->h_pin[2] = d->n_past;
    d->h_pin[3] = 0;            // history counter
    d->h_pin[4] = 0;
    d->h_pin[5] = 0;            // teacher forcing off, whatever an earlier failed call left behind
    CK(cudaMemcpyAsync(d->d_token, d->h_pin, 24, cudaMemcpyHostToDevice, s));
    if (d->trace) trace_init_kernel<<<(d->trace_n * 4 + 255) / 256, 256, 0, s>>>(d->trace, d->trace_n);
    CK(cudaGraphLaunch(d->exec, s));
    CK(cudaMemcpyAsync(d->h_pin + 8, d->d_next, 4, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    d->n_past += 1;
    *next_out = d->h_pin[8];
    return check_dev_status(d);
}

int fl_b200_decoder_run(fl_b200_decoder *d, int32_t first_token, uint32_t n, int32_t *tokens_host) {
    if (!d || !tokens_host) return set_err(FL_B200_ERR_ARG, "decoder_run: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_run: finalize first");
    if (n == 0 || n > d->hist_cap) return set_err(FL_B200_ERR_ARG, "decoder_run: n %u outside 1..%u", n, d->hist_cap);
    if ((uint64_t)d->n_past + n > d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_run: kv full (%d + %u > %u)", d->n_past, n, d->c.max_kv);
    if (first_token < 0 || (uint32_t)first_token >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_run: token outside the vocabulary");
    cudaStream_t s = d->ctx->stream;
    d->h_pin[0] = first_token;
    d->h_pin[1] = 0;
    d->h_pin[2] = d->n_past;
    d->h_pin[3] = 0;
    d->h_pin[4] = 0;
    d->h_pin[5] = 0;            // teacher forcing off
    CK(cudaMemcpyAsync(d->d_token, d->h_pin, 24, cudaMemcpyHostToDevice, s));
    for (uint32_t i = 0; i < n; ++i) CK(cudaGraphLaunch(d->exec, s));
    CK(cudaMemcpyAsync(tokens_host, d->d_hist, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    d->n_past += (int32_t)n;
    return check_dev_status(d);
}

// Greedy verification of a draft (the speculative-decoding verify step, tools/decode_main.cpp:329-400
// of the reference): the model is run on first_token, draft[0], ..., draft[n_draft-1] teacher-forced
// from position n_past; draft[i] is accepted while it equals the model's greedy token after the
// previous input. Returns the number of accepted draft tokens and the model's own next token after
// the last accepted one; n_past moves past the accepted tokens only (the cache rows of rejected
// positions are overwritten by later steps). The positions are computed one after the other with
// the single-token launch plan (no host round trip in between).
int fl_b200_decoder_verify(fl_b200_decoder *d, int32_t first_token, const int32_t *draft, uint32_t n_draft,
                           uint32_t *n_accepted_out, int32_t *next_token_out) {
    if (!d || !draft || !n_accepted_out || !next_token_out) return set_err(FL_B200_ERR_ARG, "decoder_verify: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_verify: finalize first");
    const uint32_t n = n_draft + 1;   // inputs: the last accepted token and the draft
    if (n_draft == 0 || n > d->hist_cap) return set_err(FL_B200_ERR_ARG, "decoder_verify: draft length %u outside 1..%u", n_draft, d->hist_cap - 1);
    if ((uint64_t)d->n_past + n > d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_verify: kv full (%d + %u > %u)", d->n_past, n, d->c.max_kv);
    if (first_token < 0 || (uint32_t)first_token >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_verify: token outside the vocabulary");
    for (uint32_t i = 0; i < n_draft; ++i)
        if (draft[i] < 0 || (uint32_t)draft[i] >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_verify: draft token %u outside the vocabulary", i);
    cudaStream_t s = d->ctx->stream;
    std::vector<int32_t> got(n);
    CK(cudaMemcpyAsync(d->d_forced, draft, (size_t)n_draft * 4, cudaMemcpyHostToDevice, s));   // forced[k] follows input k
    d->h_pin[0] = first_token; d->h_pin[1] = 0; d->h_pin[2] = d->n_past; d->h_pin[3] = 0; d->h_pin[4] = 0; d->h_pin[5] = 1;
    CK(cudaMemcpyAsync(d->d_token, d->h_pin, 24, cudaMemcpyHostToDevice, s));
    for (uint32_t i = 0; i < n; ++i) CK(cudaGraphLaunch(d->exec, s));
    CK(cudaMemcpyAsync(got.data(), d->d_hist, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
    CK(cudaMemsetAsync(d->d_use_forced, 0, 4, s));
    CK(cudaStreamSynchronize(s));
    uint32_t acc = 0;
    while (acc < n_draft && got[acc] == draft[acc]) ++acc;
    *n_accepted_out = acc;
    *next_token_out = got[acc];
    d->n_past += (int32_t)acc + 1;
    return check_dev_status(d);
}

// ---- Decoder::step_batch (src/model/decoder.h:64-70): m tokens at positions n_past .. n_past + m - 1 in one
// pass. Every weight tensor is walked once per pass where the multi-column kernel takes it (Q4_K, up to 8
// columns) and once per token otherwise; the attention launch covers all m positions, position b attending
// n_past + b + 1 keys of the one cache (the rows of this pass are appended first). ----
// Passes of fewer tokens than this run as teacher-forced single steps (FLB_BATCH_MIN overrides; 1 = always the batch pass).
static const uint32_t kBatchMin = getenv("FLB_BATCH_MIN") ? (uint32_t)atoi(getenv("FLB_BATCH_MIN")) : 4u;

static int batch_alloc(fl_b200_decoder *d) {
    if (d->b.ready) return FL_B200_OK;
    const fl_b200_llama_cfg &c = d->c;
    const size_t M = FL_B200_MAX_BATCH, E = c.n_embd, QD = (size_t)d->Hq * c.head_dim, KD = (size_t)d->Hkv * c.head_dim;
    CK(cudaMalloc(&d->b.x, M * E * 4)); CK(cudaMalloc(&d->b.xn, M * E * 4));
    CK(cudaMalloc(&d->b.q, M * QD * 4)); CK(cudaMalloc(&d->b.k, M * KD * 4)); CK(cudaMalloc(&d->b.v, M * KD * 4));
    CK(cudaMalloc(&d->b.att, M * QD * 4));
    CK(cudaMalloc(&d->b.g, M * (size_t)d->F * 4)); CK(cudaMalloc(&d->b.u, M * (size_t)d->F * 4));
    CK(cudaMalloc(&d->b.logits, M * (size_t)d->V * 4)); CK(cudaMalloc(&d->b.margin, M * 4));
    size_t part = 0;
    for (uint32_t m = 1; m <= M; ++m)
        part = std::max(part, attn_part_floats(d->Hq, m, attn_pick_splits(d->Hkv, m, c.max_kv, d->ctx->sms)));
    CK(cudaMalloc(&d->b.part, part * sizeof(float)));
    if (d->tp_size > 1) {
        CK(cudaMalloc(&d->b.partial, M * E * 4));
        CK(cudaMalloc(&d->b.top3, M * 16));
    }
    CK(cudaMalloc(&d->b.io, 3 * FL_B200_MAX_BATCH * sizeof(int32_t)));
    CK(cudaMalloc(&d->b.tickets, (size_t)d->Hkv * M * sizeof(uint32_t)));
    CK(cudaMemset(d->b.tickets, 0, (size_t)d->Hkv * M * sizeof(uint32_t)));
    CK(cudaMallocHost(&d->b.h_io, 4 * FL_B200_MAX_BATCH * sizeof(int32_t)));
    d->b.ready = true;
    return FL_B200_OK;
}

// seqs: the m tokens belong to m independent sequences (token i -> sequence i at its own position, its own cache)
// instead of m consecutive positions of the one sequence.
static int enqueue_batch(fl_b200_decoder *d, uint32_t m, cudaStream_t s, bool seqs = false) {
    const fl_b200_llama_cfg &c = d->c;
    fl_b200_ctx *ctx = d->ctx;
    const uint32_t E = c.n_embd, D = c.head_dim, QD = d->Hq * D, KD = d->Hkv * D, F = d->F, V = d->V;
    const float theta_scale = powf(c.rope_base, -2.0f / (float)D);
    static const int kBatchPdl = getenv("FLB_BATCH_PDL") ? atoi(getenv("FLB_BATCH_PDL")) : 1;
    auto &b = d->b;
    const bool tp = d->tp_size > 1;
    // x[i] += sum over the ranks of partial[i], token by token, through the decoder's exchange buffers (rank order)
    auto sum_ranks = [&]() -> int {
        for (uint32_t i = 0; i < m; ++i) {
            AllReduceArgs r{};
            for (uint32_t p = 0; p < d->tp_size; ++p) r.peers[p] = d->peers[p];
            r.in = b.partial + (size_t)i * E; r.resid = b.x + (size_t)i * E; r.out = b.x + (size_t)i * E; r.n = E;
            r.rank = d->tp_rank; r.world = d->tp_size; r.st = CommState{d->comm_state}; r.status = ctx->status; r.wait_ns = ctx->wait_limit_ns;
            CK(launch_allreduce_resid(r, s, false));
        }
        return FL_B200_OK;
    };
    const int32_t *tok = b.io, *pos = b.io + FL_B200_MAX_BATCH;
    int32_t *next = b.io + 2 * FL_B200_MAX_BATCH;
    for (uint32_t i = 0; i < m; ++i)
        CK(launch_embed(d->tok_embd.fmt, d->tok_embd.w, tok + i, E, b.x + (size_t)i * E, s));
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        const Tensor *w = &d->lw[(size_t)l * 7];
        CK(launch_rmsnorm(b.x, d->attn_norm[l], b.xn, c.eps, E, s, m, E));
        if (int rc = matmul(ctx, w[FL_B200_T_WQ].fmt, w[FL_B200_T_WQ].w, QD, E, b.xn, m, E, b.q, QD, 0, 0, nullptr, 0, kBatchPdl)) return rc;
        // the converted activations of the multi-column kernel are reused while the weight format stays the same
        if (int rc = matmul(ctx, w[FL_B200_T_WK].fmt, w[FL_B200_T_WK].w, KD, E, b.xn, m, E, b.k, KD, 0, 0, nullptr, 0, kBatchPdl, nullptr,
                            w[FL_B200_T_WK].fmt == w[FL_B200_T_WQ].fmt)) return rc;
        if (int rc = matmul(ctx, w[FL_B200_T_WV].fmt, w[FL_B200_T_WV].w, KD, E, b.xn, m, E, b.v, KD, 0, 0, nullptr, 0, kBatchPdl, nullptr,
                            w[FL_B200_T_WV].fmt == w[FL_B200_T_WK].fmt)) return rc;
        {   // rotate q and k of every token by its own position, append k and v
            RopeAppendArgs r{};
            r.q = b.q; r.k = b.k; r.v = b.v; r.kcache = seqs ? d->sq.kc[l] : d->kc[l]; r.vcache = seqs ? d->sq.vc[l] : d->vc[l]; r.pos = pos;
            r.seq_elems = seqs ? (uint64_t)d->Hkv * c.max_kv * D : 0;
            r.n_q_head = d->Hq; r.n_kv_head = d->Hkv; r.head_dim = D; r.kv_stride = c.max_kv; r.theta_scale = theta_scale;
            r.n_tok = m; r.q_tok_stride = QD; r.kv_tok_stride = KD;
            CK(launch_rope_append(r, s));
        }
        {
            AttnArgs a{};
            a.q = b.q; a.k = seqs ? d->sq.kc[l] : d->kc[l]; a.v = seqs ? d->sq.vc[l] : d->vc[l]; a.out = b.att; a.part = b.part; a.tickets = b.tickets;
            a.pos = pos; a.kv_len = 0; a.kv_len_step = seqs ? 0 : 1; a.shared_kv = seqs ? 0 : 1; a.pos_stride = seqs ? 1 : 0;
            a.kv_stride = c.max_kv; a.batch_stride = (uint64_t)d->Hkv * c.max_kv * D;
            a.n_q_head = d->Hq; a.n_kv_head = d->Hkv; a.batch = m;
            a.n_splits = attn_pick_splits(d->Hkv, m, c.max_kv, ctx->sms);
            a.scale = 1.0f / sqrtf((float)D); a.status = ctx->status;
            CK(attn_make_maps(a));
            CK(launch_attn_decode(a, s));
        }
        // x += Wo att (the residual stays in place); tensor parallel: the ranks' partial products are summed per token
        if (!tp) {
            if (int rc = matmul(ctx, w[FL_B200_T_WO].fmt, w[FL_B200_T_WO].w, E, QD, b.att, m, QD, b.x, E, 1, w[FL_B200_T_WO].pitch, nullptr, 0, kBatchPdl)) return rc;
        } else {
            if (int rc = matmul(ctx, w[FL_B200_T_WO].fmt, w[FL_B200_T_WO].w, E, QD, b.att, m, QD, b.partial, E, 0, w[FL_B200_T_WO].pitch, nullptr, 0, kBatchPdl)) return rc;
            if (int rc = sum_ranks()) return rc;
        }
        CK(launch_rmsnorm(b.x, d->ffn_norm[l], b.xn, c.eps, E, s, m, E));
        if (d->moe[l]) {   // every expert once for the tokens that chose it, then x += the block's output
            if (int rc = moe_enqueue_tokens(d->moe[l], b.xn, m, b.q, nullptr)) return rc;
            CK(launch_add2(b.x, b.q, b.x, m * E, s));
            continue;
        }
        if (int rc = matmul(ctx, w[FL_B200_T_GATE].fmt, w[FL_B200_T_GATE].w, F, E, b.xn, m, E, b.g, F, 0, 0, nullptr, 0, kBatchPdl)) return rc;
        if (int rc = matmul(ctx, w[FL_B200_T_UP].fmt, w[FL_B200_T_UP].w, F, E, b.xn, m, E, b.u, F, 0, 0, nullptr, 0, kBatchPdl, nullptr,
                            w[FL_B200_T_UP].fmt == w[FL_B200_T_GATE].fmt)) return rc;
        // SiLU(g) * u is built while the down projection's activation is converted (streaming formats); other formats
        // get the product from a launch of its own
        const bool fuse_silu = (w[FL_B200_T_DOWN].fmt == FL_B200_Q4_K || w[FL_B200_T_DOWN].fmt == FL_B200_Q6_K || w[FL_B200_T_DOWN].fmt == FL_B200_Q8_0) &&
                               row_bytes(w[FL_B200_T_DOWN].fmt, F) % 16 == 0;   // rows the streaming kernels take
        if (!fuse_silu) CK(launch_silu_mul(b.g, b.u, b.g, m * F, s));
        const float *down_x2 = fuse_silu ? b.u : nullptr;
        if (!tp) {
            if (int rc = matmul(ctx, w[FL_B200_T_DOWN].fmt, w[FL_B200_T_DOWN].w, E, F, b.g, m, F, b.x, E, 1, w[FL_B200_T_DOWN].pitch, nullptr, 0, kBatchPdl, down_x2)) return rc;
        } else {
            if (int rc = matmul(ctx, w[FL_B200_T_DOWN].fmt, w[FL_B200_T_DOWN].w, E, F, b.g, m, F, b.partial, E, 0, w[FL_B200_T_DOWN].pitch, nullptr, 0, kBatchPdl, down_x2)) return rc;
            if (int rc = sum_ranks()) return rc;
        }
    }
    CK(launch_rmsnorm(b.x, d->out_norm, b.xn, c.eps, E, s, m, E));
    if (int rc = matmul(ctx, d->output.fmt, d->output.w, V, E, b.xn, m, E, b.logits, V, 0, 0, nullptr, 0, kBatchPdl)) return rc;
    for (uint32_t i = 0; i < m; ++i) {
        CK(launch_argmax(b.logits + (size_t)i * V, V, next + i, b.margin + i, ctx->argmax_scratch, ctx->argmax_ticket, ctx->sms, s,
                         false, tp ? b.top3 + 4 * i : nullptr));
        if (tp) {   // merge the ranks' (best, index, runner-up) of this position: the same token on every rank
            TopExchangeArgs x{};
            for (uint32_t p = 0; p < d->tp_size; ++p) x.peers[p] = d->peers[p];
            x.top3 = b.top3 + 4 * i; x.index_base = d->tp_rank * V; x.out_idx = next + i; x.out_margin = b.margin + i;
            x.rank = d->tp_rank; x.world = d->tp_size; x.st = CommState{d->comm_state}; x.status = ctx->status; x.wait_ns = ctx->wait_limit_ns;
            CK(launch_argmax_exchange(x, s, false));
        }
    }
    return FL_B200_OK;
}

int fl_b200_decoder_step_batch(fl_b200_decoder *d, const int32_t *toks, uint32_t m, int32_t *outs, float *margins) {
    if (!d || !toks || !outs) return set_err(FL_B200_ERR_ARG, "decoder_step_batch: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_step_batch: finalize first");
    if (m == 0 || m > FL_B200_MAX_BATCH) return set_err(FL_B200_ERR_ARG, "decoder_step_batch: m %u outside 1..%d", m, FL_B200_MAX_BATCH);
    if ((uint64_t)d->n_past + m > d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_step_batch: kv full (%d + %u > %u)", d->n_past, m, d->c.max_kv);
    for (uint32_t i = 0; i < m; ++i)
        if (toks[i] < 0 || (uint32_t)toks[i] >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_step_batch: token %d outside the vocabulary", toks[i]);
    cudaStream_t s = d->ctx->stream;
    CK(cudaSetDevice(d->ctx->device));
    if (int rc = batch_alloc(d)) return rc;
    if (m < kBatchMin) {
        // Few tokens: the fused single-token step, teacher-forced m times on the device, is faster than the batch
        // pass (measured at the 8B shape: 2.1 / 4.3 / 6.4 ms against 3.5 / 5.4 / 6.6 ms for m = 1 / 2 / 3).
        if (m > 1) CK(cudaMemcpyAsync(d->d_forced, toks + 1, (size_t)(m - 1) * 4, cudaMemcpyHostToDevice, s));   // forced[k] follows input k
        d->h_pin[0] = toks[0]; d->h_pin[1] = 0; d->h_pin[2] = d->n_past; d->h_pin[3] = 0; d->h_pin[4] = 0; d->h_pin[5] = 1;
        CK(cudaMemcpyAsync(d->d_token, d->h_pin, 24, cudaMemcpyHostToDevice, s));
        for (uint32_t i = 0; i < m; ++i) {
            CK(cudaGraphLaunch(d->exec, s));
            CK(cudaMemcpyAsync(d->b.logits + (size_t)i * d->V, d->logits, (size_t)d->V * 4, cudaMemcpyDeviceToDevice, s));
        }
        CK(cudaMemcpyAsync(d->b.h_io + 2 * FL_B200_MAX_BATCH, d->d_hist, (size_t)m * 4, cudaMemcpyDeviceToHost, s));
        CK(cudaMemcpyAsync(d->b.h_io + 3 * FL_B200_MAX_BATCH, d->d_margin_hist, (size_t)m * 4, cudaMemcpyDeviceToHost, s));
        CK(cudaMemsetAsync(d->d_use_forced, 0, 4, s));
        CK(cudaStreamSynchronize(s));
        for (uint32_t i = 0; i < m; ++i) {
            outs[i] = d->b.h_io[2 * FL_B200_MAX_BATCH + i];
            if (margins) memcpy(&margins[i], &d->b.h_io[3 * FL_B200_MAX_BATCH + i], 4);
        }
        d->n_past += (int32_t)m;
        d->b.last_m = m;
        return check_dev_status(d);
    }
    if (!d->b.exec[m]) {
        CK(cudaStreamSynchronize(s));
        CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_batch(d, m, s);
        cudaGraph_t g = nullptr;
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        CK(e);
        d->b.graph[m] = g;
        CK(cudaGraphInstantiate(&d->b.exec[m], g, 0));
    }
    for (uint32_t i = 0; i < FL_B200_MAX_BATCH; ++i) {
        d->b.h_io[i] = i < m ? toks[i] : 0;
        d->b.h_io[FL_B200_MAX_BATCH + i] = d->n_past + (int32_t)i;
    }
    CK(cudaMemcpyAsync(d->b.io, d->b.h_io, 2 * FL_B200_MAX_BATCH * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    CK(cudaGraphLaunch(d->b.exec[m], s));
    CK(cudaMemcpyAsync(d->b.h_io + 2 * FL_B200_MAX_BATCH, d->b.io + 2 * FL_B200_MAX_BATCH, FL_B200_MAX_BATCH * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CK(cudaMemcpyAsync(d->b.h_io + 3 * FL_B200_MAX_BATCH, d->b.margin, FL_B200_MAX_BATCH * sizeof(float), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    for (uint32_t i = 0; i < m; ++i) {
        outs[i] = d->b.h_io[2 * FL_B200_MAX_BATCH + i];
        if (margins) memcpy(&margins[i], &d->b.h_io[3 * FL_B200_MAX_BATCH + i], 4);
    }
    d->n_past += (int32_t)m;
    d->b.last_m = m;
    return check_dev_status(d);
}

// ---- independent sequences in lock step: one pass feeds one token to each of n sequences (each with its own cache and
// position); every tensor is walked once per 8 sequences, the attention runs per sequence over its own keys. ----
int fl_b200_decoder_seqs_init(fl_b200_decoder *d, uint32_t n_seq) {
    if (!d) return set_err(FL_B200_ERR_ARG, "decoder_seqs_init: null");
    if (n_seq < 2 || n_seq > FL_B200_MAX_BATCH) return set_err(FL_B200_ERR_ARG, "decoder_seqs_init: %u sequences outside 2..%d", n_seq, FL_B200_MAX_BATCH);
    if (d->tp_size > 1) return set_err(FL_B200_ERR_ARG, "decoder_seqs_init: one GPU only");
    if (d->sq.n) return set_err(FL_B200_ERR_STATE, "decoder_seqs_init: already set up for %u sequences", d->sq.n);
    const fl_b200_llama_cfg &c = d->c;
    CK(cudaSetDevice(d->ctx->device));
    const size_t bytes = (size_t)n_seq * d->Hkv * c.max_kv * c.head_dim * sizeof(__half);
    d->sq.kc.assign(c.n_layer, nullptr);
    d->sq.vc.assign(c.n_layer, nullptr);
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        CK(cudaMalloc(&d->sq.kc[l], bytes));
        CK(cudaMalloc(&d->sq.vc[l], bytes));
        CK(cudaMemsetAsync(d->sq.kc[l], 0, bytes, d->ctx->stream));
        CK(cudaMemsetAsync(d->sq.vc[l], 0, bytes, d->ctx->stream));
    }
    CK(cudaStreamSynchronize(d->ctx->stream));
    d->sq.n = n_seq;
    return FL_B200_OK;
}

int fl_b200_decoder_seqs_kv(fl_b200_decoder *d, uint32_t layer, uint32_t seq, uint16_t **k_out, uint16_t **v_out) {
    if (!d || !k_out || !v_out) return set_err(FL_B200_ERR_ARG, "decoder_seqs_kv: null");
    if (layer >= d->c.n_layer || seq >= d->sq.n) return set_err(FL_B200_ERR_ARG, "decoder_seqs_kv: layer %u / sequence %u out of range", layer, seq);
    const size_t per_seq = (size_t)d->Hkv * d->c.max_kv * d->c.head_dim;
    *k_out = reinterpret_cast<uint16_t *>(d->sq.kc[layer] + seq * per_seq);
    *v_out = reinterpret_cast<uint16_t *>(d->sq.vc[layer] + seq * per_seq);
    return FL_B200_OK;
}

int fl_b200_decoder_seqs_set_pos(fl_b200_decoder *d, uint32_t seq, int32_t n_past) {
    if (!d || seq >= d->sq.n || n_past < 0 || (uint32_t)n_past > d->c.max_kv) return set_err(FL_B200_ERR_ARG, "decoder_seqs_set_pos: out of range");
    d->sq.pos[seq] = n_past;
    return FL_B200_OK;
}

int fl_b200_decoder_seqs_pos(fl_b200_decoder *d, uint32_t seq, int32_t *n_past_out) {
    if (!d || !n_past_out || seq >= d->sq.n) return set_err(FL_B200_ERR_ARG, "decoder_seqs_pos: out of range");
    *n_past_out = d->sq.pos[seq];
    return FL_B200_OK;
}

int fl_b200_decoder_seqs_step(fl_b200_decoder *d, const int32_t *toks, int32_t *outs, float *margins) {
    if (!d || !toks || !outs) return set_err(FL_B200_ERR_ARG, "decoder_seqs_step: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_seqs_step: finalize first");
    const uint32_t m = d->sq.n;
    if (m == 0) return set_err(FL_B200_ERR_STATE, "decoder_seqs_step: fl_b200_decoder_seqs_init first");
    for (uint32_t i = 0; i < m; ++i) {
        if (toks[i] < 0 || (uint32_t)toks[i] >= d->c.n_vocab) return set_err(FL_B200_ERR_ARG, "decoder_seqs_step: token %d outside the vocabulary", toks[i]);
        if ((uint32_t)d->sq.pos[i] >= d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_seqs_step: kv of sequence %u full", i);
    }
    cudaStream_t s = d->ctx->stream;
    CK(cudaSetDevice(d->ctx->device));
    if (int rc = batch_alloc(d)) return rc;
    if (!d->sq.exec) {
        CK(cudaStreamSynchronize(s));
        CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_batch(d, m, s, true);
        cudaGraph_t g = nullptr;
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (rc) { if (g) cudaGraphDestroy(g); return rc; }
        CK(e);
        d->sq.graph = g;
        CK(cudaGraphInstantiate(&d->sq.exec, g, 0));
    }
    for (uint32_t i = 0; i < FL_B200_MAX_BATCH; ++i) {
        d->b.h_io[i] = i < m ? toks[i] : 0;
        d->b.h_io[FL_B200_MAX_BATCH + i] = i < m ? d->sq.pos[i] : 0;
    }
    CK(cudaMemcpyAsync(d->b.io, d->b.h_io, 2 * FL_B200_MAX_BATCH * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    CK(cudaGraphLaunch(d->sq.exec, s));
    CK(cudaMemcpyAsync(d->b.h_io + 2 * FL_B200_MAX_BATCH, d->b.io + 2 * FL_B200_MAX_BATCH, FL_B200_MAX_BATCH * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CK(cudaMemcpyAsync(d->b.h_io + 3 * FL_B200_MAX_BATCH, d->b.margin, FL_B200_MAX_BATCH * sizeof(float), cudaMemcpyDeviceToHost, s));
    CK(cudaStreamSynchronize(s));
    for (uint32_t i = 0; i < m; ++i) {
        outs[i] = d->b.h_io[2 * FL_B200_MAX_BATCH + i];
        if (margins) memcpy(&margins[i], &d->b.h_io[3 * FL_B200_MAX_BATCH + i], 4);
        d->sq.pos[i] += 1;
    }
    d->b.last_m = m;   // fl_b200_decoder_batch_logits(i): the logits of sequence i
    return check_dev_status(d);
}

int fl_b200_decoder_batch_logits(fl_b200_decoder *d, uint32_t index, float *out) {
    if (!d || !out) return set_err(FL_B200_ERR_ARG, "decoder_batch_logits: null");
    if (!d->b.ready || index >= d->b.last_m) return set_err(FL_B200_ERR_STATE, "decoder_batch_logits: position %u of a pass of %u", index, d->b.last_m);
    return fl_b200_download(d->ctx, out, d->b.logits + (size_t)index * d->V, (size_t)d->V * 4);
}

int fl_b200_decoder_logits(fl_b200_decoder *d, float *out) {
    if (!d || !out) return set_err(FL_B200_ERR_ARG, "decoder_logits: null");
    return fl_b200_download(d->ctx, out, d->logits, (size_t)d->V * 4);   // this rank's slice of the vocabulary
}

int fl_b200_decoder_margin(fl_b200_decoder *d, float *out) {
    if (!d || !out) return set_err(FL_B200_ERR_ARG, "decoder_margin: null");
    return fl_b200_download(d->ctx, out, d->d_margin, 4);
}

int fl_b200_decoder_tap(fl_b200_decoder *d, int which, float *out) {
    if (!d || !out) return set_err(FL_B200_ERR_ARG, "decoder_tap: null");
    const fl_b200_llama_cfg &c = d->c;
    const uint32_t QD = d->Hq * c.head_dim, KD = d->Hkv * c.head_dim;
    const float *src = nullptr;
    size_t n = 0;
    switch (which) {
    case 0: src = d->xa; n = c.n_embd; break;        // hidden state after the last layer
    case 1:                                          // final normed vector: made here from the hidden state (the head's
        src = d->xn_final; n = c.n_embd;             // launch takes the norm inside its prologue and keeps no copy)
        if (cudaError_t e = launch_rmsnorm(d->xa, d->out_norm, d->xn_final, c.eps, c.n_embd, d->ctx->stream, 1, c.n_embd); e != cudaSuccess)
            return set_err(FL_B200_ERR_CUDA, "decoder_tap: %s", cudaGetErrorString(e));
        break;
    case 2: src = d->q; n = QD; break;               // last layer: q (before RoPE: the attention kernel rotates it)
    case 3: src = d->v; n = KD; break;               // last layer: v
    case 4: src = d->att; n = QD; break;             // last layer: attention output
    case 5: src = d->xb; n = c.n_embd; break;        // last layer: residual after attention
    case 6: src = d->g; n = d->F; break;           // last layer: silu(gate) * up (gate alone if the formats of gate and up differ)
    case 7: src = d->u; n = d->F; break;           // last layer: up (only written if the formats of gate and up differ)
    default: return set_err(FL_B200_ERR_ARG, "decoder_tap: unknown tap %d", which);
    }
    return fl_b200_download(d->ctx, out, src, n * 4);
}

// Times `reps` replays of one kernel class of the step (the same launches, in
// step order, with the decoder's real weights and buffers; the other classes
// are left out, so the activations are stale and the results meaningless) with
// CUDA events on the context's stream. The position used is the current n_past.
int fl_b200_decoder_time_class(fl_b200_decoder *d, uint32_t kernel_class, uint32_t reps, float *ms_per_step,
                               uint32_t *launches_per_step) {
    if (!d || !ms_per_step || !launches_per_step) return set_err(FL_B200_ERR_ARG, "decoder_time_class: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_time_class: finalize first");
    if (kernel_class == 0 || kernel_class > K_ALL || reps == 0) return set_err(FL_B200_ERR_ARG, "decoder_time_class: bad class / reps");
    if ((uint32_t)d->n_past >= d->c.max_kv) return set_err(FL_B200_ERR_STATE, "decoder_time_class: kv full");
    cudaStream_t s = d->ctx->stream;
    d->h_pin[0] = 0; d->h_pin[1] = 0; d->h_pin[2] = d->n_past; d->h_pin[3] = 0; d->h_pin[4] = 0; d->h_pin[5] = 0;
    CK(cudaMemcpyAsync(d->d_token, d->h_pin, 24, cudaMemcpyHostToDevice, s));
    // Bit 4 keeps the mask different from K_ALL, so the advance kernel is left
    // out and the position stays put over the replays.
    const uint32_t m = kernel_class | 16u;
    cudaGraph_t g = nullptr;
    cudaGraphExec_t ge = nullptr;
    CK(cudaStreamSynchronize(s));
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    uint32_t n = 0;
    int rc = enqueue_step(d, s, &n, m);
    cudaError_t e = cudaStreamEndCapture(s, &g);
    if (rc) { if (g) cudaGraphDestroy(g); return rc; }
    CK(e);
    CK(cudaGraphInstantiate(&ge, g, 0));
    CK(cudaGraphLaunch(ge, s));   // warm-up
    CK(cudaEventRecord(d->ctx->ev0, s));
    for (uint32_t i = 0; i < reps; ++i) CK(cudaGraphLaunch(ge, s));
    CK(cudaEventRecord(d->ctx->ev1, s));
    CK(cudaEventSynchronize(d->ctx->ev1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, d->ctx->ev0, d->ctx->ev1));
    cudaGraphExecDestroy(ge);
    cudaGraphDestroy(g);
    *ms_per_step = ms / (float)reps;
    *launches_per_step = n;
    return check_dev_status(d);
}

// Diagnostics (FLB_TRACE=1 in the environment at finalize): per launch of the
// last fl_b200_decoder_step, four %globaltimer values in ns: earliest kernel
// entry, earliest point after the dependency wait, latest end of the prologue,
// latest exit. Only the matvec and attention kernels record; the other entries
// stay {~0, ~0, 0, 0}. Returns the number of records through n_out (0 when
// tracing is off).
int fl_b200_decoder_trace(fl_b200_decoder *d, uint64_t *host_out, uint32_t cap_records, uint32_t *n_out) {
    if (!d || !n_out) return set_err(FL_B200_ERR_ARG, "decoder_trace: null");
    *n_out = 0;
    if (!d->trace) return FL_B200_OK;
    const uint32_t n = d->launches < d->trace_n ? d->launches : d->trace_n;
    if (!host_out || cap_records < n) return set_err(FL_B200_ERR_ARG, "decoder_trace: need room for %u records", n);
    *n_out = n;
    return fl_b200_download(d->ctx, host_out, d->trace, (size_t)n * 4 * sizeof(uint64_t));
}

int fl_b200_decoder_launches_per_step(fl_b200_decoder *d, uint32_t *n) {
    if (!d || !n) return set_err(FL_B200_ERR_ARG, "decoder_launches_per_step: null");
    if (!d->finalized) return set_err(FL_B200_ERR_STATE, "decoder_launches_per_step: finalize first");
    *n = d->launches;
    return FL_B200_OK;
}

int fl_b200_decoder_bytes_per_step(fl_b200_decoder *d, int32_t pos, uint64_t *wb, uint64_t *kvb) {
    if (!d || !wb || !kvb) return set_err(FL_B200_ERR_ARG, "decoder_bytes_per_step: null");
    const fl_b200_llama_cfg &c = d->c;
    // this rank's share (the whole model on one GPU)
    const uint32_t E = c.n_embd, QD = d->Hq * c.head_dim, KD = d->Hkv * c.head_dim;
    uint64_t w = 0;
    for (uint32_t l = 0; l < c.n_layer; ++l) {
        const Tensor *t = &d->lw[(size_t)l * 7];
        w += (uint64_t)QD * row_bytes(t[FL_B200_T_WQ].fmt, E) + (uint64_t)KD * row_bytes(t[FL_B200_T_WK].fmt, E) +
             (uint64_t)KD * row_bytes(t[FL_B200_T_WV].fmt, E) + (uint64_t)E * row_bytes(t[FL_B200_T_WO].fmt, QD);
        if (d->moe[l]) w += moe_bytes_per_token(d->moe[l]);   // the router and the selected experts
        else w += (uint64_t)d->F * row_bytes(t[FL_B200_T_GATE].fmt, E) + (uint64_t)d->F * row_bytes(t[FL_B200_T_UP].fmt, E) +
                  (uint64_t)E * row_bytes(t[FL_B200_T_DOWN].fmt, d->F);
        w += 2ull * E * 4;   // the two norm vectors
    }
    w += (uint64_t)d->V * row_bytes(d->output.fmt, E) + (uint64_t)E * 4;
    *wb = w;
    *kvb = (uint64_t)c.n_layer * 2ull * (uint64_t)(pos + 1) * KD * 2ull;
    return FL_B200_OK;
}

} // extern "C"
