/* Test infrastructure, not product code.
 *
 * CPU oracle for one greedy decode step of a Llama-shape decoder (RMSNorm ->
 * Q/K/V matvec -> RoPE -> KV append -> GQA attention -> O matvec + residual ->
 * RMSNorm -> SwiGLU FFN + residual, then output norm, head matvec, argmax),
 * sequenced over an operator table (flo_ops.h) so that the same driver runs on
 * the reference's own operators or on the plain-C port.
 *
 * The reference ships only a deepseek2 graph builder
 * (src/model/decoder.cpp:751-1083); this file wires the same operator kinds in
 * the Llama order. Where the reference's operators cannot express the shape, a
 * thin adapter is used and nothing inside the operator changes:
 *   - grouped-query attention: fl_op_attn_head indexes q + head*dk,
 *     k + (j*n_head + head)*dk and out + head*dv
 *     (src/runtime/decode_params.h:186-190, :221), so calling it with
 *     n_head = n_kv_head, head = hkv and q/out pointers moved back by
 *     (hq - hkv) heads makes query head hq attend over KV head hkv;
 *   - f16 KV cache: the cache the operator reads is an f32 mirror whose every
 *     value is exactly representable in f16; a newly appended row is rounded
 *     through f2h/h2f (src/runtime/quants.h:333-356, :40-64) right after
 *     KV_APPEND, which is what storing it in an f16 cache does.
 * Per-token host work follows Decoder::step_batch
 * (src/model/decoder.cpp:1176-1264): dequantise the embedding row, zero the
 * accumulate slots, run the operators, argmax with strict '>' (lowest id wins
 * ties) and the top1-top2 margin.
 *
 * Rows of a matvec and heads of attention are independent, so running them on
 * several threads (OpenMP) does not change a single bit of the result.
 */
#include "flo_ops.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

uint64_t flo_row_bytes(int fmt, uint32_t cols);

typedef struct {
    uint32_t n_layer, n_embd, n_head, n_kv_head, head_dim, n_ff, n_vocab, max_kv;
    float rope_base, eps;
} flo_llama_cfg;

enum { T_WQ, T_WK, T_WV, T_WO, T_GATE, T_UP, T_DOWN, T_PER_LAYER };
enum { G_TOK_EMBD = 0, G_OUTPUT = 1 };

typedef struct { int fmt; const uint8_t *w; } tensor_t;

/* A mixture-of-experts feed-forward block in place of a layer's dense one (the chain the reference's graph builder
 * emits per MoE layer, src/model/decoder.cpp:925-1045: router matvec -> ROUTER_SEL -> per selected expert gate, up,
 * SILU_MUL, down through STREAM_DOT_IDX -> WMERGE with the residual). Experts are stacked row-wise in each tensor. */
typedef struct {
    uint32_t n_expert, top_k, norm, n_ff;
    float scale;
    const float *router;      /* [n_expert][n_embd] f32 */
    int fmt_gu, fmt_d;
    const uint8_t *wg, *wu, *wd;
} moe_t;

typedef struct flo_llama {
    flo_llama_cfg c;
    moe_t *moe;               /* n_layer; n_expert == 0: dense layer */
    float *mo_logits, *mo_gates, *mo_parts, *mo_g, *mo_u, *mo_h;
    uint32_t *mo_ids;
    tensor_t *lw;             /* n_layer * T_PER_LAYER */
    const float **attn_norm;  /* n_layer */
    const float **ffn_norm;   /* n_layer */
    tensor_t tok_embd, output;
    const float *out_norm;
    float **kc, **vc;         /* per layer f32 mirror [max_kv][n_kv_head][head_dim] */
    int32_t n_past;
    /* activations */
    float *x, *xn, *q, *kvb, *k, *v, *att, *o, *x1, *g, *u, *h, *dn, *logits, *scratch;
    float margin;
} flo_llama;

static float *falloc(size_t n) { return (float *)calloc(n ? n : 1, sizeof(float)); }

flo_llama *flo_llama_create(const flo_llama_cfg *cfg) {
    flo_llama *m = (flo_llama *)calloc(1, sizeof(*m));
    m->c = *cfg;
    const flo_llama_cfg *c = &m->c;
    m->lw = (tensor_t *)calloc((size_t)c->n_layer * T_PER_LAYER, sizeof(tensor_t));
    m->attn_norm = (const float **)calloc(c->n_layer, sizeof(float *));
    m->ffn_norm = (const float **)calloc(c->n_layer, sizeof(float *));
    m->kc = (float **)calloc(c->n_layer, sizeof(float *));
    m->vc = (float **)calloc(c->n_layer, sizeof(float *));
    const size_t kvn = (size_t)c->max_kv * c->n_kv_head * c->head_dim;
    for (uint32_t l = 0; l < c->n_layer; ++l) {
        m->kc[l] = falloc(kvn);
        m->vc[l] = falloc(kvn);
    }
    const uint32_t qd = c->n_head * c->head_dim, kd = c->n_kv_head * c->head_dim;
    m->x = falloc(c->n_embd);  m->xn = falloc(c->n_embd);
    m->q = falloc(qd);         m->kvb = falloc(2 * (size_t)kd);
    m->k = falloc(kd);         m->v = falloc(kd);
    m->att = falloc(qd);       m->o = falloc(c->n_embd);
    m->x1 = falloc(c->n_embd); m->g = falloc(c->n_ff);
    m->u = falloc(c->n_ff);    m->h = falloc(c->n_ff);
    m->dn = falloc(c->n_embd); m->logits = falloc(c->n_vocab);
    m->scratch = falloc((size_t)c->n_head * c->max_kv);
    m->moe = (moe_t *)calloc(c->n_layer, sizeof(moe_t));
    return m;
}

void flo_llama_set_layer_moe(flo_llama *m, uint32_t layer, uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale,
                             uint32_t n_ff, const float *router, int fmt_gu, const uint8_t *wg, const uint8_t *wu,
                             int fmt_d, const uint8_t *wd) {
    moe_t *e = &m->moe[layer];
    e->n_expert = n_expert; e->top_k = top_k; e->norm = norm; e->scale = scale; e->n_ff = n_ff;
    e->router = router; e->fmt_gu = fmt_gu; e->fmt_d = fmt_d; e->wg = wg; e->wu = wu; e->wd = wd;
    if (!m->mo_logits) {   /* scratch for the widest block the tests build */
        m->mo_logits = falloc(1024); m->mo_gates = falloc(64); m->mo_ids = (uint32_t *)calloc(64, sizeof(uint32_t));
        m->mo_parts = falloc((size_t)64 * m->c.n_embd);
        m->mo_g = falloc(65536); m->mo_u = falloc(65536); m->mo_h = falloc(65536);
    }
}

void flo_llama_destroy(flo_llama *m) {
    if (!m) return;
    for (uint32_t l = 0; l < m->c.n_layer; ++l) { free(m->kc[l]); free(m->vc[l]); }
    free(m->kc); free(m->vc); free(m->lw); free(m->attn_norm); free(m->ffn_norm);
    free(m->x); free(m->xn); free(m->q); free(m->kvb); free(m->k); free(m->v);
    free(m->att); free(m->o); free(m->x1); free(m->g); free(m->u); free(m->h);
    free(m->dn); free(m->logits); free(m->scratch);
    free(m->moe); free(m->mo_logits); free(m->mo_gates); free(m->mo_ids); free(m->mo_parts); free(m->mo_g); free(m->mo_u); free(m->mo_h);
    free(m);
}

void flo_llama_set_layer_tensor(flo_llama *m, uint32_t layer, int which, int fmt, const uint8_t *w) {
    m->lw[(size_t)layer * T_PER_LAYER + which].fmt = fmt;
    m->lw[(size_t)layer * T_PER_LAYER + which].w = w;
}
void flo_llama_set_layer_norms(flo_llama *m, uint32_t layer, const float *attn_norm, const float *ffn_norm) {
    m->attn_norm[layer] = attn_norm;
    m->ffn_norm[layer] = ffn_norm;
}
void flo_llama_set_global(flo_llama *m, int which, int fmt, const uint8_t *w) {
    tensor_t *t = which == G_TOK_EMBD ? &m->tok_embd : &m->output;
    t->fmt = fmt;
    t->w = w;
}
void flo_llama_set_out_norm(flo_llama *m, const float *w) { m->out_norm = w; }

/* Seed n_pos cached positions of one layer from an f16 cache laid out
 * [n_kv_head][kv_stride][head_dim] (the layout the GPU path keeps in HBM). */
void flo_llama_seed_kv(flo_llama *m, const flo_ops_t *ops, uint32_t layer,
                       const uint16_t *k16, const uint16_t *v16,
                       uint32_t n_pos, uint64_t kv_stride) {
    const uint32_t H = m->c.n_kv_head, D = m->c.head_dim;
    #pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < (int64_t)n_pos; ++p)
        for (uint32_t h = 0; h < H; ++h)
            for (uint32_t d = 0; d < D; ++d) {
                const size_t src = ((size_t)h * kv_stride + (size_t)p) * D + d;
                const size_t dst = ((size_t)p * H + h) * D + d;
                m->kc[layer][dst] = ops->h2f(k16[src]);
                m->vc[layer][dst] = ops->h2f(v16[src]);
            }
}

void flo_llama_set_n_past(flo_llama *m, int32_t n) { m->n_past = n; }
int32_t flo_llama_n_past(const flo_llama *m) { return m->n_past; }
const float *flo_llama_logits(const flo_llama *m) { return m->logits; }
float flo_llama_margin(const flo_llama *m) { return m->margin; }

/* Read back one cached position of one layer as f16, [n_kv_head][head_dim] for
 * K then V (to compare the rows a step appended with the GPU cache). */
void flo_llama_get_kv_row(const flo_llama *m, const flo_ops_t *ops, uint32_t layer,
                          uint32_t pos, uint16_t *k16, uint16_t *v16) {
    const size_t n = (size_t)m->c.n_kv_head * m->c.head_dim;
    for (size_t i = 0; i < n; ++i) {
        k16[i] = ops->f2h(m->kc[layer][(size_t)pos * n + i]);
        v16[i] = ops->f2h(m->vc[layer][(size_t)pos * n + i]);
    }
}

/* y[0..rows) = W x, as zeroed slots plus STREAM_DOT tiles of `tile` rows (the
 * reference emits 192-row tiles at batch width 1, decoder.cpp:713-716). */
static void matvec(const flo_ops_t *ops, tensor_t t, uint32_t rows, uint32_t cols,
                   const float *x, float *y) {
    const uint32_t tile = 192;
    const uint64_t rb = flo_row_bytes(t.fmt, cols);
    const int64_t n_tiles = (rows + tile - 1) / tile;
    memset(y, 0, (size_t)rows * sizeof(float));
    #pragma omp parallel for schedule(dynamic, 1)
    for (int64_t i = 0; i < n_tiles; ++i) {
        const uint32_t r0 = (uint32_t)i * tile;
        const uint32_t nr = rows - r0 < tile ? rows - r0 : tile;
        ops->stream_dot(t.fmt, t.w + (size_t)r0 * rb, nr, cols, x, 1, 0, y + r0, 0);
    }
}

/* GQA attention for all query heads at position pos through the one-head
 * operator; see the adapter note at the top of the file. */
void flo_attn_gqa(const flo_ops_t *ops, const float *q, const float *kc, const float *vc,
                  float *scratch, float *out, int32_t pos, float scale,
                  uint32_t n_head, uint32_t n_kv_head, uint32_t d, uint32_t max_kv) {
    const uint32_t grp = n_head / n_kv_head;
    #pragma omp parallel for schedule(dynamic, 1)
    for (int64_t hq = 0; hq < (int64_t)n_head; ++hq) {
        const uint32_t hkv = (uint32_t)hq / grp;
        const ptrdiff_t shift = ((ptrdiff_t)hq - (ptrdiff_t)hkv) * (ptrdiff_t)d;
        ops->attn_head(q + shift, kc, vc, scratch + (size_t)hq * max_kv, out + shift,
                       pos, scale, hkv, n_kv_head, d, d, max_kv);
    }
}

/* Same, from an f16 cache [n_kv_head][kv_stride][d]: widens it into the f32
 * layout the operator reads, then calls flo_attn_gqa. kv_len positions. */
void flo_attn_gqa_f16(const flo_ops_t *ops, const float *q, const uint16_t *k16,
                      const uint16_t *v16, uint64_t kv_stride, uint32_t kv_len,
                      float scale, uint32_t n_head, uint32_t n_kv_head, uint32_t d,
                      float *out) {
    const size_t n = (size_t)kv_len * n_kv_head * d;
    float *kc = falloc(n), *vc = falloc(n);
    float *scratch = falloc((size_t)n_head * kv_len);
    #pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < (int64_t)kv_len; ++p)
        for (uint32_t h = 0; h < n_kv_head; ++h)
            for (uint32_t i = 0; i < d; ++i) {
                const size_t src = ((size_t)h * kv_stride + (size_t)p) * d + i;
                const size_t dst = ((size_t)p * n_kv_head + h) * d + i;
                kc[dst] = ops->h2f(k16[src]);
                vc[dst] = ops->h2f(v16[src]);
            }
    flo_attn_gqa(ops, q, kc, vc, scratch, out, (int32_t)kv_len - 1, scale,
                 n_head, n_kv_head, d, kv_len);
    free(kc); free(vc); free(scratch);
}

/* One decode step: feed `token` at position n_past, return the greedy argmax. */
int32_t flo_llama_step(flo_llama *m, const flo_ops_t *ops, int32_t token) {
    const flo_llama_cfg *c = &m->c;
    const uint32_t E = c->n_embd, D = c->head_dim, H = c->n_head, HK = c->n_kv_head;
    const int32_t pos = m->n_past;
    const float scale = 1.0f / sqrtf((float)D);
    ops->dequant(m->tok_embd.fmt,
                 m->tok_embd.w + (size_t)token * flo_row_bytes(m->tok_embd.fmt, E),
                 0, E, m->x);
    for (uint32_t l = 0; l < c->n_layer; ++l) {
        const tensor_t *w = m->lw + (size_t)l * T_PER_LAYER;
        ops->rmsnorm(m->attn_norm[l], m->x, m->xn, c->eps, E);
        matvec(ops, w[T_WQ], H * D, E, m->xn, m->q);
        matvec(ops, w[T_WK], HK * D, E, m->xn, m->k);
        matvec(ops, w[T_WV], HK * D, E, m->xn, m->v);
        ops->rope(m->q, pos, H, D, 0, D, c->rope_base);
        ops->rope(m->k, pos, HK, D, 0, D, c->rope_base);
        for (uint32_t h = 0; h < HK; ++h) {
            memcpy(m->kvb + (size_t)h * 2 * D, m->k + (size_t)h * D, D * sizeof(float));
            memcpy(m->kvb + (size_t)h * 2 * D + D, m->v + (size_t)h * D, D * sizeof(float));
        }
        ops->kv_append(m->kvb, m->kc[l], m->vc[l], pos, HK, D, D, c->max_kv);
        {
            float *kr = m->kc[l] + (size_t)pos * HK * D, *vr = m->vc[l] + (size_t)pos * HK * D;
            for (uint32_t i = 0; i < HK * D; ++i) {
                kr[i] = ops->h2f(ops->f2h(kr[i]));
                vr[i] = ops->h2f(ops->f2h(vr[i]));
            }
        }
        flo_attn_gqa(ops, m->q, m->kc[l], m->vc[l], m->scratch, m->att, pos, scale,
                     H, HK, D, c->max_kv);
        matvec(ops, w[T_WO], E, H * D, m->att, m->o);
        ops->add2(m->x, m->o, m->x1, E);
        ops->rmsnorm(m->ffn_norm[l], m->x1, m->xn, c->eps, E);
        if (m->moe[l].n_expert) {
            const moe_t *e = &m->moe[l];
            const tensor_t rt = {0 /* F32 */, (const uint8_t *)e->router};
            matvec(ops, rt, e->n_expert, E, m->xn, m->mo_logits);
            ops->router_sel(m->mo_logits, m->mo_ids, m->mo_gates, e->n_expert, e->top_k, e->norm, e->scale);
            const uint64_t sg = (uint64_t)e->n_ff * flo_row_bytes(e->fmt_gu, E), sd = (uint64_t)E * flo_row_bytes(e->fmt_d, e->n_ff);
            for (uint32_t k = 0; k < e->top_k; ++k) {
                const uint32_t id = m->mo_ids[k];
                const tensor_t tg = {e->fmt_gu, e->wg + id * sg}, tu = {e->fmt_gu, e->wu + id * sg}, td = {e->fmt_d, e->wd + id * sd};
                matvec(ops, tg, e->n_ff, E, m->xn, m->mo_g);
                matvec(ops, tu, e->n_ff, E, m->xn, m->mo_u);
                ops->silu_mul(m->mo_g, m->mo_u, m->mo_h, e->n_ff);
                matvec(ops, td, E, e->n_ff, m->mo_h, m->mo_parts + (size_t)k * E);
            }
            ops->wmerge(m->mo_parts, m->mo_gates, m->x1, 0, m->x, 1.0f, e->top_k, E);
            continue;
        }
        matvec(ops, w[T_GATE], c->n_ff, E, m->xn, m->g);
        matvec(ops, w[T_UP], c->n_ff, E, m->xn, m->u);
        ops->silu_mul(m->g, m->u, m->h, c->n_ff);
        matvec(ops, w[T_DOWN], E, c->n_ff, m->h, m->dn);
        ops->add2(m->x1, m->dn, m->x, E);
    }
    ops->rmsnorm(m->out_norm, m->x, m->xn, c->eps, E);
    matvec(ops, m->output, c->n_vocab, E, m->xn, m->logits);
    m->n_past = pos + 1;
    /* greedy argmax + margin, src/model/decoder.cpp:1253-1264 */
    uint32_t best = 0;
    float bv = m->logits[0], sv = -1e30f;
    for (uint32_t i = 1; i < c->n_vocab; ++i) {
        const float z = m->logits[i];
        if (z > bv) { sv = bv; bv = z; best = i; }
        else if (z > sv) sv = z;
    }
    m->margin = bv - sv;
    return (int32_t)best;
}

/* Threads of the row / head loops from here on (a launcher may have exported OMP_NUM_THREADS=1 before this library
 * was loaded: torchrun does). */
void flo_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* The expert ids the last mixture-of-experts layer of the last step selected (top_k of them). */
const uint32_t *flo_llama_moe_ids(const flo_llama *m) { return m->mo_ids; }

/* Taps for layer-level parity checks: the hidden state after the last layer and
 * the final normed vector of the last step. */
const float *flo_llama_hidden(const flo_llama *m) { return m->x; }
const float *flo_llama_normed(const flo_llama *m) { return m->xn; }
/* Last-layer activations of the last step, same numbering as the GPU decoder's
 * taps: 2 q after RoPE, 3 v, 4 attention output, 5 residual after attention,
 * 6 the FFN hidden vector silu(gate) * up, 7 up. */
const float *flo_llama_tap(const flo_llama *m, int which) {
    switch (which) {
    case 0: return m->x;
    case 1: return m->xn;
    case 2: return m->q;
    case 3: return m->v;
    case 4: return m->att;
    case 5: return m->x1;
    case 6: return m->h;
    case 7: return m->u;
    default: return 0;
    }
}

/* Plain multi-threaded matvec (y = W x) on an operator table, for parity tests
 * and the timed CPU baseline. */
void flo_matvec(const flo_ops_t *ops, int fmt, const uint8_t *w, uint32_t rows, uint32_t cols,
                const float *x, float *y) {
    tensor_t t = {fmt, w};
    matvec(ops, t, rows, cols, x, y);
}

/* Bulk dequantise a whole tensor, rows in parallel. */
void flo_dequant_rows(const flo_ops_t *ops, int fmt, const uint8_t *w, uint32_t rows,
                      uint32_t cols, float *out) {
    const uint64_t rb = flo_row_bytes(fmt, cols);
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r)
        ops->dequant(fmt, w + (size_t)r * rb, 0, cols, out + (size_t)r * cols);
}
