/* fl_b200 — C ABI of the B200 (sm_100a) decode hot path.
 *
 * Drop-in boundary for the CUDA execution backend of the reference runtime:
 * what its task executor calls per task (exec_task_block,
 * src/runtime/gpu_exec.cu:64-140), what its decoder does per token
 * (Decoder::step / step_batch, src/model/decoder.h:52-81,
 * src/model/decoder.cpp:1176-1301) and the device bring-up it performs
 * (gpu_make_stream / gpu_start / gpu_stop_sync,
 * src/runtime/runtime_internal.h:288-301) are exported here as plain C
 * functions over plain pointers and sizes.
 *
 * Conventions
 *   - Every function returns 0 on success and a non-zero code on failure;
 *     fl_b200_last_error() then returns a message for the calling thread. The
 *     reference prints and abort()s at the same places (FL_CUCHECK,
 *     src/runtime/gpu_exec.cu:15-17; graph die, src/runtime/graph.cpp:100-103);
 *     a C++ wrapper that wants that behaviour aborts on non-zero.
 *   - Pointers named *_dev are device pointers valid on the context's device;
 *     *_host are host pointers. The caller owns every buffer.
 *   - All work is enqueued on the context's stream, in call order. Functions
 *     with "_host" in the name copy in, run and copy out, and return after the
 *     result is in host memory; the others return without synchronising.
 *   - One context = one device = one stream; calls on a context are serialised
 *     by the caller (as Runtime::run, include/fastllm/fastllm.h:226-229).
 *   - There is no CPU fallback: without a CUDA device fl_b200_create fails.
 */
#ifndef FL_B200_H
#define FL_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FL_B200_ABI_VERSION 1

/* Weight formats: numeric values of fastllm::Fmt
 * (include/fastllm/fastllm.h:56-57). */
enum { FL_B200_F32 = 0, FL_B200_Q8_0 = 1, FL_B200_Q5_0 = 2, FL_B200_Q4_K = 3, FL_B200_Q6_K = 4 };

/* Error codes. */
enum {
    FL_B200_OK = 0,
    FL_B200_ERR_ARG = 1,      /* rejected at the boundary (shape, alignment, null) */
    FL_B200_ERR_CUDA = 2,     /* a CUDA runtime call failed */
    FL_B200_ERR_DEVICE = 3,   /* a kernel reported a status (bounded wait gave up) */
    FL_B200_ERR_STATE = 4,    /* call order (e.g. step before finalize) */
    FL_B200_ERR_IO = 5,       /* a model file is missing or cannot be mapped */
    FL_B200_ERR_FORMAT = 6    /* a model file is malformed or holds what the decoder cannot run */
};

typedef struct fl_b200_ctx fl_b200_ctx;
typedef struct fl_b200_decoder fl_b200_decoder;
typedef struct fl_b200_seqpar fl_b200_seqpar;
typedef struct fl_b200_gguf fl_b200_gguf;
typedef struct fl_b200_suffix fl_b200_suffix;
typedef struct fl_b200_moe fl_b200_moe;
typedef struct fl_b200_spec fl_b200_spec;

int fl_b200_abi_version(void);
const char *fl_b200_last_error(void);

/* ---- context: replaces gpu_make_stream / gpu_start / gpu_stop_sync
 *      (src/runtime/gpu_exec.cu:384-502). No persistent kernel is started. ---- */
int fl_b200_create(int device, fl_b200_ctx **out);
void fl_b200_destroy(fl_b200_ctx *ctx);
int fl_b200_sync(fl_b200_ctx *ctx);
/* Reads and clears the device status word (0 = no kernel reported a problem). */
int fl_b200_device_status(fl_b200_ctx *ctx, uint32_t *status_out);
int fl_b200_sm_count(fl_b200_ctx *ctx);
/* Limit, in nanoseconds of the device clock, of the waits of the exchange kernels for another rank's
 * flag (0 = the default of one second). When it runs out the kernel records status 2 ("peer time-out"),
 * leaves its output untouched and returns; nothing faults and nothing waits for ever. The reference's
 * counterpart is the 60 s stall abort of Runtime::run (src/runtime/runtime.cpp:239). */
int fl_b200_set_wait_limit(fl_b200_ctx *ctx, uint64_t nanoseconds);
/* cudaStream_t of the context, for callers that enqueue their own work. */
void *fl_b200_stream(fl_b200_ctx *ctx);

/* Device memory for callers without a CUDA runtime of their own (replaces the
 * unified-memory Arena, src/runtime/arena.cpp:54-74, for the GPU side). */
int fl_b200_malloc(fl_b200_ctx *ctx, size_t bytes, void **dev_out);
int fl_b200_free(fl_b200_ctx *ctx, void *dev);
/* src may be a host pointer or a device pointer (unified addressing). */
int fl_b200_upload(fl_b200_ctx *ctx, void *dst_dev, const void *src_host, size_t bytes);
int fl_b200_download(fl_b200_ctx *ctx, void *dst_host, const void *src_dev, size_t bytes);
/* CUDA IPC handles (64 bytes) for mapping another rank's buffer into this process. */
int fl_b200_ipc_export(fl_b200_ctx *ctx, const void *dev_ptr, uint8_t handle_out[64]);
int fl_b200_ipc_open(fl_b200_ctx *ctx, const uint8_t handle[64], void **dev_ptr_out);
int fl_b200_ipc_close(fl_b200_ctx *ctx, void *dev_ptr);
int fl_b200_memset(fl_b200_ctx *ctx, void *dst_dev, int value, size_t bytes);

/* CUDA-event stopwatch on the context's stream. */
int fl_b200_timer_start(fl_b200_ctx *ctx);
int fl_b200_timer_stop(fl_b200_ctx *ctx, float *ms_out);   /* synchronises */

/* ---- single operators (device pointers) ---- */

/* Bulk dequantise rows x cols packed weights to f32, bit-exact with
 * dequant_chunk (src/runtime/kernels.h:162-242). */
int fl_b200_dequant(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint64_t rows, uint32_t cols,
                    float *out_dev);

/* STREAM_DOT (exec_task_scalar, src/runtime/runtime_internal.h:240-257):
 *   y[p*ystride + r] += dot(W[r], x + p*xstride), r < rows, p < nx.
 * Accumulates into y like the reference (its slots are zeroed per run,
 * src/model/decoder.cpp:1206-1208). w_dev must be 16-byte aligned. */
int fl_b200_matvec(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint32_t rows, uint32_t cols,
                   const float *x_dev, uint32_t nx, uint32_t xstride, float *y_dev, uint32_t ystride);
/* Same with y = dot (no read of y). */
int fl_b200_matvec_assign(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint32_t rows, uint32_t cols,
                          const float *x_dev, float *y_dev);
/* End-to-end form: x and y in host memory (y_host receives W x). */
/* Task{STREAM_DOT_IDX} (include/fastllm/fastllm.h:33-36, fl_idx_w,
 * src/runtime/runtime_internal.h:149-152): STREAM_DOT over the rows of expert
 * *expert_id_dev (read on the device when the kernel runs, so a router kernel
 * earlier on the stream may write it): W = w_dev + *expert_id_dev *
 * expert_stride_bytes. Accumulates into y like STREAM_DOT. */
int fl_b200_matvec_expert(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint32_t rows, uint32_t cols,
                          const uint32_t *expert_id_dev, uint64_t expert_stride_bytes, const float *x_dev,
                          uint32_t nx, uint32_t xstride, float *y_dev, uint32_t ystride);
/* y = W x (assigns) for a tensor whose rows are `pitch` bytes apart (pitch >=
 * the packed row size): the layout of a column slice of a k-quant tensor, whose
 * rows are zero-padded to a multiple of 16 bytes (tensor-parallel O and down). */
int fl_b200_matvec_pitched(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint32_t rows, uint32_t cols,
                           uint32_t pitch, const float *x_dev, float *y_dev);
int fl_b200_matvec_host(fl_b200_ctx *ctx, int fmt, const void *w_dev, uint32_t rows, uint32_t cols,
                        const float *x_host, float *y_host);

/* Decode attention for all query heads (fl_op_attn_head applied per head,
 * src/runtime/decode_params.h:183-232, extended to grouped-query heads and an
 * f16 cache). q, out: [batch][n_q_head][head_dim] f32; k, v:
 * [batch][n_kv_head][kv_stride][head_dim] f16; keys 0..kv_len-1 are attended.
 * head_dim must be 128 and n_q_head == 4 * n_kv_head. */
int fl_b200_attn_decode(fl_b200_ctx *ctx, const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev,
                        uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim, uint32_t kv_len,
                        uint32_t kv_stride, uint32_t batch, float scale, float *out_dev);
/* Draft verification, causal within the draft (the speculative-verify step):
 * n_draft queries q[b][n_q_head][128] against ONE cache [n_kv_head][kv_stride][128];
 * query b attends keys 0 .. base_len + b - 1 (the draft's own K/V rows are in
 * the cache already), i.e. fl_op_attn_head with pos = base_len - 1 + b per query. */
int fl_b200_attn_verify(fl_b200_ctx *ctx, const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev,
                        uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim, uint32_t base_len,
                        uint32_t kv_stride, uint32_t n_draft, float scale, float *out_dev);
/* Sequence-parallel decode attention over the GPUs of one box (the long-context
 * configuration: every rank holds a contiguous slice of the keys; the reference
 * has no counterpart). fl_b200_attn_decode_lse is fl_b200_attn_decode over the
 * rank's own keys that also returns, per (sequence, query head), lse_out = (max
 * score, sum of exp(score - max)) [batch][n_q_head][2]. fl_b200_seqpar_combine
 * merges the ranks' (context, max, sum) records through peer memory (same
 * protocol as the tensor-parallel all-reduce: push, release flag, bounded wait)
 * in rank order, so every rank gets identical bits. Set-up like the decoder's:
 * create, export fl_b200_seqpar_comm's buffer, open the peers', set_peers. */
int fl_b200_attn_decode_lse(fl_b200_ctx *ctx, const float *q_dev, const uint16_t *k_dev, const uint16_t *v_dev,
                            uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim, uint32_t kv_len,
                            uint32_t kv_stride, uint32_t batch, float scale, float *out_dev, float *lse_out_dev);
int fl_b200_seqpar_create(fl_b200_ctx *ctx, uint32_t rank, uint32_t world, uint32_t max_records, fl_b200_seqpar **out);
void fl_b200_seqpar_destroy(fl_b200_seqpar *h);
int fl_b200_seqpar_comm(fl_b200_seqpar *h, void **buf_dev_out, size_t *bytes_out);
int fl_b200_seqpar_set_peers(fl_b200_seqpar *h, void *const *bufs_dev, uint32_t n);
int fl_b200_seqpar_combine(fl_b200_seqpar *h, const float *out_local_dev, const float *lse_local_dev,
                           uint32_t n_records, float *out_dev);
/* fl_b200_attn_decode for callers that must not allocate device memory at call
 * time. It has no counterpart in the reference, whose operators keep their
 * temporaries in the caller's buffers. The split-KV scratch is a fixed array in
 * the library image: at most 4096 records of n_q_head * batch * splits (splits
 * <= 64, chosen from the SM count and kv_len) and n_kv_head * batch <= 256;
 * larger calls return FL_B200_ERR_ARG and leave `out` untouched. Arguments and
 * results are those of fl_b200_attn_decode. The first call on a device looks up
 * the array's address and should be made before any stream capture. All calls
 * on a device share the array: calls that overlap in time race on it. */
int fl_b200_attn_decode_static(fl_b200_ctx *ctx, const float *q_dev, const uint16_t *k_dev,
                               const uint16_t *v_dev, uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim,
                               uint32_t kv_len, uint32_t kv_stride, uint32_t batch, float scale, float *out_dev);
int fl_b200_attn_decode_host(fl_b200_ctx *ctx, const float *q_host, const uint16_t *k_dev,
                             const uint16_t *v_dev, uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim,
                             uint32_t kv_len, uint32_t kv_stride, uint32_t batch, float scale,
                             float *out_host);

/* fl_op_rmsnorm / fl_op_add2 / fl_op_silu_mul (decode_params.h:101-110, :267-272) */
int fl_b200_rmsnorm(fl_b200_ctx *ctx, const float *x_dev, const float *wnorm_dev, float *y_dev, float eps,
                    uint32_t n);
int fl_b200_add2(fl_b200_ctx *ctx, const float *a_dev, const float *b_dev, float *y_dev, uint32_t n);
int fl_b200_silu_mul(fl_b200_ctx *ctx, const float *gate_dev, const float *up_dev, float *h_dev, uint32_t n);
/* fl_op_router_sel (decode_params.h:234-265): softmax over n_expert (<= 256)
 * logits, top_k by weight, ties to the lower index, optional renormalisation,
 * times scale. fl_op_wmerge (decode_params.h:274-295): y = add1 + add2 + scale *
 * sum_q gates[q] * parts[q*n + i] (gates, add1, add2 may be null; n_full > n_parts
 * rescales the gates to carry the truncated tail's mass). */
int fl_b200_router_sel(fl_b200_ctx *ctx, const float *logits_dev, uint32_t *ids_dev, float *gates_dev,
                       uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale);
int fl_b200_wmerge(fl_b200_ctx *ctx, const float *parts_dev, const float *gates_dev, const float *add1_dev,
                   const float *add2_dev, float *y_dev, float scale, uint32_t n_parts, uint32_t n, uint32_t n_full);
/* fl_op_rope_ds2 (plain RoPE, adjacent pairs, decode_params.h:124-160) on q in
 * place and on k, then fl_op_kv_append (decode_params.h:162-175) of k and v
 * into an f16 cache [n_kv_head][kv_stride][head_dim] at row *pos_dev. */
int fl_b200_rope_kv_append(fl_b200_ctx *ctx, float *q_dev, const float *k_dev, const float *v_dev,
                           uint16_t *kcache_dev, uint16_t *vcache_dev, const int32_t *pos_dev,
                           uint32_t n_q_head, uint32_t n_kv_head, uint32_t head_dim, uint32_t kv_stride,
                           float freq_base);
/* Greedy argmax, lowest index on ties, and top1 - top2 margin
 * (src/model/decoder.cpp:1253-1264). */
int fl_b200_argmax(fl_b200_ctx *ctx, const float *logits_dev, uint32_t n, int32_t *idx_dev,
                   float *margin_dev);

/* ---- task-level entry: one reference Task on the device ------------------
 * Field-for-field image of fastllm::Task (include/fastllm/fastllm.h:65-97);
 * oracle/abi_check.cpp asserts the offsets against the reference header. All
 * pointers inside (and inside the aux parameter block) must be device
 * pointers. Kinds 0..12 keep the reference's numbers; 13 and 14 are appended
 * for the shapes the reference cannot express (grouped-query heads, f16
 * cache). */
enum {
    FL_B200_STREAM_DOT = 0, FL_B200_MERGE = 1, FL_B200_SIGNAL = 2, FL_B200_ACT_Q8 = 3,
    FL_B200_STREAM_DOT_IDX = 4, FL_B200_RMSNORM = 5, FL_B200_ADD2 = 6, FL_B200_ROPE_DS2 = 7,
    FL_B200_KV_APPEND = 8, FL_B200_ATTN_HEAD = 9, FL_B200_ROUTER_SEL = 10, FL_B200_SILU_MUL = 11,
    FL_B200_WMERGE = 12,
    FL_B200_ATTN_GQA_F16 = 13, FL_B200_ROPE_KV_APPEND_F16 = 14
};

typedef struct
#if defined(__GNUC__)
    __attribute__((aligned(128)))
#endif
    fl_b200_task {
    uint32_t id;
    uint8_t kind, affinity, fmt;
    uint16_t n_consumers;
    uint32_t consumers[6];
    const void *w;
    uint64_t w_bytes;
    const void *x;
    void *y;
    uint32_t rows, cols;
    int32_t dep_init, dep_count;
    uint32_t epoch;
    uint64_t handoff_ts;
    const void *aux;
    uint64_t aux2;
    uint32_t nx, xstride, ystride;
} fl_b200_task;

/* Parameter blocks of the reference operators (src/runtime/decode_params.h:23-97),
 * same field order, so a block built for the reference can be passed as is
 * once its pointers are device pointers. */
typedef struct { const float *wnorm, *x; float *y; float eps; uint32_t n; } fl_b200_rmsnorm_p;
typedef struct { const float *a, *b; float *y; uint32_t n; } fl_b200_add2_p;
typedef struct { const float *gate, *up; float *h; uint32_t n; } fl_b200_silu_mul_p;
typedef struct { const float *logits; uint32_t *ids; float *gates; uint32_t n_expert, top_k, norm; float scale; } fl_b200_router_p;
typedef struct {
    const float *parts, *gates, *add1, *add2; float *y; float scale; uint32_t n_parts, n, n_full;
} fl_b200_wmerge_p;
/* Appended kinds. */
typedef struct {
    const float *q; const uint16_t *kcache, *vcache; float *out; const int32_t *pos;
    float scale; uint32_t n_q_head, n_kv_head, head_dim, kv_stride;
} fl_b200_attn_gqa_f16_p;
typedef struct {
    float *q; const float *k, *v; uint16_t *kcache, *vcache; const int32_t *pos;
    uint32_t n_q_head, n_kv_head, head_dim, kv_stride; float freq_base;
} fl_b200_rope_kv_append_f16_p;

/* Executes one task (what exec_task_block does for the whole block,
 * src/runtime/gpu_exec.cu:64-140). SIGNAL is a no-op. Kinds without a device
 * implementation here (MERGE, ACT_Q8, ROPE_DS2, KV_APPEND, ATTN_HEAD: the
 * DeepSeek-specific forms) return FL_B200_ERR_ARG. */
int fl_b200_exec_task(fl_b200_ctx *ctx, const fl_b200_task *task);

/* ---- a frozen task table as one CUDA graph: Graph::freeze + Runtime::run for
 *      the GPU side (src/runtime/graph.cpp:48-148, src/runtime/runtime.cpp:178-292).
 * `tasks` is the host copy of the table (ids 0..n-1, consumers / dep_init as
 * Graph::edge leaves them; every pointer inside is a device pointer). The table
 * is validated with the reference's freeze rules (no cycle, exactly one sink,
 * which is a SIGNAL, aux blocks present, STREAM_DOT shapes consistent), ordered
 * by dependency level, row tiles of one weight tensor are merged into one matvec
 * launch, and the launches are recorded once. fl_b200_plan_run replays them
 * (asynchronous; fl_b200_sync waits). Parameter blocks are read at plan time:
 * they are immutable after freeze in the reference too. STREAM_DOT accumulates
 * into y: zero the slots per run as the reference does. ---- */
typedef struct fl_b200_plan fl_b200_plan;
int fl_b200_plan_create(fl_b200_ctx *ctx, const fl_b200_task *tasks_host, uint32_t n, fl_b200_plan **out);
int fl_b200_plan_run(fl_b200_plan *plan);
int fl_b200_plan_info(fl_b200_plan *plan, uint32_t *n_tasks, uint32_t *n_launches, uint32_t *n_merged_tiles);
void fl_b200_plan_destroy(fl_b200_plan *plan);

/* ---- Llama-shape greedy decoder: Decoder::step for the GQA / f16-cache
 *      shape (src/model/decoder.h:52-81). ---- */
typedef struct {
    uint32_t n_layer, n_embd, n_head, n_kv_head, head_dim, n_ff, n_vocab, max_kv;
    float rope_base, eps;
} fl_b200_llama_cfg;

enum { FL_B200_T_WQ = 0, FL_B200_T_WK, FL_B200_T_WV, FL_B200_T_WO, FL_B200_T_GATE, FL_B200_T_UP,
       FL_B200_T_DOWN };
enum { FL_B200_G_TOK_EMBD = 0, FL_B200_G_OUTPUT = 1 };

int fl_b200_decoder_create(fl_b200_ctx *ctx, const fl_b200_llama_cfg *cfg, fl_b200_decoder **out);
/* Tensor-parallel decoder: rank `rank` of `world` (<= 8) ranks, one process and
 * one GPU per rank (the reference has no multi-GPU path). cfg describes the
 * WHOLE model; this rank holds n_kv_head / world KV heads with their query heads
 * (rows of wq, wk, wv; its slice of the KV cache), the matching columns of wo,
 * n_ff / world rows of gate and up and the matching columns of down, and
 * n_vocab / world rows of the head; the hidden state is replicated. Tensors are
 * handed over already sliced: row slices are plain row ranges; a column slice
 * keeps every row's blocks [first, first + n) and stores each row zero-padded to
 * a multiple of 16 bytes. The embedding table is whole on every rank. After O
 * and after down the ranks' partial vectors are summed (in rank order, so all
 * ranks hold identical bits) by a one-shot exchange through peer memory, and the
 * per-rank argmax records are merged likewise: every rank returns the same
 * token. fl_b200_decoder_logits returns this rank's slice. Set-up: create on
 * every rank, export fl_b200_decoder_comm's buffer (fl_b200_ipc_export), open
 * the other ranks' handles (fl_b200_ipc_open), pass all `world` pointers in
 * rank order to fl_b200_decoder_set_peers (own buffer at index `rank`), then
 * finalize. All ranks must issue the same sequence of step / run / time_class
 * calls. */
int fl_b200_decoder_create_tp(fl_b200_ctx *ctx, const fl_b200_llama_cfg *cfg, uint32_t rank, uint32_t world,
                              fl_b200_decoder **out);
int fl_b200_decoder_comm(fl_b200_decoder *dec, void **buf_dev_out, size_t *bytes_out);
int fl_b200_decoder_set_peers(fl_b200_decoder *dec, void *const *bufs_dev, uint32_t n);
void fl_b200_decoder_destroy(fl_b200_decoder *dec);
/* Weights stay where the caller put them (device memory, GGUF block layout,
 * 16-byte aligned); the decoder keeps the pointers. */
int fl_b200_decoder_set_layer_tensor(fl_b200_decoder *dec, uint32_t layer, int which, int fmt,
                                     const void *w_dev);
int fl_b200_decoder_set_layer_norms(fl_b200_decoder *dec, uint32_t layer, const float *attn_norm_dev,
                                    const float *ffn_norm_dev);
/* A mixture-of-experts feed-forward block in place of the layer's dense one (a Mixtral-shape layer: the chain the
 * reference's graph builder emits per MoE layer, src/model/decoder.cpp:925-1045): the layer then needs no gate / up /
 * down tensor. The block (fl_b200_moe_create on the same context, one GPU, n_embd of the model, its weights set) stays
 * the caller's; per token it runs router -> top-k -> the selected experts through the expert-indexed matvec -> merge,
 * inside the decoder's captured step. Before fl_b200_decoder_finalize. */
int fl_b200_decoder_set_layer_moe(fl_b200_decoder *dec, uint32_t layer, fl_b200_moe *moe);
int fl_b200_decoder_set_global(fl_b200_decoder *dec, int which, int fmt, const void *w_dev);
int fl_b200_decoder_set_out_norm(fl_b200_decoder *dec, const float *w_dev);
/* The decoder owns the KV cache: per layer K and V, each
 * [n_kv_head][max_kv][head_dim] f16. Returns the device pointers so a caller
 * can prefill it. */
int fl_b200_decoder_kv(fl_b200_decoder *dec, uint32_t layer, uint16_t **k_dev_out, uint16_t **v_dev_out);
/* Freezes the configuration and records the per-token launch sequence as a
 * CUDA graph (the counterpart of Graph::freeze, src/runtime/graph.cpp:48-93). */
int fl_b200_decoder_finalize(fl_b200_decoder *dec);
int fl_b200_decoder_set_n_past(fl_b200_decoder *dec, int32_t n_past);   /* rewind_to */
int fl_b200_decoder_n_past(fl_b200_decoder *dec, int32_t *n_past_out);
/* Feed one token at position n_past; returns the greedy next token. The token
 * goes host -> device and the result device -> host inside the call. */
int fl_b200_decoder_step(fl_b200_decoder *dec, int32_t token, int32_t *next_out);
/* Runs `n` steps feeding each step's argmax back on the device (no host round
 * trip between steps); writes the n produced tokens to tokens_host. */
int fl_b200_decoder_run(fl_b200_decoder *dec, int32_t first_token, uint32_t n, int32_t *tokens_host);
/* Greedy verification of a draft (speculative decoding): runs the model on
 * first_token, draft[0..n_draft-1] teacher-forced from position n_past and
 * accepts draft[i] while it equals the model's greedy token; returns how many
 * were accepted and the model's own token after the last accepted one. n_past
 * advances by n_accepted + 1. */
int fl_b200_decoder_verify(fl_b200_decoder *dec, int32_t first_token, const int32_t *draft_host, uint32_t n_draft,
                           uint32_t *n_accepted_out, int32_t *next_token_out);
/* After a step: logits (n_vocab floats) and the top1 - top2 margin. */
/* Decoder::step_batch (src/model/decoder.h:64-70): feeds m <= FL_B200_MAX_BATCH
 * tokens at positions n_past .. n_past + m - 1 in one pass; outs_host[i] is the
 * greedy token after position i, margins_host[i] (optional) its top1 - top2
 * margin (Decoder::last_margins, :73); n_past advances by m, and rewind_to
 * (fl_b200_decoder_set_n_past) commits or discards the rows as in the
 * reference. One pass over a tensor serves up to 8 tokens where the multi-column
 * kernel takes its shape (Q4_K and Q6_K; 9 to 16 tokens: two passes); other
 * tensors are walked once per token; passes of fewer than 4 tokens run as
 * teacher-forced single steps on the device. Used for draft verification and for
 * prompt ingestion in chunks. On a tensor-parallel decoder all ranks make
 * the same call; the partial O / down outputs and the argmax records are
 * exchanged per token, and fl_b200_decoder_batch_logits returns this rank's
 * slice. */
#define FL_B200_MAX_BATCH 16
int fl_b200_decoder_step_batch(fl_b200_decoder *dec, const int32_t *toks_host, uint32_t m, int32_t *outs_host,
                               float *margins_host);
/* Several independent sequences decoded in lock step (nothing in the reference: its decoder holds one sequence): after
 * fl_b200_decoder_seqs_init(n), 2 <= n <= FL_B200_MAX_BATCH, the decoder owns n more KV caches (per layer
 * [n][n_kv_head][max_kv][head_dim] f16 for K and for V; fl_b200_decoder_seqs_kv returns sequence seq's part so that a
 * caller can prefill it) and a position per sequence (fl_b200_decoder_seqs_set_pos = rewind_to of that sequence).
 * fl_b200_decoder_seqs_step feeds toks_host[i] to sequence i at its own position and returns each sequence's greedy
 * token (and margin): one pass, every weight tensor walked once per 8 sequences, the attention per sequence over its own
 * keys; every position advances by one. fl_b200_decoder_batch_logits(i) then returns the logits of sequence i. The
 * single-sequence calls (step, run, step_batch) keep working on their own cache. One GPU. */
int fl_b200_decoder_seqs_init(fl_b200_decoder *dec, uint32_t n_seq);
int fl_b200_decoder_seqs_kv(fl_b200_decoder *dec, uint32_t layer, uint32_t seq, uint16_t **k_dev_out, uint16_t **v_dev_out);
int fl_b200_decoder_seqs_set_pos(fl_b200_decoder *dec, uint32_t seq, int32_t n_past);
int fl_b200_decoder_seqs_pos(fl_b200_decoder *dec, uint32_t seq, int32_t *n_past_out);
int fl_b200_decoder_seqs_step(fl_b200_decoder *dec, const int32_t *toks_host, int32_t *outs_host, float *margins_host);
/* Logits of position `index` of the last fl_b200_decoder_step_batch pass. */
int fl_b200_decoder_batch_logits(fl_b200_decoder *dec, uint32_t index, float *logits_host);
int fl_b200_decoder_logits(fl_b200_decoder *dec, float *logits_host);
int fl_b200_decoder_margin(fl_b200_decoder *dec, float *margin_out);
/* Activations of the last step, for layer-level parity. which: 0 hidden state
 * after the last layer (n_embd), 1 final normed vector (n_embd); of the last
 * layer: 2 q after RoPE (n_head*head_dim), 3 v (n_kv_head*head_dim), 4 attention
 * output (n_head*head_dim), 5 residual after attention (n_embd), 6 the FFN
 * hidden vector silu(gate)*up (n_ff). */
int fl_b200_decoder_tap(fl_b200_decoder *dec, int which, float *host_out);
/* Times `reps` replays of one class of the step's kernels in isolation (same
 * launches, real weights and buffers, CUDA events on the context's stream).
 * kernel_class: 1 matvec launches, 2 attention launches, 4 the small
 * operators, 7 all of them. Results of the replays are not meaningful. */
int fl_b200_decoder_time_class(fl_b200_decoder *dec, uint32_t kernel_class, uint32_t reps,
                               float *ms_per_step_out, uint32_t *launches_per_step_out);
/* Diagnostics. With FLB_TRACE=1 in the environment when the decoder is
 * finalized, every matvec and attention launch of a step records four device
 * timestamps (ns): earliest kernel entry, earliest point after its dependency
 * wait, latest end of its prologue, latest exit. Copies the records of the last
 * fl_b200_decoder_step (4 values per launch, launch order) to host_out. */
int fl_b200_decoder_trace(fl_b200_decoder *dec, uint64_t *host_out, uint32_t cap_records, uint32_t *n_out);
/* Number of kernels this library launches per decoder step. */
int fl_b200_decoder_launches_per_step(fl_b200_decoder *dec, uint32_t *n_out);
/* Weight + KV bytes one step at position `pos` must read (the roofline numerator). */
int fl_b200_decoder_bytes_per_step(fl_b200_decoder *dec, int32_t pos, uint64_t *weight_bytes,
                                   uint64_t *kv_bytes);

/* ---- GGUF model files: the reader that feeds the decoder (class Gguf,
 *      src/model/gguf.h:28-79, src/model/gguf.cpp:133-266). Host only: these
 *      calls need no GPU. Files are mapped read-only and stay mapped until
 *      fl_b200_gguf_close; tensor payloads are handed out in place. ---- */
/* ggml tensor type ids as stored in the file (src/model/gguf.h:14-19). */
enum { FL_B200_GGML_F32 = 0, FL_B200_GGML_F16 = 1, FL_B200_GGML_Q5_0 = 6, FL_B200_GGML_Q8_0 = 8,
       FL_B200_GGML_Q4_K = 12, FL_B200_GGML_Q6_K = 14, FL_B200_GGML_IQ2_XXS = 16, FL_B200_GGML_IQ3_XXS = 18 };
typedef struct {
    int32_t fmt;          /* fastllm::Fmt value (IQ2_XXS = 5, IQ3_XXS = 6 included), -1 for any other type */
    uint32_t ggml_type;
    uint32_t n_dims;      /* 1..4 */
    uint32_t shard;       /* index of the file that holds the payload */
    uint64_t ne[4];       /* ne[0] = columns (innermost), ne[1] = rows, unused dims = 1 */
    uint64_t offset;      /* from the start of its shard's data section */
    uint64_t nbytes;      /* payload size; 0 for a type whose size is unknown */
    const void *data;     /* host pointer into the mapping */
} fl_b200_gguf_tensor;
/* GGUF versions 2 and 3. A name of the form "<stem>-00001-of-000NN.gguf" opens
 * every shard: metadata comes from the file named, tensors from all of them,
 * and "split.tensors.count", when present, must match (Gguf::open,
 * src/model/gguf.cpp:133-159). A missing file returns FL_B200_ERR_IO (the
 * reference returns false); a truncated or malformed one FL_B200_ERR_FORMAT (the
 * reference aborts), and so does a payload that runs past the end of its file. */
int fl_b200_gguf_open(const char *path, fl_b200_gguf **out);
void fl_b200_gguf_close(fl_b200_gguf *g);
int fl_b200_gguf_counts(const fl_b200_gguf *g, uint32_t *n_tensors, uint32_t *n_shards, uint32_t *alignment);
/* Tensor `index` in file order (shards in order); its name goes to name_out
 * (truncated to cap - 1 characters, always terminated). */
int fl_b200_gguf_tensor_at(const fl_b200_gguf *g, uint32_t index, char *name_out, size_t cap,
                           fl_b200_gguf_tensor *info_out);
/* First tensor of that name (Gguf::find, src/model/gguf.cpp:291-295);
 * FL_B200_ERR_ARG when there is none. */
int fl_b200_gguf_find(const fl_b200_gguf *g, const char *name, fl_b200_gguf_tensor *info_out);
/* Metadata (Gguf::kv_i / kv_f / kv_s / kv_sarr, src/model/gguf.cpp:271-289):
 * integer and boolean scalars read as int64, floats as double, each falling
 * back to the other kind and then to `dflt`. kv_s copies the string (or dflt
 * when the key is absent or not a string; dflt may be null = "") and returns
 * its full length in len_out. */
int fl_b200_gguf_has(const fl_b200_gguf *g, const char *key);
int64_t fl_b200_gguf_kv_i(const fl_b200_gguf *g, const char *key, int64_t dflt);
double fl_b200_gguf_kv_f(const fl_b200_gguf *g, const char *key, double dflt);
int fl_b200_gguf_kv_s(const fl_b200_gguf *g, const char *key, const char *dflt, char *out, size_t cap, size_t *len_out);
/* String arrays (tokenizer.ggml.tokens and the like): the count, or -1 when
 * the key is absent or not a string array; then item i as kv_s does. */
int64_t fl_b200_gguf_kv_sarr_count(const fl_b200_gguf *g, const char *key);
int fl_b200_gguf_kv_sarr_at(const fl_b200_gguf *g, const char *key, uint64_t i, char *out, size_t cap, size_t *len_out);
/* Hyper-parameters of a "llama" architecture file as the decoder wants them
 * (what DecoderImpl::load_hparams, src/model/decoder.cpp:208-275, does for the
 * reference's architecture): "llama.embedding_length", "llama.block_count",
 * "llama.attention.head_count", "llama.attention.head_count_kv" (default: the
 * head count), "llama.feed_forward_length",
 * "llama.attention.layer_norm_rms_epsilon" (1e-5), "llama.rope.freq_base"
 * (10000), head size from "llama.attention.key_length" (default n_embd /
 * n_head), vocabulary from token_embd.weight's row count. A file that asks for
 * RoPE scaling (a "llama.rope.scaling.type" other than "none", or a
 * rope_freqs.weight tensor) is refused with FL_B200_ERR_FORMAT. */
int fl_b200_gguf_llama_cfg(const fl_b200_gguf *g, uint32_t max_kv, fl_b200_llama_cfg *cfg_out);
/* ---- Mixture-of-experts feed-forward block (the MoE configuration: 8 experts,
 *      top-2), single GPU or expert parallel. The reference builds the chain
 *      router matvec -> ROUTER_SEL -> STREAM_DOT_IDX x3 with SILU_MUL -> WMERGE
 *      as tasks (src/model/decoder.cpp:925-1045, src/runtime/decode_params.h:
 *      234-295) and has no multi-GPU form. ---- */
typedef struct {
    uint32_t n_embd, n_ff, n_expert, top_k;
    uint32_t norm;         /* RouterP::norm: renormalise the chosen weights */
    float scale;           /* RouterP::scale (expert_weights_scale) */
    int32_t fmt_gate_up, fmt_down;   /* Q4_K or Q6_K */
    uint32_t max_tokens;   /* tokens per fl_b200_moe_forward call */
} fl_b200_moe_cfg;
/* Rank `rank` of `world` (0 of 1: single GPU) holds experts
 * [rank * n_expert / world, (rank + 1) * n_expert / world). The hidden states are
 * replicated over the ranks, so dispatch moves nothing: every rank routes every
 * token and runs only the slots whose expert it holds; the combine is one sum of
 * the ranks' partial outputs through peer memory, in rank order (all ranks end
 * with identical bits). Set-up for world > 1 is the decoder's: export
 * fl_b200_moe_comm's buffer, open the others', fl_b200_moe_set_peers. */
int fl_b200_moe_create(fl_b200_ctx *ctx, const fl_b200_moe_cfg *cfg, uint32_t rank, uint32_t world, fl_b200_moe **out);
void fl_b200_moe_destroy(fl_b200_moe *moe);
/* router_dev: f32 [n_expert][n_embd], whole on every rank. gate / up: this rank's
 * experts stacked, [n_local][n_ff rows of n_embd columns]; down: [n_local][n_embd
 * rows of n_ff columns]; GGUF block layout, 16-byte aligned. The block keeps the
 * pointers. */
int fl_b200_moe_set_weights(fl_b200_moe *moe, const float *router_dev, const void *gate_dev, const void *up_dev,
                            const void *down_dev);
int fl_b200_moe_comm(fl_b200_moe *moe, void **buf_dev_out, size_t *bytes_out);
int fl_b200_moe_set_peers(fl_b200_moe *moe, void *const *bufs_dev, uint32_t n);
/* y[t] = sum over the top_k experts e of token t of weight_e * down_e(silu(gate_e x[t]) * up_e x[t]), t < n_tok;
 * x_dev, y_dev: [n_tok][n_embd] f32. Enqueued on the context's stream. With
 * world > 1 all ranks call it with the same x. */
int fl_b200_moe_forward(fl_b200_moe *moe, const float *x_dev, uint32_t n_tok, float *y_dev);
/* Expert ids and weights chosen in the last forward call, [n_tok][top_k]. */
int fl_b200_moe_routing(fl_b200_moe *moe, uint32_t n_tok, uint32_t *ids_host, float *gates_host);

/* ---- Speculative decoding around fl_b200_decoder_step_batch (host code). ---- */
/* Draft source: longest-suffix match over the token stream pushed so far (class
 * SuffixIndex, src/spec/suffix_index.h:16-114). Every position is indexed by its
 * trailing 3 tokens; a draft walks at most chain_cap earlier occurrences of the
 * current tail (most recent first, the tail's own entry included in the count),
 * keeps the longest match of the whole suffix (ties: the most recent) and, when
 * it is at least min_match long, proposes the tokens that followed it, up to
 * n_max and never past the end of the stream. */
int fl_b200_suffix_create(uint32_t chain_cap, uint32_t min_match, fl_b200_suffix **out);
void fl_b200_suffix_destroy(fl_b200_suffix *s);
void fl_b200_suffix_reset(fl_b200_suffix *s);
void fl_b200_suffix_push(fl_b200_suffix *s, int32_t token);
uint64_t fl_b200_suffix_size(const fl_b200_suffix *s);
/* Returns the number of draft tokens written to out (0 = no usable match).
 * diag_out (optional, 4 values; SuffixIndex::Diag, :41-46): the tail's gram was
 * indexed, candidates compared, longest match found, entries walked. */
int fl_b200_suffix_draft(const fl_b200_suffix *s, int32_t n_max, int32_t *out, int32_t *diag_out);
/* Draft-length controller (class SpecController, src/spec/spec_controller.h:16-107):
 * choose() = the n in 0..n_max that maximises (1 + a + ... + a^n) / latency(n),
 * a = running mean of the accepted fraction, latency(n) = running mean per draft
 * length, unseen lengths seeded from the nearest measured one; n_max before
 * anything is measured; after probe_iv draftless rounds in a row, probe_n. */
typedef struct {
    int32_t n_max;         /* 7 */
    double alpha0;         /* 0.75 */
    double alpha_decay;    /* 0.90 */
    double lat_decay;      /* 0.80 */
    int32_t probe_iv;      /* 16 */
    int32_t probe_n;       /* 2 */
    double seed_slope;     /* 0.15 */
} fl_b200_spec_cfg;
void fl_b200_spec_cfg_default(fl_b200_spec_cfg *cfg);
int fl_b200_spec_create(const fl_b200_spec_cfg *cfg /* null: the defaults */, fl_b200_spec **out);
void fl_b200_spec_destroy(fl_b200_spec *s);
int32_t fl_b200_spec_choose(fl_b200_spec *s);
void fl_b200_spec_observe(fl_b200_spec *s, int32_t n_drafted, int32_t n_accepted, double pass_ms);
double fl_b200_spec_alpha(const fl_b200_spec *s);
double fl_b200_spec_lat_est(const fl_b200_spec *s, int32_t n);
double fl_b200_spec_expected_emitted(const fl_b200_spec *s, int32_t n);
typedef struct {
    uint32_t passes, drafted, accepted, emitted;
    uint32_t n_hist[17];   /* passes by number of drafts */
    double pass_ms;        /* wall time of all batch passes */
} fl_b200_spec_stats;
/* The speculative generation loop of the reference's decode tool
 * (tools/decode_main.cpp:329-400): writes n_gen tokens to out_tokens_host,
 * first_token (not yet fed to the model) first. Every round drafts up to
 * min(spec_max, spec_fixed or the controller's choice) tokens from `idx`,
 * verifies them in one fl_b200_decoder_step_batch pass, emits the accepted
 * prefix and takes the model's own token after it; rejected rows of the cache
 * are dropped by rewinding. spec_fixed < 0: the controller decides and learns
 * (ctrl required). spec_max <= FL_B200_MAX_BATCH - 1. The reference's margin
 * gate is not needed: no position of this decoder's batch pass is approximated. */
int fl_b200_decoder_generate_spec(fl_b200_decoder *dec, int32_t first_token, uint32_t n_gen, int32_t spec_max,
                                  int32_t spec_fixed, fl_b200_suffix *idx, fl_b200_spec *ctrl,
                                  int32_t *out_tokens_host, fl_b200_spec_stats *stats_out);

/* Creates the decoder (rank `rank` of `world`; 0 of 1 = single GPU) of a llama
 * GGUF and uploads its tensors, each from the mapping straight to device memory
 * the decoder owns: blk.N.{attn_norm, attn_q, attn_k, attn_v, attn_output,
 * ffn_norm, ffn_gate, ffn_up, ffn_down}.weight, token_embd.weight,
 * output_norm.weight, output.weight (token_embd.weight again when the file ties
 * them); the tensor-parallel slices are cut during the upload (DecoderImpl::load
 * / load_tensor, src/model/decoder.cpp:185-206, :277-321, map in place instead).
 * Matrices must be Q4_K, Q6_K or Q8_0, norms F32. Not finalized: call
 * fl_b200_decoder_finalize (after fl_b200_decoder_set_peers when world > 1). */
int fl_b200_decoder_create_gguf(fl_b200_ctx *ctx, const fl_b200_gguf *g, uint32_t max_kv, uint32_t rank,
                                uint32_t world, fl_b200_decoder **out);

#ifdef __cplusplus
}
#endif
#endif
