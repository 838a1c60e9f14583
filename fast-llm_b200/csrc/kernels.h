// Internal launch interface between the C ABI (capi.cu), the decoder
// (decoder.cu) and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flb {

// ---- dequant.cu ---------------------------------------------------------
cudaError_t launch_dequant(int fmt, const void *w, uint64_t rows, uint32_t cols, float *out, int sms,
                           cudaStream_t stream);

// ---- matvec.cu ----------------------------------------------------------
// One weight tensor of a (possibly multi-tensor) matvec launch. All tensors of
// a launch share the activation vector and the column count.
struct MatvecTensor {
    const uint8_t *w;     // packed rows, GGUF block layout, 16-byte aligned
    float *y;             // rows outputs
    const float *resid;   // optional: y[r] = resid[r] + dot   (nullptr: none)
    uint32_t rows;
    int fmt;
    uint32_t pitch;       // bytes between rows; 0 = packed (row_bytes(fmt, cols)). A column slice of a Q6_K
                          // tensor is stored with its rows zero-padded to a multiple of 16 bytes.
    // Expert indirection (STREAM_DOT_IDX, fl_idx_w, src/runtime/runtime_internal.h:149-152): the rows used
    // are those of expert *expert_id, expert_rows rows further down per expert (nullptr: none).
    // *t[0].expert_id == kExpertSkip: the whole launch returns at once and leaves y as it is (expert
    // parallelism: the expert lives on another GPU). The id is read at kernel entry, so such a launch is not
    // made a programmatic dependent of the kernel that writes the id.
    const uint32_t *expert_id;
    uint32_t expert_rows;
};
constexpr uint32_t kExpertSkip = 0xFFFFFFFFu;

enum : int {
    MV_X_PLAIN = 0,    // activation = x
    MV_X_RMSNORM = 1,  // activation = x * rsqrt(mean(x^2)+eps) * wnorm
    MV_X_SILU_MUL = 2, // activation = silu(x) * x2
};

struct MatvecArgs {
    MatvecTensor t[4];
    int n_tensors;
    const float *x;
    const float *x2;      // MV_X_SILU_MUL: the "up" vector
    const float *wnorm;   // MV_X_RMSNORM
    float eps;
    uint32_t cols;
    int x_mode;
    int accumulate;       // 1: y[r] += dot (STREAM_DOT semantics); 0: y[r] = dot (+ resid)
    int swiglu;           // 1: t[0] = gate, t[1] = up (same shape and format): t[0].y[r] = silu(gate_r . x) * (up_r . x)
    uint32_t *status;     // device status word
    float *xn_out;        // optional: CTA 0 also writes the activation it built (nullptr: no)
    int pdl;              // launch with programmatic dependent launch (inside the decoder's step)
    int issue_late;       // 1: request the first weight stages after the activation loads are in flight instead of
                          // before the dependency wait (for launches whose CTAs only become resident when the previous
                          // kernel's CTAs leave, so that nothing is gained by requesting early)
    unsigned long long *trace;   // optional 4-entry timeline record of this launch (diagnostics)
    uint32_t *grid_bar;          // chained launches (launch_matvec_tc_chain): two zeroed words of device memory, the
                                 // state of the grid-wide barrier; one launch at a time may use them
    int expert_ids_ready;        // 1: the expert ids were complete before the previous kernel started, so the first
                                 // weight stages are requested before the dependency wait, as for a plain tensor
    // Tensor parallel: the activation is the sum of the ranks' partial vectors that an exchange launch
    // (launch_allreduce_push) is delivering into this rank's exchange buffer, plus a residual:
    // x = xr_resid + sum_r recv[r]. The kernel waits (bounded) for the ranks' flags of the epoch the
    // push launch recorded, adds in rank order (identical bits on all ranks) and CTA 0 also stores the
    // sum to xr_out (the new residual stream). nullptr: x is read as usual.
    const uint8_t *xr_buf;
    const uint32_t *xr_epoch;    // kCommChunks epoch counters of this rank's push launches
    const float *xr_resid;
    float *xr_out;
    uint32_t xr_world;
};

// Streaming kernel (Q4_K / Q6_K, cols a multiple of 256 and >= 512, rows 16-byte pitched) or the generic
// kernel (every other supported shape). Returns cudaErrorInvalidValue for
// unsupported arguments.
// 2-D tiled TMA descriptor over a row-major array (rows x dim0 elements, row pitch stride_bytes).
cudaError_t tensor_map_2d(CUtensorMap *m, uint32_t elem_bytes, const void *base, uint64_t dim0, uint64_t rows,
                          uint64_t stride_bytes, uint32_t box0, uint32_t box_rows, bool swizzle128);
cudaError_t tensor_map_lines_swz(CUtensorMap *m, const void *base, uint64_t rows, uint64_t pitch, uint32_t box_lines,
                                 uint32_t box_rows);   // [rows][pitch / 128][128 bytes], 128-byte swizzle (matvec.cu)
cudaError_t launch_matvec(const MatvecArgs &a, int sms, cudaStream_t stream);
// Q4_K / Q6_K launches that qualify run on the tensor-core streaming kernel (matvec_tc.cu).
bool matvec_tc_eligible(const MatvecArgs &a);
cudaError_t launch_matvec_tc(const MatvecArgs &a, int sms, cudaStream_t stream);
// n (1..4) matvecs in ONE launch, each consuming what the one before it wrote (O -> gate|up -> down -> next Q/K/V),
// with grid-wide barriers in between and the weights of the next phase streaming meanwhile. cudaErrorNotSupported
// when a phase does not qualify: launch them one by one then. args[0].grid_bar names the barrier state.
cudaError_t launch_matvec_tc_chain(const MatvecArgs *args, int n, int sms, cudaStream_t stream);
cudaError_t matvec_tc_init(void);
// Several activation columns (P <= 8) in one pass over a Q4_K / Q6_K tensor on the tensor cores (matvec_tc_nx.cu):
// y[p * ystride + r] (+)= dot(W[r], x + p * xstride). xq: device scratch of matmul_tc_nx_scratch_bytes(cols, P) bytes
// that holds the converted activations during the call. cudaErrorNotSupported when the shape does not qualify.
struct NxCall {
    int fmt;
    const void *w;           // rows x cols, GGUF block layout
    uint32_t rows, cols, pitch;   // pitch 0 = packed rows
    const float *x;          // columns: rows of x, xstride floats apart
    const float *x2;         // optional: the column is SiLU(x) * x2 (same stride)
    uint32_t P, xstride;     // columns of this call (<= 8)
    float *y;                // output row blocks, ystride floats apart
    uint32_t ystride;
    int accumulate;
    int skip_convert;        // 1: xq already holds exactly these columns in this format's layout (the call before used them)
    // Device-side column list (mixture of experts): column p is row col_idx[col_off + p] of x and goes to output row
    // block out_idx[col_off + p]; only columns col_off + p < *cnt exist. All nullptr: column p = row p -> row block p.
    const uint32_t *cnt, *col_idx, *out_idx;
    uint32_t col_off;
    int pdl;                 // the launches of this call are programmatic dependents of the launch before them
};
cudaError_t launch_matmul_tc_nx(const NxCall &c, uint8_t *xq, uint32_t *status, int sms, cudaStream_t stream);
size_t matmul_tc_nx_scratch_bytes(uint32_t cols, uint32_t P);
cudaError_t matmul_tc_nx_init(void);
// The same call on tcgen05 with the accumulator in tensor memory (matmul_umma.cu; Q4_K). xu: device scratch of
// matmul_umma_xu_bytes(cols) bytes for the converted activations; scratch / tickets: split-K partial results and their
// counters (matmul_umma_scratch_bytes() bytes, matmul_umma_ticket_count() zeroed words).
cudaError_t launch_matmul_umma(const NxCall &c, uint8_t *xu, float *scratch, uint32_t *tickets, uint32_t *status, int sms,
                               cudaStream_t stream);
size_t matmul_umma_xu_bytes(uint32_t cols);
size_t matmul_umma_scratch_bytes(void);
size_t matmul_umma_ticket_count(void);
cudaError_t matmul_umma_init(void);
// True when launch_matvec would take the streaming kernel for this shape.
bool matvec_is_streaming(int fmt, uint32_t cols);
// Dynamic shared memory the streaming kernel needs for (cols, formats used).
size_t matvec_smem_bytes(uint32_t cols, bool use_q4k, bool use_q6k, int *stages_out, int *warps_out, bool use_q8_0 = false);
cudaError_t matvec_init(void);   // sets the dynamic shared memory attribute once

// ---- attn.cu ------------------------------------------------------------
struct AttnArgs {
    const float *q;        // [batch][n_q_head][128] f32 (post-RoPE unless rope fused)
    const __half *k;       // [batch][n_kv_head][kv_stride][128] f16
    const __half *v;       // same layout
    float *out;            // [batch][n_q_head][128]
    float *part;           // scratch: [batch][n_q_head][n_splits][132] (context[128], max, sum, pad)
    uint32_t *tickets;     // scratch: [batch][n_kv_head], zero before first use; self-resetting
    const int32_t *pos;    // device scalar: last valid position of sequence 0 (kv_len = *pos + 1); nullptr -> kv_len
    uint32_t kv_len;       // used when pos == nullptr
    uint32_t kv_len_step;  // sequence b attends kv_len + b * kv_len_step keys (draft verification: step 1)
    uint32_t shared_kv;    // 1: all sequences read the same cache (batch_stride ignored)
    uint32_t pos_stride;   // sequence b takes its position from pos[b * pos_stride] (0: all from pos[0]; independent sequences: 1)
    uint32_t kv_stride;    // positions allocated per head
    uint64_t batch_stride; // elements between sequences in k / v
    uint32_t n_q_head, n_kv_head, batch, n_splits;
    float scale;
    uint32_t *status;
    int pdl;
    unsigned long long *trace;   // optional 4-entry timeline record (diagnostics)
    // Fused RoPE + KV append (the decoder's launch plan): q arrives un-rotated; rope_k / rope_v are this
    // token's k and v ([batch][n_kv_head][128] f32, k un-rotated); the kernel rotates q and k by the angle
    // of position *pos and appends k, v (f16) at row *pos of k_append / v_append (the same arrays as k, v).
    float2 *lse_out;                // optional [batch][n_q_head]: (max score, sum of exp(score - max)) of each head
    const float *rope_k, *rope_v;   // nullptr: q is already rotated and the cache is complete
    __half *k_append, *v_append;
    float theta_scale;              // freq_base^(-2/128)
    const float2 *rope_table;       // optional: (cos, sin) of the 64 angles of position *pos, computed once per step
                                    // (launch_rope_table); nullptr: every CTA computes them itself
    CUtensorMap kmap, vmap;         // filled by attn_make_maps
};
cudaError_t attn_make_maps(AttnArgs &a);
cudaError_t launch_attn_decode(const AttnArgs &a, cudaStream_t stream);
// Same kernel with the split-KV scratch in a fixed file-scope device array
// (no allocation at call time); cudaErrorMemoryAllocation when the launch needs
// more than attn_static_max_records() records or attn_static_max_tickets()
// (KV head, sequence) pairs.
cudaError_t launch_attn_decode_static(AttnArgs a, int device, cudaStream_t stream, size_t *records_needed);
size_t attn_static_max_records(void);
uint32_t attn_static_max_tickets(void);
cudaError_t attn_init(void);
uint32_t attn_pick_splits(uint32_t n_kv_head, uint32_t batch, uint32_t kv_len, int sms);
size_t attn_part_floats(uint32_t n_q_head, uint32_t batch, uint32_t n_splits);

// ---- comm.cu: exchange steps of the tensor-parallel step ----------------------
constexpr uint32_t kCommMaxRanks = 8;
constexpr uint32_t kCommMaxVec = 8192;     // floats per partial vector (hidden size)
constexpr uint32_t kCommChunks = 8;        // CTAs (and flags) per all-reduce
constexpr size_t kCommFlagsOff = (size_t)2 * kCommMaxRanks * kCommMaxVec * 4;
constexpr size_t kCommTopOff = kCommFlagsOff + (size_t)2 * kCommMaxRanks * kCommChunks * 4;
constexpr size_t kCommTFlagOff = kCommTopOff + (size_t)2 * kCommMaxRanks * 16;
constexpr size_t kCommBytes = kCommTFlagOff + (size_t)2 * kCommMaxRanks * 4;
struct CommState {
    uint32_t *epoch;   // kCommChunks + 1 device counters: epoch of the last exchange per chunk, then of the argmax exchange
};
struct AllReduceArgs {
    uint8_t *peers[kCommMaxRanks];   // every rank's communication buffer as mapped here; peers[rank] is local
    const float *in;                 // this rank's partial vector
    const float *resid;              // optional, added once (local)
    float *out;
    uint32_t n, rank, world;
    CommState st;
    uint32_t *status;
    uint64_t wait_ns;                // limit of the wait for the peers' flags (0 = one second)
};
struct TopExchangeArgs {
    uint8_t *peers[kCommMaxRanks];
    const float *top3;               // {best, index bits, runner-up} of this rank's slice
    uint32_t index_base;             // first global index of the slice
    int32_t *out_idx;
    float *out_margin;
    uint32_t rank, world;
    CommState st;
    uint32_t *status;
    uint64_t wait_ns;
};
// Sequence-parallel attention: every rank attended its slice of the keys and holds, per (sequence,
// query head) record, the normalised context and (max, sum); the exchange merges the ranks' records.
struct LseCombineArgs {
    uint8_t *peers[kCommMaxRanks];   // exchange buffers: [2 slots][world][max_records][132] f32, then flags [2][world][kLseChunks]
    const float *out_local;          // [n][128]
    const float2 *lse_local;         // [n]
    float *out;                      // [n][128]
    uint32_t n, max_records, rank, world;
    uint32_t *epoch;                 // kLseChunks device counters
    uint32_t *status;
    uint64_t wait_ns;                // limit of the wait for the peers' flags (0 = one second)
};
constexpr uint32_t kLseChunks = 32;
size_t lse_buffer_bytes(uint32_t max_records);
cudaError_t launch_lse_combine(const LseCombineArgs &a, cudaStream_t stream);
size_t comm_buffer_bytes(void);
cudaError_t launch_allreduce_resid(const AllReduceArgs &a, cudaStream_t stream, bool pdl);
// The push half alone (stores + flags; resid / out unused): the consumer matvec waits and adds.
cudaError_t launch_allreduce_push(const AllReduceArgs &a, cudaStream_t stream, bool pdl);
cudaError_t launch_argmax_exchange(const TopExchangeArgs &a, cudaStream_t stream, bool pdl);

// ---- glue.cu ------------------------------------------------------------
// rows vectors of n floats, `stride` floats apart in x and in y (one weight vector for all).
cudaError_t launch_rmsnorm(const float *x, const float *wnorm, float *y, float eps, uint32_t n,
                           cudaStream_t stream, uint32_t rows = 1, uint32_t stride = 0);
cudaError_t launch_add2(const float *a, const float *b, float *y, uint32_t n, cudaStream_t stream);
// fl_op_router_sel (src/runtime/decode_params.h:234-265) for n_tok tokens in one launch (one warp per token):
// softmax over n_expert logits, top_k by weight; logits [n_tok][n_expert], ids / gates [n_tok][top_k]. Expert
// parallel (lids, mgates != nullptr): also the expert's index among this rank's experts [base, base + n_local)
// or the skip mark, and the gate or 0.
cudaError_t launch_router_sel(const float *logits, uint32_t *ids, float *gates, uint32_t n_tok, uint32_t n_expert, uint32_t top_k,
                              uint32_t norm, float scale, cudaStream_t stream, uint32_t *lids = nullptr,
                              float *mgates = nullptr, uint32_t base = 0, uint32_t n_local = 0);
// The (token, slot) pairs of a block, grouped by the local expert they chose (a stable counting sort: within an
// expert the pairs stay in ascending order): cnt[e] pairs for expert e, their tokens in tok_list[e * cap + i] and
// their pair indices (token * top_k + slot) in pair_list[e * cap + i]. lids: local expert of every pair or kExpertSkip.
cudaError_t launch_group_by_expert(const uint32_t *lids, uint32_t n_pairs, uint32_t top_k, uint32_t n_local, uint32_t cap,
                                   uint32_t *cnt, uint32_t *tok_list, uint32_t *pair_list, cudaStream_t stream);
// fl_op_wmerge (src/runtime/decode_params.h:274-295).
cudaError_t launch_wmerge(const float *parts, const float *gates, const float *add1, const float *add2, float *y,
                          float scale, uint32_t n_parts, uint32_t n, uint32_t n_full, cudaStream_t stream);
// fl_op_wmerge for n_tok tokens in one launch: y[t] = sum_q gates[t][q] * parts[t][q] (products and sums rounded in
// the reference's order; no residual terms).
cudaError_t launch_wmerge_tokens(const float *parts, const float *gates, float *y, uint32_t n_parts, uint32_t n, uint32_t n_tok,
                                 cudaStream_t stream);
cudaError_t launch_silu_mul(const float *gate, const float *up, float *h, uint32_t n, cudaStream_t stream);
// RoPE (adjacent pairs) on q in place and on k, then store k and v as f16 at
// row *pos of a cache laid out [n_kv_head][kv_stride][head_dim].
struct RopeAppendArgs {
    float *q;              // [n_q_head][head_dim], rotated in place (nullptr: skip)
    const float *k;        // [n_kv_head][head_dim] (pre-RoPE)
    const float *v;        // [n_kv_head][head_dim]
    __half *kcache, *vcache;
    const int32_t *pos;
    uint32_t n_q_head, n_kv_head, head_dim, kv_stride;
    float theta_scale;     // freq_base^(-2/head_dim), computed on the host
    int pdl;
    // batch pass: n_tok tokens (0 = 1), token i at q + i * q_tok_stride, k / v + i * kv_tok_stride, position pos[i]
    uint32_t n_tok, q_tok_stride, kv_tok_stride;
    uint64_t seq_elems;    // independent sequences: token i appends to the cache of sequence i, seq_elems halves further (0: one cache)
};
cudaError_t launch_rope_append(const RopeAppendArgs &a, cudaStream_t stream);
// (cos, sin) of pos * theta_scale^i, i < head_dim / 2, with the angle built by repeated multiplication exactly as
// fl_op_rope_ds2 does (src/runtime/decode_params.h:124-160); table: head_dim / 2 float2.
cudaError_t launch_rope_table(const int32_t *pos, float theta_scale, uint32_t head_dim, float2 *table, cudaStream_t stream);
// Greedy argmax with the reference's tie rule (lowest index) and the
// top1 - top2 margin. out_idx: int32, out_margin: float; scratch: 2*blocks*2 floats.
cudaError_t launch_argmax(const float *logits, uint32_t n, int32_t *out_idx, float *out_margin,
                          float *scratch, uint32_t *ticket, int sms, cudaStream_t stream, bool pdl = false,
                          float *top3 = nullptr);   // top3: optional {best, index bits, runner-up}
// Embedding row gather + dequant: out[0..cols) = dequant(table row *token).
cudaError_t launch_embed(int fmt, const void *table, const int32_t *token, uint32_t cols, float *out,
                         cudaStream_t stream, bool pdl = false);

} // namespace flb
