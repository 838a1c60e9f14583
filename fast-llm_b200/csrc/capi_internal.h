// Shared between capi.cu and decoder.cu: the context object and error helpers.
#pragma once
#include "../../include/fl_b200.h"
#include "common.cuh"
#include "kernels.h"

#include <vector>

struct fl_b200_ctx {
    int device = 0;
    int sms = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    uint32_t *status = nullptr;          // device status word (+ small counters behind it)
    uint32_t *argmax_ticket = nullptr;
    uint32_t *attn_tickets = nullptr;    // zero between launches (kernels reset them)
    uint32_t attn_tickets_cap = 0;
    float *attn_part = nullptr;          // split-KV partials (scratch, grown on demand)
    size_t attn_part_cap = 0;
    // Scratch buffers that were outgrown. A recorded plan (fl_b200_plan) keeps the address it was
    // captured with, so an outgrown buffer stays allocated until the context goes.
    std::vector<void *> retired;
    float *argmax_scratch = nullptr;
    void *small = nullptr;
    uint8_t *xq = nullptr;               // converted activations of the multi-column matmul (fixed size, see fl_b200_create)
    uint8_t *xu = nullptr;               // the same for the tcgen05 matmul, with its split-K scratch and tickets
    float *um_scratch = nullptr;
    uint32_t *um_tickets = nullptr;
    uint32_t *grid_bar = nullptr;        // barrier state of the chained matvec launches (two words, zero between launches)
    uint64_t wait_limit_ns = 0;          // limit of the exchange kernels' waits for other ranks (0 = one second)
    void *stage = nullptr;               // device staging for the *_host entry points
    size_t stage_cap = 0;
};

namespace flb {
int set_err(int code, const char *fmt, ...);
// Makes c->attn_part at least `bytes` large (never frees a buffer a recorded plan may still use).
int grow_attn_part(fl_b200_ctx *c, size_t bytes);
int cuda_err(cudaError_t e, const char *what);
// y[p * ystride + r] (+)= dot(W[r], x + p * xstride), p < nx, enqueued on the context's stream: up to 8
// columns per pass over the weights where the multi-column kernel takes the shape, one column per pass otherwise
// (pdl: those one-column launches are programmatic dependents of the launch before them).
int matmul(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t nx,
           uint32_t xstride, float *y, uint32_t ystride, int accumulate, uint32_t pitch = 0,
           const uint32_t *expert_id = nullptr, uint64_t expert_stride = 0, int pdl = 0, const float *x2 = nullptr,
           int same_columns = 0);
// x2 != nullptr: column p is SiLU(x_p) * x2_p (fl_op_silu_mul fused into the matmul's activation prologue).
// same_columns: x, nx and the weight format are those of the matmul call before this one on the same context, so the
// converted activations of the multi-column kernel are reused (Q/K after Q, up after gate).
// Hands device memory to the decoder, which frees it when it is destroyed.
void decoder_adopt(fl_b200_decoder *d, void *dev);
// The MoE block inside a decoder step (moe.cu): y[t] = sum over the selected experts of gate * expert(x[t]) for
// n_tok <= the block's max_tokens rows of x, enqueued on the block's context's stream (one token: one expert walk per
// selected expert through the expert-indexed matvec; more: every expert once through the multi-column matmul).
// *n_launch: launches enqueued.
// wnorm / eps / resid (one token): x is the raw hidden state, RMSNorm(x) * wnorm is taken inside the block's first
// kernels, and y = resid + the block's output.
int moe_enqueue_tokens(fl_b200_moe *m, const float *x, uint32_t n_tok, float *y, uint32_t *n_launch, const float *wnorm = nullptr,
                       float eps = 0.f, const float *resid = nullptr);
fl_b200_ctx *moe_ctx(const fl_b200_moe *m);
const fl_b200_moe_cfg *moe_cfg(const fl_b200_moe *m);
uint32_t moe_world(const fl_b200_moe *m);
// Packed weight bytes one token reads in the block: the router and top_k experts.
uint64_t moe_bytes_per_token(const fl_b200_moe *m);
} // namespace flb
