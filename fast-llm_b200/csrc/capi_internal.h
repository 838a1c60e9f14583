// Shared between capi.cu and decoder.cu: the context object and error helpers.
#pragma once
#include "../../include/fl_b200.h"
#include "common.cuh"
#include "kernels.h"

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
    float *argmax_scratch = nullptr;
    void *small = nullptr;
    void *stage = nullptr;               // device staging for the *_host entry points
    size_t stage_cap = 0;
};

namespace flb {
int set_err(int code, const char *fmt, ...);
int cuda_err(cudaError_t e, const char *what);
// y[p * ystride + r] (+)= dot(W[r], x + p * xstride), p < nx, enqueued on the context's stream: up to 8
// columns per pass over the weights where the multi-column kernel takes the shape, one column per pass otherwise
// (pdl: those one-column launches are programmatic dependents of the launch before them).
int matmul(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t nx,
           uint32_t xstride, float *y, uint32_t ystride, int accumulate, uint32_t pitch = 0,
           const uint32_t *expert_id = nullptr, uint64_t expert_stride = 0, int pdl = 0);
// Hands device memory to the decoder, which frees it when it is destroyed.
void decoder_adopt(fl_b200_decoder *d, void *dev);
} // namespace flb
