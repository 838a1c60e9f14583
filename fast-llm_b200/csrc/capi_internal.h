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
    struct MatvecScratchFwd *mv = nullptr;   // scratch of ad-hoc matvec calls (MatvecScratch)
    void *stage = nullptr;               // device staging for the *_host entry points
    size_t stage_cap = 0;
};

namespace flb {
int set_err(int code, const char *fmt, ...);
int cuda_err(cudaError_t e, const char *what);
// Scratch of the streaming matvec: partial row sums of units shared between
// warps and their arrival counters (zero between launches).
struct MatvecScratch {
    float *buf = nullptr;
    size_t cap = 0;          // floats
    uint32_t *tickets = nullptr;
    size_t tickets_cap = 0;
};
// Grows the scratch for this launch if needed (synchronises; not allowed during
// stream capture) and points the arguments at it.
int ensure_matvec_scratch(fl_b200_ctx *c, MatvecScratch &s, MatvecArgs &a);
void free_matvec_scratch(MatvecScratch &s);
} // namespace flb
