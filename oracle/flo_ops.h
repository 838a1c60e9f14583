/* Test infrastructure, not product code.
 *
 * C operator table shared by the two CPU oracles of the decode hot path:
 *   - oracle/oracle.c     : a plain-C restatement of the reference's canonical
 *                           CPU semantics ("port"), and
 *   - oracle/ref_shim.cpp : the reference's own functions, compiled from the
 *                           reference sources where they lie and re-exported
 *                           ("reference").
 * Both fill the same table so that the model-level driver (oracle/llama_oracle.c)
 * and the Python tests can run either one through identical call sites.
 *
 * Format ids follow fastllm::Fmt (include/fastllm/fastllm.h:56-57):
 *   0 F32, 1 Q8_0, 2 Q5_0, 3 Q4_K, 4 Q6_K.
 */
#ifndef FLO_OPS_H
#define FLO_OPS_H
#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { FLO_F32 = 0, FLO_Q8_0 = 1, FLO_Q5_0 = 2, FLO_Q4_K = 3, FLO_Q6_K = 4 };

typedef struct flo_ops {
    const char *name;   /* "port" or "reference" */
    /* software half conversions (src/runtime/quants.h:40-64, :333-356) */
    float    (*h2f)(uint16_t h);
    uint16_t (*f2h)(float f);
    /* bulk dequantise elements [elem0, elem0+n) of one packed row
     * (dequant_chunk, src/runtime/kernels.h:162-242) */
    void (*dequant)(int fmt, const uint8_t *row, uint32_t elem0, uint32_t n, float *out);
    /* STREAM_DOT tile: y[p*ystride + r] += dot(W[r], x + p*xstride)
     * (exec_task_scalar, src/runtime/runtime_internal.h:240-257) */
    void (*stream_dot)(int fmt, const uint8_t *w, uint32_t rows, uint32_t cols,
                       const float *x, uint32_t nx, uint32_t xstride,
                       float *y, uint32_t ystride);
    /* fl_op_rmsnorm (src/runtime/decode_params.h:101-106) */
    void (*rmsnorm)(const float *wnorm, const float *x, float *y, float eps, uint32_t n);
    /* fl_op_add2 (decode_params.h:108-110) */
    void (*add2)(const float *a, const float *b, float *y, uint32_t n);
    /* fl_op_rope_ds2 (decode_params.h:124-160), plain RoPE: freq_scale 1,
     * ext_factor 0, attn_factor 1 */
    void (*rope)(float *buf, int32_t pos, uint32_t n_head, uint32_t head_stride,
                 uint32_t rot_off, uint32_t n_rot, float freq_base);
    /* fl_op_kv_append (decode_params.h:162-175) with d_rope = 0:
     * kvb is n_head * (d_k + d_v), per head [k | v] */
    void (*kv_append)(const float *kvb, float *kcache, float *vcache, int32_t pos,
                      uint32_t n_head, uint32_t d_k, uint32_t d_v, uint32_t max_kv);
    /* fl_op_attn_head (decode_params.h:183-232): one head over keys 0..pos of
     * an f32 cache laid out [max_kv][n_head][d] */
    void (*attn_head)(const float *q, const float *kcache, const float *vcache,
                      float *scratch, float *out, int32_t pos, float scale,
                      uint32_t head, uint32_t n_head, uint32_t dk, uint32_t dv,
                      uint32_t max_kv);
    /* fl_op_silu_mul (decode_params.h:267-272) */
    void (*silu_mul)(const float *gate, const float *up, float *h, uint32_t n);
    /* fl_op_router_sel (decode_params.h:234-265) */
    void (*router_sel)(const float *logits, uint32_t *ids, float *gates,
                       uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale);
    /* fl_op_wmerge (decode_params.h:274-295) with n_full = 0 */
    void (*wmerge)(const float *parts, const float *gates, const float *add1,
                   const float *add2, float *y, float scale, uint32_t n_parts, uint32_t n);
} flo_ops_t;

/* Provided by oracle/oracle.c (liboracle.so). */
const flo_ops_t *flo_port_ops(void);
/* Provided by oracle/ref_shim.cpp (oracle/_ref/libflref.so). */
const flo_ops_t *flref_ops(void);

#ifdef __cplusplus
}
#endif
#endif
