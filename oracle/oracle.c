/* Test infrastructure, not product code.
 *
 * A plain-C restatement ("port") of the reference's canonical CPU semantics for
 * the decode hot path: the GGUF k-quant block layouts, the bulk dequantiser,
 * the canonical elementwise-ascending row dots and the small decode operators.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may call
 * it; the product path never does.
 *
 * Parity status: PINNED. tests/test_oracle.py checks every function here
 * bit-for-bit against the reference's own code (oracle/_ref/libflref.so, built
 * from the reference sources by oracle/Makefile) on seeded inputs, against the
 * reference's known-answer vectors for the f16 conversions
 * (tests/test_runtime.cpp:540-544), and against the fixtures in tests/golden/
 * that were generated from the reference build.
 *
 * Numerics contract reproduced here: plain f32, every multiply and add rounded
 * separately (the reference builds with -ffp-contract=off, CMakeLists.txt:13;
 * this file must be compiled the same way), sequential ascending accumulation,
 * fused multiply-add only where the reference calls fmaf() explicitly.
 *
 * Each function names the reference lines it follows.
 */
#include "flo_ops.h"
#include <math.h>
#include <string.h>

/* ------------------------------------------------------------ f16 <-> f32 -- */

/* fl_half2float, src/runtime/quants.h:40-64. Exact widening; subnormal halves
 * are renormalised. Here the subnormal case is done by an exact integer-to-
 * float scaling (m * 2^-24 is exactly representable in f32). */
static float o_h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0x1Fu) {
        bits = sign | 0x7F800000u | (man << 13);
    } else if (exp != 0) {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    } else if (man == 0) {
        bits = sign;
    } else {
        float v = (float)man * 5.9604644775390625e-08f; /* 2^-24, exact */
        uint32_t vb;
        memcpy(&vb, &v, 4);
        bits = sign | vb;
    }
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

/* fl_float2half, src/runtime/quants.h:333-356: round to nearest even, overflow
 * to inf, NaN to 0x7E00, gradual underflow. */
static uint16_t o_f2h(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t mag = u & 0x7FFFFFFFu;
    if (mag > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (mag >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);
    uint32_t sig, drop; /* significand incl. hidden bit; number of bits dropped */
    uint32_t base;      /* half bits before adding the kept significand */
    if (mag >= 0x38800000u) {
        /* normal half: drop 13 mantissa bits */
        sig = mag & 0x7FFFFFu;
        drop = 13;
        base = ((mag >> 23) - 112u) << 10;
    } else {
        const uint32_t e = mag >> 23;
        if (e < 102u) return sign; /* below half of the smallest subnormal */
        sig = (mag & 0x7FFFFFu) | 0x800000u;
        drop = 126u - e; /* 14..24 */
        base = 0;
    }
    uint32_t kept = sig >> drop;
    const uint32_t rem = sig & ((1u << drop) - 1u);
    const uint32_t halfway = 1u << (drop - 1);
    uint32_t h = base + kept; /* a carry out of the mantissa bumps the exponent */
    if (rem > halfway || (rem == halfway && (h & 1u))) h += 1;
    return (uint16_t)(sign | h);
}

/* -------------------------------------------------------- block geometry -- */
/* fl_blk_elems / fl_blk_bytes / fl_row_bytes, src/runtime/quants.h:76-99 */
static uint32_t blk_elems(int fmt) {
    switch (fmt) {
    case FLO_F32: return 1;
    case FLO_Q8_0: case FLO_Q5_0: return 32;
    default: return 256;
    }
}
static uint32_t blk_bytes(int fmt) {
    switch (fmt) {
    case FLO_F32: return 4;
    case FLO_Q8_0: return 34;
    case FLO_Q5_0: return 22;
    case FLO_Q4_K: return 144;
    default: return 210;
    }
}
uint64_t flo_row_bytes(int fmt, uint32_t cols) {
    return (uint64_t)(cols / blk_elems(fmt)) * blk_bytes(fmt);
}

static uint16_t ld16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Q4_K 6-bit scale / min of sub-block j (fl_q4k_scale_min, quants.h:121-129).
 * The 12 bytes hold, for j < 4, scale j in the low 6 bits of byte j and min j
 * in the low 6 bits of byte 4+j; for j >= 4 the low 4 bits sit in byte 4+j
 * (scale in the low nibble, min in the high nibble) and the top 2 bits in the
 * top 2 bits of bytes j-4 (scale) and j (min). */
static void q4k_scale_min(const uint8_t *s, int j, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = s[j] & 0x3F;
        *mn = s[4 + j] & 0x3F;
    } else {
        *sc = (uint8_t)((s[4 + j] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *mn = (uint8_t)((s[4 + j] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* One Q4_K super-block (144 B: f16 d, f16 dmin, 12 B scales, 128 B nibbles) to
 * 256 floats: value = (d*sc)*q - (dmin*mn), two roundings for the products and
 * one for the subtraction (dequant_chunk, kernels.h:182-200). Chunk c of 64
 * elements takes the low nibbles of bytes 32c..32c+31 for its first 32 elements
 * and the high nibbles for the next 32. */
static void q4k_block(const uint8_t *b, float *o) {
    const float d = o_h2f(ld16(b)), dmin = o_h2f(ld16(b + 2));
    const uint8_t *sc12 = b + 4, *q = b + 16;
    for (int c = 0; c < 4; ++c) {
        uint8_t s0, m0, s1, m1;
        q4k_scale_min(sc12, 2 * c, &s0, &m0);
        q4k_scale_min(sc12, 2 * c + 1, &s1, &m1);
        const float dl = d * (float)s0, ml = dmin * (float)m0;
        const float dh = d * (float)s1, mh = dmin * (float)m1;
        for (int l = 0; l < 32; ++l) {
            const uint8_t v = q[32 * c + l];
            o[64 * c + l] = dl * (float)(v & 0x0F) - ml;
            o[64 * c + 32 + l] = dh * (float)(v >> 4) - mh;
        }
    }
}

/* One Q6_K super-block (210 B: 128 B low nibbles, 64 B 2-bit highs, 16 int8
 * scales, f16 d at offset 208) to 256 floats: value = (d*sc)*(q-32)
 * (dequant_chunk, kernels.h:221-240). Half hf of 128 elements uses ql[64hf..],
 * qh[32hf..], scales[8hf..]; within a half, element 32g+l (g = 0..3) takes its
 * low 4 bits from ql[32(g&1)+l] (low nibble for g<2, high for g>=2), its high
 * 2 bits from qh[l] >> 2g, and scale index 2g + l/16. */
static void q6k_block(const uint8_t *b, float *o) {
    const float d = o_h2f(ld16(b + 208));
    for (int hf = 0; hf < 2; ++hf) {
        const uint8_t *ql = b + 64 * hf, *qh = b + 128 + 32 * hf;
        const int8_t *sc = (const int8_t *)(b + 192 + 8 * hf);
        for (int g = 0; g < 4; ++g) {
            for (int l = 0; l < 32; ++l) {
                const uint8_t lo = ql[32 * (g & 1) + l];
                const int q4 = g < 2 ? (lo & 0x0F) : (lo >> 4);
                const int q6 = q4 | (((qh[l] >> (2 * g)) & 3) << 4);
                o[128 * hf + 32 * g + l] =
                    d * (float)sc[2 * g + l / 16] * (float)(q6 - 32);
            }
        }
    }
}

/* Q8_0 block (34 B: f16 d, 32 int8): value = d*q (kernels.h:203-214). */
static void q8_0_block(const uint8_t *b, float *o) {
    const float d = o_h2f(ld16(b));
    const int8_t *q = (const int8_t *)(b + 2);
    for (int i = 0; i < 32; ++i) o[i] = d * (float)q[i];
}

/* Q5_0 block (22 B: f16 d, 4 B fifth bits, 16 B nibbles): value = d*(q-16),
 * elements 0..15 from the low nibbles with fifth bit j, 16..31 from the high
 * nibbles with fifth bit 16+j (kernels.h:169-181). */
static void q5_0_block(const uint8_t *b, float *o) {
    const float d = o_h2f(ld16(b));
    uint32_t qh;
    memcpy(&qh, b + 2, 4);
    const uint8_t *q = b + 6;
    for (int j = 0; j < 16; ++j) {
        const int lo = (q[j] & 0x0F) | (int)(((qh >> j) & 1u) << 4);
        const int hi = (q[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
        o[j] = d * (float)(lo - 16);
        o[16 + j] = d * (float)(hi - 16);
    }
}

static void block_to_f32(int fmt, const uint8_t *b, float *o) {
    switch (fmt) {
    case FLO_Q8_0: q8_0_block(b, o); break;
    case FLO_Q5_0: q5_0_block(b, o); break;
    case FLO_Q4_K: q4k_block(b, o); break;
    case FLO_Q6_K: q6k_block(b, o); break;
    default: memcpy(o, b, 4); break;
    }
}

/* dequant_chunk, src/runtime/kernels.h:162-242 (block-aligned spans). */
static void o_dequant(int fmt, const uint8_t *row, uint32_t elem0, uint32_t n, float *out) {
    const uint32_t be = blk_elems(fmt), bb = blk_bytes(fmt);
    const uint8_t *b = row + (size_t)(elem0 / be) * bb;
    for (uint32_t e = 0; e + be <= n; e += be, b += bb) block_to_f32(fmt, b, out + e);
}

/* Canonical row dot: one f32 accumulator, elements ascending, each term
 * dequant(w_i) * x_i added with its own rounding (fl_dot_row_any,
 * src/runtime/quants.h:625-642). The per-element value expressions are those of
 * the per-format loops at quants.h:132-230: they equal the bulk dequantiser's
 * value followed by one multiply by x_i, because both keep the same
 * left-to-right association. */
static float dot_row(int fmt, const uint8_t *row, const float *x, uint32_t cols) {
    float acc = 0.f;
    if (fmt == FLO_F32) {
        const float *w = (const float *)row;
        for (uint32_t c = 0; c < cols; ++c) acc += w[c] * x[c];
        return acc;
    }
    const uint32_t be = blk_elems(fmt), bb = blk_bytes(fmt);
    float v[256];
    for (uint32_t e = 0; e < cols; e += be, row += bb) {
        block_to_f32(fmt, row, v);
        for (uint32_t i = 0; i < be; ++i) acc += v[i] * x[e + i];
    }
    return acc;
}

float flo_dot_row(int fmt, const uint8_t *row, const float *x, uint32_t cols) {
    return dot_row(fmt, row, x, cols);
}

/* STREAM_DOT, src/runtime/runtime_internal.h:240-257: accumulates into y. */
static void o_stream_dot(int fmt, const uint8_t *w, uint32_t rows, uint32_t cols,
                         const float *x, uint32_t nx, uint32_t xstride,
                         float *y, uint32_t ystride) {
    const uint64_t rb = flo_row_bytes(fmt, cols);
    if (nx == 0) nx = 1;
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t p = 0; p < nx; ++p)
            y[(size_t)p * ystride + r] +=
                dot_row(fmt, w + (size_t)r * rb, x + (size_t)p * xstride, cols);
}

/* fl_op_rmsnorm, src/runtime/decode_params.h:101-106 */
static void o_rmsnorm(const float *wnorm, const float *x, float *y, float eps, uint32_t n) {
    float ss = 0.f;
    for (uint32_t i = 0; i < n; ++i) ss += x[i] * x[i];
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = 0; i < n; ++i) y[i] = x[i] * inv * wnorm[i];
}

/* fl_op_add2, decode_params.h:108-110 */
static void o_add2(const float *a, const float *b, float *y, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) y[i] = a[i] + b[i];
}

/* fl_op_rope_ds2, decode_params.h:124-160, with freq_scale 1, ext_factor 0,
 * attn_factor 1: adjacent pairs (i, i+1); the angle starts at pos and is
 * multiplied by base^(-2/n_rot) after every pair. */
static void o_rope(float *buf, int32_t pos, uint32_t n_head, uint32_t head_stride,
                   uint32_t rot_off, uint32_t n_rot, float freq_base) {
    const float step = powf(freq_base, -2.0f / (float)n_rot);
    for (uint32_t h = 0; h < n_head; ++h) {
        float *v = buf + (size_t)h * head_stride + rot_off;
        float theta = (float)pos;
        for (uint32_t i = 0; i < n_rot; i += 2) {
            const float th = 1.0f * theta;
            const float c = cosf(th) * 1.0f, s = sinf(th) * 1.0f;
            const float a = v[i], b = v[i + 1];
            v[i] = a * c - b * s;
            v[i + 1] = a * s + b * c;
            theta *= step;
        }
    }
}

/* fl_op_kv_append, decode_params.h:162-175, with d_rope = 0 */
static void o_kv_append(const float *kvb, float *kcache, float *vcache, int32_t pos,
                        uint32_t n_head, uint32_t d_k, uint32_t d_v, uint32_t max_kv) {
    (void)max_kv;
    float *kr = kcache + (size_t)pos * n_head * d_k;
    float *vr = vcache + (size_t)pos * n_head * d_v;
    for (uint32_t h = 0; h < n_head; ++h) {
        const float *src = kvb + (size_t)h * (d_k + d_v);
        memcpy(kr + (size_t)h * d_k, src, d_k * sizeof(float));
        memcpy(vr + (size_t)h * d_v, src + d_k, d_v * sizeof(float));
    }
}

/* fl_op_attn_head, decode_params.h:183-232. Scores: eight interleaved fmaf
 * chains over the head dimension folded left to right, times scale; softmax
 * with the running maximum, expf and a sequential sum; context: weights
 * e/sum applied with one fmaf per element, positions ascending. Head sizes that
 * are not multiples of 8 (dk) and 4 (dv) use plain multiply-add instead. */
static void o_attn_head(const float *q, const float *kcache, const float *vcache,
                        float *scratch, float *out, int32_t pos, float scale,
                        uint32_t head, uint32_t n_head, uint32_t dk, uint32_t dv,
                        uint32_t max_kv) {
    (void)max_kv;
    const uint32_t n = (uint32_t)pos + 1;
    const float *qh = q + (size_t)head * dk;
    const int striped = (dk % 8u) == 0 && (dv % 4u) == 0;
    float mx = -1e30f;
    for (uint32_t j = 0; j < n; ++j) {
        const float *k = kcache + ((size_t)j * n_head + head) * dk;
        float s;
        if (striped) {
            float lane[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (uint32_t d = 0; d < dk; d += 8)
                for (int t = 0; t < 8; ++t) lane[t] = fmaf(qh[d + t], k[d + t], lane[t]);
            s = lane[0];
            for (int t = 1; t < 8; ++t) s = s + lane[t];
        } else {
            s = 0.f;
            for (uint32_t d = 0; d < dk; ++d) s += qh[d] * k[d];
        }
        s *= scale;
        scratch[j] = s;
        if (s > mx) mx = s;
    }
    float sum = 0.f;
    for (uint32_t j = 0; j < n; ++j) {
        const float e = expf(scratch[j] - mx);
        scratch[j] = e;
        sum += e;
    }
    const float inv = 1.0f / sum;
    float *o = out + (size_t)head * dv;
    for (uint32_t d = 0; d < dv; ++d) o[d] = 0.f;
    for (uint32_t j = 0; j < n; ++j) {
        const float w = scratch[j] * inv;
        const float *v = vcache + ((size_t)j * n_head + head) * dv;
        if (striped)
            for (uint32_t d = 0; d < dv; ++d) o[d] = fmaf(w, v[d], o[d]);
        else
            for (uint32_t d = 0; d < dv; ++d) o[d] += w * v[d];
    }
}

/* fl_op_silu_mul, decode_params.h:267-272 */
static void o_silu_mul(const float *gate, const float *up, float *h, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) {
        const float g = gate[i];
        h[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

/* fl_op_router_sel, decode_params.h:234-265: softmax over all experts, then k
 * rounds of "largest remaining weight, lowest index on ties", optional
 * renormalisation by the selected mass, then the global scale. */
static void o_router_sel(const float *logits, uint32_t *ids, float *gates,
                         uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale) {
    float w[256];
    float mx = -1e30f;
    for (uint32_t i = 0; i < n_expert; ++i)
        if (logits[i] > mx) mx = logits[i];
    float sum = 0.f;
    for (uint32_t i = 0; i < n_expert; ++i) {
        w[i] = expf(logits[i] - mx);
        sum += w[i];
    }
    for (uint32_t i = 0; i < n_expert; ++i) w[i] /= sum;
    float picked = 0.f;
    for (uint32_t k = 0; k < top_k; ++k) {
        uint32_t best = 0;
        float bw = -1.f;
        for (uint32_t i = 0; i < n_expert; ++i) {
            int used = 0;
            for (uint32_t p = 0; p < k; ++p) used |= (ids[p] == i);
            if (!used && w[i] > bw) { bw = w[i]; best = i; }
        }
        ids[k] = best;
        gates[k] = bw;
        picked += bw;
    }
    for (uint32_t k = 0; k < top_k; ++k) {
        if (norm) gates[k] /= picked;
        gates[k] *= scale;
    }
}

/* fl_op_wmerge, decode_params.h:274-295, exact merge (n_full = 0, so the gate
 * rescale factor is exactly 1 and is still multiplied in, as the reference
 * does). */
static void o_wmerge(const float *parts, const float *gates, const float *add1,
                     const float *add2, float *y, float scale, uint32_t n_parts, uint32_t n) {
    const float gsc = 1.0f;
    for (uint32_t i = 0; i < n; ++i) {
        float acc = 0.f;
        for (uint32_t p = 0; p < n_parts; ++p)
            acc += (gates ? gsc * gates[p] : 1.0f) * parts[(size_t)p * n + i];
        acc *= scale;
        if (add1) acc += add1[i];
        if (add2) acc += add2[i];
        y[i] = acc;
    }
}

static const flo_ops_t kPortOps = {
    "port", o_h2f, o_f2h, o_dequant, o_stream_dot, o_rmsnorm, o_add2, o_rope,
    o_kv_append, o_attn_head, o_silu_mul, o_router_sel, o_wmerge,
};

const flo_ops_t *flo_port_ops(void) { return &kPortOps; }
