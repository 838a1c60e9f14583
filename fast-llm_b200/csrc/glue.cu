// Small decode operators around the matvecs and attention. Each follows one
// canonical operator of the reference (src/runtime/decode_params.h) and keeps
// its rounding where that is cheap: separate multiplies / adds via __fmul_rn,
// __fadd_rn, __fsub_rn, IEEE division and square root.
#include "common.cuh"
#include "kernels.h"

namespace flb {

namespace {

// fl_op_rmsnorm, decode_params.h:101-106. The sum of squares is a tree
// reduction here (the reference sums sequentially); everything after it rounds
// like the reference: 1/sqrtf(ss/n + eps), then (x*s)*w.
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                       float *__restrict__ y, float eps, uint32_t n, uint32_t stride) {
    __shared__ float red[32];
    __shared__ float inv;
    x += (size_t)blockIdx.y * stride;   // one block per vector
    y += (size_t)blockIdx.y * stride;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (uint32_t k = 0; k < (blockDim.x + 31) / 32; ++k) t += red[k];
        inv = 1.0f / sqrtf(__fadd_rn(t / (float)n, eps));
    }
    __syncthreads();
    const float s = inv;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) y[i] = __fmul_rn(__fmul_rn(x[i], s), w[i]);
}

// fl_op_add2, decode_params.h:108-110
__global__ void add2_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ y,
                            uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(a[i], b[i]);
}

// Expert selection of the MoE router (fl_op_router_sel, src/runtime/decode_params.h:234-265): softmax over the
// expert logits of a token, the top_k largest weights (ties go to the lower index), optionally renormalised
// over the chosen ones. One warp per token, every token of the block in one launch. What the warp does in
// parallel: the maximum, the exponentials, the divisions and each round's arg-max. What stays sequential,
// because f32 sums depend on their order and the results have to equal the reference's bit for bit: the sum of
// the exponentials (ascending expert index, one lane) and the sum of the chosen weights (selection order).
// With expert parallelism (lids != nullptr) the kernel also writes, per (token, slot), the index of the expert
// among this rank's experts [base, base + n_local) or the skip mark, and the gate or 0.
constexpr int kRouterWarps = 4;
__global__ void __launch_bounds__(kRouterWarps * 32) router_sel_kernel(const float *__restrict__ logits, uint32_t *ids, float *gates,
                                                                     uint32_t *lids, float *mgates, uint32_t n_tok,
                                                                     uint32_t n_expert, uint32_t top_k, uint32_t norm, float scale,
                                                                     uint32_t base, uint32_t n_local) {
    __shared__ float w_s[kRouterWarps][256], g_s[kRouterWarps][256];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t tok = blockIdx.x * kRouterWarps + warp;
    if (tok >= n_tok) return;
    const float *l = logits + (size_t)tok * n_expert;
    float *w = w_s[warp], *gk = g_s[warp];
    float mx = -1e30f;
    for (uint32_t i = lane; i < n_expert; i += 32) mx = fmaxf(mx, l[i]);
    mx = warp_max(mx);
    for (uint32_t i = lane; i < n_expert; i += 32) w[i] = expf(__fsub_rn(l[i], mx));
    __syncwarp();
    float sum = 0.f;
    if (lane == 0)
        for (uint32_t i = 0; i < n_expert; ++i) sum = __fadd_rn(sum, w[i]);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    for (uint32_t i = lane; i < n_expert; i += 32) w[i] = __fdiv_rn(w[i], sum);
    __syncwarp();
    float tsum = 0.f;
    for (uint32_t k = 0; k < top_k; ++k) {
        // the largest weight not chosen yet; a chosen entry is overwritten with -2, below the starting value -1
        float bw = -1.f;
        uint32_t best = 0;
        for (uint32_t i = lane; i < n_expert; i += 32)
            if (w[i] > bw) { bw = w[i]; best = i; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ow = __shfl_xor_sync(0xffffffffu, bw, o);
            const uint32_t ob = __shfl_xor_sync(0xffffffffu, best, o);
            if (ow > bw || (ow == bw && ob < best)) { bw = ow; best = ob; }
        }
        tsum = __fadd_rn(tsum, bw);   // every lane keeps the same running sum, in selection order
        if (lane == 0) {
            ids[(size_t)tok * top_k + k] = best;
            gk[k] = bw;
            if (bw >= 0.f) w[best] = -2.f;
        }
        __syncwarp();
    }
    for (uint32_t k = lane; k < top_k; k += 32) {
        float g = gk[k];
        if (norm) g = __fdiv_rn(g, tsum);
        g = __fmul_rn(g, scale);
        gates[(size_t)tok * top_k + k] = g;
        if (lids) {
            const uint32_t e = ids[(size_t)tok * top_k + k];
            const bool mine = e >= base && e - base < n_local;
            lids[(size_t)tok * top_k + k] = mine ? e - base : kExpertSkip;
            mgates[(size_t)tok * top_k + k] = mine ? g : 0.f;
        }
    }
}

// fl_op_wmerge, decode_params.h:274-295: y = add1 + add2 + scale * sum_q gate_q * part_q,
// products and sums rounded separately and in the reference's order.
__global__ void wmerge_kernel(const float *__restrict__ parts, const float *__restrict__ gates,
                              const float *__restrict__ add1, const float *__restrict__ add2, float *__restrict__ y,
                              float scale, uint32_t n_parts, uint32_t n, uint32_t n_full) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float gsc = 1.0f;
    if (gates && n_full > n_parts) {
        float s = 0.f, sf = 0.f;
        for (uint32_t q = 0; q < n_parts; ++q) s = __fadd_rn(s, gates[q]);
        for (uint32_t q = 0; q < n_full; ++q) sf = __fadd_rn(sf, gates[q]);
        if (s > 0.f) gsc = __fdiv_rn(sf, s);
    }
    float acc = 0.f;
    for (uint32_t q = 0; q < n_parts; ++q) {
        const float g = gates ? __fmul_rn(gsc, gates[q]) : 1.0f;
        acc = __fadd_rn(acc, __fmul_rn(g, parts[(size_t)q * n + i]));
    }
    acc = __fmul_rn(acc, scale);
    if (add1) acc = __fadd_rn(acc, add1[i]);
    if (add2) acc = __fadd_rn(acc, add2[i]);
    y[i] = acc;
}

// y[t][i] = sum_q (gates[t][q] * parts[t][q][i]), the arithmetic of fl_op_wmerge (decode_params.h:274-295) without its
// residual terms, for every token of a block in one launch. grid (ceil(n / 256), n_tok).
__global__ void wmerge_tokens_kernel(const float *__restrict__ parts, const float *__restrict__ gates, float *__restrict__ y,
                                     uint32_t n_parts, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (i >= n) return;
    float acc = 0.f;
    for (uint32_t q = 0; q < n_parts; ++q)
        acc = __fadd_rn(acc, __fmul_rn(gates[(size_t)t * n_parts + q], parts[((size_t)t * n_parts + q) * n + i]));
    y[(size_t)t * n + i] = __fmul_rn(acc, 1.0f);
}

// One warp: a stable counting sort of the pairs by local expert.
__global__ void __launch_bounds__(32) group_by_expert_kernel(const uint32_t *__restrict__ lids, uint32_t n_pairs, uint32_t top_k,
                                                             uint32_t n_local, uint32_t cap, uint32_t *__restrict__ cnt,
                                                             uint32_t *__restrict__ tok_list, uint32_t *__restrict__ pair_list) {
    const uint32_t lane = threadIdx.x;
    for (uint32_t e = lane; e < n_local; e += 32) cnt[e] = 0;
    __syncwarp();
    for (uint32_t b = 0; b < n_pairs; b += 32) {
        const uint32_t pair = b + lane;
        const uint32_t e = pair < n_pairs ? lids[pair] : 0xFFFFFFFFu;
        for (uint32_t x = 0; x < n_local; ++x) {
            const uint32_t mask = __ballot_sync(0xffffffffu, e == x);
            if (mask == 0) continue;
            const uint32_t base = cnt[x];
            if (e == x) {
                const uint32_t pos = base + __popc(mask & ((1u << lane) - 1u));
                if (pos < cap) { tok_list[(size_t)x * cap + pos] = pair / top_k; pair_list[(size_t)x * cap + pos] = pair; }
            }
            __syncwarp();
            if (lane == 0) cnt[x] = min(base + __popc(mask), cap);
            __syncwarp();
        }
    }
}

// fl_op_silu_mul, decode_params.h:267-272: (g / (1 + expf(-g))) * u
__global__ void silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ h,
                                uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float v = g[i];
        h[i] = __fmul_rn(v / __fadd_rn(1.0f, expf(-v)), u[i]);
    }
}

// fl_op_rope_ds2 (decode_params.h:124-160, plain RoPE: adjacent pairs, angle
// pos * theta_scale^i built by repeated multiplication exactly as the reference
// does, so the angle is bit-identical; cosf/sinf differ from the host libm by at
// most a few ulp) followed by the f16 KV append (fl_op_kv_append,
// decode_params.h:162-175, with the cache kept in f16, head-major).
__global__ void __launch_bounds__(128) rope_append_kernel(const RopeAppendArgs a) {
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t half = a.head_dim / 2;
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t n_rot_heads = (a.q ? a.n_q_head : 0) + a.n_kv_head;
    const uint32_t tokn = blockIdx.y;   // token of a batch pass (0 in a single step)
    const uint32_t pos = (uint32_t)a.pos[tokn];
    if (t < n_rot_heads * half) {
        const uint32_t h = t / half, i = t % half;
        float theta = (float)(int32_t)pos;
        for (uint32_t k = 0; k < i; ++k) theta = __fmul_rn(theta, a.theta_scale);
        const float c = cosf(theta), s = sinf(theta);
        const uint32_t nq = a.q ? a.n_q_head : 0;
        if (h < nq) {
            float *v = a.q + (size_t)tokn * a.q_tok_stride + (size_t)h * a.head_dim + 2 * i;
            const float x0 = v[0], x1 = v[1];
            v[0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            v[1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
        } else {
            const uint32_t hk = h - nq;
            const float *v = a.k + (size_t)tokn * a.kv_tok_stride + (size_t)hk * a.head_dim + 2 * i;
            const float x0 = v[0], x1 = v[1];
            __half *dst = a.kcache + (size_t)tokn * a.seq_elems + ((size_t)hk * a.kv_stride + pos) * a.head_dim + 2 * i;
            dst[0] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
            dst[1] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
        }
    } else if (t < (n_rot_heads + a.n_kv_head) * half) {
        const uint32_t u = t - n_rot_heads * half;
        const uint32_t hk = u / half, i = u % half;
        const float *v = a.v + (size_t)tokn * a.kv_tok_stride + (size_t)hk * a.head_dim + 2 * i;
        __half *dst = a.vcache + (size_t)tokn * a.seq_elems + ((size_t)hk * a.kv_stride + pos) * a.head_dim + 2 * i;
        dst[0] = __float2half_rn(v[0]);
        dst[1] = __float2half_rn(v[1]);
    }
}

__global__ void rope_table_kernel(const int32_t *pos, float theta_scale, uint32_t half, float2 *table) {
    const uint32_t i = threadIdx.x;
    if (i >= half) return;
    float theta = (float)*pos;
    for (uint32_t k = 0; k < i; ++k) theta = __fmul_rn(theta, theta_scale);
    table[i] = make_float2(cosf(theta), sinf(theta));
}

// Greedy argmax: strict '>' scan order of the reference (lowest index wins
// ties) and the runner-up value for the margin (src/model/decoder.cpp:1253-1264).
struct Top { float b; uint32_t i; float s; };

__device__ __forceinline__ Top top_merge(const Top &x, const Top &y) {
    const bool y_wins = y.b > x.b || (y.b == x.b && y.i < x.i);
    Top r;
    if (y_wins) { r.b = y.b; r.i = y.i; r.s = fmaxf(x.b, fmaxf(x.s, y.s)); }
    else { r.b = x.b; r.i = x.i; r.s = fmaxf(y.b, fmaxf(x.s, y.s)); }
    return r;
}
__device__ __forceinline__ Top top_warp(Top t) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Top u;
        u.b = __shfl_xor_sync(0xffffffffu, t.b, o);
        u.i = __shfl_xor_sync(0xffffffffu, t.i, o);
        u.s = __shfl_xor_sync(0xffffffffu, t.s, o);
        t = top_merge(t, u);
    }
    return t;
}

__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ lg, uint32_t n, int32_t *out_idx,
                                                     float *out_margin, float *scratch, uint32_t *ticket, float *top3) {
    griddep_launch_dependents();
    griddep_wait();
    __shared__ Top wtop[8];
    __shared__ uint32_t last;
    Top t{-INFINITY, 0xFFFFFFFFu, -INFINITY};
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = lg[i];
        if (v > t.b) { t.s = t.b; t.b = v; t.i = i; }   // indices ascend within a thread
        else if (v > t.s) t.s = v;
    }
    t = top_warp(t);
    if ((threadIdx.x & 31u) == 0) wtop[threadIdx.x >> 5] = t;
    __syncthreads();
    if (threadIdx.x == 0) {
        Top r = wtop[0];
        for (int w = 1; w < 8; ++w) r = top_merge(r, wtop[w]);
        float *slot = scratch + 3 * blockIdx.x;
        slot[0] = r.b; slot[1] = __uint_as_float(r.i); slot[2] = r.s;
        __threadfence();
        last = atomicAdd(ticket, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        Top r{-INFINITY, 0xFFFFFFFFu, -INFINITY};
        for (uint32_t k = threadIdx.x; k < gridDim.x; k += 32) {
            Top u;
            u.b = __ldcg(scratch + 3 * k);
            u.i = __float_as_uint(__ldcg(scratch + 3 * k + 1));
            u.s = __ldcg(scratch + 3 * k + 2);
            r = top_merge(r, u);
        }
        r = top_warp(r);
        if (threadIdx.x == 0) {
            *out_idx = (int32_t)r.i;
            *out_margin = r.b - r.s;
            if (top3) { top3[0] = r.b; top3[1] = __uint_as_float(r.i); top3[2] = r.s; }   // for the cross-rank merge
            *ticket = 0;
        }
    }
}

} // namespace

cudaError_t launch_rmsnorm(const float *x, const float *wnorm, float *y, float eps, uint32_t n,
                           cudaStream_t stream, uint32_t rows, uint32_t stride) {
    if (rows == 0) return cudaErrorInvalidValue;
    rmsnorm_kernel<<<dim3(1, rows), 1024, 0, stream>>>(x, wnorm, y, eps, n, stride);
    return cudaGetLastError();
}

cudaError_t launch_add2(const float *a, const float *b, float *y, uint32_t n, cudaStream_t stream) {
    add2_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a, b, y, n);
    return cudaGetLastError();
}

cudaError_t launch_router_sel(const float *logits, uint32_t *ids, float *gates, uint32_t n_tok, uint32_t n_expert, uint32_t top_k,
                              uint32_t norm, float scale, cudaStream_t stream, uint32_t *lids, float *mgates, uint32_t base,
                              uint32_t n_local) {
    if (n_tok == 0 || n_expert == 0 || n_expert > 256 || top_k == 0 || top_k > n_expert) return cudaErrorInvalidValue;
    if ((lids == nullptr) != (mgates == nullptr)) return cudaErrorInvalidValue;
    router_sel_kernel<<<(n_tok + kRouterWarps - 1) / kRouterWarps, kRouterWarps * 32, 0, stream>>>(
        logits, ids, gates, lids, mgates, n_tok, n_expert, top_k, norm, scale, base, n_local);
    return cudaGetLastError();
}

cudaError_t launch_wmerge(const float *parts, const float *gates, const float *add1, const float *add2, float *y,
                          float scale, uint32_t n_parts, uint32_t n, uint32_t n_full, cudaStream_t stream) {
    if (n == 0 || n_parts == 0) return cudaErrorInvalidValue;
    wmerge_kernel<<<(n + 255) / 256, 256, 0, stream>>>(parts, gates, add1, add2, y, scale, n_parts, n, n_full);
    return cudaGetLastError();
}

cudaError_t launch_wmerge_tokens(const float *parts, const float *gates, float *y, uint32_t n_parts, uint32_t n, uint32_t n_tok,
                                 cudaStream_t stream) {
    if (n == 0 || n_parts == 0 || n_tok == 0) return cudaErrorInvalidValue;
    wmerge_tokens_kernel<<<dim3((n + 255) / 256, n_tok), 256, 0, stream>>>(parts, gates, y, n_parts, n);
    return cudaGetLastError();
}

cudaError_t launch_group_by_expert(const uint32_t *lids, uint32_t n_pairs, uint32_t top_k, uint32_t n_local, uint32_t cap,
                                   uint32_t *cnt, uint32_t *tok_list, uint32_t *pair_list, cudaStream_t stream) {
    if (n_pairs == 0 || top_k == 0 || n_local == 0 || cap == 0) return cudaErrorInvalidValue;
    group_by_expert_kernel<<<1, 32, 0, stream>>>(lids, n_pairs, top_k, n_local, cap, cnt, tok_list, pair_list);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const float *gate, const float *up, float *h, uint32_t n, cudaStream_t stream) {
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, stream>>>(gate, up, h, n);
    return cudaGetLastError();
}

cudaError_t launch_rope_append(const RopeAppendArgs &a, cudaStream_t stream) {
    if (a.head_dim == 0 || (a.head_dim & 1u)) return cudaErrorInvalidValue;
    const uint32_t half = a.head_dim / 2;
    const uint32_t n = ((a.q ? a.n_q_head : 0) + 2 * a.n_kv_head) * half;
    return launch_kernel(rope_append_kernel, dim3((n + 127) / 128, a.n_tok ? a.n_tok : 1), dim3(128), 0, stream, a.pdl != 0, a);
}

cudaError_t launch_rope_table(const int32_t *pos, float theta_scale, uint32_t head_dim, float2 *table, cudaStream_t stream) {
    if (head_dim == 0 || (head_dim & 1u) || head_dim > 2048) return cudaErrorInvalidValue;
    rope_table_kernel<<<1, head_dim / 2, 0, stream>>>(pos, theta_scale, head_dim / 2, table);
    return cudaGetLastError();
}

cudaError_t launch_argmax(const float *logits, uint32_t n, int32_t *out_idx, float *out_margin,
                          float *scratch, uint32_t *ticket, int sms, cudaStream_t stream, bool pdl, float *top3) {
    uint32_t grid = (n + 255) / 256;
    if (grid > (uint32_t)sms) grid = (uint32_t)sms;
    if (grid == 0) return cudaErrorInvalidValue;
    return launch_kernel(argmax_kernel, dim3(grid), dim3(256), 0, stream, pdl, logits, n, out_idx, out_margin, scratch,
                         ticket, top3);
}

} // namespace flb
