// Single-token (decode) grouped-query attention over an f16 KV cache, split
// along the sequence with an in-kernel log-sum-exp combine. Semantics follow the
// reference's one-head operator fl_op_attn_head
// (src/runtime/decode_params.h:183-232): scores = scale * (q . k_j) over keys
// 0..pos, softmax, context = sum softmax_j * v_j, all in f32; the reference has
// no GPU attention kernel (it runs the operator on one thread,
// src/runtime/gpu_exec.cu:84-88), no GQA and no f16 cache, so layout and
// parallelisation here are new.
//
// Cache layout in HBM: [batch][n_kv_head][kv_stride][128] f16 for K and for V,
// described to the TMA unit as a 2-D tensor [rows][128]. A tile is 64 positions:
// four boxes of 64 rows x 64 columns (K and V, low and high half of the head
// dimension), written to shared memory with the 128-byte swizzle so that the
// 8 x 8 matrix loads below are free of bank conflicts. 3-stage ring per CTA.
//
// Grid = (n_splits, n_kv_head, batch), 128 threads, two or more CTAs per SM. A
// CTA serves the 4 query heads of its KV head, so every K/V byte is read from HBM
// once per group. Warp w owns positions 16w .. 16w+15 of every tile and runs an
// independent online softmax over them (no block barrier between scores,
// softmax and context):
//   scores : mma.sync m16n8k16 (f16 x f16 -> f32), A = K rows (ldmatrix), B = q.
//            The 8 columns are the 4 heads, each as (hi, lo) with q = hi + lo in
//            f16, so the product is exact to 2^-22 although the multiplier is f16;
//   softmax: lane (g, t) holds head t for positions g and g + 8; max / sum over
//            the 8 lanes of a head by shuffles;
//   context: mma.sync with A = V^T (ldmatrix.trans), B = probabilities as
//            (hi, lo) f16 pairs, accumulators 128 dims x 4 heads in registers.
// The warps' (max, sum, context) are merged through shared memory, each CTA
// writes one record per head to scratch and takes a ticket; the CTA that draws
// the last ticket of its (batch, kv head) rescales and sums the partials in split
// order (deterministic) and writes the output. No CTA ever waits for another one.
//
// Fused mode of the decoder (rope_k != nullptr): q arrives un-rotated, and this
// token's K and V rows are not in the cache yet. Every CTA rotates q itself
// (fl_op_rope_ds2, plain RoPE on adjacent pairs, angle built by repeated
// multiplication like the reference, src/runtime/decode_params.h:124-160); the CTA
// whose range holds the current position also rotates k, rounds k and v to f16,
// appends them to the cache (fl_op_kv_append, decode_params.h:162-175) and patches
// the rows into its shared-memory tile. Tiles are requested before the dependency
// wait: older rows cannot change.
#include "common.cuh"
#include "kernels.h"

namespace flb {

namespace {

constexpr int kD = 128;              // head dimension
constexpr int kGroup = 4;            // query heads per KV head handled by one CTA
constexpr int kTile = 64;            // positions per stage
constexpr int kStages = 3;
constexpr int kAttnWarps = 4;        // warp w <-> positions 16w .. 16w+15 of a tile
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr uint32_t kHalfBytes = kTile * 128;        // one box: 64 rows x 64 f16 (128 bytes), swizzled
constexpr uint32_t kStageBytes = 4 * kHalfBytes;    // K lo, K hi, V lo, V hi = 32 KB
constexpr int kPartStride = kD + 4;  // o[128], m, l, pad (keeps o 16-byte aligned)

struct AttnSmem {
    uint8_t ring[kStages][kStageBytes];   // 1024-byte aligned (swizzle atom)
    float wo[kAttnWarps][kGroup][kD];     // per-warp context, for the merge
    float wm[kAttnWarps][kGroup], wl[kAttnWarps][kGroup];
    float2 cs[kD / 2];                    // cos / sin of this position's rotation angles (fused mode)
    uint64_t full[kStages];
    uint32_t is_last;
};

// Byte offset of (row r, 16-byte chunk c of the 128-byte row) inside a swizzled box.
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// x as an f16 pair: part 0 = the nearest f16, part 1 = the f16 nearest to the remainder.
__device__ __forceinline__ __half split_part(float x, uint32_t part) {
    const __half hi = __float2half_rn(x);
    return part ? __float2half_rn(x - __half2float(hi)) : hi;
}
__device__ __forceinline__ uint32_t pack_h2(__half lo, __half hi) {
    return (uint32_t)__half_as_ushort(lo) | ((uint32_t)__half_as_ushort(hi) << 16);
}

__global__ void __launch_bounds__(kAttnThreads, 2) attn_decode_kernel(const __grid_constant__ AttnArgs a) {
    extern __shared__ uint8_t smem_dyn[];
    AttnSmem &sm = *reinterpret_cast<AttnSmem *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const uint32_t group = a.n_q_head / a.n_kv_head;   // == kGroup (checked on the host)
    const bool fused = a.rope_k != nullptr;
    if (tid == 0) trace_min(a.trace, 0);
    griddep_launch_dependents();
    // *pos was written at the end of the previous step (or is kv_len - 1 of a single call): stable here.
    const uint32_t kv_len = (a.pos ? (uint32_t)a.pos[b * a.pos_stride] + 1u : a.kv_len) + b * a.kv_len_step;
    const uint32_t tiles_total = (kv_len + kTile - 1) / kTile;
    const uint32_t tps = (tiles_total + a.n_splits - 1) / a.n_splits;
    const uint32_t t0 = split * tps;
    const uint32_t t1 = min(t0 + tps, tiles_total);
    const uint32_t n_tiles = t1 > t0 ? t1 - t0 : 0;
    const uint32_t row0 = ((a.shared_kv ? 0u : b) * a.n_kv_head + hkv) * a.kv_stride;   // first row of this head in the 2-D view

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&sm.full[s], 1);
        sm.is_last = 0;
        fence_barrier_init();
    }
    if (fused && tid < kD / 2) {
        if (a.rope_table) {
            sm.cs[tid] = a.rope_table[tid];   // computed once per step, before this launch's predecessors
        } else {
            // angle of pair i: pos * theta_scale^i by repeated multiplication (bit-identical to the reference)
            float theta = (float)(int32_t)(kv_len - 1u);
            for (uint32_t k = 0; k < tid; ++k) theta = __fmul_rn(theta, a.theta_scale);
            sm.cs[tid] = make_float2(cosf(theta), sinf(theta));
        }
    }
    __syncthreads();

    const uint32_t ring = smem_u32(&sm.ring[0][0]);
    auto issue = [&](uint32_t i) {   // thread 0 only: tile t0 + i into slot i % kStages
        const uint32_t slot = i % kStages, r = row0 + (t0 + i) * kTile;
        const uint32_t dst = ring + slot * kStageBytes;
        mbar_arrive_expect_tx(&sm.full[slot], kStageBytes);
        // rows past the end of the whole cache are filled with zeros; rows past kv_len are masked below
        tma_box(dst, &a.kmap, 0, r, &sm.full[slot]);
        tma_box(dst + kHalfBytes, &a.kmap, 64, r, &sm.full[slot]);
        tma_box(dst + 2 * kHalfBytes, &a.vmap, 0, r, &sm.full[slot]);
        tma_box(dst + 3 * kHalfBytes, &a.vmap, 64, r, &sm.full[slot]);
    };
    // Older cache rows never change: request the first tiles while the previous kernel still runs.
    if (tid == 0)
        for (uint32_t i = 0; i < (uint32_t)kStages && i < n_tiles; ++i) issue(i);

    griddep_wait();   // q (and, fused, this token's k and v) come from the previous kernel
    if (tid == 0) trace_min(a.trace, 1);

    // ---- q as the B operand of the score MMAs: column n = g is head g/2, part g&1 (hi / lo);
    //      for k-step kb this lane holds dims 16kb + {2t, 2t+1} and 16kb + {2t+8, 2t+9}. ----
    uint32_t qb[8][2];
    {
        const uint32_t h = g >> 1, part = g & 1u;
        const float *qg = a.q + ((uint64_t)b * a.n_q_head + (uint64_t)hkv * group + h) * kD;
#pragma unroll
        for (int kb = 0; kb < 8; ++kb)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t d = kb * 16 + 2 * t + 8 * j;
                float2 v = *reinterpret_cast<const float2 *>(qg + d);
                if (fused) {
                    const float2 cs = sm.cs[d >> 1];
                    const float x0 = v.x, x1 = v.y;
                    v.x = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
                    v.y = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
                }
                qb[kb][j] = pack_h2(split_part(v.x * a.scale, part), split_part(v.y * a.scale, part));
            }
    }

    // ---- fused mode: the CTA whose tiles hold the current position appends this token's K / V ----
    const uint32_t pos = kv_len - 1u;
    const bool owner = fused && n_tiles > 0 && pos / kTile >= t0 && pos / kTile < t1;
    if (owner) {
        // thread i < 64: pair i of k (rotated) ; thread 64 + i: elements 2i, 2i+1 of v
        const uint32_t i = tid & 63u;
        const float *src = (tid < 64 ? a.rope_k : a.rope_v) + ((uint64_t)b * a.n_kv_head + hkv) * kD + 2 * i;
        float x0 = src[0], x1 = src[1];
        if (tid < 64) {
            const float2 cs = sm.cs[i];
            const float y0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
            const float y1 = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
            x0 = y0; x1 = y1;
        }
        const uint32_t packed = pack_h2(__float2half_rn(x0), __float2half_rn(x1));
        __half *cache = (tid < 64 ? a.k_append : a.v_append) + ((uint64_t)row0 + pos) * kD + 2 * i;
        *reinterpret_cast<uint32_t *>(cache) = packed;
        sm.wo[0][0][tid] = __uint_as_float(packed);   // staged: patched into the tile once it has landed
    }

    // ---- main loop ----
    float o[8][4];                       // context^T: dim tile dt, {(dim g, hi), (dim g, lo), (dim g+8, hi), (dim g+8, lo)} of head t
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) o[dt][0] = o[dt][1] = o[dt][2] = o[dt][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;   // of head t over this warp's positions (replicated over g)

    for (uint32_t it = 0; it < n_tiles; ++it) {
        const uint32_t slot = it % kStages;
        const uint32_t p0 = (t0 + it) * kTile;
        const uint32_t n = min((uint32_t)kTile, kv_len - p0);   // valid positions of this tile
        const uint32_t st = ring + slot * kStageBytes;
        if (!mbar_wait_bounded(&sm.full[slot], (it / kStages) & 1u, a.status)) return;
        if (owner && pos >= p0 && pos < p0 + kTile) {
            // overwrite the (stale) row of the current position with the values staged above
            __syncthreads();   // staging complete (all warps pass here: `owner` and the tile are CTA-uniform)
            const uint32_t r = pos - p0, i = tid & 63u;
            const uint32_t off = (tid < 64 ? 0u : 2u * kHalfBytes) + (i >= 32 ? kHalfBytes : 0u) + swz(r, (i & 31u) >> 2) + (i & 3u) * 4u;
            *reinterpret_cast<uint32_t *>(&sm.ring[slot][off]) = __float_as_uint(sm.wo[0][0][tid]);
            __syncthreads();
        }
        const uint32_t wrow = warp * 16;       // this warp's rows of the tile
        if (wrow < n) {
            if (n < wrow + 16) {
                // ragged end: rows >= n may hold anything (even NaN): clear them in V so that 0 * V stays 0
                for (uint32_t k = lane; k < 16 * 16; k += 32) {
                    const uint32_t r = wrow + (k >> 4), c = k & 15u;
                    if (r >= n)
                        *reinterpret_cast<uint4 *>(&sm.ring[slot][2 * kHalfBytes + (c >> 3) * kHalfBytes + swz(r, c & 7u)]) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
            // ---- scores: S[16 positions][8 columns] ----
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const uint32_t r = wrow + ((lane >> 3) & 1u) * 8 + (lane & 7u);   // row this lane addresses
#pragma unroll
                for (int kb = 0; kb < 8; ++kb) {
                    uint32_t ka[4];
                    ldsm_x4(st + (kb >> 2) * kHalfBytes + swz(r, 2 * (kb & 3) + (lane >> 4)), ka);
                    mma_f16(sc, ka, qb[kb][0], qb[kb][1]);
                }
            }
            // lane (g, t): head t, positions wrow + g and wrow + g + 8 (hi + lo columns)
            float s0 = sc[0] + sc[1], s1 = sc[2] + sc[3];
            if (wrow + g >= n) s0 = -INFINITY;
            if (wrow + g + 8 >= n) s1 = -INFINITY;
            float mt = fmaxf(s0, s1);
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
            mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
            const float m_new = fmaxf(m_run, mt);   // finite: row wrow < n is valid
            const float p0v = expf(s0 - m_new), p1v = expf(s1 - m_new);
            const float al = expf(m_run - m_new);   // 0 on the first tile (m_run = -inf)
            float ps = p0v + p1v;
            ps += __shfl_xor_sync(0xffffffffu, ps, 4);
            ps += __shfl_xor_sync(0xffffffffu, ps, 8);
            ps += __shfl_xor_sync(0xffffffffu, ps, 16);
            l_run = l_run * al + ps;
            m_run = m_new;
            // ---- probabilities as the B operand: column g = head g/2, part g&1; k = positions 2t, 2t+1, 2t+8, 2t+9 ----
            const uint32_t srcA = (2 * t) * 4 + (g >> 1), srcB = srcA + 4;
            const float a0 = __shfl_sync(0xffffffffu, p0v, srcA), b0 = __shfl_sync(0xffffffffu, p0v, srcB);
            const float a1 = __shfl_sync(0xffffffffu, p1v, srcA), b1 = __shfl_sync(0xffffffffu, p1v, srcB);
            const uint32_t part = g & 1u;
            const uint32_t pb0 = pack_h2(split_part(a0, part), split_part(b0, part));
            const uint32_t pb1 = pack_h2(split_part(a1, part), split_part(b1, part));
            // ---- context: O^T[128 dims][8 columns] = alpha * O^T + V^T P ----
            {
                const uint32_t mi = lane >> 3;
                const uint32_t r = wrow + (mi >> 1) * 8 + (lane & 7u);
#pragma unroll
                for (int dt = 0; dt < 8; ++dt) {
                    uint32_t va[4];
                    ldsm_x4_trans(st + 2 * kHalfBytes + (dt >> 2) * kHalfBytes + swz(r, 2 * (dt & 3) + (mi & 1u)), va);
                    o[dt][0] *= al; o[dt][1] *= al; o[dt][2] *= al; o[dt][3] *= al;
                    mma_f16(o[dt], va, pb0, pb1);
                }
            }
        }
        __syncthreads();   // tile fully consumed by all warps: the slot can be refilled
        if (tid == 0 && it + kStages < n_tiles) issue(it + kStages);
    }

    // ---- merge the 4 warps' (max, sum, context) and write this split's partial ----
    // o[dt][0] + o[dt][1] = context of head t at dim 16dt + g; o[dt][2] + o[dt][3] at dim 16dt + g + 8.
#pragma unroll
    for (int dt = 0; dt < 8; ++dt) {
        sm.wo[warp][t][16 * dt + g] = o[dt][0] + o[dt][1];
        sm.wo[warp][t][16 * dt + g + 8] = o[dt][2] + o[dt][3];
    }
    if (g == 0) { sm.wm[warp][t] = m_run; sm.wl[warp][t] = l_run; }
    __syncthreads();
    {
        const uint32_t h = warp;   // warp h <-> head h of the group, lane <-> 4 dims
        float mw[kAttnWarps], M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) { mw[w] = sm.wm[w][h]; M = fmaxf(M, mw[w]); }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float sc = mw[w] == -INFINITY ? 0.f : expf(mw[w] - M);
            L = fmaf(sm.wl[w][h], sc, L);
            const float4 v = *reinterpret_cast<const float4 *>(&sm.wo[w][h][lane * 4]);
            acc.x = fmaf(v.x, sc, acc.x); acc.y = fmaf(v.y, sc, acc.y);
            acc.z = fmaf(v.z, sc, acc.z); acc.w = fmaf(v.w, sc, acc.w);
        }
        float *part = a.part + (((uint64_t)b * a.n_q_head + (uint64_t)hkv * group + h) * a.n_splits + split) * kPartStride;
        *reinterpret_cast<float4 *>(part + lane * 4) = acc;
        if (lane == 0) { part[kD] = M; part[kD + 1] = L; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        trace_max(a.trace, 2);
        const uint32_t tk = atomicAdd(&a.tickets[b * a.n_kv_head + hkv], 1u);
        sm.is_last = (tk == a.n_splits - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!sm.is_last) return;
    __threadfence();

    // ---- combine (last CTA of this batch / KV head): warp h <-> head h. Every lane derives the
    // global maximum and the rescaled sum from all splits' (m, l), then accumulates the contexts
    // in split order, 4 dims per lane, 16 loads in flight. ----
    {
        const uint32_t h = warp;
        const uint64_t hq = (uint64_t)b * a.n_q_head + (uint64_t)hkv * group + h;
        const float *part = a.part + hq * a.n_splits * kPartStride;
        const uint32_t S = a.n_splits;
        const float m0 = lane < S ? __ldcg(part + (uint64_t)lane * kPartStride + kD) : -INFINITY;
        const float m1 = lane + 32 < S ? __ldcg(part + (uint64_t)(lane + 32) * kPartStride + kD) : -INFINITY;
        const float l0 = lane < S ? __ldcg(part + (uint64_t)lane * kPartStride + kD + 1) : 0.f;
        const float l1 = lane + 32 < S ? __ldcg(part + (uint64_t)(lane + 32) * kPartStride + kD + 1) : 0.f;
        // The contexts of up to kCombineChunk splits are requested before anything waits for the maxima: the tail of a
        // launch is a chain of L2 round trips (ticket, maxima, contexts), and with 16 loads in flight the contexts of
        // 37 splits alone were three of them.
        constexpr int kCombineChunk = 40;
        float4 ov[kCombineChunk];
#pragma unroll
        for (int j = 0; j < kCombineChunk; ++j)
            ov[j] = (uint32_t)j < S ? __ldcg(reinterpret_cast<const float4 *>(part + (uint64_t)j * kPartStride) + lane)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
        const float mx = warp_max(fmaxf(m0, m1));
        const float w0 = m0 == -INFINITY ? 0.f : expf(m0 - mx);
        const float w1 = m1 == -INFINITY ? 0.f : expf(m1 - mx);
        const float L = warp_sum(l0 * w0 + l1 * w1);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < kCombineChunk; ++j) {
            const float w = __shfl_sync(0xffffffffu, j < 32 ? w0 : w1, j & 31);
            acc.x = fmaf(ov[j].x, w, acc.x); acc.y = fmaf(ov[j].y, w, acc.y);
            acc.z = fmaf(ov[j].z, w, acc.z); acc.w = fmaf(ov[j].w, w, acc.w);
        }
        for (uint32_t s = kCombineChunk; s < S; ++s) {   // more splits than one chunk: the rest one by one, in split order
            const float4 o = __ldcg(reinterpret_cast<const float4 *>(part + (uint64_t)s * kPartStride) + lane);
            const float w = __shfl_sync(0xffffffffu, s < 32 ? w0 : w1, s & 31u);
            acc.x = fmaf(o.x, w, acc.x); acc.y = fmaf(o.y, w, acc.y);
            acc.z = fmaf(o.z, w, acc.z); acc.w = fmaf(o.w, w, acc.w);
        }
        const float inv = 1.0f / L;
        acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
        reinterpret_cast<float4 *>(a.out + hq * kD)[lane] = acc;
        if (a.lse_out && lane == 0) a.lse_out[hq] = make_float2(mx, L);
    }
    if (tid == 0) {
        a.tickets[b * a.n_kv_head + hkv] = 0;   // ready for the next launch
        trace_max(a.trace, 3);
    }
}

constexpr size_t kAttnSmemBytes = sizeof(AttnSmem) + 1024;   // + slack to align the ring to the swizzle atom

} // namespace

// K and V as 2-D f16 tensors [rows][128] for the TMA unit: box = 64 rows x 64 columns, 128-byte swizzle.
cudaError_t attn_make_maps(AttnArgs &a) {
    const uint64_t rows = (uint64_t)(a.shared_kv ? 1u : a.batch) * a.n_kv_head * a.kv_stride;
    if (!a.shared_kv && a.batch_stride != (uint64_t)a.n_kv_head * a.kv_stride * kD) return cudaErrorInvalidValue;   // sequences are contiguous
    cudaError_t e = tensor_map_2d(&a.kmap, /*elem_bytes=*/2, a.k, kD, rows, kD * 2, 64, kTile, /*swizzle128=*/true);
    if (e != cudaSuccess) return e;
    return tensor_map_2d(&a.vmap, 2, a.v, kD, rows, kD * 2, 64, kTile, true);
}

cudaError_t attn_init(void) {
    return cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmemBytes);
}

uint32_t attn_pick_splits(uint32_t n_kv_head, uint32_t batch, uint32_t kv_len, int sms) {
    const uint32_t tiles = (kv_len + kTile - 1) / kTile;
    const uint32_t heads = n_kv_head * batch;
    uint32_t s = (2u * (uint32_t)sms + heads - 1) / heads;   // two resident CTAs per SM
    if (s > tiles) s = tiles;
    if (s > 64) s = 64;   // the combine gives each lane two splits
    if (s < 1) s = 1;
    return s;
}

size_t attn_part_floats(uint32_t n_q_head, uint32_t batch, uint32_t n_splits) {
    return (size_t)n_q_head * batch * n_splits * kPartStride;
}

// ---- Split-KV scratch that lives in the module image instead of the heap ----
//
// Some callers may not allocate device memory at call time at all: a serving
// loop that promised its embedder a fixed memory footprint after start-up, or a
// host thread that runs between two points where cudaMalloc's implicit
// device-wide synchronisation would stall other streams. For them the partial
// results of the split-KV kernel (one 132-float record per query head and split)
// and the per-KV-head arrival counters sit in this fixed array. Its size is the
// limit of the variant: kStaticMaxRecords records (4096 x 528 B = 2.1 MB, e.g.
// 64 query heads x 64 splits) and kStaticMaxTickets (KV head, sequence) pairs.
// Every call on a device shares the one array, so two calls that overlap in
// time (different streams or host threads) race on it; calls on one stream are
// ordered and safe.
constexpr size_t kStaticMaxRecords = 4096;
constexpr uint32_t kStaticMaxTickets = 256;
constexpr size_t kStaticPartFloats = kStaticMaxRecords * kPartStride;
static __device__ __align__(256) float g_attn_static_scratch[kStaticPartFloats + kStaticMaxTickets];

constexpr int kMaxDevices = 64;
static float *g_static_ptr[kMaxDevices];   // device address of the array, per device; nullptr = not asked yet

// Launches the split-KV kernel with its scratch in the static array. a.part and
// a.tickets are ignored. The first call on a device resolves the array's device
// address (cudaGetSymbolAddress; that first call may initialise the module, so
// make it before any stream capture). The counters have to be zero when the
// kernel starts: the kernel leaves them at zero, but a launch that gave up on a
// bounded wait may not, so they are cleared on the stream in front of every
// launch (a memset node: no allocation).
cudaError_t launch_attn_decode_static(AttnArgs a, int device, cudaStream_t stream, size_t *records_needed) {
    const size_t records = (size_t)a.n_q_head * a.batch * a.n_splits;
    if (records_needed) *records_needed = records;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    if (a.n_splits == 0 || a.n_splits > 64) return cudaErrorInvalidValue;   // the combine gives each lane two splits
    if (records > kStaticMaxRecords || (uint64_t)a.n_kv_head * a.batch > kStaticMaxTickets)
        return cudaErrorMemoryAllocation;   // the caller turns this into its size message
    // cudaGetSymbolAddress answers for the device that is current on this thread: the address is only
    // cached under `device` when that is the current one.
    int cur = -1;
    cudaError_t e0 = cudaGetDevice(&cur);
    if (e0 != cudaSuccess) return e0;
    if (cur != device) return cudaErrorInvalidDevice;
    float *ptr = __atomic_load_n(&g_static_ptr[device], __ATOMIC_ACQUIRE);
    if (!ptr) {
        const cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_attn_static_scratch);
        if (e != cudaSuccess) return e;
        __atomic_store_n(&g_static_ptr[device], ptr, __ATOMIC_RELEASE);   // every thread stores the same value
    }
    a.part = ptr;
    a.tickets = reinterpret_cast<uint32_t *>(ptr + kStaticPartFloats);
    cudaError_t e = cudaMemsetAsync(a.tickets, 0, (size_t)a.n_kv_head * a.batch * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    e = attn_make_maps(a);   // host-side descriptors only
    if (e != cudaSuccess) return e;
    return launch_attn_decode(a, stream);
}

size_t attn_static_max_records(void) { return kStaticMaxRecords; }
uint32_t attn_static_max_tickets(void) { return kStaticMaxTickets; }

cudaError_t launch_attn_decode(const AttnArgs &a, cudaStream_t stream) {
    if (a.n_kv_head == 0 || a.n_q_head != a.n_kv_head * kGroup || a.n_splits == 0 || a.batch == 0)
        return cudaErrorInvalidValue;
    if (a.pos == nullptr && a.kv_len == 0) return cudaErrorInvalidValue;
    if (a.rope_k && (!a.rope_v || !a.k_append || !a.v_append || !a.pos)) return cudaErrorInvalidValue;
    const dim3 grid(a.n_splits, a.n_kv_head, a.batch);
    return launch_kernel(attn_decode_kernel, grid, dim3(kAttnThreads), kAttnSmemBytes, stream, a.pdl != 0, a);
}

} // namespace flb
