// k-quant dequantize-matvec for single-token decode (replaces the reference's
// warp-per-row gdot_q4_K / gdot_q6_K / gdot_q8_0, src/runtime/kernels_gpu.h:65-205,
// and the STREAM_DOT branch of exec_task_block, src/runtime/gpu_exec.cu:64-140).
//
// Streaming kernel (Q4_K and Q6_K, cols a multiple of 2048)
// ---------------------------------------------------------
// HBM-bound: every packed weight byte is read exactly once. Each warp owns a
// private ring of shared-memory stages that its lane 0 keeps filled with 1-D
// bulk copies (TMA engine, completion on an mbarrier), so the bytes in flight
// per SM do not depend on registers and no warp ever synchronises with another.
//   stage  = the same 8-super-block column segment (2048 weights) of 4
//            consecutive rows (a "row quad"): 4 x 1152 B (Q4_K) or 4 x 1680 B
//            (Q6_K), each a contiguous, 16-byte aligned slice of a packed row;
//   lane   = one quarter of a super-block (64 weights) of each of the 4 rows:
//            block = lane/4, quarter = lane%4. The activation slice a lane
//            needs is the same for all 4 rows, so it is read from shared memory
//            once per stage (float4, conflict-free thanks to a per-format
//            permuted copy of x built once per CTA) and reused 4 times;
//   math   = quants are converted to f32 in registers and multiplied with f32
//            activations (packed f32x2 FMA), accumulated per 32- or 16-element
//            sub-block; the sub-block scale (and, for Q4_K, the min times the
//            precomputed sum of the activations of that sub-block) is applied
//            once per sub-block, the super-block scale d / dmin once per
//            quarter. All accumulation is f32 in a fixed order, so results
//            are reproducible run to run.
// A row's 32-lane partials are reduced with shuffles when its last segment is
// done; lane 0 writes y. Several tensors that share x (Q/K/V, gate/up) run in
// one launch. The activation can be built on the fly from the residual stream
// (RMSNorm) or from gate/up (SiLU * up), which removes those launches.
//
// Generic kernel: any other shape / format (Q8_0, Q5_0, F32, cols not a
// multiple of 2048): warp per row, element-wise, same f32 accumulation.
#include "common.cuh"
#include "kernels.h"

namespace flb {

namespace {

constexpr int kWarps = 12;            // warps per CTA (all are consumers + self-producers)
constexpr int kThreads = kWarps * 32;
constexpr int kRowsPerStage = 4;
constexpr uint32_t kSeg4 = 8 * 144;   // bytes of one Q4_K segment (8 super-blocks)
constexpr uint32_t kSeg6 = 8 * 210;   // bytes of one Q6_K segment
constexpr uint32_t kStage4 = kRowsPerStage * kSeg4;       // ring slot size, Q4_K only
constexpr uint32_t kStage6 = kRowsPerStage * kSeg6;       // ring slot size when Q6_K is present

// ---- u8 -> f32 without the conversion pipe --------------------------------
// Integer-to-float conversion instructions issue at a fraction of the FMA rate,
// so bytes are turned into floats with a byte permute instead: placing byte k
// of w under the constant 0x4B000000 gives the float 2^23 + byte exactly; a
// packed f32x2 add of -2^23 removes the offset for two values at once.
constexpr float kMagic = 8388608.0f;   // 2^23

template <int K>
__device__ __forceinline__ float u8_biased(uint32_t w) {   // 2^23 + byte K of w
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K));
}
template <int K>
__device__ __forceinline__ float u8f(uint32_t w) { return u8_biased<K>(w) - kMagic; }

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }

// acc += (bytes of w as floats) . x4
__device__ __forceinline__ void dot4_u8(uint32_t w, const float4 &x, float2 &acc) {
    const float2 nm = make_float2(-kMagic, -kMagic);
    const float2 q01 = add2(make_float2(u8_biased<0>(w), u8_biased<1>(w)), nm);
    const float2 q23 = add2(make_float2(u8_biased<2>(w), u8_biased<3>(w)), nm);
    acc = fma2(q01, make_float2(x.x, x.y), acc);
    acc = fma2(q23, make_float2(x.z, x.w), acc);
}

// ---- permuted activation layouts -------------------------------------------
// Both layouts store, for segment s and float4 slot f (0..15), the 32 lanes'
// float4 contiguously: index ((s*16 + f)*32 + lane)*4 + i.
// Q4_K: lane = blk*4 + chunk(64); f = (element within chunk)/4: f 0..7 are the
//       low-nibble sub-block, 8..15 the high-nibble sub-block.
// Q6_K: lane = blk*4 + half*2 + hq where the quarter covers, in each of the 4
//       32-element groups g of the half, elements 16*hq .. 16*hq+15;
//       f = g*4 + (element within the 16)/4.
__device__ __forceinline__ uint32_t perm4(uint32_t col) {
    const uint32_t blk = col >> 8, seg = blk >> 3, sbi = blk & 7u;
    const uint32_t c = (col >> 6) & 3u, k = col & 63u;
    return ((seg * 16 + (k >> 2)) * 32 + sbi * 4 + c) * 4 + (k & 3u);
}
__device__ __forceinline__ uint32_t perm6(uint32_t col) {
    const uint32_t blk = col >> 8, seg = blk >> 3, sbi = blk & 7u;
    const uint32_t e = col & 255u;
    const uint32_t hf = e >> 7, g = (e >> 5) & 3u, hq = (e >> 4) & 1u, j = (e >> 2) & 3u;
    return ((seg * 16 + g * 4 + j) * 32 + sbi * 4 + hf * 2 + hq) * 4 + (e & 3u);
}

struct Smem {
    float *x4, *s4;   // Q4_K: permuted x, per-lane sums of its two 32-element sub-blocks
    float *x6, *s6;   // Q6_K: permuted x, per-lane sums of its four 16-element groups
    uint64_t *bars;   // [kWarps][stages]
    uint8_t *ring;    // [kWarps][stages][stage bytes]
};

__device__ __forceinline__ Smem carve(uint8_t *base, uint32_t cols, bool q4, bool q6, int stages) {
    Smem s;
    uint8_t *p = base;
    s.x4 = s.s4 = s.x6 = s.s6 = nullptr;
    if (q4) { s.x4 = (float *)p; p += (size_t)cols * 4; s.s4 = (float *)p; p += (size_t)cols / 32 * 4; }
    if (q6) { s.x6 = (float *)p; p += (size_t)cols * 4; s.s6 = (float *)p; p += (size_t)cols / 16 * 4; }
    s.bars = (uint64_t *)p; p += (size_t)kWarps * stages * 8;
    p = (uint8_t *)(((uintptr_t)p + 127) & ~(uintptr_t)127);
    s.ring = p;
    return s;
}

// ---- per-stage math ----------------------------------------------------------

// Q4_K quarter (64 weights) of one row: returns its contribution to the dot.
__device__ __forceinline__ float q4k_quarter(const uint8_t *blk, uint32_t c, const float4 *xs,
                                             float2 sx) {
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * c);
    const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * c);
    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    float2 pa = make_float2(0.f, 0.f), pb = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t lo = qw[i] & 0x0F0F0F0Fu, hi = qw[i] & 0xF0F0F0F0u;   // hi holds 16 * q
        dot4_u8(lo, xs[i * 32], pa);
        dot4_u8(hi, xs[(8 + i) * 32], pb);
    }
    // 6-bit scales / mins of sub-blocks 2c and 2c+1 (packing: fl_q4k_scale_min,
    // src/runtime/quants.h:121-129), both pairs decoded byte-parallel.
    const uint32_t sh = 16u * (c & 1u);
    const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, e = hdr.w >> sh;
    const uint32_t sc_lo = a & 0x3F3Fu, mn_lo = b & 0x3F3Fu;
    const uint32_t sc_hi = (e & 0x0F0Fu) | ((a >> 2) & 0x3030u);
    const uint32_t mn_hi = ((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
    const uint32_t sc = c >= 2 ? sc_hi : sc_lo, mn = c >= 2 ? mn_hi : mn_lo;
    const float d = h2f_bits((uint16_t)(hdr.x & 0xFFFFu)), dmin = h2f_bits((uint16_t)(hdr.x >> 16));
    const float t = u8f<0>(sc) * (pa.x + pa.y) + u8f<1>(sc) * (0.0625f * (pb.x + pb.y));
    const float m = u8f<0>(mn) * sx.x + u8f<1>(mn) * sx.y;
    return d * t - dmin * m;
}

// Aligned-word fetch from a 2-byte aligned position inside a stage.
__device__ __forceinline__ uint32_t ldw2(const uint32_t *w, uint32_t sel) {
    return __byte_perm(w[0], w[1], sel);
}

// Q6_K quarter (64 weights: 16 elements of each of the 4 groups of one half).
__device__ __forceinline__ float q6k_quarter(const uint8_t *stage_row, uint32_t sbi, uint32_t qt,
                                             const float4 *xs, float4 sx) {
    const uint32_t hf = qt >> 1, hq = qt & 1u;
    const uint32_t ob = sbi * 210u;                  // block offset: 2 mod 4 for odd blocks
    const uint32_t sel = (ob & 2u) ? 0x5432u : 0x3210u;
    const uint32_t *wbase = reinterpret_cast<const uint32_t *>(stage_row + (ob & ~3u));
    const uint32_t *wa = wbase + (64 * hf + 16 * hq) / 4;          // ql: groups 0 (low) / 2 (high)
    const uint32_t *wb = wa + 8;                                   // ql + 32: groups 1 / 3
    const uint32_t *wh = wbase + (128 + 32 * hf + 16 * hq) / 4;    // qh
    float2 p0 = make_float2(0.f, 0.f), p1 = p0, p2 = p0, p3 = p0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a = ldw2(wa + j, sel), b = ldw2(wb + j, sel), h = ldw2(wh + j, sel);
        const uint32_t g0 = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
        const uint32_t g1 = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
        const uint32_t g2 = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
        const uint32_t g3 = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
        dot4_u8(g0, xs[(0 + j) * 32], p0);
        dot4_u8(g1, xs[(4 + j) * 32], p1);
        dot4_u8(g2, xs[(8 + j) * 32], p2);
        dot4_u8(g3, xs[(12 + j) * 32], p3);
    }
    const uint8_t *scp = stage_row + ob + 192 + 8 * hf + hq;
    // int8 scales -> f32 through the same trick: (s ^ 0x80) = s + 128 as an unsigned byte
    const uint32_t sw = ((uint32_t)scp[0] | ((uint32_t)scp[2] << 8) | ((uint32_t)scp[4] << 16) | ((uint32_t)scp[6] << 24)) ^ 0x80808080u;
    const float kOff = kMagic + 128.0f;
    const float d = h2f_bits(*reinterpret_cast<const uint16_t *>(stage_row + ob + 208));
    // value = d * sc * (q - 32): sum q*x minus 32 * sum x per 16-element group
    float t = (u8_biased<0>(sw) - kOff) * ((p0.x + p0.y) - 32.f * sx.x);
    t += (u8_biased<1>(sw) - kOff) * ((p1.x + p1.y) - 32.f * sx.y);
    t += (u8_biased<2>(sw) - kOff) * ((p2.x + p2.y) - 32.f * sx.z);
    t += (u8_biased<3>(sw) - kOff) * ((p3.x + p3.y) - 32.f * sx.w);
    return d * t;
}

// ---- the streaming kernel ---------------------------------------------------

struct QuadRef {
    const uint8_t *row[kRowsPerStage];
    float *y;
    const float *resid;
    uint32_t r0, rows;
    int fmt;
};

__device__ __forceinline__ QuadRef locate_quad(const MatvecArgs &a, uint32_t quad) {
    QuadRef q;
    int ti = 0;
    uint32_t base = 0;
#pragma unroll 1
    for (; ti < a.n_tensors - 1; ++ti) {
        const uint32_t nq = (a.t[ti].rows + kRowsPerStage - 1) / kRowsPerStage;
        if (quad < base + nq) break;
        base += nq;
    }
    const MatvecTensor &t = a.t[ti];
    const uint64_t rb = row_bytes(t.fmt, a.cols);
    q.r0 = (quad - base) * kRowsPerStage;
    q.rows = t.rows;
    q.fmt = t.fmt;
    q.y = t.y;
    q.resid = t.resid;
#pragma unroll
    for (int r = 0; r < kRowsPerStage; ++r) {
        const uint32_t rr = q.r0 + r < t.rows ? q.r0 + r : t.rows - 1;   // clamp: tail rows re-read the last row
        q.row[r] = t.w + (uint64_t)rr * rb;
    }
    return q;
}

__global__ void __launch_bounds__(kThreads, 1)
matvec_stream_kernel(const MatvecArgs a, const uint32_t total_quads, const int stages, const int use_q4,
                     const int use_q6) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.cols, use_q4 != 0, use_q6 != 0, stages);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t nseg = a.cols / 2048u;
    const uint32_t kStageBytes = use_q6 ? kStage6 : kStage4;
    __shared__ float red[kWarps];
    __shared__ float inv_rms;

    uint64_t *bars = sm.bars + warp * stages;
    uint8_t *ring = sm.ring + (size_t)warp * stages * kStageBytes;
    if (lane == 0)
        for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    __syncwarp();

    // This warp's quads: gw, gw + W, ... ; its stage i is (quad i / nseg, segment i % nseg).
    const uint32_t gw = blockIdx.x * kWarps + warp, W = gridDim.x * kWarps;
    const uint32_t my_quads = gw < total_quads ? (total_quads - gw + W - 1) / W : 0;
    const uint32_t my_stages = my_quads * nseg;

    auto issue = [&](uint32_t i) {   // lane 0 only
        const QuadRef q = locate_quad(a, gw + (i / nseg) * W);
        const uint32_t seg = i % nseg, slot = i % stages;
        const uint32_t sb = q.fmt == FMT_Q4_K ? kSeg4 : kSeg6;
        mbar_arrive_expect_tx(&bars[slot], kRowsPerStage * sb);
#pragma unroll
        for (int r = 0; r < kRowsPerStage; ++r)
            bulk_g2s(ring + (size_t)slot * kStageBytes + r * sb, q.row[r] + (size_t)seg * sb, sb, &bars[slot]);
    };
    // Weights do not depend on the activation: start streaming before x is built.
    if (lane == 0)
        for (uint32_t i = 0; i < (uint32_t)stages && i < my_stages; ++i) issue(i);

    // ---- build the activation in shared memory (permuted, per format) ----
    if (a.x_mode == MV_X_RMSNORM) {
        float ss = 0.f;
        for (uint32_t c = tid; c < a.cols; c += kThreads) { const float v = a.x[c]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (tid == 0) {
            float t = 0.f;
            for (int w = 0; w < kWarps; ++w) t += red[w];
            inv_rms = 1.0f / sqrtf(t / (float)a.cols + a.eps);
        }
        __syncthreads();
    }
    for (uint32_t c = tid; c < a.cols; c += kThreads) {
        float v = a.x[c];
        if (a.x_mode == MV_X_RMSNORM) v = v * inv_rms * a.wnorm[c];
        else if (a.x_mode == MV_X_SILU_MUL) v = (v / (1.0f + expf(-v))) * a.x2[c];
        if (use_q4) sm.x4[perm4(c)] = v;
        if (use_q6) sm.x6[perm6(c)] = v;
        if (a.xn_out != nullptr && blockIdx.x == 0) a.xn_out[c] = v;
    }
    __syncthreads();
    if (use_q4) {   // sums of each lane's two 32-element sub-blocks
        for (uint32_t i = tid; i < a.cols / 32; i += kThreads) {
            const uint32_t seg = i >> 6, ln = (i >> 1) & 31u, which = i & 1u;
            const float *p = sm.x4 + ((size_t)(seg * 16 + which * 8) * 32 + ln) * 4;
            float s = 0.f;
            for (int f = 0; f < 8; ++f) { const float4 v = *(const float4 *)(p + f * 128); s += (v.x + v.y) + (v.z + v.w); }
            sm.s4[i] = s;
        }
    }
    if (use_q6) {   // sums of each lane's four 16-element groups
        for (uint32_t i = tid; i < a.cols / 16; i += kThreads) {
            const uint32_t seg = i >> 7, ln = (i >> 2) & 31u, g = i & 3u;
            const float *p = sm.x6 + ((size_t)(seg * 16 + g * 4) * 32 + ln) * 4;
            float s = 0.f;
            for (int f = 0; f < 4; ++f) { const float4 v = *(const float4 *)(p + f * 128); s += (v.x + v.y) + (v.z + v.w); }
            sm.s6[i] = s;
        }
    }
    __syncthreads();

    // ---- consume ----
    float acc[kRowsPerStage] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t sbi = lane >> 2, qt = lane & 3u;
    QuadRef cur;
    for (uint32_t i = 0; i < my_stages; ++i) {
        const uint32_t seg = i % nseg, slot = i % stages;
        if (seg == 0) cur = locate_quad(a, gw + (i / nseg) * W);
        if (!mbar_wait_bounded(&bars[slot], (i / stages) & 1u, a.status)) return;
        const uint8_t *st = ring + (size_t)slot * kStageBytes;
        if (cur.fmt == FMT_Q4_K) {
            const float4 *xs = reinterpret_cast<const float4 *>(sm.x4) + (size_t)seg * 16 * 32 + lane;
            const float2 sx = reinterpret_cast<const float2 *>(sm.s4)[seg * 32 + lane];
#pragma unroll
            for (int r = 0; r < kRowsPerStage; ++r)
                acc[r] += q4k_quarter(st + r * kSeg4 + sbi * 144, qt, xs, sx);
        } else {
            const float4 *xs = reinterpret_cast<const float4 *>(sm.x6) + (size_t)seg * 16 * 32 + lane;
            const float4 sx = reinterpret_cast<const float4 *>(sm.s6)[seg * 32 + lane];
#pragma unroll
            for (int r = 0; r < kRowsPerStage; ++r)
                acc[r] += q6k_quarter(st + r * kSeg6, sbi, qt, xs, sx);
        }
        __syncwarp();
        if (lane == 0 && i + stages < my_stages) {
            fence_proxy_async_smem();
            issue(i + stages);
        }
        if (seg == nseg - 1) {
#pragma unroll
            for (int r = 0; r < kRowsPerStage; ++r) {
                const float v = warp_sum(acc[r]);
                acc[r] = 0.f;
                const uint32_t row = cur.r0 + r;
                if (lane == 0 && row < cur.rows) {
                    float o = v;
                    if (cur.resid) o = cur.resid[row] + v;
                    if (a.accumulate) o = cur.y[row] + o;
                    cur.y[row] = o;
                }
            }
        }
    }
}

// ---- generic kernel: warp per row, element-wise -------------------------------

__device__ __forceinline__ float dequant_elem(int fmt, const uint8_t *row, uint32_t e) {
    switch (fmt) {
    case FMT_F32: return reinterpret_cast<const float *>(row)[e];
    case FMT_Q8_0: {
        const uint8_t *b = row + (size_t)(e >> 5) * 34;
        return h2f_bits(*reinterpret_cast<const uint16_t *>(b)) * (float)(int)(int8_t)b[2 + (e & 31u)];
    }
    case FMT_Q5_0: {
        const uint8_t *b = row + (size_t)(e >> 5) * 22;
        const uint32_t l = e & 31u, j = l & 15u;
        const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
        const uint32_t nib = l < 16 ? (b[6 + j] & 15u) : (uint32_t)(b[6 + j] >> 4);
        const int q = (int)(nib | (((qh >> l) & 1u) << 4)) - 16;
        return h2f_bits(*reinterpret_cast<const uint16_t *>(b)) * (float)q;
    }
    case FMT_Q4_K: {
        const uint8_t *b = row + (size_t)(e >> 8) * 144;
        const uint32_t i = e & 255u, c = i >> 6, hi = (i >> 5) & 1u, l = i & 31u, j = 2 * c + hi;
        const uint8_t *s = b + 4;
        uint32_t sc, mn;
        if (j < 4) { sc = s[j] & 63u; mn = s[j + 4] & 63u; }
        else { sc = (s[j + 4] & 15u) | ((uint32_t)(s[j - 4] >> 6) << 4); mn = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4); }
        const uint32_t q = hi ? (uint32_t)(b[16 + 32 * c + l] >> 4) : (b[16 + 32 * c + l] & 15u);
        return h2f_bits(*reinterpret_cast<const uint16_t *>(b)) * (float)sc * (float)q -
               h2f_bits(*reinterpret_cast<const uint16_t *>(b + 2)) * (float)mn;
    }
    default: {
        const uint8_t *b = row + (size_t)(e >> 8) * 210;
        const uint32_t i = e & 255u, hf = i >> 7, g = (i >> 5) & 3u, l = i & 31u;
        const uint32_t lo = b[64 * hf + 32 * (g & 1u) + l];
        const uint32_t q4 = g < 2 ? (lo & 15u) : (lo >> 4);
        const int q = (int)(q4 | (((b[128 + 32 * hf + l] >> (2 * g)) & 3u) << 4)) - 32;
        return h2f_bits(*reinterpret_cast<const uint16_t *>(b + 208)) * (float)(int)(int8_t)b[192 + 8 * hf + 2 * g + (l >> 4)] * (float)q;
    }
    }
}

__global__ void __launch_bounds__(256) matvec_generic_kernel(const MatvecArgs a, const uint32_t total_rows) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, W = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t vr = gw; vr < total_rows; vr += W) {
        int ti = 0;
        uint32_t base = 0;
        for (; ti < a.n_tensors - 1; ++ti) {
            if (vr < base + a.t[ti].rows) break;
            base += a.t[ti].rows;
        }
        const MatvecTensor &t = a.t[ti];
        const uint32_t r = vr - base;
        const uint8_t *row = t.w + (uint64_t)r * row_bytes(t.fmt, a.cols);
        float acc = 0.f;
        for (uint32_t e = lane; e < a.cols; e += 32) acc += dequant_elem(t.fmt, row, e) * a.x[e];
        acc = warp_sum(acc);
        if (lane == 0) {
            float o = acc;
            if (t.resid) o = t.resid[r] + acc;
            if (a.accumulate) o = t.y[r] + o;
            t.y[r] = o;
        }
    }
}

} // namespace

bool matvec_is_streaming(int fmt, uint32_t cols) {
    return (fmt == FMT_Q4_K || fmt == FMT_Q6_K) && cols >= 2048 && cols % 2048 == 0;
}

size_t matvec_smem_bytes(uint32_t cols, bool q4, bool q6, int *stages_out) {
    size_t fixed = 0;
    if (q4) fixed += (size_t)cols * 4 + (size_t)cols / 32 * 4;
    if (q6) fixed += (size_t)cols * 4 + (size_t)cols / 16 * 4;
    fixed += 128;   // ring alignment slack
    const size_t limit = 227 * 1024 - 1024;   // leave room for static shared memory
    int stages = 4;
    const size_t slot = q6 ? kStage6 : kStage4;
    while (stages > 1 && fixed + (size_t)kWarps * stages * (8 + slot) > limit) --stages;
    if (stages_out) *stages_out = stages;
    return fixed + (size_t)kWarps * stages * (8 + slot);
}

cudaError_t matvec_init(void) {
    return cudaFuncSetAttribute(matvec_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
}

cudaError_t launch_matvec(const MatvecArgs &a, int sms, cudaStream_t stream) {
    if (a.n_tensors < 1 || a.n_tensors > 4 || a.cols == 0) return cudaErrorInvalidValue;
    bool streaming = true, q4 = false, q6 = false;
    uint32_t total_rows = 0, total_quads = 0;
    for (int i = 0; i < a.n_tensors; ++i) {
        const MatvecTensor &t = a.t[i];
        if (t.rows == 0 || a.cols % blk_elems(t.fmt) != 0) return cudaErrorInvalidValue;
        if (t.fmt < FMT_F32 || t.fmt > FMT_Q6_K) return cudaErrorInvalidValue;
        streaming = streaming && matvec_is_streaming(t.fmt, a.cols) && (((uintptr_t)t.w) & 15u) == 0;
        q4 = q4 || t.fmt == FMT_Q4_K;
        q6 = q6 || t.fmt == FMT_Q6_K;
        total_rows += t.rows;
        total_quads += (t.rows + kRowsPerStage - 1) / kRowsPerStage;
    }
    if (streaming) {
        int stages = 0;
        const size_t smem = matvec_smem_bytes(a.cols, q4, q6, &stages);
        if (smem <= 227 * 1024 - 1024 && stages >= 2) {
            uint32_t grid = (total_quads + kWarps - 1) / kWarps;
            if (grid > (uint32_t)sms) grid = (uint32_t)sms;
            matvec_stream_kernel<<<grid, kThreads, smem, stream>>>(a, total_quads, stages, q4 ? 1 : 0, q6 ? 1 : 0);
            return cudaGetLastError();
        }
    }
    if (a.x_mode != MV_X_PLAIN) return cudaErrorInvalidValue;   // prologues exist only in the streaming kernel
    uint32_t grid = (total_rows + 7) / 8;
    if (grid > (uint32_t)sms * 8) grid = (uint32_t)sms * 8;
    matvec_generic_kernel<<<grid, 256, 0, stream>>>(a, total_rows);
    return cudaGetLastError();
}

} // namespace flb
