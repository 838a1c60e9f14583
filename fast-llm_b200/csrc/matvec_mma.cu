// Q4_K dequantize-matvec on the integer tensor-core path (mma.sync m16n8k32,
// u8 x s8 -> s32) for Q4_K-only launches (O, gate|up). EXPERIMENTAL and off by
// default (FLB_MMA=1 turns it on): correct, but not faster than the scalar
// kernel at one activation column; see matvec_mma_eligible().
// Same contract as the streaming kernel in matvec.cu (STREAM_DOT of the
// reference, src/runtime/runtime_internal.h:240-257, over blk_q4_K rows,
// src/runtime/quants.h:25, :121-129): packed weights cross HBM once through
// per-warp TMA rings, the activation is the same 21-bit fixed point
// (x = s * (a0*2^14 + a1*2^7 + a2) per 256-column block, balanced base-128
// digits), all integer sums are exact.
//
// What changes is who multiplies. A stage is 16 rows x 1 super-block. For one
// 32-weight sub-block the MMA's A operand is the 16 x 32 tile of 4-bit quants
// (masked out of the packed words, no further unpacking) and its B operand
// holds the three digit planes of the 32 activation columns in columns 0, 2, 4
// of the 8 (so that lane t of a quad ends up with plane t of its two rows): one
// instruction replaces the 3 x 8 x 16 dp4a of the scalar loop. The per-sub-block
// 6-bit scale, the min term and d / dmin stay in f32 as in the reference's
// formula  w = d * sc * q - dmin * m; integers become floats by adding a magic
// constant (no conversion instructions: they run at a quarter of the rate).
//
// Work split: a unit is 16 rows (gate|up: 8 gate rows + the 8 matching up rows)
// over all columns and belongs to one CTA; warp w takes super-blocks w, w + 16,
// ... of it. The 16 warps add their partial row sums through shared memory in a
// fixed order and warp 0 runs the epilogue (residual add or SwiGLU), so results
// are reproducible and nothing waits across CTAs. Units are dealt to the CTAs
// round robin; the per-warp TMA rings run ahead across unit boundaries.
#include "common.cuh"
#include "kernels.h"

#include <cuda.h>
#include <cstdlib>
#include <cstring>

namespace flb {

namespace {

constexpr int kWarps = 16;                         // = column pieces per unit
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kStageBytes = 16 * 144;         // 16 rows x one super-block (256 columns)
constexpr int kStages = 4;
constexpr uint32_t kPlanePad = 16;                 // keeps the three planes on different banks
constexpr float kFixMax = 1040000.0f;              // 63*2^14 + 63*2^7 + 63 = 1040447

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// D(16x8, s32) = A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// D += A * B
__device__ __forceinline__ void mma_u8s8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// byte K of w as a float (no integer->float conversion instruction): 2^23 + byte under 0x4B000000
template <int K>
__device__ __forceinline__ float u8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K)) - 8388608.0f;
}
__device__ __forceinline__ float u8f_dyn(uint32_t w, uint32_t k) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | k)) - 8388608.0f;
}
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// small integer (|v| < 2^22) as a float without a conversion instruction
__device__ __forceinline__ float i2f_small(int v) {
    return __int_as_float(0x4B400000 + v) - 12582912.0f;
}

struct Maps { CUtensorMap m[2]; };

struct Smem {
    int8_t *planes;   // [3][cols + kPlanePad]
    float *sx;        // [cols / 32]: sum of the fixed-point activation over each 32-column sub-block
    float *xs;        // [cols / 256]: activation scale of each block
    float *part;      // [kWarps][16]: partial row sums of a piece
    uint64_t *bars;   // [kWarps][kStages]
    uint8_t *ring;    // [kWarps][kStages][kStageBytes]
};
__host__ __device__ inline size_t fixed_bytes(uint32_t cols) {
    return (size_t)3 * (cols + kPlanePad) + (size_t)cols / 32 * 4 + (size_t)cols / 256 * 4 + kWarps * 16 * 4 + kWarps * kStages * 8;
}
__device__ __forceinline__ Smem carve(uint8_t *p, uint32_t cols) {
    Smem s;
    s.planes = (int8_t *)p; p += (size_t)3 * (cols + kPlanePad);   // cols and the pad are multiples of 16
    s.sx = (float *)p; p += (size_t)cols / 32 * 4;
    s.xs = (float *)p; p += (size_t)cols / 256 * 4;
    s.part = (float *)p; p += kWarps * 16 * 4;
    p = (uint8_t *)(((uintptr_t)p + 7) & ~(uintptr_t)7);
    s.bars = (uint64_t *)p; p += kWarps * kStages * 8;
    p = (uint8_t *)(((uintptr_t)p + 127) & ~(uintptr_t)127);
    s.ring = p;
    return s;
}

__global__ void __launch_bounds__(kThreads, 1)
matvec_q4k_mma_kernel(const MatvecArgs a, const __grid_constant__ Maps maps, const uint32_t n_units) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const Smem sm = carve(smem_raw, a.cols);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t nblk = a.cols / 256;
    const uint32_t spu = nblk / kWarps;   // stages (super-blocks) of a unit per warp; checked on the host: nblk % kWarps == 0
    __shared__ float red[kWarps];

    uint64_t *bars = sm.bars + warp * kStages;
    const uint32_t ring = smem_u32(sm.ring) + warp * kStages * kStageBytes;
    if (lane == 0)
        for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    __syncwarp();

    // Units of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
    const uint32_t my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t my_stages = my_units * spu;

    // Producer (lane 0): stage i of this warp = unit blockIdx.x + (i / spu) * gridDim.x, super-block warp + (i % spu) * kWarps.
    uint32_t p_i = 0, p_slot = 0, p_unit = blockIdx.x, p_s = 0;
    auto issue = [&]() {
        const uint32_t dst = ring + p_slot * kStageBytes;
        const uint32_t blk = warp + p_s * kWarps;
        mbar_arrive_expect_tx(&bars[p_slot], kStageBytes);
        if (a.swiglu) {   // rows 0..7 of the tile: gate rows 8u .. 8u+7; rows 8..15: the same rows of up
            tma_load_box(dst, &maps.m[0], blk * 18, p_unit * 8, &bars[p_slot]);
            tma_load_box(dst + 8 * 144, &maps.m[1], blk * 18, p_unit * 8, &bars[p_slot]);
        } else {
            tma_load_box(dst, &maps.m[0], blk * 18, p_unit * 16, &bars[p_slot]);
        }
        ++p_i;
        if (++p_slot == (uint32_t)kStages) p_slot = 0;
        if (++p_s == spu) { p_s = 0; p_unit += gridDim.x; }
    };
    if (tid == 0) trace_min(a.trace, 0);
    griddep_launch_dependents();
    if (lane == 0)
        while (p_i < (uint32_t)kStages && p_i < my_stages) issue();

    // ---- the fixed-point activation: one warp per 256-column block, lane l <-> columns 8l .. 8l+7 ----
    constexpr int kMaxBlk = 2;   // cols <= 2 * 256 * kWarps = 8192
    float4 ra[kMaxBlk][2], rw[kMaxBlk][2];
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b) ra[b][0] = ra[b][1] = rw[b][0] = rw[b][1] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.x_mode == MV_X_RMSNORM) {
#pragma unroll
        for (int b = 0; b < kMaxBlk; ++b) {
            const uint32_t blk = warp + b * kWarps;
            if (blk < nblk) {
                rw[b][0] = __ldg(reinterpret_cast<const float4 *>(a.wnorm + blk * 256 + lane * 8));
                rw[b][1] = __ldg(reinterpret_cast<const float4 *>(a.wnorm + blk * 256 + lane * 8 + 4));
            }
        }
    }
    griddep_wait();   // the activation (and resid) come from the previous kernel
    if (tid == 0) trace_min(a.trace, 1);
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b) {
        const uint32_t blk = warp + b * kWarps;
        if (blk < nblk) {
            ra[b][0] = *reinterpret_cast<const float4 *>(a.x + blk * 256 + lane * 8);
            ra[b][1] = *reinterpret_cast<const float4 *>(a.x + blk * 256 + lane * 8 + 4);
        }
    }
    float ss = 0.f;
    if (a.x_mode == MV_X_RMSNORM) {
#pragma unroll
        for (int b = 0; b < kMaxBlk; ++b) {
            const float4 u0 = ra[b][0], u1 = ra[b][1];
            ss += (u0.x * u0.x + u0.y * u0.y) + (u0.z * u0.z + u0.w * u0.w);
            ss += (u1.x * u1.x + u1.y * u1.y) + (u1.z * u1.z + u1.w * u1.w);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
    }
    const uint32_t pstride = a.cols + kPlanePad;
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b) {
        const uint32_t blk = warp + b * kWarps;
        if (blk >= nblk) break;
        float v[8] = {ra[b][0].x, ra[b][0].y, ra[b][0].z, ra[b][0].w, ra[b][1].x, ra[b][1].y, ra[b][1].z, ra[b][1].w};
        const float w2[8] = {rw[b][0].x, rw[b][0].y, rw[b][0].z, rw[b][0].w, rw[b][1].x, rw[b][1].y, rw[b][1].z, rw[b][1].w};
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (a.x_mode == MV_X_RMSNORM) v[i] = v[i] * w2[i];   // the common factor 1/rms is applied to the row sums
            amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = warp_max(amax);
        const float s = amax > 0.f ? amax / kFixMax : 1.0f;
        const float inv_s = 1.0f / s;
        int sum = 0;
        uint32_t pk[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int X = __float2int_rn(v[i] * inv_s);
            const int d2 = ((X + 64) & 127) - 64;
            const int X1 = (X - d2) >> 7;
            const int d1 = ((X1 + 64) & 127) - 64;
            const int d0 = (X1 - d1) >> 7;
            sum += X;
            pk[0][i >> 2] |= (uint32_t)(d0 & 0xFF) << (8 * (i & 3));
            pk[1][i >> 2] |= (uint32_t)(d1 & 0xFF) << (8 * (i & 3));
            pk[2][i >> 2] |= (uint32_t)(d2 & 0xFF) << (8 * (i & 3));
        }
        const uint32_t c0 = blk * 256 + lane * 8;
#pragma unroll
        for (int d = 0; d < 3; ++d) *reinterpret_cast<uint2 *>(sm.planes + d * pstride + c0) = make_uint2(pk[d][0], pk[d][1]);
        int s32 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
        s32 += __shfl_xor_sync(0xffffffffu, s32, 2);
        if ((lane & 3u) == 0) sm.sx[blk * 8 + (lane >> 2)] = (float)s32;
        if (lane == 0) sm.xs[blk] = s;
    }
    __syncthreads();
    float inv_rms = 1.f;
    if (a.x_mode == MV_X_RMSNORM) {
        float tt = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tt += red[w];
        inv_rms = 1.0f / sqrtf(tt / (float)a.cols + a.eps);
    }
    if (tid == 0) trace_max(a.trace, 2);

    // ---- consume ----
    // B operand: column n = g of the MMA; planes 0, 1, 2 sit in columns 0, 2, 4, the other columns are zero.
    const bool feeds = (g & 1u) == 0 && g < 6;
    const uint32_t planes_addr = smem_u32(sm.planes) + (feeds ? (g >> 1) : 0u) * pstride;
    // lane t owns columns (2t, 2t+1) of the accumulator tile = (plane t, zero): weight of its plane
    const float pw = t == 0 ? 16384.f : t == 1 ? 128.f : t == 2 ? 1.f : 0.f;
    const float pwm = -8388608.0f * pw;   // scale byte -> float times pw in one fma
    float acc_g = 0.f, acc_h = 0.f;   // rows g and g + 8 of the tile, this lane's share
    uint32_t slot = 0, parity = 0, unit = blockIdx.x, s_in = 0;
    bool dead = false;
    for (uint32_t i = 0; i < my_stages; ++i) {
        const uint32_t st = ring + slot * kStageBytes;
        const uint32_t blk = warp + s_in * kWarps;
        // B operands of the 8 sub-blocks: bytes 4t..4t+3 and 16+4t.. of each sub-block's plane slice
        uint32_t bq[8][2];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t adr = planes_addr + (blk * 256 + j * 32) + 4 * t;
            const uint32_t v0 = lds32(adr), v1 = lds32(adr + 16);
            bq[j][0] = feeds ? v0 : 0u;
            bq[j][1] = feeds ? v1 : 0u;
        }
        const float sx0 = sm.sx[blk * 8 + t], sx1 = sm.sx[blk * 8 + 4 + t];
        const float xs = sm.xs[blk];
        // A wait that gives up has set the status word; the warp then skips the arithmetic but keeps its
        // place in the block barriers below (a warp that left would block the CTA for ever).
        if (!dead && !mbar_wait_bounded(&bars[slot], parity, a.status)) dead = true;
        if (!dead) {
            const uint32_t rg = st + g * 144, rh = st + (g + 8) * 144;
            const uint4 hg = lds128(rg), hh = lds128(rh);
            // 6-bit scales / mins of the 8 sub-blocks, 4 to a word (fl_q4k_scale_min, src/runtime/quants.h:121-129)
            const uint32_t scg_lo = hg.y & 0x3F3F3F3Fu, mng_lo = hg.z & 0x3F3F3F3Fu;
            const uint32_t scg_hi = (hg.w & 0x0F0F0F0Fu) | ((hg.y >> 2) & 0x30303030u);
            const uint32_t mng_hi = ((hg.w >> 4) & 0x0F0F0F0Fu) | ((hg.z >> 2) & 0x30303030u);
            const uint32_t sch_lo = hh.y & 0x3F3F3F3Fu, mnh_lo = hh.z & 0x3F3F3F3Fu;
            const uint32_t sch_hi = (hh.w & 0x0F0F0F0Fu) | ((hh.y >> 2) & 0x30303030u);
            const uint32_t mnh_hi = ((hh.w >> 4) & 0x0F0F0F0Fu) | ((hh.z >> 2) & 0x30303030u);
            float pg = 0.f, ph = 0.f;   // sum_j sc_j * (q . X) of this block, this lane's plane, times its weight
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t wg0 = lds32(rg + 16 + 32 * c + 4 * t), wg1 = lds32(rg + 32 + 32 * c + 4 * t);
                const uint32_t wh0 = lds32(rh + 16 + 32 * c + 4 * t), wh1 = lds32(rh + 32 + 32 * c + 4 * t);
                int lo[4], hi[4];
                mma_u8s8(lo, wg0 & 0x0F0F0F0Fu, wh0 & 0x0F0F0F0Fu, wg1 & 0x0F0F0F0Fu, wh1 & 0x0F0F0F0Fu,
                         bq[2 * c][0], bq[2 * c][1]);
                mma_u8s8(hi, (wg0 >> 4) & 0x0F0F0F0Fu, (wh0 >> 4) & 0x0F0F0F0Fu, (wg1 >> 4) & 0x0F0F0F0Fu, (wh1 >> 4) & 0x0F0F0F0Fu,
                         bq[2 * c + 1][0], bq[2 * c + 1][1]);
                // sub-blocks 2c (low nibbles) and 2c + 1 (high nibbles): bytes (2c & 3), (2c & 3) + 1 of the lo / hi scale word;
                // (2^23 + byte) * pw - 2^23 * pw = byte * pw
                const uint32_t wsg = c < 2 ? scg_lo : scg_hi, wsh = c < 2 ? sch_lo : sch_hi;
                const uint32_t sel0 = 0x7650u | (c & 1 ? 2u : 0u), sel1 = 0x7650u | (c & 1 ? 3u : 1u);
                const float s0g = fmaf(__uint_as_float(__byte_perm(wsg, 0x4B000000u, sel0)), pw, pwm);
                const float s1g = fmaf(__uint_as_float(__byte_perm(wsg, 0x4B000000u, sel1)), pw, pwm);
                const float s0h = fmaf(__uint_as_float(__byte_perm(wsh, 0x4B000000u, sel0)), pw, pwm);
                const float s1h = fmaf(__uint_as_float(__byte_perm(wsh, 0x4B000000u, sel1)), pw, pwm);
                pg = fmaf(s0g, i2f_small(lo[0]), pg);   // |q . digit plane| <= 15 * 64 * 32
                ph = fmaf(s0h, i2f_small(lo[2]), ph);
                pg = fmaf(s1g, i2f_small(hi[0]), pg);
                ph = fmaf(s1h, i2f_small(hi[2]), ph);
            }
            // min term: sum_j m_j * sum(X over sub-block j); lane t takes sub-blocks t and t + 4
            const float mg = u8f_dyn(mng_lo, t) * sx0 + u8f_dyn(mng_hi, t) * sx1;
            const float mh = u8f_dyn(mnh_lo, t) * sx0 + u8f_dyn(mnh_hi, t) * sx1;
            const float dg = h2f_bits((uint16_t)(hg.x & 0xFFFFu)), dming = h2f_bits((uint16_t)(hg.x >> 16));
            const float dh = h2f_bits((uint16_t)(hh.x & 0xFFFFu)), dminh = h2f_bits((uint16_t)(hh.x >> 16));
            acc_g = fmaf(xs, dg * pg - dming * mg, acc_g);
            acc_h = fmaf(xs, dh * ph - dminh * mh, acc_h);
        }
        __syncwarp();
        if (lane == 0 && p_i < my_stages && !dead) issue();   // the slot was only read (generic proxy loads): no proxy fence needed
        if (++slot == (uint32_t)kStages) { slot = 0; parity ^= 1u; }
        if (++s_in == spu) {
            s_in = 0;
            // ---- this warp's part of the unit is done: add the 4 lanes of a row, then the 16 warps ----
            acc_g += __shfl_xor_sync(0xffffffffu, acc_g, 1); acc_h += __shfl_xor_sync(0xffffffffu, acc_h, 1);
            acc_g += __shfl_xor_sync(0xffffffffu, acc_g, 2); acc_h += __shfl_xor_sync(0xffffffffu, acc_h, 2);
            if (t == 0) { sm.part[warp * 16 + g] = acc_g; sm.part[warp * 16 + g + 8] = acc_h; }
            acc_g = acc_h = 0.f;
            __syncthreads();
            if (warp == 0 && lane < 16) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < kWarps; ++w) v += sm.part[w * 16 + lane];   // fixed order over the warps
                v *= inv_rms;
                if (a.swiglu) {
                    // rows 0..7 = gate rows, 8..15 = the same rows of up: h = silu(gate) * up (fl_op_silu_mul,
                    // src/runtime/decode_params.h:267-272)
                    const float up = __shfl_down_sync(0x0000ffffu, v, 8);
                    const uint32_t row = unit * 8 + lane;
                    if (lane < 8 && row < a.t[0].rows) a.t[0].y[row] = (v / (1.0f + expf(-v))) * up;
                } else {
                    const uint32_t row = unit * 16 + lane;
                    if (row < a.t[0].rows) {
                        float o = v;
                        if (a.t[0].resid) o = a.t[0].resid[row] + v;
                        if (a.accumulate) o = a.t[0].y[row] + o;
                        a.t[0].y[row] = o;
                    }
                }
            }
            __syncthreads();   // sm.part is reused by the next unit
            unit += gridDim.x;
        }
    }
    if (lane == 0) trace_max(a.trace, 3);
}


// ---- several activation columns at once (draft verification: Task::nx > 1) ---------------------
//
// y[p][r] (+)= dot(W[r], x[p]) for p < nt <= 8 columns in ONE pass over the weights
// (include/fastllm/fastllm.h:87-96: "the weight row is read ONCE for all nx columns"). Same stage
// geometry as above. What makes several columns cheap is that the per-sub-block scale moves into the
// A operand: sc = 8 sh + sl with sh, sl in 0..7, and q * sh, q * sl (<= 105) are still bytes, one
// integer multiply on the packed word. The MMAs then accumulate over the 8 sub-blocks of a super-block,
// and the scalar epilogue runs once per super-block instead of once per sub-block. The min term goes the
// same way (A = the 6-bit min broadcast to the 32 weights). B holds two columns per MMA: columns
// n = 3 * (p & 1) + plane of the 8, for the column pair p / 2. Per super-block, lane t of a quad then
// owns accumulator columns 2t, 2t + 1 of each pair and applies d, dmin, the plane weight and the
// column's activation scale in f32.
constexpr int kNxMaxCols = 8;
constexpr int kNxStages = 3;

struct NxArgs {
    const uint8_t *w;      // packed Q4_K rows
    const float *x;        // nt activation columns, xstride floats apart
    float *y;              // nt output columns, ystride floats apart
    uint32_t rows, cols, nt, xstride, ystride;
    int accumulate;
    uint32_t *status;
};

struct NxSmem {
    int8_t *planes;   // [nt_pad][3][cols + kPlanePad], nt_pad = nt rounded up to even (a zero column pads)
    float *xs;        // [nt_pad][cols / 256]
    float *part;      // [kWarps][16 rows][kNxMaxCols]
    uint64_t *bars;
    uint8_t *ring;
};
__host__ __device__ inline size_t nx_fixed_bytes(uint32_t cols, uint32_t nt_pad) {
    return (size_t)nt_pad * 3 * (cols + kPlanePad) + (size_t)nt_pad * (cols / 256) * 4 + (size_t)kWarps * 16 * kNxMaxCols * 4 +
           (size_t)kWarps * kNxStages * 8;
}

__global__ void __launch_bounds__(kThreads, 1)
matvec_q4k_mma_nx_kernel(const NxArgs a, const __grid_constant__ CUtensorMap map, const uint32_t n_units) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t nblk = a.cols / 256, spu = nblk / kWarps;
    const uint32_t nt_pad = (a.nt + 1u) & ~1u, npair = nt_pad / 2;
    const uint32_t pstride = a.cols + kPlanePad;
    NxSmem sm;
    {
        uint8_t *p = smem_raw;
        sm.planes = (int8_t *)p; p += (size_t)nt_pad * 3 * pstride;
        sm.xs = (float *)p; p += (size_t)nt_pad * nblk * 4;
        sm.part = (float *)p; p += (size_t)kWarps * 16 * kNxMaxCols * 4;
        p = (uint8_t *)(((uintptr_t)p + 7) & ~(uintptr_t)7);
        sm.bars = (uint64_t *)p; p += (size_t)kWarps * kNxStages * 8;
        p = (uint8_t *)(((uintptr_t)p + 127) & ~(uintptr_t)127);
        sm.ring = p;
    }
    uint64_t *bars = sm.bars + warp * kNxStages;
    const uint32_t ring = smem_u32(sm.ring) + warp * kNxStages * kStageBytes;
    if (lane == 0)
        for (int s = 0; s < kNxStages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    __syncwarp();

    const uint32_t my_units = blockIdx.x < n_units ? (n_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t my_stages = my_units * spu;
    uint32_t p_i = 0, p_slot = 0, p_unit = blockIdx.x, p_s = 0;
    auto issue = [&]() {
        mbar_arrive_expect_tx(&bars[p_slot], kStageBytes);
        tma_load_box(ring + p_slot * kStageBytes, &map, (warp + p_s * kWarps) * 18, p_unit * 16, &bars[p_slot]);
        ++p_i;
        if (++p_slot == (uint32_t)kNxStages) p_slot = 0;
        if (++p_s == spu) { p_s = 0; p_unit += gridDim.x; }
    };
    if (lane == 0)
        while (p_i < (uint32_t)kNxStages && p_i < my_stages) issue();

    // ---- fixed-point planes of every column: warp w takes blocks w, w + 16, ... of each column in turn ----
    for (uint32_t p = 0; p < nt_pad; ++p) {
        for (uint32_t blk = warp; blk < nblk; blk += kWarps) {
            float v[8];
            if (p < a.nt) {
                const float4 u0 = *reinterpret_cast<const float4 *>(a.x + (size_t)p * a.xstride + blk * 256 + lane * 8);
                const float4 u1 = *reinterpret_cast<const float4 *>(a.x + (size_t)p * a.xstride + blk * 256 + lane * 8 + 4);
                v[0] = u0.x; v[1] = u0.y; v[2] = u0.z; v[3] = u0.w; v[4] = u1.x; v[5] = u1.y; v[6] = u1.z; v[7] = u1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f;
            }
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            amax = warp_max(amax);
            const float s = amax > 0.f ? amax / kFixMax : 1.0f;
            const float inv_s = 1.0f / s;
            uint32_t pk[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int X = __float2int_rn(v[i] * inv_s);
                const int d2 = ((X + 64) & 127) - 64;
                const int X1 = (X - d2) >> 7;
                const int d1 = ((X1 + 64) & 127) - 64;
                const int d0 = (X1 - d1) >> 7;
                pk[0][i >> 2] |= (uint32_t)(d0 & 0xFF) << (8 * (i & 3));
                pk[1][i >> 2] |= (uint32_t)(d1 & 0xFF) << (8 * (i & 3));
                pk[2][i >> 2] |= (uint32_t)(d2 & 0xFF) << (8 * (i & 3));
            }
#pragma unroll
            for (int d = 0; d < 3; ++d)
                *reinterpret_cast<uint2 *>(sm.planes + ((size_t)p * 3 + d) * pstride + blk * 256 + lane * 8) = make_uint2(pk[d][0], pk[d][1]);
            if (lane == 0) sm.xs[p * nblk + blk] = s;
        }
    }
    __syncthreads();

    // B operand: MMA column n = g holds column 2 * pair + n / 3 of the activation, plane n % 3 (n < 6).
    const bool feeds = g < 6;
    const uint32_t bcol = g < 3 ? 0u : 1u, bplane = g < 3 ? g : g - 3u;
    // accumulator columns of this lane: n = 2t and 2t + 1
    const uint32_t n0 = 2 * t, n1 = 2 * t + 1;
    const float pwt[3] = {16384.f, 128.f, 1.f};
    const float pw0 = n0 < 6 ? pwt[n0 % 3] : 0.f, pw1 = n1 < 6 ? pwt[n1 % 3] : 0.f;
    const uint32_t c0 = n0 < 6 ? n0 / 3 : 0u, c1 = n1 < 6 ? n1 / 3 : 0u;   // which column of the pair

    float acc[kNxMaxCols / 2][2][2];   // [pair][row g / g + 8][accumulator column]
#pragma unroll
    for (int q = 0; q < kNxMaxCols / 2; ++q) acc[q][0][0] = acc[q][0][1] = acc[q][1][0] = acc[q][1][1] = 0.f;
    uint32_t slot = 0, parity = 0, unit = blockIdx.x, s_in = 0;
    bool dead = false;
    for (uint32_t i = 0; i < my_stages; ++i) {
        const uint32_t st = ring + slot * kStageBytes;
        const uint32_t blk = warp + s_in * kWarps;
        if (!dead && !mbar_wait_bounded(&bars[slot], parity, a.status)) dead = true;
        if (!dead) {
            const uint32_t rg = st + g * 144, rh = st + (g + 8) * 144;
            const uint4 hg = lds128(rg), hh = lds128(rh);
            const uint32_t scg_lo = hg.y & 0x3F3F3F3Fu, mng_lo = hg.z & 0x3F3F3F3Fu;
            const uint32_t scg_hi = (hg.w & 0x0F0F0F0Fu) | ((hg.y >> 2) & 0x30303030u);
            const uint32_t mng_hi = ((hg.w >> 4) & 0x0F0F0F0Fu) | ((hg.z >> 2) & 0x30303030u);
            const uint32_t sch_lo = hh.y & 0x3F3F3F3Fu, mnh_lo = hh.z & 0x3F3F3F3Fu;
            const uint32_t sch_hi = (hh.w & 0x0F0F0F0Fu) | ((hh.y >> 2) & 0x30303030u);
            const uint32_t mnh_hi = ((hh.w >> 4) & 0x0F0F0F0Fu) | ((hh.z >> 2) & 0x30303030u);
            int chi[kNxMaxCols / 2][4], clo[kNxMaxCols / 2][4], cmn[kNxMaxCols / 2][4];
#pragma unroll
            for (int q = 0; q < kNxMaxCols / 2; ++q)
#pragma unroll
                for (int e = 0; e < 4; ++e) chi[q][e] = clo[q][e] = cmn[q][e] = 0;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t wg0 = lds32(rg + 16 + 32 * c + 4 * t), wg1 = lds32(rg + 32 + 32 * c + 4 * t);
                const uint32_t wh0 = lds32(rh + 16 + 32 * c + 4 * t), wh1 = lds32(rh + 32 + 32 * c + 4 * t);
#pragma unroll
                for (int hn = 0; hn < 2; ++hn) {   // sub-block j = 2c + hn: low / high nibbles
                    const int j = 2 * c + hn;
                    const uint32_t qg0 = (hn ? wg0 >> 4 : wg0) & 0x0F0F0F0Fu, qg1 = (hn ? wg1 >> 4 : wg1) & 0x0F0F0F0Fu;
                    const uint32_t qh0 = (hn ? wh0 >> 4 : wh0) & 0x0F0F0F0Fu, qh1 = (hn ? wh1 >> 4 : wh1) & 0x0F0F0F0Fu;
                    const uint32_t scg = ((j < 4 ? scg_lo : scg_hi) >> (8 * (j & 3))) & 0xFFu;
                    const uint32_t sch = ((j < 4 ? sch_lo : sch_hi) >> (8 * (j & 3))) & 0xFFu;
                    const uint32_t mg = (((j < 4 ? mng_lo : mng_hi) >> (8 * (j & 3))) & 0xFFu) * 0x01010101u;
                    const uint32_t mh = (((j < 4 ? mnh_lo : mnh_hi) >> (8 * (j & 3))) & 0xFFu) * 0x01010101u;
                    const uint32_t shg = scg >> 3, slg = scg & 7u, shh = sch >> 3, slh = sch & 7u;
                    const uint32_t adr = smem_u32(sm.planes) + (blk * 256 + j * 32) + 4 * t;
#pragma unroll
                    for (int q = 0; q < kNxMaxCols / 2; ++q) {
                        if (q < (int)npair) {
                            const uint32_t pa = adr + ((2 * q + bcol) * 3 + bplane) * pstride;
                            const uint32_t v0 = lds32(pa), v1 = lds32(pa + 16);
                            const uint32_t b0 = feeds ? v0 : 0u, b1 = feeds ? v1 : 0u;
                            mma_u8s8_acc(chi[q], qg0 * shg, qh0 * shh, qg1 * shg, qh1 * shh, b0, b1);
                            mma_u8s8_acc(clo[q], qg0 * slg, qh0 * slh, qg1 * slg, qh1 * slh, b0, b1);
                            mma_u8s8_acc(cmn[q], mg, mh, mg, mh, b0, b1);
                        }
                    }
                }
            }
            const float dg = h2f_bits((uint16_t)(hg.x & 0xFFFFu)), dming = h2f_bits((uint16_t)(hg.x >> 16));
            const float dh = h2f_bits((uint16_t)(hh.x & 0xFFFFu)), dminh = h2f_bits((uint16_t)(hh.x >> 16));
#pragma unroll
            for (int q = 0; q < kNxMaxCols / 2; ++q) {
                if (q < (int)npair) {
                    const float xs0 = sm.xs[(2 * q + c0) * nblk + blk] * pw0, xs1 = sm.xs[(2 * q + c1) * nblk + blk] * pw1;
                    // accumulator entries: [0] (row g, col n0), [1] (row g, col n1), [2] (row g + 8, n0), [3] (row g + 8, n1)
                    acc[q][0][0] = fmaf(xs0, dg * (float)(8 * chi[q][0] + clo[q][0]) - dming * (float)cmn[q][0], acc[q][0][0]);
                    acc[q][0][1] = fmaf(xs1, dg * (float)(8 * chi[q][1] + clo[q][1]) - dming * (float)cmn[q][1], acc[q][0][1]);
                    acc[q][1][0] = fmaf(xs0, dh * (float)(8 * chi[q][2] + clo[q][2]) - dminh * (float)cmn[q][2], acc[q][1][0]);
                    acc[q][1][1] = fmaf(xs1, dh * (float)(8 * chi[q][3] + clo[q][3]) - dminh * (float)cmn[q][3], acc[q][1][1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && p_i < my_stages && !dead) issue();
        if (++slot == (uint32_t)kNxStages) { slot = 0; parity ^= 1u; }
        if (++s_in == spu) {
            s_in = 0;
            // per (row, column) totals of this warp: columns n = 0..2 of a pair are its even column, 3..5 its odd one
#pragma unroll
            for (int q = 0; q < kNxMaxCols / 2; ++q) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    float ev = t == 0 ? acc[q][r][0] + acc[q][r][1] : t == 1 ? acc[q][r][0] : 0.f;
                    float od = t == 2 ? acc[q][r][0] + acc[q][r][1] : t == 1 ? acc[q][r][1] : 0.f;
                    ev += __shfl_xor_sync(0xffffffffu, ev, 1); od += __shfl_xor_sync(0xffffffffu, od, 1);
                    ev += __shfl_xor_sync(0xffffffffu, ev, 2); od += __shfl_xor_sync(0xffffffffu, od, 2);
                    if (t == 0) {
                        sm.part[(warp * 16 + g + 8 * r) * kNxMaxCols + 2 * q] = ev;
                        sm.part[(warp * 16 + g + 8 * r) * kNxMaxCols + 2 * q + 1] = od;
                    }
                    acc[q][r][0] = acc[q][r][1] = 0.f;
                }
            }
            __syncthreads();
            if (tid < 16 * kNxMaxCols) {
                const uint32_t row = tid / kNxMaxCols, col = tid % kNxMaxCols;
                if (col < a.nt) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w) v += sm.part[(w * 16 + row) * kNxMaxCols + col];   // fixed order
                    float *dst = a.y + (size_t)col * a.ystride + unit * 16 + row;
                    *dst = a.accumulate ? *dst + v : v;
                }
            }
            __syncthreads();
            unit += gridDim.x;
        }
    }
}

} // namespace

static bool g_mma_init = false;

// True when the launch can take the tensor-core kernel: Q4_K only, one tensor (or the gate|up pair with the
// SwiGLU epilogue), plain or RMSNorm activation, columns a multiple of 256 * 16 and at most 8192,
// rows a multiple of 16 (8 for the pair), packed rows, 16-byte aligned pointers.
bool matvec_mma_eligible(const MatvecArgs &a) {
    // Opt-in (FLB_MMA=1). Measured on the 8B-shape step against the scalar dp4a kernel: the O projection alone
    // is faster (4.2 vs 5.5 us: 16 warps build the activation in one round), gate|up is slower (21.7 vs 19.3 us:
    // a block barrier per 16-row unit, and the instruction count is not lower: 11.1 M vs 10.0 M warp
    // instructions), and the whole step is slower either way (443 vs 457 tokens/s). Kept as the base of the
    // multi-column (draft verification) matmul, where one A operand serves several B operands.
    const char *on = getenv("FLB_MMA");
    if (!on || on[0] != '1') return false;
    if (a.swiglu && !getenv("FLB_MMA_SWIGLU")) return false;
    if (a.n_tensors != (a.swiglu ? 2 : 1)) return false;
    for (int i = 0; i < a.n_tensors; ++i) {
        const MatvecTensor &t = a.t[i];
        if (t.fmt != FMT_Q4_K || t.expert_id || (t.pitch && t.pitch != row_bytes(FMT_Q4_K, a.cols))) return false;
        if ((((uintptr_t)t.w) & 15u) != 0) return false;
        if (t.rows % (a.swiglu ? 8u : 16u) != 0) return false;
    }
    if (a.swiglu && (a.t[0].rows != a.t[1].rows || a.accumulate)) return false;
    if (a.x_mode != MV_X_PLAIN && a.x_mode != MV_X_RMSNORM) return false;
    if (a.cols % (256u * kWarps) != 0 || a.cols > 2u * 256u * kWarps) return false;
    if ((((uintptr_t)a.x) & 15u) != 0 || (((uintptr_t)a.wnorm) & 15u) != 0) return false;
    if (a.xn_out) return false;
    return true;
}

// y[p * ystride + r] (+)= dot(W[r], x + p * xstride), p < nt, in one pass over a Q4_K tensor. Returns
// cudaErrorNotSupported when the shape does not qualify (the caller then runs the columns one by one).
cudaError_t launch_matmul_q4k_nx(const void *w, uint32_t rows, uint32_t cols, const float *x, uint32_t nt, uint32_t xstride,
                                 float *y, uint32_t ystride, int accumulate, uint32_t *status, int sms, cudaStream_t stream) {
    static bool init = false;
    if (nt < 2 || nt > kNxMaxCols || rows % 16 != 0 || cols % (256u * kWarps) != 0) return cudaErrorNotSupported;
    if ((((uintptr_t)w) & 15u) != 0 || (((uintptr_t)x) & 15u) != 0 || (xstride & 3u) != 0 || ystride < rows) return cudaErrorNotSupported;
    const uint32_t nt_pad = (nt + 1u) & ~1u;
    const size_t smem = nx_fixed_bytes(cols, nt_pad) + 8 + 128 + (size_t)kWarps * kNxStages * kStageBytes;
    if (smem > 227 * 1024 - 1024) return cudaErrorNotSupported;
    if (!init) {
        const cudaError_t e = cudaFuncSetAttribute(matvec_q4k_mma_nx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return e;
        init = true;
    }
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    const uint64_t rb = row_bytes(FMT_Q4_K, cols);
    cudaError_t e = tensor_map_2d(&map, 8, w, rb / 8, rows, rb, 18, 16, false);
    if (e != cudaSuccess) return e;
    NxArgs a{};
    a.w = (const uint8_t *)w; a.x = x; a.y = y; a.rows = rows; a.cols = cols; a.nt = nt; a.xstride = xstride; a.ystride = ystride;
    a.accumulate = accumulate; a.status = status;
    const uint32_t n_units = rows / 16;
    const uint32_t grid = n_units < (uint32_t)sms ? n_units : (uint32_t)sms;
    return launch_kernel(matvec_q4k_mma_nx_kernel, dim3(grid), dim3(kThreads), smem, stream, false, a, map, n_units);
}

cudaError_t launch_matvec_mma(const MatvecArgs &a, int sms, cudaStream_t stream) {
    const size_t smem = fixed_bytes(a.cols) + 128 + (size_t)kWarps * kStages * kStageBytes;
    if (!g_mma_init) {
        const cudaError_t e = cudaFuncSetAttribute(matvec_q4k_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return e;
        g_mma_init = true;
    }
    if (smem > 227 * 1024 - 1024) return cudaErrorInvalidValue;
    const uint32_t rows_per_unit = a.swiglu ? 8u : 16u;
    const uint32_t n_units = a.t[0].rows / rows_per_unit;
    Maps maps;
    memset(&maps, 0, sizeof(maps));
    for (int i = 0; i < a.n_tensors; ++i) {
        const uint64_t rb = row_bytes(FMT_Q4_K, a.cols);
        const cudaError_t e = tensor_map_2d(&maps.m[i], 8, a.t[i].w, rb / 8, a.t[i].rows, rb, 18, rows_per_unit, false);
        if (e != cudaSuccess) return e;
    }
    uint32_t grid = n_units < (uint32_t)sms ? n_units : (uint32_t)sms;
    return launch_kernel(matvec_q4k_mma_kernel, dim3(grid), dim3(kThreads), smem, stream, a.pdl != 0, a, maps, n_units);
}

} // namespace flb
