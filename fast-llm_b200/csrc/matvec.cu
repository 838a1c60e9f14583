// k-quant dequantize-matvec for single-token decode (replaces the reference's
// warp-per-row gdot_q4_K / gdot_q6_K / gdot_q8_0, src/runtime/kernels_gpu.h:65-205,
// and the STREAM_DOT branch of exec_task_block, src/runtime/gpu_exec.cu:64-140).
//
// Streaming kernel (Q4_K and Q6_K, cols a multiple of 256)
// ---------------------------------------------------------
// HBM-bound by design: every packed weight byte is read exactly once. Each warp
// owns a private ring of shared-memory stages that its lane 0 keeps filled with
// 2-D TMA box loads (cp.async.bulk.tensor.2d over a [rows][row bytes / 8]
// view of the packed tensor, completion on an mbarrier), so the bytes in flight
// per SM do not depend on registers and no warp synchronises with another one.
//   stage  = the same 8-super-block column segment (2048 weights) of 4
//            consecutive rows (a "row quad"): one box of 4 x 1152 B (Q4_K) or
//            4 x 1680 B (Q6_K); a last partial segment and rows past the end
//            of the tensor are filled with zeros by the TMA unit;
//   lane   = one quarter of a super-block (64 weights) of each of the 4 rows:
//            block = lane/4, quarter = lane%4. The activation slice a lane
//            needs is the same for the 4 rows: it is read from shared memory
//            once per stage and reused 4 times.
//   math   = a first version converted every quant to f32 and used f32 FMAs; ncu
//            showed it issue-bound at 4.5 instructions per weight (the byte ->
//            float conversions dominate). The activation is therefore kept in
//            21-bit fixed point per 256-column block: x = s * (a0*2^14 + a1*2^7
//            + a2) with balanced base-128 digits a_i in [-64, 63] stored as
//            int8. The 4/6-bit quants, masked four to a word, are multiplied
//            with the three digit planes by dp4a (exact int32 sums over a 32- or
//            16-element sub-block); one int->float conversion per sub-block,
//            then f32: times the sub-block scale, minus min * (sum of the
//            sub-block's activations) for Q4_K, times d / dmin and the block's
//            activation scale. The fixed-point step is amax * 2^-20 of each
//            256-column block, i.e. about 1e-6 of the row dot in the
//            S-normalised metric (the canonical f32 sequential dot is itself
//            8e-6 from the f64 value), far inside the 1e-3 gate; all sums are
//            in a fixed order, so results are reproducible run to run.
// A row's 32-lane partials are reduced with shuffles when its last segment is
// done; lane 0 writes y. Several tensors that share x (Q/K/V, gate/up) run in
// one launch. The activation can be built on the fly from the residual stream
// (RMSNorm) or from gate/up (SiLU * up), which removes those launches.
//
// Generic kernel: any other shape / format (Q8_0, Q5_0, F32, cols not a
// multiple of 256, rows not 16-byte pitched): warp per row, element-wise f32.
#include "common.cuh"
#include "kernels.h"

#include <cuda.h>
#include <cstdlib>
#include <cstring>

namespace flb {

namespace {

constexpr int kWarps = 12;            // warps per CTA (each consumes and feeds its own ring); 16 warps with two ring
                                      // stages each were measured slower (they cap the kernel at 128 registers)
constexpr int kMaxThreads = kWarps * 32;
constexpr int kRowsPerStage = 4;
constexpr uint32_t kSeg4 = 8 * 144;   // bytes of one Q4_K segment (8 super-blocks)
constexpr uint32_t kSeg6 = 8 * 210;   // bytes of one Q6_K segment
constexpr uint32_t kStage4 = kRowsPerStage * kSeg4;       // ring slot size, Q4_K only
constexpr uint32_t kStage6 = (kRowsPerStage * kSeg6 + 127u) & ~127u;   // ring slot size when Q6_K is present (128-byte aligned for TMA)
constexpr uint32_t kSeg8 = 64 * 34;   // bytes of one Q8_0 segment (64 blocks of 32 weights = 2048 columns)
constexpr uint32_t kHalf8 = kSeg8 / 2;                    // a TMA box is at most 256 eight-byte elements wide: two boxes per segment
constexpr uint32_t kStage8 = kRowsPerStage * kSeg8;       // ring slot size, Q8_0 only: [half][row][1088 bytes]
constexpr float kFixMax = 1040000.0f; // largest fixed-point magnitude (63*2^14 + 63*2^7 + 63 = 1040447)

// byte K of w as a float, without the integer->float conversion pipe: the byte
// placed under 0x4B000000 is the float 2^23 + byte.
template <int K>
__device__ __forceinline__ float u8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K)) - 8388608.0f;
}

// 4 x (u8 * s8) + c
__device__ __forceinline__ int dp4a_us(uint32_t a_u8x4, uint32_t b_s8x4, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_u8x4), "r"(b_s8x4), "r"(c));
    return d;
}

// ---- activation layouts in shared memory --------------------------------------
// For segment s (2048 columns), 16-byte slot f (0..11) and lane l the slot sits at
// byte ((s*12 + f)*32 + l)*16, so a warp's 16-byte loads are contiguous.
// slot f = digit*4 + part, digit 0 = most significant.
// Q4_K: lane = blk*4 + chunk(64 columns); parts 0,1 = the 32 columns of the
//       low-nibble sub-block (16 each), parts 2,3 = the high-nibble sub-block.
// Q6_K: lane = blk*4 + half*2 + hq; the quarter covers columns 16*hq..16*hq+15
//       of each 32-column group g of the half; part = g.
__device__ __forceinline__ uint32_t pos4(uint32_t col, uint32_t digit) {
    const uint32_t blk = col >> 8, seg = blk >> 3, sbi = blk & 7u;
    const uint32_t c = (col >> 6) & 3u, k = col & 63u;
    return (((seg * 12 + digit * 4 + (k >> 4)) * 32) + sbi * 4 + c) * 16 + (k & 15u);
}
__device__ __forceinline__ uint32_t pos6(uint32_t col, uint32_t digit) {
    const uint32_t blk = col >> 8, seg = blk >> 3, sbi = blk & 7u;
    const uint32_t e = col & 255u;
    const uint32_t hf = e >> 7, g = (e >> 5) & 3u, hq = (e >> 4) & 1u;
    return (((seg * 12 + digit * 4 + g) * 32) + sbi * 4 + hf * 2 + hq) * 16 + (e & 15u);
}

struct Smem {
    int8_t *q4;      // Q4_K layout of the digit planes: cols * 3 bytes
    float *s4;       // per lane: sums of its two 32-column sub-blocks (in units of the block scale)
    int8_t *q6;      // Q6_K layout: cols * 3 bytes
    float *s6;       // per lane: sums of its four 16-column groups
    float *xs;       // activation scale of each 256-column block
    uint64_t *bars;  // [warps][stages]
    uint8_t *ring;   // [warps][stages][stage bytes]
};

// Columns rounded up to whole 2048-column segments: the shared-memory layouts are
// per segment, and the blocks past the end of a shorter row hold zeros.
__host__ __device__ inline uint32_t padded_cols(uint32_t cols) { return (cols + 2047u) & ~2047u; }

__host__ __device__ inline size_t smem_fixed_bytes(uint32_t cols, bool q4, bool q6) {
    cols = padded_cols(cols);
    size_t n = (size_t)cols / 256 * 4;                               // xs
    if (q4) n += (size_t)cols * 3 + (size_t)cols / 32 * 4;
    if (q6) n += (size_t)cols * 3 + (size_t)cols / 16 * 4;
    return n;
}

__device__ __forceinline__ Smem carve(uint8_t *base, uint32_t cols, bool q4, bool q6, int stages, uint32_t nw) {
    Smem s;
    uint8_t *p = base;
    cols = padded_cols(cols);
    s.q4 = s.q6 = nullptr;
    s.s4 = s.s6 = nullptr;
    if (q4) { s.q4 = (int8_t *)p; p += (size_t)cols * 3; }     // cols*3 is a multiple of 16
    if (q6) { s.q6 = (int8_t *)p; p += (size_t)cols * 3; }
    if (q4) { s.s4 = (float *)p; p += (size_t)cols / 32 * 4; }
    if (q6) { s.s6 = (float *)p; p += (size_t)cols / 16 * 4; }
    s.xs = (float *)p; p += (size_t)cols / 256 * 4;
    p = (uint8_t *)(((uintptr_t)p + 7) & ~(uintptr_t)7);
    s.bars = (uint64_t *)p; p += (size_t)nw * stages * 8;
    p = (uint8_t *)(((uintptr_t)p + 127) & ~(uintptr_t)127);
    s.ring = p;
    return s;
}

// ---- shared-memory loads by 32-bit shared address ------------------------------
// (explicit .shared loads: ring pointers derived from the dynamic shared base
// would otherwise compile to generic loads)
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// ---- per-stage math ----------------------------------------------------------

// The 12 activation slots of one lane for one segment: v[digit*4 + part].
struct XSlots { uint4 v[12]; };

__device__ __forceinline__ XSlots load_slots(uint32_t base_addr, uint32_t seg, uint32_t lane) {
    XSlots s;
    const uint32_t p = base_addr + ((seg * 12 * 32) + lane) * 16;
#pragma unroll
    for (int f = 0; f < 12; ++f) s.v[f] = lds128(p + f * 32 * 16);
    return s;
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// digits -> one integer: a0*2^14 + a1*2^7 + a2 (fits int32 for a sub-block)
__device__ __forceinline__ float fix_to_float(int i0, int i1, int i2) {
    return (float)((i0 << 14) + (i1 << 7) + i2);
}

// Q4_K quarter (64 weights) of one row: its contribution to the dot, in units
// of the block's activation scale. blk: shared address of the super-block.
__device__ __forceinline__ float q4k_quarter(uint32_t blk, uint32_t c, const XSlots &xq, float2 sx) {
    const uint4 hdr = lds128(blk);
    const uint4 qa = lds128(blk + 16 + 32 * c);
    const uint4 qb = lds128(blk + 32 + 32 * c);
    int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w = i < 4 ? word_of(qa, i) : word_of(qb, i - 4);
        const uint32_t lo = w & 0x0F0F0F0Fu, hi = w & 0xF0F0F0F0u;   // hi holds 16 * q
        const int part = i >> 2, wi = i & 3;
        a0 = dp4a_us(lo, word_of(xq.v[0 + part], wi), a0);
        a1 = dp4a_us(lo, word_of(xq.v[4 + part], wi), a1);
        a2 = dp4a_us(lo, word_of(xq.v[8 + part], wi), a2);
        b0 = dp4a_us(hi, word_of(xq.v[2 + part], wi), b0);
        b1 = dp4a_us(hi, word_of(xq.v[6 + part], wi), b1);
        b2 = dp4a_us(hi, word_of(xq.v[10 + part], wi), b2);
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
    // the high-nibble sums are exact multiples of 16: fold the 1/16 into the digit shifts
    const float fb = (float)((b0 << 10) + (b1 << 3) + (b2 >> 4));
    const float t = u8f<0>(sc) * fix_to_float(a0, a1, a2) + u8f<1>(sc) * fb;
    const float m = u8f<0>(mn) * sx.x + u8f<1>(mn) * sx.y;
    return d * t - dmin * m;
}

// Q6_K quarter (64 weights: 16 columns of each of the 4 groups of one half).
// row: shared address of this row's segment in the stage. Blocks are 210 bytes,
// so odd blocks start 2 bytes past a word boundary: every field is read as the
// two aligned words around it and realigned with a byte permute.
__device__ __forceinline__ float q6k_quarter(uint32_t row, uint32_t sbi, uint32_t qt, const XSlots &xq, float4 sx) {
    const uint32_t hf = qt >> 1, hq = qt & 1u;
    const uint32_t ob = sbi * 210u;
    const uint32_t sel = (ob & 2u) ? 0x5432u : 0x3210u;
    const uint32_t wbase = row + (ob & ~3u);
    const uint32_t pa = wbase + 64 * hf + 16 * hq;          // ql: groups 0 (low nibbles) / 2 (high)
    const uint32_t ph = wbase + 128 + 32 * hf + 16 * hq;    // qh
    uint32_t wa[5], wb[5], wh[5];
#pragma unroll
    for (int j = 0; j < 5; ++j) {
        wa[j] = lds32(pa + 4 * j);
        wb[j] = lds32(pa + 32 + 4 * j);                    // ql + 32: groups 1 / 3
        wh[j] = lds32(ph + 4 * j);
    }
    int acc[4][3];
#pragma unroll
    for (int g = 0; g < 4; ++g) acc[g][0] = acc[g][1] = acc[g][2] = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t a = __byte_perm(wa[j], wa[j + 1], sel), b = __byte_perm(wb[j], wb[j + 1], sel);
        const uint32_t h = __byte_perm(wh[j], wh[j + 1], sel);
        uint32_t q[4];
        q[0] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
        q[1] = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
        q[2] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
        q[3] = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            acc[g][0] = dp4a_us(q[g], word_of(xq.v[0 + g], j), acc[g][0]);
            acc[g][1] = dp4a_us(q[g], word_of(xq.v[4 + g], j), acc[g][1]);
            acc[g][2] = dp4a_us(q[g], word_of(xq.v[8 + g], j), acc[g][2]);
        }
    }
    // the 8 int8 scales of this half: bytes hq, hq+2, hq+4, hq+6 are this quarter's
    const uint32_t ps = wbase + 192 + 8 * hf;
    const uint32_t s0 = lds32(ps), s1 = lds32(ps + 4), s2 = lds32(ps + 8);
    const uint32_t lo = __byte_perm(s0, s1, sel), hi = __byte_perm(s1, s2, sel);
    // (s ^ 0x80) is s + 128 as an unsigned byte
    const uint32_t sw = __byte_perm(lo, hi, hq ? 0x7531u : 0x6420u) ^ 0x80808080u;
    const float d = h2f_bits((uint16_t)lds16(row + ob + 208));
    // value = d * sc * (q - 32): sum q*x minus 32 * sum x per 16-column group
    float t = (u8f<0>(sw) - 128.f) * (fix_to_float(acc[0][0], acc[0][1], acc[0][2]) - 32.f * sx.x);
    t += (u8f<1>(sw) - 128.f) * (fix_to_float(acc[1][0], acc[1][1], acc[1][2]) - 32.f * sx.y);
    t += (u8f<2>(sw) - 128.f) * (fix_to_float(acc[2][0], acc[2][1], acc[2][2]) - 32.f * sx.z);
    t += (u8f<3>(sw) - 128.f) * (fix_to_float(acc[3][0], acc[3][1], acc[3][2]) - 32.f * sx.w);
    return d * t;
}

// Q8_0: the lane's 64 columns are two blocks of 34 bytes (f16 d + 32 int8), 68 bytes from `blk` (4-byte
// aligned). The first block's quants start 2 bytes into a word and are realigned with byte permutes.
// Value in units of the block's activation scale. Same digit-plane layout as Q4_K (16 columns per slot).
__device__ __forceinline__ float q8_0_pair(uint32_t blk, const XSlots &xq) {
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = lds32(blk + 4 * i);
    int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int qa = (int)__byte_perm(w[k], w[k + 1], 0x5432u);   // bytes 2, 3 of word k, then 0, 1 of word k + 1
        const int qb = (int)w[9 + k];
        const int part = k >> 2, wi = k & 3;
        a0 = __dp4a(qa, (int)word_of(xq.v[0 + part], wi), a0);
        a1 = __dp4a(qa, (int)word_of(xq.v[4 + part], wi), a1);
        a2 = __dp4a(qa, (int)word_of(xq.v[8 + part], wi), a2);
        b0 = __dp4a(qb, (int)word_of(xq.v[2 + part], wi), b0);
        b1 = __dp4a(qb, (int)word_of(xq.v[6 + part], wi), b1);
        b2 = __dp4a(qb, (int)word_of(xq.v[10 + part], wi), b2);
    }
    const float d0 = h2f_bits((uint16_t)(w[0] & 0xFFFFu)), d1 = h2f_bits((uint16_t)(w[8] >> 16));
    return d0 * fix_to_float(a0, a1, a2) + d1 * fix_to_float(b0, b1, b2);
}

// ---- the streaming kernel ---------------------------------------------------

// One TMA descriptor per tensor of the launch: the packed tensor as a 2-D array
// of 8-byte elements [rows][row_bytes / 8]; a box is 4 rows x one column segment.
struct TensorMaps { CUtensorMap m[4]; };

// A row quad of one of the launch's tensors.
struct QuadRef {
    float *y;
    const float *resid;
    uint32_t r0, rows;     // first row index, rows in the tensor
    uint32_t row_off;      // rows to skip in the weight array (expert indirection)
    int fmt, ti;           // format, tensor index
};

// 2-D tiled TMA load (box = 4 rows x one segment) into shared memory; x counts
// 8-byte elements (always a multiple of 2, so the copy starts 16-byte aligned).
__device__ __forceinline__ void tma_load_box(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ QuadRef locate_quad(const MatvecArgs &a, uint32_t quad) {
    QuadRef q;
    if (a.swiglu) {   // quad = rows 2q, 2q+1 of the gate tensor and the same rows of the up tensor
        q.r0 = quad * 2;
        q.rows = a.t[0].rows;
        q.fmt = a.t[0].fmt;
        q.ti = 0;
        q.y = a.t[0].y;
        q.resid = nullptr;
        q.row_off = 0;
        return q;
    }
    int ti = 0;
    uint32_t base = 0;
#pragma unroll 1
    for (; ti < a.n_tensors - 1; ++ti) {
        const uint32_t nq = (a.t[ti].rows + kRowsPerStage - 1) / kRowsPerStage;
        if (quad < base + nq) break;
        base += nq;
    }
    const MatvecTensor &t = a.t[ti];
    q.r0 = (quad - base) * kRowsPerStage;
    q.rows = t.rows;
    q.fmt = t.fmt;
    q.ti = ti;
    q.y = t.y;
    q.resid = t.resid;
    q.row_off = t.expert_id ? *t.expert_id * t.expert_rows : 0u;
    return q;
}

// XR: the activation is the sum of the ranks' partial vectors arriving in the exchange buffer (tensor
// parallel); a separate instantiation so that the single-GPU kernel does not pay for it in registers.
// Q8: a launch of Q8_0 tensors (never mixed with the K-quants) has an instantiation of its own. All K-quant
// launches of a decode step share ONE kernel body on purpose: the step alternates between launch shapes every
// few microseconds, and instruction fetch is a visible part of these short kernels. Measured on the 8B-shape
// step: taking the Q8_0 unpack code out of the shared body gave +2 % (452 -> 461 tokens/s), while one
// instantiation per format combination, each smaller still, lost 13 % (395 tokens/s) because consecutive
// launches then no longer ran the same code.
template <bool XR, bool Q8>
__global__ void __launch_bounds__(kMaxThreads, 1)
matvec_stream_kernel(const MatvecArgs a, const __grid_constant__ TensorMaps maps, const uint32_t total_quads,
                     const int stages, const int use_q4, const int use_q6) {
    constexpr bool use_q8 = Q8;   // use_q4 is set for Q8_0 launches: they use the Q4_K plane layout
    extern __shared__ __align__(128) uint8_t smem_raw[];
    if (a.t[0].expert_id != nullptr && *a.t[0].expert_id == kExpertSkip) return;   // not this GPU's expert (see MatvecTensor)
    const uint32_t nw = blockDim.x >> 5;   // warps of this launch
    const Smem sm = carve(smem_raw, a.cols, use_q4 != 0, use_q6 != 0, stages, nw);   // Q8_0 uses the Q4_K plane layout (use_q4 is set)
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t nseg = (a.cols + 2047u) / 2048u;   // the last segment may be partial: the TMA unit fills the rest with zeros
    const uint32_t stage_bytes = use_q8 ? kStage8 : use_q6 ? kStage6 : kStage4;
    __shared__ float red[kWarps];

    bool indirect = false;
    for (int i = 0; i < a.n_tensors; ++i) indirect = indirect || a.t[i].expert_id != nullptr;
    indirect = indirect && !a.expert_ids_ready;   // ids written before the previous kernel started are read like constants
    uint64_t *bars = sm.bars + warp * stages;
    const uint32_t ring = smem_u32(sm.ring) + warp * stages * stage_bytes;   // shared address
    if (lane == 0)
        for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    fence_barrier_init();
    __syncwarp();

    // This warp's quads: gw, gw + W, ... ; per quad nseg stages (one per column segment).
    // Warps are numbered CTA-fastest, so a launch with few quads spreads them over
    // all SMs instead of filling the first CTAs.
    const uint32_t gw = warp * gridDim.x + blockIdx.x, W = gridDim.x * nw;
    const uint32_t my_quads = gw < total_quads ? (total_quads - gw + W - 1) / W : 0;
    const uint32_t my_stages = my_quads * nseg;

    // Producer state (meaningful in lane 0): next stage to request.
    uint32_t p_i = 0, p_seg = 0, p_slot = 0, p_quad = gw;
    QuadRef pq;
    auto issue = [&]() {   // lane 0 only; requests stage p_i and advances
        if (p_seg == 0) pq = locate_quad(a, p_quad);
        if (use_q8) {   // two boxes of 4 rows x 1088 bytes: the halves of the segment
            mbar_arrive_expect_tx(&bars[p_slot], kStage8);
            tma_load_box(ring + p_slot * stage_bytes, &maps.m[pq.ti], p_seg * (kSeg8 / 8), pq.r0, &bars[p_slot]);
            tma_load_box(ring + p_slot * stage_bytes + kRowsPerStage * kHalf8, &maps.m[pq.ti], p_seg * (kSeg8 / 8) + kHalf8 / 8, pq.r0,
                         &bars[p_slot]);
            ++p_i;
            if (++p_slot == (uint32_t)stages) p_slot = 0;
            if (++p_seg == nseg) { p_seg = 0; p_quad += W; }
            return;
        }
        const uint32_t sb = pq.fmt == FMT_Q4_K ? kSeg4 : kSeg6;
        mbar_arrive_expect_tx(&bars[p_slot], kRowsPerStage * sb);
        // rows past the end of the tensor are filled with zeros by the TMA unit (their results are dropped)
        if (a.swiglu) {   // two boxes of 2 rows: gate rows, then up rows
            tma_load_box(ring + p_slot * stage_bytes, &maps.m[0], p_seg * (sb / 8), pq.r0, &bars[p_slot]);
            tma_load_box(ring + p_slot * stage_bytes + 2 * sb, &maps.m[1], p_seg * (sb / 8), pq.r0, &bars[p_slot]);
        } else {
            tma_load_box(ring + p_slot * stage_bytes, &maps.m[pq.ti], p_seg * (sb / 8), pq.r0 + pq.row_off, &bars[p_slot]);
        }
        ++p_i;
        if (++p_slot == (uint32_t)stages) p_slot = 0;
        if (++p_seg == nseg) { p_seg = 0; p_quad += W; }
    };
    // Weights do not depend on the activation: start streaming before x is built
    // (unless the expert to stream is itself a result of the previous kernel).
    if (tid == 0) trace_min(a.trace, 0);
    griddep_launch_dependents();
    if (lane == 0 && !indirect && !a.issue_late)
        while (p_i < (uint32_t)stages && p_i < my_stages) issue();

    // ---- build the fixed-point activation in shared memory ----
    // Half a warp per 256-column block (blocks h, h + 2 nw, ... with h = 2 warp + lane / 16); lane l of
    // the half holds columns 16 l .. 16 l + 15 of the block, so the 16 blocks of a 4096-column
    // activation are one round for 12 warps (a block's chain of reduce -> scale -> digits is latency
    // bound; a second round would double it). All global loads of all the blocks are issued first, so
    // the prologue costs one memory round trip; the norm weights are constants and are fetched before
    // the dependency wait.
    constexpr int kMaxBlk = 3;   // blocks per half-warp: cols <= 3 * 256 * 2 * kWarps = 18432
    const uint32_t nblk = a.cols / 256, nblk_pad = nseg * 8;   // blocks nblk .. nblk_pad-1 are zeros
    const uint32_t hw = 2 * warp + (lane >> 4), hl = lane & 15u, nhw = 2 * nw;
    float4 ra[kMaxBlk][4], rb2[kMaxBlk][4];
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b)
#pragma unroll
        for (int k = 0; k < 4; ++k) ra[b][k] = rb2[b][k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.x_mode == MV_X_RMSNORM) {
#pragma unroll
        for (int b = 0; b < kMaxBlk; ++b) {
            const uint32_t blk = hw + b * nhw;
            if (blk < nblk) {
                const float4 *src = reinterpret_cast<const float4 *>(a.wnorm + blk * 256 + hl * 16);
#pragma unroll
                for (int k = 0; k < 4; ++k) rb2[b][k] = __ldg(src + k);
            }
        }
    }
    griddep_wait();   // the activation (and y, resid) come from the previous kernel
    if (tid == 0) trace_min(a.trace, 1);
    if (lane == 0 && indirect)
        while (p_i < (uint32_t)stages && p_i < my_stages) issue();
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b) {
        const uint32_t blk = hw + b * nhw;
        if (XR && blk < nblk) {
            // x = residual + the ranks' partial vectors, as they land in this rank's exchange buffer
            const uint32_t c0 = blk * 256 + hl * 16;
            const uint32_t chunk = c0 / (a.cols / kCommChunks);        // the lane's 16 columns lie in one chunk
            const uint32_t e = __ldcg(a.xr_epoch + chunk), slot = e & 1u;
            const float *recv = reinterpret_cast<const float *>(a.xr_buf) + (size_t)slot * kCommMaxRanks * kCommMaxVec;
            const uint32_t *flags = reinterpret_cast<const uint32_t *>(a.xr_buf + kCommFlagsOff) +
                                    (size_t)slot * kCommMaxRanks * kCommChunks + chunk;
            const float4 *rs = reinterpret_cast<const float4 *>(a.xr_resid + c0);
#pragma unroll
            for (int k = 0; k < 4; ++k) ra[b][k] = rs[k];
            for (uint32_t r = 0; r < a.xr_world; ++r) {
                if (!wait_flag(flags + r * kCommChunks, e, a.status)) break;   // status word set; the result is void
                const float4 *pv = reinterpret_cast<const float4 *>(recv + (size_t)r * kCommMaxVec + c0);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 v = __ldcg(pv + k);
                    ra[b][k].x += v.x; ra[b][k].y += v.y; ra[b][k].z += v.z; ra[b][k].w += v.w;
                }
            }
            if (blockIdx.x == 0) {
                float4 *dst = reinterpret_cast<float4 *>(a.xr_out + c0);
#pragma unroll
                for (int k = 0; k < 4; ++k) dst[k] = ra[b][k];
            }
        } else if (blk < nblk) {
            const float4 *src = reinterpret_cast<const float4 *>(a.x + blk * 256 + hl * 16);
#pragma unroll
            for (int k = 0; k < 4; ++k) ra[b][k] = src[k];
            if (a.x_mode == MV_X_SILU_MUL) {
                const float4 *src2 = reinterpret_cast<const float4 *>(a.x2 + blk * 256 + hl * 16);
#pragma unroll
                for (int k = 0; k < 4; ++k) rb2[b][k] = src2[k];
            }
        }
    }
    if (lane == 0 && a.issue_late && !indirect)
        while (p_i < (uint32_t)stages && p_i < my_stages) issue();   // the activation loads are in flight meanwhile
    // RMSNorm: the digits are those of x*w (the common factor 1/rms is applied to
    // the row sums at the end), so the sum of squares and the quantisation need
    // only one block-wide barrier between them and the consumers.
    float ss = 0.f;
    if (a.x_mode == MV_X_RMSNORM) {
#pragma unroll
        for (int b = 0; b < kMaxBlk; ++b)   // blocks that were not loaded hold zeros
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 u = ra[b][k];
                ss += (u.x * u.x + u.y * u.y) + (u.z * u.z + u.w * u.w);
            }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
    }
#pragma unroll
    for (int b = 0; b < kMaxBlk; ++b) {
        // nblk_pad is even and the warp's two blocks are 2 warp + b nhw (+1): both halves leave together
        if (2 * warp + b * nhw >= nblk_pad) break;
        const uint32_t blk = hw + b * nhw;
        const uint32_t c0 = blk * 256 + hl * 16;
        float v[16], w2[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[4 * k] = ra[b][k].x; v[4 * k + 1] = ra[b][k].y; v[4 * k + 2] = ra[b][k].z; v[4 * k + 3] = ra[b][k].w;
            w2[4 * k] = rb2[b][k].x; w2[4 * k + 1] = rb2[b][k].y; w2[4 * k + 2] = rb2[b][k].z; w2[4 * k + 3] = rb2[b][k].w;
        }
        // one branch around each form: chosen per element, the compiler evaluates the exponential in every mode
        if (a.x_mode == MV_X_RMSNORM) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = v[i] * w2[i];
        } else if (a.x_mode == MV_X_SILU_MUL) {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = (v[i] / (1.0f + expf(-v[i]))) * w2[i];   // 0 for padding: silu(0) = 0
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // over the half-warp
        const float s = amax > 0.f ? amax / kFixMax : 1.0f;
        const float inv_s = 1.0f / s;
        int sum = 0;
        uint32_t pk[3][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};   // this lane's 16 columns of each digit plane
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int X = __float2int_rn(v[i] * inv_s);          // |X| <= 1040000
            const int d2 = ((X + 64) & 127) - 64;                // balanced base-128 digits
            const int X1 = (X - d2) >> 7;
            const int d1 = ((X1 + 64) & 127) - 64;
            const int d0 = (X1 - d1) >> 7;
            sum += X;
            pk[0][i >> 2] |= (uint32_t)(d0 & 0xFF) << (8 * (i & 3));
            pk[1][i >> 2] |= (uint32_t)(d1 & 0xFF) << (8 * (i & 3));
            pk[2][i >> 2] |= (uint32_t)(d2 & 0xFF) << (8 * (i & 3));
        }
        // the lane's 16 columns are exactly one 16-byte slot in both layouts
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            const uint4 w4 = make_uint4(pk[d][0], pk[d][1], pk[d][2], pk[d][3]);
            if (use_q4) *reinterpret_cast<uint4 *>(sm.q4 + pos4(c0, d)) = w4;
            if (use_q6) *reinterpret_cast<uint4 *>(sm.q6 + pos6(c0, d)) = w4;
        }
        // sums over 16 columns (this lane) and 32 columns (lane pairs), exact in int32
        const int s16 = sum;
        const int s32 = s16 + __shfl_xor_sync(0xffffffffu, s16, 1);
        const uint32_t seg = blk >> 3, sbi = blk & 7u;
        if (use_q4 && (hl & 1u) == 0) {
            // 32-column sub-block j = hl / 2 -> consumer lane sbi*4 + j/2, component j & 1
            const uint32_t j = hl >> 1;
            sm.s4[((seg * 32 + sbi * 4 + (j >> 1)) << 1) + (j & 1u)] = (float)s32;
        }
        if (use_q6) {
            // 16-column run r = hl (0..15): half = r/8, group g = (r/2)%4, hq = r%2
            const uint32_t r = hl, hf = r >> 3, g = (r >> 1) & 3u, hq = r & 1u;
            sm.s6[((seg * 32 + sbi * 4 + hf * 2 + hq) << 2) + g] = (float)s16;
        }
        if (hl == 0) sm.xs[blk] = s;
    }
    __syncthreads();
    float inv_rms = 1.f;
    if (a.x_mode == MV_X_RMSNORM) {
        float t = 0.f;
#pragma unroll
        for (uint32_t w = 0; w < nw; ++w) t += red[w];   // same order in every thread
        inv_rms = 1.0f / sqrtf(t / (float)a.cols + a.eps);
    }
    if (a.xn_out != nullptr && blockIdx.x == 0) {   // the activation as f32, for layer-level checks
        for (uint32_t c = tid; c < a.cols; c += blockDim.x) {
            float v = a.x[c];
            if (a.x_mode == MV_X_RMSNORM) v = v * inv_rms * a.wnorm[c];
            else if (a.x_mode == MV_X_SILU_MUL) v = (v / (1.0f + expf(-v))) * a.x2[c];
            a.xn_out[c] = v;
        }
    }
    if (tid == 0) trace_max(a.trace, 2);

    // ---- consume ----
    const uint32_t q4_addr = use_q4 ? smem_u32(sm.q4) : 0, q6_addr = use_q6 ? smem_u32(sm.q6) : 0;
    float acc[kRowsPerStage] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t sbi = lane >> 2, qt = lane & 3u;
    uint32_t seg = 0, slot = 0, parity = 0, quad = gw;
    QuadRef cur;
    for (uint32_t i = 0; i < my_stages; ++i) {
        if (seg == 0) cur = locate_quad(a, quad);
        const float xs = sm.xs[seg * 8 + sbi];
        const uint32_t st = ring + slot * stage_bytes;
        if constexpr (use_q8) {
            const XSlots xq = load_slots(q4_addr, seg, lane);
            if (!mbar_wait_bounded(&bars[slot], parity, a.status)) return;
            const uint32_t base = st + (lane >> 4) * (kRowsPerStage * kHalf8) + (lane & 15u) * 68u;
#pragma unroll
            for (int r = 0; r < kRowsPerStage; ++r) acc[r] = fmaf(xs, q8_0_pair(base + r * kHalf8, xq), acc[r]);
        } else if (cur.fmt == FMT_Q4_K) {
            const XSlots xq = load_slots(q4_addr, seg, lane);
            const float2 sx = reinterpret_cast<const float2 *>(sm.s4)[seg * 32 + lane];
            if (!mbar_wait_bounded(&bars[slot], parity, a.status)) return;
            // Two rows per trip of a rolled loop, not four unrolled: the smaller body measured +0.9 % on the whole
            // step (instruction fetch). The accumulator pairs swap places each trip so that they stay in registers.
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const uint32_t rs = st + (2 * h) * kSeg4 + sbi * 144;
                acc[0] = fmaf(xs, q4k_quarter(rs, qt, xq, sx), acc[0]);
                acc[1] = fmaf(xs, q4k_quarter(rs + kSeg4, qt, xq, sx), acc[1]);
                const float t0 = acc[0], t1 = acc[1];
                acc[0] = acc[2]; acc[1] = acc[3]; acc[2] = t0; acc[3] = t1;
            }
        } else {
            const XSlots xq = load_slots(q6_addr, seg, lane);
            const float4 sx = reinterpret_cast<const float4 *>(sm.s6)[seg * 32 + lane];
            if (!mbar_wait_bounded(&bars[slot], parity, a.status)) return;
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const uint32_t rs = st + (2 * h) * kSeg6;
                acc[0] = fmaf(xs, q6k_quarter(rs, sbi, qt, xq, sx), acc[0]);
                acc[1] = fmaf(xs, q6k_quarter(rs + kSeg6, sbi, qt, xq, sx), acc[1]);
                const float t0 = acc[0], t1 = acc[1];
                acc[0] = acc[2]; acc[1] = acc[3]; acc[2] = t0; acc[3] = t1;
            }
        }
        __syncwarp();
        if (lane == 0 && p_i < my_stages) {
            fence_proxy_async_smem();
            issue();
        }
        if (++slot == (uint32_t)stages) { slot = 0; parity ^= 1u; }
        if (++seg == nseg) {
            seg = 0;
            quad += W;
            // 4 row sums over 32 lanes in 6 shuffles: halve the number of live
            // values at each of the first two steps, then a 3-step butterfly.
            // Afterwards lanes 0, 8, 16, 24 hold the totals of rows 0, 2, 1, 3.
            const bool up16 = (lane & 16u) != 0, up8 = (lane & 8u) != 0;
            float k0 = up16 ? acc[1] : acc[0], g0 = up16 ? acc[0] : acc[1];
            float k1 = up16 ? acc[3] : acc[2], g1 = up16 ? acc[2] : acc[3];
            k0 += __shfl_xor_sync(0xffffffffu, g0, 16);   // lanes <16: row 0, lanes >=16: row 1
            k1 += __shfl_xor_sync(0xffffffffu, g1, 16);   // lanes <16: row 2, lanes >=16: row 3
            float k = up8 ? k1 : k0, g = up8 ? k0 : k1;
            k += __shfl_xor_sync(0xffffffffu, g, 8);      // row = (lane>>4 & 1) + 2*(lane>>3 & 1)
            k += __shfl_xor_sync(0xffffffffu, k, 4);
            k += __shfl_xor_sync(0xffffffffu, k, 2);
            k += __shfl_xor_sync(0xffffffffu, k, 1);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            if (a.swiglu) {
                // stage rows 0,1 = gate rows r0, r0+1 (lanes 0, 16), rows 2,3 = up rows (lanes 8, 24):
                // h = silu(gate) * up (fl_op_silu_mul, src/runtime/decode_params.h:267-272)
                k *= inv_rms;
                const float up = __shfl_xor_sync(0xffffffffu, k, 8);
                const uint32_t row = cur.r0 + ((lane >> 4) & 1u);
                if ((lane & 15u) == 0 && row < cur.rows) cur.y[row] = (k / (1.0f + expf(-k))) * up;
                continue;
            }
            const uint32_t row = cur.r0 + ((lane >> 4) & 1u) + 2u * ((lane >> 3) & 1u);
            if ((lane & 7u) == 0 && row < cur.rows) {
                k *= inv_rms;
                float o = k;
                if (cur.resid) o = cur.resid[row] + k;
                if (a.accumulate) o = cur.y[row] + o;
                cur.y[row] = o;
            }
        }
    }
    if (lane == 0) trace_max(a.trace, 3);
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
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, W = (gridDim.x * blockDim.x) >> 5;
    if (a.t[0].expert_id != nullptr && *a.t[0].expert_id == kExpertSkip) return;   // not this GPU's expert (see MatvecTensor)
    for (uint32_t vr = gw; vr < total_rows; vr += W) {
        int ti = 0;
        uint32_t base = 0;
        for (; ti < a.n_tensors - 1; ++ti) {
            if (vr < base + a.t[ti].rows) break;
            base += a.t[ti].rows;
        }
        const MatvecTensor &t = a.t[ti];
        const uint32_t r = vr - base;
        const uint64_t pitch = t.pitch ? t.pitch : row_bytes(t.fmt, a.cols);
        const uint8_t *row = t.w + ((uint64_t)r + (t.expert_id ? (uint64_t)*t.expert_id * t.expert_rows : 0ull)) * pitch;
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
    return (fmt == FMT_Q4_K || fmt == FMT_Q6_K || fmt == FMT_Q8_0) && cols >= 512 && cols % 256 == 0;
}

// Shared memory of a launch and its shape: kWarps rings with as many stages (at most 4) as fit.
size_t matvec_smem_bytes(uint32_t cols, bool q4, bool q6, int *stages_out, int *warps_out, bool q8) {
    const size_t fixed = smem_fixed_bytes(cols, q4 || q8, q6) + 8 + 128;   // + alignment slack
    const size_t limit = 227 * 1024 - 1024;   // leave room for static shared memory
    const size_t slot = q8 ? kStage8 : q6 ? kStage6 : kStage4;
    const int warps = kWarps;
    int stages = 4;
    while (stages > 1 && fixed + (size_t)warps * stages * (8 + slot) > limit) --stages;
    if (stages_out) *stages_out = stages;
    if (warps_out) *warps_out = warps;
    return fixed + (size_t)warps * stages * (8 + slot);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

cudaError_t matvec_init(void) {
    if (!g_encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        g_encode = (EncodeTiledFn)fn;
    }
    const void *kernels[] = {(const void *)matvec_stream_kernel<false, false>, (const void *)matvec_stream_kernel<true, false>,
                             (const void *)matvec_stream_kernel<false, true>};
    for (const void *k : kernels) {
        const cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// The packed tensor as [rows][row_bytes / 8] 8-byte elements, box = 4 rows x one segment.
static cudaError_t encode_map(CUtensorMap *m, const MatvecTensor &t, uint32_t cols, uint32_t box_rows) {
    if (!g_encode) return cudaErrorNotSupported;
    const uint64_t rb = t.pitch ? t.pitch : row_bytes(t.fmt, cols);   // a multiple of 16 (checked by the caller)
    const uint32_t seg = t.fmt == FMT_Q4_K ? kSeg4 : t.fmt == FMT_Q8_0 ? kHalf8 : kSeg6;
    // With expert indirection the rows of all experts are one array; its end is not known here, and
    // no box reaches past an expert (rows % 4 == 0 is required), so the row bound is left open.
    const cuuint64_t gdim[2] = {rb / 8, t.expert_id ? (cuuint64_t)0x7fffffffu : (cuuint64_t)t.rows};
    const cuuint64_t gstride[1] = {rb};
    const cuuint32_t box[2] = {seg / 8, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, (void *)t.w, gdim, gstride, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t tensor_map_2d(CUtensorMap *m, uint32_t elem_bytes, const void *base, uint64_t dim0, uint64_t rows,
                          uint64_t stride_bytes, uint32_t box0, uint32_t box_rows, bool swizzle128) {
    if (!g_encode) {
        const cudaError_t e = matvec_init();
        if (e != cudaSuccess) return e;
    }
    const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                 : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64;
    const cuuint64_t gdim[2] = {dim0, rows};
    const cuuint64_t gstride[1] = {stride_bytes};
    const cuuint32_t box[2] = {box0, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(m, dt, 2, const_cast<void *>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// A row-major byte array of rows whose pitch is a multiple of 128 bytes, seen as [rows][pitch / 128][128 bytes] with
// the 128-byte swizzle: a box of box_rows x box_lines lines lands in shared memory as lines of 128 bytes whose
// 16-byte chunks are permuted by the line index (chunk ^ (line & 7)), so that the same chunk of 8 consecutive
// rows falls into 8 different bank groups whatever the row pitch is.
cudaError_t tensor_map_lines_swz(CUtensorMap *m, const void *base, uint64_t rows, uint64_t pitch, uint32_t box_lines,
                                 uint32_t box_rows) {
    if (!g_encode) {
        const cudaError_t e = matvec_init();
        if (e != cudaSuccess) return e;
    }
    if (pitch % 128 != 0) return cudaErrorInvalidValue;
    const cuuint64_t gdim[3] = {16, pitch / 128, rows};      // 8-byte elements per line, lines per row, rows
    const cuuint64_t gstride[2] = {128, pitch};
    const cuuint32_t box[3] = {16, box_lines, box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), gdim, gstride, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

cudaError_t launch_matvec(const MatvecArgs &a, int sms, cudaStream_t stream) {
    if (a.n_tensors < 1 || a.n_tensors > 4 || a.cols == 0) return cudaErrorInvalidValue;
    if (matvec_tc_eligible(a)) return launch_matvec_tc(a, sms, stream);
    bool streaming = true, q4 = false, q6 = false, q8 = false;
    uint32_t total_rows = 0, total_quads = 0;
    for (int i = 0; i < a.n_tensors; ++i) {
        const MatvecTensor &t = a.t[i];
        if (t.rows == 0 || a.cols % blk_elems(t.fmt) != 0) return cudaErrorInvalidValue;
        if (t.fmt < FMT_F32 || t.fmt > FMT_Q6_K) return cudaErrorInvalidValue;
        const uint64_t pitch = t.pitch ? t.pitch : row_bytes(t.fmt, a.cols);
        if (pitch < row_bytes(t.fmt, a.cols)) return cudaErrorInvalidValue;
        streaming = streaming && matvec_is_streaming(t.fmt, a.cols) && (((uintptr_t)t.w) & 15u) == 0 && (pitch & 15u) == 0;
        if (t.expert_id && (t.rows % kRowsPerStage != 0 || a.swiglu)) streaming = false;
        streaming = streaming && a.cols <= 6u * 256u * kWarps && (((uintptr_t)a.x) & 15u) == 0 &&
                    (((uintptr_t)a.x2) & 15u) == 0 && (((uintptr_t)a.wnorm) & 15u) == 0;
        q4 = q4 || t.fmt == FMT_Q4_K;
        q6 = q6 || t.fmt == FMT_Q6_K;
        q8 = q8 || t.fmt == FMT_Q8_0;
        if (t.fmt == FMT_Q8_0 && (t.expert_id || a.swiglu)) streaming = false;
        total_rows += t.rows;
        total_quads += (t.rows + kRowsPerStage - 1) / kRowsPerStage;
    }
    if (a.swiglu) {
        if (a.n_tensors != 2 || a.t[0].rows != a.t[1].rows || a.t[0].fmt != a.t[1].fmt || a.accumulate || !streaming)
            return cudaErrorInvalidValue;
        total_quads = (a.t[0].rows + 1) / 2;
    }
    if (q8 && (q4 || q6)) streaming = false;   // Q8_0 streams only in launches of its own (another stage layout)
    if (streaming) {
        int stages = 0, warps = 0;
        const size_t smem = matvec_smem_bytes(a.cols, q4, q6, &stages, &warps, q8);
        if (smem <= 227 * 1024 - 1024 && stages >= 2) {
            uint32_t grid = total_quads < (uint32_t)sms ? total_quads : (uint32_t)sms;
            TensorMaps maps;
            memset(&maps, 0, sizeof(maps));
            for (int i = 0; i < a.n_tensors; ++i) {
                const cudaError_t e = encode_map(&maps.m[i], a.t[i], a.cols, a.swiglu ? 2 : kRowsPerStage);
                if (e != cudaSuccess) return e;
            }
            if (a.xr_buf && q8) return cudaErrorInvalidValue;   // the exchange prologue is not instantiated for Q8_0
            if (q8)
                return launch_kernel(matvec_stream_kernel<false, true>, dim3(grid), dim3(warps * 32), smem, stream, a.pdl != 0, a,
                                     maps, total_quads, stages, 1, 0);
            if (a.xr_buf)
                return launch_kernel(matvec_stream_kernel<true, false>, dim3(grid), dim3(warps * 32), smem, stream, a.pdl != 0, a,
                                     maps, total_quads, stages, q4 ? 1 : 0, q6 ? 1 : 0);
            return launch_kernel(matvec_stream_kernel<false, false>, dim3(grid), dim3(warps * 32), smem, stream, a.pdl != 0, a,
                                 maps, total_quads, stages, q4 ? 1 : 0, q6 ? 1 : 0);
        }
    }
    if (a.x_mode != MV_X_PLAIN || a.xr_buf) return cudaErrorInvalidValue;   // prologues exist only in the streaming kernel
    uint32_t grid = (total_rows + 7) / 8;
    if (grid > (uint32_t)sms * 8) grid = (uint32_t)sms * 8;
    return launch_kernel(matvec_generic_kernel, dim3(grid), dim3(256), 0, stream, a.pdl != 0, a, total_rows);
}

} // namespace flb
