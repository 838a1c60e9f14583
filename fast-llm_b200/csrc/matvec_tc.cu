// k-quant dequantize-matvec for single-token decode, tensor-core form (replaces the
// reference's warp-per-row gdot_q4_K / gdot_q6_K, src/runtime/kernels_gpu.h:65-205,
// and the STREAM_DOT branch of exec_task_block, src/runtime/gpu_exec.cu:64-140).
//
// HBM-bound by design: every packed weight byte crosses HBM -> shared memory once,
// as tiled TMA boxes issued by a producer warp into a CTA-wide ring and completed on
// mbarriers. What this kernel changes against the dp4a streaming kernel (matvec.cu) is
// the arithmetic: there the consume loop was bound by instruction issue (about 2.7
// instructions per weight, the integer dot products at half rate). Here
//   * a unit of work is 16 rows x all columns; a stage is the same 8-super-block
//     column segment (2048 columns) of the unit's 16 rows, one box per stage;
//     consumer warp w of a group owns super-block w of the segment for all 16 rows;
//   * the products run on the tensor cores through mma.sync, lane (g, t) holding rows
//     g and g + 8 and the k-slots of lane column t. Column n of the B operand is
//     non-zero only for the k-slots of lane column t = n / 2, so that the accumulator
//     a lane reads back, C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1], is the dot
//     product of exactly the weights the lane unpacked with their activations: every
//     lane column accumulates its own sub-block, the sub-block scales / mins are
//     applied once per super-block in f32, and no shuffle is needed until a row is
//     complete;
//   * integer forms (the default for Q4_K and Q6_K; q4k_block_i8, q6k_block_i8): the
//     quants go in as they are, as unsigned 8-bit operands of m16n8k32 (a masked word
//     is four weights: one logic operation per four weights for Q4_K), the activation
//     as fixed point per 32-column sub-block, x = 2^e n with |n| < 2^30, cut into four
//     signed 8-bit digit planes that are the two B columns of a lane column in two
//     instructions. Products and sums are exact integers; one huge element costs the
//     other 31 of its sub-block at most the digits it pushes out of 30 bits;
//   * f16 forms (FLB_TC_I8=0, and every launch that holds a Q8_0 tensor): the quants
//     become f16 values with two logic operations per PAIR of weights (the quant lands
//     in the mantissa of a constant that an exact f16 subtraction takes off again), the
//     activation per 256-column block as x = 2^e (hi + lo) with hi, lo f16: 22 bits;
//   * sums are taken in a fixed order: results are reproducible run to run;
//   * a unit's partial row sums (one per warp) are added in warp order by a finalizer
//     warp, which also applies the fused epilogues (1/rms, residual, accumulate,
//     SiLU(gate) * up).
// Fused prologues as in the dp4a kernel: plain x, RMSNorm(x) * w, SiLU(x) * x2.
// The kernel is instantiated once per format set of a decode launch (template F) beside
// the form that decides everything at run time: see matvec_tc_kernel.
#include "common.cuh"
#include "kernels.h"

#include <cuda.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace flb {

namespace {

constexpr int kCW = 8;                          // consumer warps per group (one per super-block of a segment)
constexpr uint32_t kSeg4 = 8 * 144, kSeg6 = 8 * 210, kSeg8 = 64 * 34;
// A stage of Q4_K / Q6_K rows arrives as ONE tiled TMA box (16 rows x the segment): one bulk copy per row was
// measured to cost the TMA unit about 130 cycles each, which capped the stream at 2.6 TB/s. The row pitch in
// shared memory is therefore the segment's own size.
// Q6_K: 1680 bytes (105 x 16: odd), which with the per-t rotation of the word order makes the 32-bit loads
// conflict free. Q4_K: 1152 = 9 x 128 bytes: plain, the block headers of 8 rows would collide 8-way and the
// quants 2-way (measured 2.2 x the shared-memory wavefronts). The rows are therefore fetched as lines of 128 bytes
// with the 128-byte swizzle (tensor_map_lines_swz), which spreads the same 16-byte chunk of 8 consecutive rows
// over 8 bank groups; the consumer addresses chunk c of line l at l * 128 + ((c ^ (l & 7)) << 4). Rows whose
// pitch in memory is not a multiple of 128 bytes (columns not a multiple of 2048) fall back to the plain box.
// Q8_0 (a segment is wider than a box may be): one bulk copy per row, pitch + 16 (548 words = 4 mod 32).
constexpr uint32_t kPitch4 = kSeg4, kPitch6 = kSeg6, kPitch8 = kSeg8 + 16;
// ring slots are multiples of 1024 bytes: the swizzle pattern of a Q4_K stage is tied to the address
constexpr uint32_t slot_round(uint32_t b) { return (b + 1023u) & ~1023u; }
constexpr uint32_t kSlot4 = slot_round(16 * kPitch4), kSlot6 = slot_round(16 * kPitch6), kSlot8 = slot_round(16 * kPitch8);
// 256-column blocks a half-warp of the prologue converts (bounds the column count: see matvec_tc_eligible)
__host__ __device__ constexpr int max_blk_per_half_warp(int groups) { return groups == 1 ? 4 : 2; }

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
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t a) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Tiled TMA loads into shared memory (2-D: x counts 8-byte elements, a multiple of 2; 3-D: lines of 128 bytes).
__device__ __forceinline__ void tma_box2(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_box3(uint32_t dst, const CUtensorMap *map, uint32_t line, uint32_t row, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(0), "r"(line), "r"(row), "r"(smem_u32(bar))
        : "memory");
}
// The same with an L2 eviction policy for the lines the copy touches (the weights pass through L2 once).
__device__ __forceinline__ void tma_box2_hint(uint32_t dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void tma_box3_hint(uint32_t dst, const CUtensorMap *map, uint32_t line, uint32_t row, uint64_t *bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
        "l"(map), "r"(0), "r"(line), "r"(row), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Read-only 16-byte load whose line is kept in L2 in preference to others (small tensors every launch reads again)
__device__ __forceinline__ float4 ldg_keep(const float4 *p, uint64_t pol) {
    float4 v;
    asm volatile("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(pol));
    return v;
}
// All threads of the prologue (every warp but the producer) meet here.
__device__ __forceinline__ void prologue_barrier(uint32_t nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col). Lane (g, t): a0 / a1 = rows g / g + 8, k-slots 4t..4t+3;
// a2 / a3 = the same rows, k-slots 16+4t..; b0 / b1 = column g, the same two k-slot runs; c as for the f16 form.
__device__ __forceinline__ void imma16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (a & b) | c in one instruction; b and c are constants the compiler keeps in registers
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// h - off for both halves (exact: the operands are small integers)
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t h, __half2 off) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), off);
    return *reinterpret_cast<const uint32_t *>(&r);
}
// The common case of a wait: the phase is already complete. The bounded polling loop stays out of line.
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, uint32_t *status) {
    return mbar_wait_bounded(bar, parity, status);
}
// The form the consumer loops use: no exit out of the loop. `dead` (warp-uniform) is set when a wait ran out;
// from then on the warp waits for nothing any more (its results are void, the status word says so) and the
// launch still ends.
__device__ __forceinline__ void mbar_wait_or_die(uint64_t *bar, uint32_t parity, uint32_t *status, bool &dead) {
    if (dead || mbar_try_wait(bar, parity)) return;
    dead = !mbar_wait_slow(bar, parity, status);
}
// byte K of w as a float without the conversion pipe (the byte under 0x4B000000 is 2^23 + byte)
template <int K>
__device__ __forceinline__ float u8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K)) - 8388608.0f;
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// ---- the activation in shared memory ---------------------------------------------------------
// Per 256-column block 1024 bytes per layout: f16 hi and lo parts in the order the B operand wants.
// "lane8" = 2 t + h is the slot of the lane (g = 2 t + h, t) that feeds column 2 t + h of B.
// Q4_K layout: for word j (0..7) of a 32-byte chunk: 128 bytes = 8 lane8 x 16; a lane8's 16 bytes are the
//   B registers (b0, b1) of the low-nibble MMA (columns 64 c + 4 j + {0, 2, 1, 3}) and of the high-nibble
//   MMA (columns 64 c + 32 + 4 j + {0, 2, 1, 3}), c = t.
// Q6_K layout: for step s (0..3; the lane column t works on word (s + t) & 3 of its 16-byte runs):
//   256 bytes = 2 x (8 lane8 x 16); a lane8's 2 x 16 bytes are (b0, b1) of the four 32-column groups
//   gq = 0..3 (columns 128 hf + 32 gq + 16 hq + 4 j + {0, 2, 1, 3}, t = 2 hf + hq).
__device__ __forceinline__ uint32_t x4_off(uint32_t j, uint32_t lane8, uint32_t sub) { return j * 128u + lane8 * 16u + sub * 8u; }
__device__ __forceinline__ uint32_t x6_off(uint32_t s, uint32_t lane8, uint32_t gq) {
    return s * 256u + (gq >> 1) * 128u + lane8 * 16u + (gq & 1u) * 8u;
}

struct TcTensor {
    CUtensorMap map;               // Q4_K / Q6_K: the tiled view a stage's box is cut from
    const uint8_t *w;
    float *y;
    const float *resid;
    uint32_t rows, pitch, unit0;   // unit0: index of the tensor's first unit in the launch
    int fmt, swz;                  // swz: Q4_K rows fetched as swizzled 128-byte lines
};

// One matvec of a launch. A launch is a sequence of up to four phases that depend on one another
// (phase p + 1 reads as its activation what phase p wrote): O -> gate|up -> down -> next Q/K/V.
struct TcPhase {
    TcTensor t[3];
    int n_tensors;
    const float *x, *x2, *wnorm;
    float eps;
    uint32_t cols;
    int x_mode, accumulate, swiglu;
    uint32_t total_units;
    int use_q4, use_q6;
    int q4_i8;                     // the phase runs on the integer forms (q4k_block_i8, q6k_block_i8): no Q8_0 tensor in it
    float *xn_out;
};

// Grid-wide barrier between the phases of a launch: an arrival counter and a generation number in
// global memory; the counter returns to zero by itself, so the state serves every launch.
struct GridBar { uint32_t count, gen; };

struct TcArgs {
    TcPhase ph[4];
    int n_phases;
    uint32_t nslots, slot_bytes, ring_off;   // ring_off: bytes from the start of shared memory to the ring
    uint32_t *status;
    int l2_hints;                            // weights evict-first, norm weights evict-last in L2
    GridBar *bar;                            // n_phases > 1
    unsigned long long *trace;
};

struct TcSmem {
    uint64_t *full, *empty;        // [nslots]
    uint64_t *red_full, *red_empty;   // [2]
    float *red;                    // [2][groups * 8][16]
    float *ssq;                    // per-warp sums of squares of the prologue
    uint8_t *zero;                 // 16 zero bytes (the B operand of lanes that feed no column)
    float *xs;                     // [nblk] block scale 2^e
    float *xs8;                    // integer form, Q4_K: [nblk][8] sub-block scales 2^e (odd sub-blocks: 2^e / 16)
    float *xsp;                    // integer form, Q6_K: [nblk][8] sub-block scales 2^e
    float *s16;                    // integer form, Q6_K: [nblk][4 lane columns][4 groups] sums of the 16-column groups
    float *s4;                     // [nblk][8] sums of the 32-column sub-blocks, in units of the block scale (integer form: as they are)
    uint8_t *x4, *x6;              // [nblk][1024]
    uint8_t *ring;
};

// Shared memory in front of the ring: barriers and reduction buffers (the same for every phase), then
// the activation of the current phase. The ring starts at the same offset in every phase.
__host__ __device__ inline size_t tc_head_bytes(uint32_t nslots, int groups) {
    size_t n = (size_t)nslots * 16 + 32;                  // barriers
    n += (size_t)2 * groups * kCW * 16 * 4;              // red
    n += 36 * 4 + 16;                                     // ssq, 16 zero bytes
    return (n + 15) & ~(size_t)15;
}
__host__ __device__ inline size_t tc_x_bytes(uint32_t cols, bool q4, bool q6, bool i8) {
    const size_t nblk = cols / 256;
    size_t n = (nblk * 4 + 15) & ~(size_t)15;             // xs
    if (i8 && q4) n += nblk * 32;                         // xs8
    if (i8 && q6) n += nblk * 32 + nblk * 64;             // xsp, s16
    if (q4) n += nblk * 32 + nblk * 1024;
    if (q6) n += nblk * 1024;
    return n;
}

template <int G>
__device__ __forceinline__ TcSmem tc_carve(uint8_t *base, uint32_t cols, bool q4, bool q6, bool i8, uint32_t nslots, uint32_t ring_off) {
    TcSmem s;
    const uint32_t nblk = cols / 256;
    uint8_t *p = base;
    s.full = (uint64_t *)p; p += nslots * 8;
    s.empty = (uint64_t *)p; p += nslots * 8;
    s.red_full = (uint64_t *)p; p += 16;
    s.red_empty = (uint64_t *)p; p += 16;
    s.red = (float *)p; p += 2 * G * kCW * 16 * 4;
    s.ssq = (float *)p; p += 36 * 4;
    s.zero = p;
    p = base + tc_head_bytes(nslots, G);
    s.xs = (float *)p; p += (nblk * 4 + 15) & ~15u;
    s.xs8 = s.xsp = s.s16 = nullptr;
    if (i8 && q4) { s.xs8 = (float *)p; p += nblk * 32; }
    if (i8 && q6) { s.xsp = (float *)p; p += nblk * 32; s.s16 = (float *)p; p += nblk * 64; }
    s.s4 = nullptr; s.x4 = s.x6 = nullptr;
    if (q4) { s.s4 = (float *)p; p += nblk * 32; s.x4 = p; p += (size_t)nblk * 1024; }
    if (q6) { s.x6 = p; p += (size_t)nblk * 1024; }
    s.ring = base + ring_off;
    return s;
}

// Which tensor and which first row a unit covers (non-SwiGLU launches).
__device__ __forceinline__ int unit_tensor(const TcPhase &a, uint32_t u) {
    int ti = 0;
#pragma unroll 1
    for (; ti < a.n_tensors - 1; ++ti)
        if (u < a.t[ti + 1].unit0) break;
    return ti;
}

// ---- per-super-block math ------------------------------------------------------------------

// Q4_K: rows g (r0) and g + 8 (r1) of one super-block; chunk c = t. Returns the two rows' contributions in
// units of the block's activation scale. All shared-memory loads of the block are issued first (they are
// volatile asm statements, which the compiler keeps in program order), so that their latency overlaps.
// xaddr: this lane's 16-byte B slot of word 0 (lanes that feed no column of B point at 16 zero bytes and
// use a stride of 0).
// Byte offset o of a row as the stage holds it: as it is, or in the swizzled 128-byte lines (see kPitch4).
__device__ __forceinline__ uint32_t q4_row_off(uint32_t o, uint32_t g, bool swz) {
    return swz ? (o & ~127u) + ((((o >> 4) ^ (g + (o >> 7))) & 7u) << 4) : o;
}
// r0: row g of the stage; row g + 8 is 8 * kPitch4 further (the same swizzle: 72 lines further). oh / oa / ob: offsets
// of the block's header and of the two 16-byte halves of chunk t in the row (q4_row_off).
__device__ __forceinline__ void q4k_block(uint32_t r0, uint32_t oh, uint32_t oa, uint32_t ob, uint32_t t, uint32_t xaddr,
                                          uint32_t xstride, float2 sx, float &out0, float &out1) {
    const uint32_t r1 = r0 + 8 * kPitch4;
    const uint4 wa0 = lds128(r0 + oa), wa1 = lds128(r1 + oa);
    uint4 bx[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) bx[j] = lds128(xaddr + j * xstride);
    const uint4 wb0 = lds128(r0 + ob), wb1 = lds128(r1 + ob);
#pragma unroll
    for (int j = 4; j < 8; ++j) bx[j] = lds128(xaddr + j * xstride);
    const uint4 h0 = lds128(r0 + oh), h1 = lds128(r1 + oh);
    // two accumulator chains per nibble kind: a chain of eight dependent tensor-core instructions measured 25 % slower
    float cL[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, cH[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    // A quant lands in the mantissa of a constant: bits 0..3 under 0x6400 give 1024 + q, bits 4..7 under 0x5400 give
    // 64 + q; the constant is taken off again exactly (f16 subtraction on the other pipe). Bytes 1 and 3 come
    // down by one shift. Five logic operations and four subtractions per 8 weights.
    const uint32_t ML = 0x000F000Fu, KL = 0x64006400u, MH = 0x00F000F0u, KH = 0x54005400u;
    const __half2 oL = __floats2half2_rn(1024.f, 1024.f), oH = __floats2half2_rn(64.f, 64.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t W0 = j < 4 ? word_of(wa0, j) : word_of(wb0, j - 4);
        const uint32_t W1 = j < 4 ? word_of(wa1, j) : word_of(wb1, j - 4);
        const uint32_t V0 = W0 >> 8, V1 = W1 >> 8;
        // low nibbles (sub-block 2t): bytes 0, 2 -> k-slots 2t, 2t+1; bytes 1, 3 -> k-slots 2t+8, 2t+9
        mma16816(cL[j & 1], hsub2_u32(and_or(W0, ML, KL), oL), hsub2_u32(and_or(W1, ML, KL), oL),
                 hsub2_u32(and_or(V0, ML, KL), oL), hsub2_u32(and_or(V1, ML, KL), oL), bx[j].x, bx[j].y);
        // high nibbles (sub-block 2t+1)
        mma16816(cH[j & 1], hsub2_u32(and_or(W0, MH, KH), oH), hsub2_u32(and_or(W1, MH, KH), oH),
                 hsub2_u32(and_or(V0, MH, KH), oH), hsub2_u32(and_or(V1, MH, KH), oH), bx[j].z, bx[j].w);
    }
    // 6-bit scales / mins of sub-blocks 2t, 2t+1 (packing: fl_q4k_scale_min, src/runtime/quants.h:121-129). One form
    // for both kinds of sub-block, the lane's shifts and masks being loop constants: sub-blocks 0..3 are the low six
    // bits of bytes 0..3 (4..7 for the mins); sub-blocks 4..7 a nibble of bytes 8..11 under the top two bits of those.
    const uint32_t sh = 16u * (t & 1u);
    const uint32_t shA = t >= 2 ? sh + 2u : sh, mA = t >= 2 ? 0x3030u : 0x3F3Fu, mE = t >= 2 ? 0x0F0Fu : 0u;
    const float s0 = sx.x, s1 = sx.y;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 hdr = r ? h1 : h0;
        const uint32_t sc = ((hdr.y >> shA) & mA) | ((hdr.w >> sh) & mE);
        const uint32_t mn = ((hdr.z >> shA) & mA) | ((hdr.w >> (sh + 4u)) & mE);
        const float d = h2f_bits((uint16_t)(hdr.x & 0xFFFFu)), dmin = h2f_bits((uint16_t)(hdr.x >> 16));
        const float tl = (cL[0][2 * r] + cL[1][2 * r]) + (cL[0][2 * r + 1] + cL[1][2 * r + 1]);
        const float th = (cH[0][2 * r] + cH[1][2 * r]) + (cH[0][2 * r + 1] + cH[1][2 * r + 1]);
        const float q = u8f<0>(sc) * tl + u8f<1>(sc) * th;
        const float m = u8f<0>(mn) * s0 + u8f<1>(mn) * s1;
        (r ? out1 : out0) = d * q - dmin * m;
    }
}

// Q4_K, integer form (the default for Q4_K). The nibbles are used as they are: word & 0x0F0F0F0F is four unsigned
// 8-bit quants of sub-block 2t, word & 0xF0F0F0F0 four quants of sub-block 2t+1 times 16 (the 1/16 sits in that
// sub-block's activation scale): one logic operation per four weights, and the products and sums are exact. The
// activation is fixed point per 32-column sub-block, x = 2^e * n with |n| < 2^30, n cut into four signed 8-bit digits
// n = D0 2^24 + D1 2^16 + D2 2^8 + D3; digit planes (D0, D1) are the two columns of B that belong to the lane column
// in the first instruction of a pair, (D2, D3) in the second, so that a lane reads back its own rows' four plane
// sums: c[0] = {D0, D1 of row g; D0, D1 of row g + 8}, c[1] the same for D2, D3. Word pair (2m, 2m+1) of the chunk
// is one instruction's k range (8 weights per row). sx: sums of the activation over sub-blocks 2t, 2t+1; xs2: their
// scales. Results come back in final units (no block scale left to apply).
__device__ __forceinline__ void q4k_block_i8(uint32_t r0, uint32_t oh, uint32_t oa, uint32_t ob, uint32_t t, uint32_t xaddr,
                                             uint32_t xstride, float2 sx, float2 xs2, float &out0, float &out1) {
    const uint32_t r1 = r0 + 8 * kPitch4;
    const uint4 wa0 = lds128(r0 + oa), wa1 = lds128(r1 + oa);
    uint4 bx[8];   // slot 2m + h: (b0, b1) of planes 0, 1 and of planes 2, 3 for word pair m, nibble kind h
#pragma unroll
    for (int j = 0; j < 4; ++j) bx[j] = lds128(xaddr + j * xstride);
    const uint4 wb0 = lds128(r0 + ob), wb1 = lds128(r1 + ob);
#pragma unroll
    for (int j = 4; j < 8; ++j) bx[j] = lds128(xaddr + j * xstride);
    const uint4 h0 = lds128(r0 + oh), h1 = lds128(r1 + oh);
    int cL[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, cH[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    const uint32_t ML = 0x0F0F0F0Fu, MH = 0xF0F0F0F0u;
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t A0 = m < 2 ? word_of(wa0, 2 * m) : word_of(wb0, 2 * m - 4), B0 = m < 2 ? word_of(wa0, 2 * m + 1) : word_of(wb0, 2 * m - 3);
        const uint32_t A1 = m < 2 ? word_of(wa1, 2 * m) : word_of(wb1, 2 * m - 4), B1 = m < 2 ? word_of(wa1, 2 * m + 1) : word_of(wb1, 2 * m - 3);
        const uint32_t l0 = A0 & ML, l1 = A1 & ML, l2 = B0 & ML, l3 = B1 & ML;
        const uint32_t g0 = A0 & MH, g1 = A1 & MH, g2 = B0 & MH, g3 = B1 & MH;
        imma16832(cL[0], l0, l1, l2, l3, bx[2 * m].x, bx[2 * m].y);
        imma16832(cH[0], g0, g1, g2, g3, bx[2 * m + 1].x, bx[2 * m + 1].y);
        imma16832(cL[1], l0, l1, l2, l3, bx[2 * m].z, bx[2 * m].w);
        imma16832(cH[1], g0, g1, g2, g3, bx[2 * m + 1].z, bx[2 * m + 1].w);
    }
    // 6-bit scales / mins of sub-blocks 2t, 2t+1 (fl_q4k_scale_min, src/runtime/quants.h:121-129), as in q4k_block
    const uint32_t sh = 16u * (t & 1u);
    const uint32_t shA = t >= 2 ? sh + 2u : sh, mA = t >= 2 ? 0x3030u : 0x3F3Fu, mE = t >= 2 ? 0x0F0Fu : 0u;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 hdr = r ? h1 : h0;
        const uint32_t sc = ((hdr.y >> shA) & mA) | ((hdr.w >> sh) & mE);
        const uint32_t mn = ((hdr.z >> shA) & mA) | ((hdr.w >> (sh + 4u)) & mE);
        const float d = h2f_bits((uint16_t)(hdr.x & 0xFFFFu)), dmin = h2f_bits((uint16_t)(hdr.x >> 16));
        // the four plane sums of a sub-block as one number: two exact integer steps (|.| < 2^28), then f32
        const float tl = fmaf((float)(cL[0][2 * r] * 256 + cL[0][2 * r + 1]), 65536.f, (float)(cL[1][2 * r] * 256 + cL[1][2 * r + 1]));
        const float th = fmaf((float)(cH[0][2 * r] * 256 + cH[0][2 * r + 1]), 65536.f, (float)(cH[1][2 * r] * 256 + cH[1][2 * r + 1]));
        const float q = u8f<0>(sc) * (xs2.x * tl) + u8f<1>(sc) * (xs2.y * th);   // the sums in the activation's units first
        const float mm = u8f<0>(mn) * sx.x + u8f<1>(mn) * sx.y;
        (r ? out1 : out0) = d * q - dmin * mm;
    }
}

// Q6_K: lane column t = 2 hf + hq works on the 16-byte runs ql[64 hf + 16 hq ..], ql[64 hf + 32 + 16 hq ..],
// qh[32 hf + 16 hq ..] of rows g and g + 8 (q = nibble | two high bits << 4, value d * sc * (q - 32);
// fl_dot_row_q6_K, src/runtime/quants.h:194-230). ODD: the block starts 2 bytes past a word boundary
// (r0, r1 are then the word-aligned addresses 2 bytes in front of it). Loads first, as for Q4_K.
template <bool ODD>
__device__ __forceinline__ void q6k_block(uint32_t r0, uint32_t r1, uint32_t t, uint32_t xaddr, uint32_t xstride, float &out0,
                                          float &out1) {
    const uint32_t hf = t >> 1, hq = t & 1u;
    const uint32_t oa = 64 * hf + 16 * hq, oh = 128 + 32 * hf + 16 * hq;   // byte offsets in the block
    uint32_t wa[2][4], wb[2][4], wh[2][4];
    uint4 bA[4], bB[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t js = ((uint32_t)s + t) & 3u;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t rb = r ? r1 : r0;
            if (ODD) {
                const uint32_t a0 = lds32(rb + oa + 4 * js), a1 = lds32(rb + oa + 4 * js + 4);
                const uint32_t b0 = lds32(rb + oa + 32 + 4 * js), b1 = lds32(rb + oa + 36 + 4 * js);
                const uint32_t h0 = lds32(rb + oh + 4 * js), h1 = lds32(rb + oh + 4 * js + 4);
                wa[r][s] = __byte_perm(a0, a1, 0x5432u);
                wb[r][s] = __byte_perm(b0, b1, 0x5432u);
                wh[r][s] = __byte_perm(h0, h1, 0x5432u);
            } else {
                wa[r][s] = lds32(rb + oa + 4 * js);
                wb[r][s] = lds32(rb + oa + 32 + 4 * js);
                wh[r][s] = lds32(rb + oh + 4 * js);
            }
        }
        bA[s] = lds128(xaddr + s * 2 * xstride);
        bB[s] = lds128(xaddr + s * 2 * xstride + xstride);
    }
    // scales: int8 sc[8 hf + 2 gq + hq]; d at byte 208
    uint32_t sw[2];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t rb = r ? r1 : r0;
        const uint32_t ps = rb + 192 + 8 * hf;
        uint32_t lo, hi;
        if (ODD) {
            const uint32_t s0 = lds32(ps), s1 = lds32(ps + 4), s2 = lds32(ps + 8);
            lo = __byte_perm(s0, s1, 0x5432u);
            hi = __byte_perm(s1, s2, 0x5432u);
        } else {
            lo = lds32(ps);
            hi = lds32(ps + 4);
        }
        sw[r] = __byte_perm(lo, hi, hq ? 0x7531u : 0x6420u) ^ 0x80808080u;   // s + 128 as unsigned bytes
        dd[r] = h2f_bits((uint16_t)lds16(rb + (ODD ? 2u : 0u) + 208));
    }
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) c[i][k] = 0.f;
    const __half2 off = __floats2half2_rn(1056.f, 1056.f);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        uint32_t a_[2][8];   // per row: A registers (k-slots 2t.. , 2t+8..) of the four groups
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t a = wa[r][s], b = wb[r][s], h = wh[r][s];
            uint32_t q[4];
            q[0] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
            q[1] = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
            q[2] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
            q[3] = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                // bytes 0, 2 / 1, 3 under 0x64: f16 1024 + q; minus 1056 is q - 32, exact
                const uint32_t e02 = __byte_perm(q[gq], 0x64646464u, 0x4240u), e13 = __byte_perm(q[gq], 0x64646464u, 0x4341u);
                __half2 h02 = *reinterpret_cast<const __half2 *>(&e02), h13 = *reinterpret_cast<const __half2 *>(&e13);
                h02 = __hsub2(h02, off);
                h13 = __hsub2(h13, off);
                a_[r][2 * gq] = *reinterpret_cast<const uint32_t *>(&h02);
                a_[r][2 * gq + 1] = *reinterpret_cast<const uint32_t *>(&h13);
            }
        }
        mma16816(c[0], a_[0][0], a_[1][0], a_[0][1], a_[1][1], bA[s].x, bA[s].y);
        mma16816(c[1], a_[0][2], a_[1][2], a_[0][3], a_[1][3], bA[s].z, bA[s].w);
        mma16816(c[2], a_[0][4], a_[1][4], a_[0][5], a_[1][5], bB[s].x, bB[s].y);
        mma16816(c[3], a_[0][6], a_[1][6], a_[0][7], a_[1][7], bB[s].z, bB[s].w);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float v = (u8f<0>(sw[r]) - 128.f) * (c[0][2 * r] + c[0][2 * r + 1]);
        v += (u8f<1>(sw[r]) - 128.f) * (c[1][2 * r] + c[1][2 * r + 1]);
        v += (u8f<2>(sw[r]) - 128.f) * (c[2][2 * r] + c[2][2 * r + 1]);
        v += (u8f<3>(sw[r]) - 128.f) * (c[3][2 * r] + c[3][2 * r + 1]);
        (r ? out1 : out0) = dd[r] * v;
    }
}

// byte K of w, which holds s + 128, as the float s (the byte under 0x4B000000 is 2^23 + 128 + s)
template <int K>
__device__ __forceinline__ float s8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u + K)) - 8388736.f;
}

// Q6_K, integer form: the same loads and the same assembly of the 6-bit quants as q6k_block, but the four bytes
// q (0 .. 63) of a word are used as they are, as unsigned 8-bit operands of mma.sync m16n8k32; the - 32 of the format
// comes off through the activation's group sums (sum (q - 32) x = sum q x - 32 sum x). Steps (2 sp, 2 sp + 1) of group gq
// are one instruction's k range; the activation is the fixed-point form of q4k_block_i8 (scale per 32 columns: the
// lane column's groups gq = 0..3 have their own sub-blocks), digit planes (D0, D1) in the first instruction of a pair,
// (D2, D3) in the second. xs4: the scales of the lane's four groups; sx4: the sums of the activation over them.
template <bool ODD>
__device__ __forceinline__ void q6k_block_i8(uint32_t r0, uint32_t r1, uint32_t t, uint32_t xaddr, uint32_t xstride, float4 xs4,
                                             float4 sx4, float &out0, float &out1) {
    const uint32_t hf = t >> 1, hq = t & 1u;
    const uint32_t oa = 64 * hf + 16 * hq, oh = 128 + 32 * hf + 16 * hq;   // byte offsets in the block
    uint32_t wa[2][4], wb[2][4], wh[2][4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const uint32_t js = ((uint32_t)s + t) & 3u;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t rb = r ? r1 : r0;
            if (ODD) {
                const uint32_t a0 = lds32(rb + oa + 4 * js), a1 = lds32(rb + oa + 4 * js + 4);
                const uint32_t b0 = lds32(rb + oa + 32 + 4 * js), b1 = lds32(rb + oa + 36 + 4 * js);
                const uint32_t h0 = lds32(rb + oh + 4 * js), h1 = lds32(rb + oh + 4 * js + 4);
                wa[r][s] = __byte_perm(a0, a1, 0x5432u);
                wb[r][s] = __byte_perm(b0, b1, 0x5432u);
                wh[r][s] = __byte_perm(h0, h1, 0x5432u);
            } else {
                wa[r][s] = lds32(rb + oa + 4 * js);
                wb[r][s] = lds32(rb + oa + 32 + 4 * js);
                wh[r][s] = lds32(rb + oh + 4 * js);
            }
        }
    }
    uint4 bx[8];   // slot 4 sp + gq
#pragma unroll
    for (int q = 0; q < 8; ++q) bx[q] = lds128(xaddr + q * xstride);
    // scales: int8 sc[8 hf + 2 gq + hq]; d at byte 208
    uint32_t sw[2];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t rb = r ? r1 : r0;
        const uint32_t ps = rb + 192 + 8 * hf;
        uint32_t lo, hi;
        if (ODD) {
            const uint32_t s0 = lds32(ps), s1 = lds32(ps + 4), s2 = lds32(ps + 8);
            lo = __byte_perm(s0, s1, 0x5432u);
            hi = __byte_perm(s1, s2, 0x5432u);
        } else {
            lo = lds32(ps);
            hi = lds32(ps + 4);
        }
        sw[r] = __byte_perm(lo, hi, hq ? 0x7531u : 0x6420u) ^ 0x80808080u;   // s + 128 as unsigned bytes
        dd[r] = h2f_bits((uint16_t)lds16(rb + (ODD ? 2u : 0u) + 208));
    }
    const float xs_[4] = {xs4.x, xs4.y, xs4.z, xs4.w};
    const float m32[4] = {-32.f * sx4.x, -32.f * sx4.y, -32.f * sx4.z, -32.f * sx4.w};
    float v[2] = {0.f, 0.f};
#pragma unroll
    for (int gq = 0; gq < 4; ++gq) {
        uint32_t q[2][4];   // [row][step]
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t a = wa[r][s], b = wb[r][s], h = wh[r][s];
                q[r][s] = gq == 0   ? (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u)
                          : gq == 1 ? (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u)
                          : gq == 2 ? ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u)
                                    : ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
            }
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
        imma16832(c0, q[0][0], q[1][0], q[0][1], q[1][1], bx[gq].x, bx[gq].y);
        imma16832(c1, q[0][0], q[1][0], q[0][1], q[1][1], bx[gq].z, bx[gq].w);
        imma16832(c0, q[0][2], q[1][2], q[0][3], q[1][3], bx[4 + gq].x, bx[4 + gq].y);
        imma16832(c1, q[0][2], q[1][2], q[0][3], q[1][3], bx[4 + gq].z, bx[4 + gq].w);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float f = fmaf((float)(c0[2 * r] * 256 + c0[2 * r + 1]), 65536.f, (float)(c1[2 * r] * 256 + c1[2 * r + 1]));
            const float sc = gq == 0 ? s8f<0>(sw[r]) : gq == 1 ? s8f<1>(sw[r]) : gq == 2 ? s8f<2>(sw[r]) : s8f<3>(sw[r]);
            v[r] = fmaf(sc, fmaf(xs_[gq], f, m32[gq]), v[r]);
        }
    }
    out0 = dd[0] * v[0];
    out1 = dd[1] * v[1];
}

// Q8_0 (blocks of 32 int8 with one f16 d, 34 bytes; fl_dot_row_q8_0, src/runtime/quants.h:132-142): the 256
// columns of warp w are blocks 8 w .. 8 w + 7 of the segment; lane column t takes blocks 2 t and 2 t + 1, 68 bytes
// from `r0` / `r1` (4-byte aligned). The first block's quants start 2 bytes into a word and are realigned with
// byte permutes; the second block's are aligned. An int8 s becomes f16 through (s ^ 0x80) under 0x64: 1024 + 128 + s,
// minus 1152, exact. The activation uses the Q4_K layout (64 consecutive columns per lane column, words of 4).
__device__ __forceinline__ void q8_0_block(uint32_t r0, uint32_t r1, uint32_t xaddr, uint32_t xstride, float &out0, float &out1) {
    uint32_t w0[17], w1[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) { w0[i] = lds32(r0 + 4 * i); w1[i] = lds32(r1 + 4 * i); }
    uint4 bx[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) bx[j] = lds128(xaddr + j * xstride);
    float cA[2][4], cB[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int k = 0; k < 4; ++k) cA[i][k] = cB[i][k] = 0.f;
    const __half2 off = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t a0 = __byte_perm(w0[j], w0[j + 1], 0x5432u) ^ 0x80808080u, a1 = __byte_perm(w1[j], w1[j + 1], 0x5432u) ^ 0x80808080u;
        const uint32_t b0 = w0[9 + j] ^ 0x80808080u, b1 = w1[9 + j] ^ 0x80808080u;
        mma16816(cA[j & 1], hsub2_u32(__byte_perm(a0, 0x64646464u, 0x4240u), off), hsub2_u32(__byte_perm(a1, 0x64646464u, 0x4240u), off),
                 hsub2_u32(__byte_perm(a0, 0x64646464u, 0x4341u), off), hsub2_u32(__byte_perm(a1, 0x64646464u, 0x4341u), off), bx[j].x, bx[j].y);
        mma16816(cB[j & 1], hsub2_u32(__byte_perm(b0, 0x64646464u, 0x4240u), off), hsub2_u32(__byte_perm(b1, 0x64646464u, 0x4240u), off),
                 hsub2_u32(__byte_perm(b0, 0x64646464u, 0x4341u), off), hsub2_u32(__byte_perm(b1, 0x64646464u, 0x4341u), off), bx[j].z, bx[j].w);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t *w = r ? w1 : w0;
        const float dA = h2f_bits((uint16_t)(w[0] & 0xFFFFu)), dB = h2f_bits((uint16_t)(w[8] >> 16));
        const float ta = (cA[0][2 * r] + cA[1][2 * r]) + (cA[0][2 * r + 1] + cA[1][2 * r + 1]);
        const float tb = (cB[0][2 * r] + cB[1][2 * r]) + (cB[0][2 * r + 1] + cB[1][2 * r + 1]);
        (r ? out1 : out0) = dA * ta + dB * tb;
    }
}

// ---- grid barrier --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t atom_add_release_gpu(uint32_t *p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.add.release.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
// One thread per CTA. All CTAs of the launch are resident (one per SM, grid <= SM count; no kernel that
// could hold an SM depends on this one), so every arrival comes. The wait is bounded all the same: after
// about a second it records ST_WAIT_TIMEOUT and gives up.
__device__ __forceinline__ bool grid_barrier(GridBar *b, uint32_t nblocks, uint32_t *status) {
    const uint32_t gen = ld_acquire_gpu(&b->gen);          // cannot advance before this CTA has arrived
    const uint32_t old = atom_add_release_gpu(&b->count, 1u);
    if (old == nblocks - 1u) {
        b->count = 0u;                                     // ordered before the release below
        atom_add_release_gpu(&b->gen, 1u);
        return true;
    }
    if (ld_acquire_gpu(&b->gen) != gen) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 16; ++i)
            if (ld_acquire_gpu(&b->gen) != gen) return true;
        if (globaltimer_ns() - t0 > 1000000000ull) {
            atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
            return false;
        }
    }
}

// ---- the kernel ----------------------------------------------------------------------------
// Warps: G groups of 8 consumer warps (group i takes stages i, i + G, ...), then the producer warp,
// then the finalizer warp. A launch runs its phases one after the other with a grid-wide barrier in
// between; the producer does not take part in the barriers: the weights of the next phase are already
// streaming into the ring while the current phase drains and the next activation is built.
// F: 0 = every format and form, decided per phase at run time (f16 forms, Q8_0, several phases); 1 / 2 / 3 = one phase
// on the integer forms holding Q4_K tensors only / Q6_K only / both: what a decode step launches. The specialised
// instances carry only their own code (the whole kernel is some 7000 instructions, and a launch that has to fetch its
// path out of that from L2 starts later) and get their own register allocation.
// R: 256-column blocks a half-warp of the prologue converts (F != 0: 1 up to 34 blocks = 8704 columns, else 2; the
// specialised instances also leave out the SiLU prologue, the second copy of the activation and several phases).
template <int G, int F, int R>
__global__ void __launch_bounds__((G * kCW + 2) * 32) matvec_tc_kernel(const __grid_constant__ TcArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr uint32_t kConsumers = G * kCW;
    constexpr uint32_t kProducer = kConsumers, kFinal = kConsumers + 1;
    constexpr uint32_t kPrologueThreads = (kConsumers + 1) * 32;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t S = a.nslots;
    {
        const TcSmem sm = tc_carve<G>(smem_raw, 256, false, false, false, S, a.ring_off);
        if (tid == 0) {
            for (uint32_t s = 0; s < S; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], kCW); }
            for (int i = 0; i < 2; ++i) { mbar_init(&sm.red_full[i], kConsumers); mbar_init(&sm.red_empty[i], 1); }
            *reinterpret_cast<uint4 *>(sm.zero) = make_uint4(0u, 0u, 0u, 0u);
            fence_barrier_init();
            trace_min(a.trace, 0);
        }
    }
    __syncthreads();
    griddep_launch_dependents();
    const uint32_t ring = smem_u32(smem_raw) + a.ring_off;

    if (warp == kProducer) {
        // ---- producer: one bulk copy per row and stage; the weights do not depend on any activation ----
        const TcSmem sm = tc_carve<G>(smem_raw, 256, false, false, false, S, a.ring_off);
        uint32_t slot = 0, par = 1;   // a fresh barrier passes a wait on parity 1
        const uint64_t pol = a.l2_hints ? l2_policy_evict_first() : 0ull;
#pragma unroll 1
        for (int p = 0; p < a.n_phases; ++p) {
            const TcPhase &ph = a.ph[p];
            const uint32_t nblk = ph.cols / 256, nseg = (nblk + 7) / 8;
            const uint32_t my_units = blockIdx.x < ph.total_units ? (ph.total_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
            for (uint32_t k = 0; k < my_units; ++k) {
                const uint32_t u = blockIdx.x + k * gridDim.x;
                const uint8_t *src = nullptr;
                uint32_t pitch = 0, fmt;
                bool valid = false;
                if (ph.swiglu) {
                    const TcTensor &t = ph.t[(lane >> 3) & 1u];
                    const uint32_t row = 8 * u + (lane & 7u);
                    fmt = (uint32_t)ph.t[0].fmt;
                    valid = lane < 16 && row < t.rows;
                    pitch = t.pitch;
                    src = t.w + (size_t)row * t.pitch;
                } else {
                    const TcTensor &t = ph.t[unit_tensor(ph, u)];
                    const uint32_t row = 16 * (u - t.unit0) + lane;
                    fmt = (uint32_t)t.fmt;
                    valid = lane < 16 && row < t.rows;
                    pitch = t.pitch;
                    src = t.w + (size_t)row * t.pitch;
                }
                const uint32_t segb = fmt == FMT_Q4_K ? kSeg4 : fmt == FMT_Q6_K ? kSeg6 : kSeg8;
                const uint32_t rp = fmt == FMT_Q4_K ? kPitch4 : fmt == FMT_Q6_K ? kPitch6 : kPitch8;
                const uint32_t nvalid = __popc(__ballot_sync(0xffffffffu, valid));
                const int ti = ph.swiglu ? 0 : unit_tensor(ph, u);
                const uint32_t row0 = ph.swiglu ? 8 * u : 16 * (u - ph.t[ti].unit0);
                for (uint32_t seg = 0; seg < nseg; ++seg) {
                    const uint32_t off = seg * segb;
                    if (!mbar_wait_bounded(&sm.empty[slot], par, a.status)) return;
                    fence_proxy_async_smem();
                    const uint32_t dst = ring + slot * a.slot_bytes;
                    if (F == 0 && fmt == FMT_Q8_0) {   // one bulk copy per row
                        const uint32_t bytes = min(segb, pitch - off);   // pitch and off are multiples of 16
                        if (lane == 0) mbar_arrive_expect_tx(&sm.full[slot], nvalid * bytes);
                        __syncwarp();
                        if (valid) bulk_g2s_addr(dst + lane * rp, src + off, bytes, &sm.full[slot]);
                    } else if (lane == 0) {
                        // one box of 16 rows x the segment (SwiGLU: 8 gate rows, then 8 up rows); rows past the end of the
                        // tensor and blocks past the end of a row arrive as zeros and count as bytes all the same
                        mbar_arrive_expect_tx(&sm.full[slot], 16 * segb);
                        const TcTensor &t0 = ph.t[ti];
                        if (t0.swz && a.l2_hints) {
                            tma_box3_hint(dst, &t0.map, off / 128, row0, &sm.full[slot], pol);
                            if (ph.swiglu) tma_box3_hint(dst + 8 * segb, &ph.t[1].map, off / 128, row0, &sm.full[slot], pol);
                        } else if (t0.swz) {
                            tma_box3(dst, &t0.map, off / 128, row0, &sm.full[slot]);
                            if (ph.swiglu) tma_box3(dst + 8 * segb, &ph.t[1].map, off / 128, row0, &sm.full[slot]);
                        } else if (a.l2_hints) {
                            tma_box2_hint(dst, &t0.map, off / 8, row0, &sm.full[slot], pol);
                            if (ph.swiglu) tma_box2_hint(dst + 8 * segb, &ph.t[1].map, off / 8, row0, &sm.full[slot], pol);
                        } else {
                            tma_box2(dst, &t0.map, off / 8, row0, &sm.full[slot]);
                            if (ph.swiglu) tma_box2(dst + 8 * segb, &ph.t[1].map, off / 8, row0, &sm.full[slot]);
                        }
                    }
                    if (++slot == S) { slot = 0; par ^= 1u; }
                }
            }
        }
        return;
    }

    uint32_t it_base = 0;    // stages of this CTA in earlier phases
    // consumer warps: the next stage of this warp's group (index over the whole launch), its ring slot and parity
    uint32_t c_it = (warp / kCW) % G, c_slot = c_it % a.nslots, c_par = 0;
    bool dead = false;       // a bounded wait of this warp ran out
    uint32_t kk = 0;         // units of this CTA so far (all phases): selects the reduction buffer
#pragma unroll 1
    for (int p = 0; p < a.n_phases; ++p) {
        const TcPhase &ph = a.ph[p];
        const uint32_t nblk = ph.cols / 256, nseg = (nblk + 7) / 8;
        const bool I8 = F ? true : ph.q4_i8 != 0, UQ4 = F ? (F & 1) != 0 : ph.use_q4 != 0, UQ6 = F ? (F & 2) != 0 : ph.use_q6 != 0;
        const TcSmem sm = tc_carve<G>(smem_raw, ph.cols, UQ4, UQ6, I8, S, a.ring_off);
        const uint32_t my_units = blockIdx.x < ph.total_units ? (ph.total_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const bool late = F == 0 && p > 0;   // the activation was written by the previous phase of this launch: read it past L1

        // ---- prologue (consumers and the finalizer): the activation as f16 (hi, lo) pairs ----
        {
            const uint32_t pw = warp < kProducer ? warp : warp - 1;   // 0 .. kConsumers
            const uint32_t hw = 2 * pw + (lane >> 4), hl = lane & 15u;
            constexpr uint32_t nhw = 2 * (kConsumers + 1);
            constexpr int kMaxBlkPerHalfWarp = F ? R : max_blk_per_half_warp(G);
            float4 ra[kMaxBlkPerHalfWarp][4], rb[kMaxBlkPerHalfWarp][4];
#pragma unroll
            for (int b = 0; b < kMaxBlkPerHalfWarp; ++b)
#pragma unroll
                for (int k = 0; k < 4; ++k) ra[b][k] = rb[b][k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ph.x_mode == MV_X_RMSNORM) {   // the norm weights are constants: fetch them before the dependency is met
                const uint64_t keep = a.l2_hints ? l2_policy_evict_last() : 0ull;
#pragma unroll
                for (int b = 0; b < kMaxBlkPerHalfWarp; ++b) {
                    const uint32_t blk = hw + b * nhw;
                    if (blk < nblk) {
                        const float4 *src = reinterpret_cast<const float4 *>(ph.wnorm + blk * 256 + hl * 16);
#pragma unroll
                        for (int k = 0; k < 4; ++k) rb[b][k] = a.l2_hints ? ldg_keep(src + k, keep) : __ldg(src + k);
                    }
                }
            }
            if (!late) {
                griddep_wait();   // the activation (and y, resid) come from the previous kernel
                if (tid == 0) trace_min(a.trace, 1);
            } else {
                // every output of the previous phase, from every CTA, has to be visible: the finalizer (which wrote
                // this CTA's share) meets the other CTAs, then this CTA's warps meet here
                if (warp == kFinal) {
                    __threadfence();
                    __syncwarp();
                    bool ok = true;
                    if (lane == 0) ok = grid_barrier(a.bar, gridDim.x, a.status);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    (void)ok;   // on a time-out the status word is set; the launch runs on with void results
                }
                prologue_barrier(kPrologueThreads);
            }
#pragma unroll
            for (int b = 0; b < kMaxBlkPerHalfWarp; ++b) {
                const uint32_t blk = hw + b * nhw;
                if (blk < nblk) {
                    const float4 *src = reinterpret_cast<const float4 *>(ph.x + blk * 256 + hl * 16);
#pragma unroll
                    for (int k = 0; k < 4; ++k) ra[b][k] = late ? __ldcg(src + k) : src[k];
                    if (F == 0 && ph.x_mode == MV_X_SILU_MUL) {
                        const float4 *src2 = reinterpret_cast<const float4 *>(ph.x2 + blk * 256 + hl * 16);
#pragma unroll
                        for (int k = 0; k < 4; ++k) rb[b][k] = late ? __ldcg(src2 + k) : src2[k];
                    }
                }
            }
            // RMSNorm: hi / lo are those of x * w; the common factor 1 / rms goes onto the row sums at the end
            if (ph.x_mode == MV_X_RMSNORM) {
                float ss = 0.f;
#pragma unroll
                for (int b = 0; b < kMaxBlkPerHalfWarp; ++b)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float4 u = ra[b][k];
                        ss += (u.x * u.x + u.y * u.y) + (u.z * u.z + u.w * u.w);
                    }
                ss = warp_sum(ss);
                if (lane == 0) sm.ssq[pw] = ss;
            }
#pragma unroll
            for (int b = 0; b < kMaxBlkPerHalfWarp; ++b) {
                const uint32_t blk = hw + b * nhw;
                if (2 * pw + b * nhw >= nblk) break;   // warp-uniform
                const bool live = blk < nblk;          // the second half-warp of the last warp may be past the end
                float v[16];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[4 * k] = ra[b][k].x; v[4 * k + 1] = ra[b][k].y; v[4 * k + 2] = ra[b][k].z; v[4 * k + 3] = ra[b][k].w;
                }
                if (ph.x_mode != MV_X_PLAIN) {
                    float w2[16];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        w2[4 * k] = rb[b][k].x; w2[4 * k + 1] = rb[b][k].y; w2[4 * k + 2] = rb[b][k].z; w2[4 * k + 3] = rb[b][k].w;
                    }
                    // one branch around each form (a per-element choice made the compiler evaluate the exponential and
                    // the division in RMSNorm launches too: measured 1.1 us per launch)
                    if (F != 0 || ph.x_mode == MV_X_RMSNORM) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] *= w2[i];
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = (v[i] / (1.0f + expf(-v[i]))) * w2[i];
                    }
                }
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
                if (I8) {
                    // ---- integer form: fixed point per 32-column sub-block (this lane and its neighbour hl ^ 1) ----
                    const float am = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    int e = (int)((__float_as_uint(am) >> 23) & 0xFFu) - 127 - 29;   // am / 2^e in [2^29, 2^30)
                    e = am > 0.f ? max(-122, min(e, 98)) : 0;                          // 2^-e and 2^(e - 4) are normal floats
                    const float inv_s = __uint_as_float((uint32_t)(127 - e) << 23);
                    float sum = 0.f;
                    uint32_t V[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        sum += v[i];
                        // n + 0x808080 has the balanced digits of n, each plus 128, in its low three bytes
                        V[i] = ((uint32_t)__float2int_rn(v[i] * inv_s) + 0x00808080u) ^ 0x00808080u;
                    }
                    const float sum32 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
                    uint32_t P[4][4];   // [plane: 0 = most significant digit][group of four elements]
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t t0 = __byte_perm(V[4 * k], V[4 * k + 1], 0x5140u), t1 = __byte_perm(V[4 * k + 2], V[4 * k + 3], 0x5140u);
                        const uint32_t t2 = __byte_perm(V[4 * k], V[4 * k + 1], 0x7362u), t3 = __byte_perm(V[4 * k + 2], V[4 * k + 3], 0x7362u);
                        P[3][k] = __byte_perm(t0, t1, 0x5410u);
                        P[2][k] = __byte_perm(t0, t1, 0x7632u);
                        P[1][k] = __byte_perm(t2, t3, 0x5410u);
                        P[0][k] = __byte_perm(t2, t3, 0x7632u);
                    }
                    if (live && UQ4) {
                        // columns 16 hl ..: chunk c, nibble kind h, elements 16 (hl & 1) .. of the sub-block = word pairs m0, m0 + 1
                        const uint32_t c = hl >> 2, h = (hl >> 1) & 1u, m0 = 2 * (hl & 1u);
                        const uint32_t base = smem_u32(sm.x4) + blk * 1024u + h * 128u + c * 32u;
#pragma unroll
                        for (int mm = 0; mm < 2; ++mm)
#pragma unroll
                            for (int pl = 0; pl < 4; ++pl)
                                sts64(base + (m0 + mm) * 256u + (pl & 1) * 16u + (pl >> 1) * 8u, P[pl][2 * mm], P[pl][2 * mm + 1]);
                        if ((hl & 1u) == 0) {
                            sm.s4[blk * 8 + (hl >> 1)] = sum32;
                            sm.xs8[blk * 8 + (hl >> 1)] = __uint_as_float((uint32_t)(127 + e - (h ? 4 : 0)) << 23);
                        }
                    }
                    if (live && UQ6) {
                        // Q6_K: these 16 columns are one scale group (half hf, group gq, run hq) of lane column t = 2 hf + hq;
                        // word js of the run is the lane column's step s = (js - t) & 3: register s & 1 of slot (s / 2, gq)
                        const uint32_t hf = hl >> 3, gq = (hl >> 1) & 3u, hq = hl & 1u, t = 2 * hf + hq;
                        const uint32_t base = smem_u32(sm.x6) + blk * 1024u + gq * 128u + t * 32u;
                        // words (hq, hq + 1) of the run are steps (2 sp, 2 sp + 1) of slot sp = hf, words (hq + 2, hq + 3) those
                        // of slot hf ^ 1: one select per word for the odd lane columns, the slot by address
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int pp = 0; pp < 2; ++pp) {
                                const uint32_t a0 = hq ? P[pp][2 * q + 1] : P[pp][2 * q], a1 = hq ? P[pp][(2 * q + 2) & 3] : P[pp][2 * q + 1];
                                const uint32_t a2 = hq ? P[pp + 2][2 * q + 1] : P[pp + 2][2 * q], a3 = hq ? P[pp + 2][(2 * q + 2) & 3] : P[pp + 2][2 * q + 1];
                                sts128(base + ((uint32_t)q ^ hf) * 512u + pp * 16u, a0, a1, a2, a3);
                            }
                        sm.s16[blk * 16 + t * 4 + gq] = sum;
                        if (hq == 0) sm.xsp[blk * 8 + (hl >> 1)] = __uint_as_float((uint32_t)(127 + e) << 23);
                    }
                    continue;   // warp-uniform: the f16 images belong to the other form
                }
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // over the half-warp
                // block scale 2^e with amax / 2^e in [2^13, 2^14); e clamped so that both 2^e and 2^-e are normal floats
                int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 13;
                e = amax > 0.f ? max(-126, min(e, 114)) : 0;
                const float inv_s = __uint_as_float((uint32_t)(127 - e) << 23);
                uint32_t hi2[8], lo2[8];   // element pairs (i, i + 2) of each group of four: the B operand's k order
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    // converted two at a time, already as the pairs the operand wants (one conversion instruction per pair)
                    const float s0 = v[4 * j] * inv_s, s1 = v[4 * j + 1] * inv_s, s2 = v[4 * j + 2] * inv_s, s3 = v[4 * j + 3] * inv_s;
                    const __half2 h02 = __floats2half2_rn(s0, s2), h13 = __floats2half2_rn(s1, s3);
                    const float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
                    const __half2 l02 = __floats2half2_rn(s0 - f02.x, s2 - f02.y), l13 = __floats2half2_rn(s1 - f13.x, s3 - f13.y);
                    const float2 g02 = __half22float2(l02), g13 = __half22float2(l13);
                    sum += f02.x + g02.x;   // elements 0, 1, 2, 3 in this order
                    sum += f13.x + g13.x;
                    sum += f02.y + g02.y;
                    sum += f13.y + g13.y;
                    hi2[2 * j] = *reinterpret_cast<const uint32_t *>(&h02);
                    hi2[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&h13);
                    lo2[2 * j] = *reinterpret_cast<const uint32_t *>(&l02);
                    lo2[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&l13);
                }
                const float sum32 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
                if (live) {
                    if (F == 0 && UQ4 && !I8) {
                        // columns 16 hl .. 16 hl + 15: chunk c = hl / 4, sub-block half (hl / 2) & 1, words 4 (hl & 1) + j
                        const uint32_t c = hl >> 2, sub = (hl >> 1) & 1u, j0 = 4 * (hl & 1u);
                        const uint32_t base = smem_u32(sm.x4) + blk * 1024u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            sts64(base + x4_off(j0 + j, 2 * c, sub), hi2[2 * j], hi2[2 * j + 1]);
                            sts64(base + x4_off(j0 + j, 2 * c + 1, sub), lo2[2 * j], lo2[2 * j + 1]);
                        }
                        if ((hl & 1u) == 0) sm.s4[blk * 8 + (hl >> 1)] = sum32;
                    }
                    if (F == 0 && UQ6) {
                        // columns 16 hl ..: half hf = hl / 8, group gq = (hl / 2) & 3, run hq = hl & 1, words j = 0..3
                        const uint32_t hf = hl >> 3, gq = (hl >> 1) & 3u, hq = hl & 1u, t = 2 * hf + hq;
                        const uint32_t base = smem_u32(sm.x6) + blk * 1024u;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t s = ((uint32_t)j - t) & 3u;
                            sts64(base + x6_off(s, 2 * t, gq), hi2[2 * j], hi2[2 * j + 1]);
                            sts64(base + x6_off(s, 2 * t + 1, gq), lo2[2 * j], lo2[2 * j + 1]);
                        }
                    }
                    if (hl == 0) sm.xs[blk] = __uint_as_float((uint32_t)(127 + e) << 23);
                }
            }
            prologue_barrier(kPrologueThreads);
            if (F == 0 && ph.xn_out != nullptr && blockIdx.x == 0) {   // the activation as f32, for layer-level checks
                float t = 0.f;
                for (uint32_t w = 0; w <= kConsumers; ++w) t += sm.ssq[w];
                const float inv_rms = 1.0f / sqrtf(t / (float)ph.cols + ph.eps);
                const uint32_t ptid = pw * 32 + lane;
                for (uint32_t c = ptid; c < ph.cols; c += kPrologueThreads) {
                    float v = late ? __ldcg(ph.x + c) : ph.x[c];
                    if (ph.x_mode == MV_X_RMSNORM) v = v * inv_rms * ph.wnorm[c];
                    else if (ph.x_mode == MV_X_SILU_MUL) v = (v / (1.0f + expf(-v))) * (late ? __ldcg(ph.x2 + c) : ph.x2[c]);
                    ph.xn_out[c] = v;
                }
            }
            if (tid == 0 && !late) trace_max(a.trace, 2);
        }

        if (warp == kFinal) {
            // ---- finalizer: adds the warps' partial row sums of a unit in warp order, applies the epilogue ----
            float inv_rms = 1.f;
            if (ph.x_mode == MV_X_RMSNORM) {
                float t = 0.f;
                for (uint32_t w = 0; w <= kConsumers; ++w) t += sm.ssq[w];   // the same order in every CTA
                inv_rms = 1.0f / sqrtf(t / (float)ph.cols + ph.eps);
            }
            for (uint32_t k = 0; k < my_units; ++k, ++kk) {
                const uint32_t u = blockIdx.x + k * gridDim.x, buf = kk & 1u;
                if (!mbar_wait_bounded(&sm.red_full[buf], (kk >> 1) & 1u, a.status)) return;
                float v = 0.f;
                if (lane < 16) {
                    const float *pp = sm.red + buf * kConsumers * 16 + lane;
#pragma unroll
                    for (uint32_t w = 0; w < kConsumers; ++w) v += pp[w * 16];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.red_empty[buf]);
                v *= inv_rms;
                if (ph.swiglu) {
                    // rows 0..7 = gate rows 8u.., rows 8..15 = up rows: h = silu(gate) * up (fl_op_silu_mul,
                    // src/runtime/decode_params.h:267-272)
                    const float up = __shfl_down_sync(0xffffffffu, v, 8);
                    const uint32_t row = 8 * u + lane;
                    if (lane < 8 && row < ph.t[0].rows) ph.t[0].y[row] = (v / (1.0f + expf(-v))) * up;
                } else {
                    const TcTensor &t = ph.t[unit_tensor(ph, u)];
                    const uint32_t row = 16 * (u - t.unit0) + lane;
                    if (lane < 16 && row < t.rows) {
                        float o = v;
                        if (t.resid) o = __ldcg(t.resid + row) + v;
                        if (ph.accumulate) o = __ldcg(t.y + row) + o;
                        t.y[row] = o;
                    }
                }
            }
        } else {
            // ---- consumers ----
            const uint32_t w = warp % kCW;
            const uint32_t g = lane >> 2, t = lane & 3u;
            const bool has_b = (g >> 1) == t;   // this lane feeds column g of the B operand; the others feed zeros
            const uint32_t lane8 = 2 * t + (g & 1u);
            const uint32_t zero16 = smem_u32(sm.zero);
            const uint32_t x4 = UQ4 ? smem_u32(sm.x4) + lane8 * 16u : 0u, x6 = UQ6 ? smem_u32(sm.x6) + lane8 * 16u : 0u;
            const uint32_t xstride = has_b ? 128u : 0u;
            const uint32_t xb = has_b ? 1024u : 0u;   // lanes that feed zeros stay on the zero slot
            const uint32_t xa4 = has_b ? x4 : zero16, xa6 = has_b ? x6 : zero16;
            // the tensor of the current unit: its format and the Q4_K offsets change only where a unit enters the next
            // tensor of the launch (a CTA's units ascend), so they are set there and not once per unit
            uint32_t ti_end = 0;     // first unit past the current tensor
            int fmt = 0;
            uint32_t oh = 0, oa = 0, ob = 0;
            for (uint32_t k = 0; k < my_units; ++k, ++kk) {
                const uint32_t u = blockIdx.x + k * gridDim.x;
                if (u >= ti_end) {
                    const int ti = ph.swiglu ? 0 : unit_tensor(ph, u);
                    ti_end = (ph.swiglu || ti + 1 >= ph.n_tensors) ? 0xFFFFFFFFu : ph.t[ti + 1].unit0;
                    fmt = ph.t[ti].fmt;
                    const bool swz = ph.t[ti].swz != 0;
                    oh = q4_row_off(w * 144u, g, swz);
                    oa = q4_row_off(w * 144u + 16u + 32u * t, g, swz);
                    ob = q4_row_off(w * 144u + 32u + 32u * t, g, swz);
                }
                float acc0 = 0.f, acc1 = 0.f;
                // this group's stages of unit k: those of its stage sequence (grp, grp + G, ... over the whole launch)
                // that fall into [it_base + k nseg, it_base + (k + 1) nseg)
                const uint32_t it0 = it_base + k * nseg, it1 = it0 + nseg;
                const bool is4 = F == 1 ? true : F == 2 ? false : fmt == FMT_Q4_K;
                if (is4 && I8) {
#pragma unroll 1
                    for (; c_it < it1; c_it += G) {
                        const uint32_t blk = (c_it - it0) * 8 + w;
                        mbar_wait_or_die(&sm.full[c_slot], c_par, a.status, dead);
                        if (blk < nblk) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch4;
                            const float2 sx = *reinterpret_cast<const float2 *>(sm.s4 + blk * 8 + 2 * t);
                            const float2 xs2 = *reinterpret_cast<const float2 *>(sm.xs8 + blk * 8 + 2 * t);
                            float o0, o1;
                            q4k_block_i8(r0, oh, oa, ob, t, xa4 + blk * xb, xstride, sx, xs2, o0, o1);
                            acc0 += o0;
                            acc1 += o1;
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm.empty[c_slot]);
                        c_slot += G;
                        if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                    }
                } else if (F == 0 && fmt == FMT_Q4_K) {
#pragma unroll 1
                    for (; c_it < it1; c_it += G) {
                        const uint32_t blk = (c_it - it0) * 8 + w;
                        mbar_wait_or_die(&sm.full[c_slot], c_par, a.status, dead);
                        if (blk < nblk) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch4;
                            const float2 sx = *reinterpret_cast<const float2 *>(sm.s4 + blk * 8 + 2 * t);
                            float o0, o1;
                            q4k_block(r0, oh, oa, ob, t, xa4 + blk * xb, xstride, sx, o0, o1);
                            const float xs = sm.xs[blk];
                            acc0 = fmaf(xs, o0, acc0);
                            acc1 = fmaf(xs, o1, acc1);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm.empty[c_slot]);
                        c_slot += G;
                        if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                    }
                } else if (F == 0 && fmt == FMT_Q8_0) {
#pragma unroll 1
                    for (; c_it < it1; c_it += G) {
                        const uint32_t blk = (c_it - it0) * 8 + w;
                        mbar_wait_or_die(&sm.full[c_slot], c_par, a.status, dead);
                        if (blk < nblk) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch8 + w * 272u + t * 68u;
                            float o0, o1;
                            q8_0_block(r0, r0 + 8 * kPitch8, xa4 + blk * xb, xstride, o0, o1);
                            const float xs = sm.xs[blk];
                            acc0 = fmaf(xs, o0, acc0);
                            acc1 = fmaf(xs, o1, acc1);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm.empty[c_slot]);
                        c_slot += G;
                        if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                    }
                } else if (I8) {
#pragma unroll 1
                    for (; c_it < it1; c_it += G) {
                        const uint32_t blk = (c_it - it0) * 8 + w;
                        mbar_wait_or_die(&sm.full[c_slot], c_par, a.status, dead);
                        if (blk < nblk) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch6 + w * 210u;
                            const float4 xs4 = *reinterpret_cast<const float4 *>(sm.xsp + blk * 8 + 4 * (t >> 1));
                            const float4 sx4 = *reinterpret_cast<const float4 *>(sm.s16 + blk * 16 + 4 * t);
                            float o0, o1;
                            if (w & 1u) q6k_block_i8<true>(r0 - 2, r0 + 8 * kPitch6 - 2, t, xa6 + blk * xb, xstride, xs4, sx4, o0, o1);
                            else q6k_block_i8<false>(r0, r0 + 8 * kPitch6, t, xa6 + blk * xb, xstride, xs4, sx4, o0, o1);
                            acc0 += o0;
                            acc1 += o1;
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm.empty[c_slot]);
                        c_slot += G;
                        if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                    }
                } else if (F == 0) {
#pragma unroll 1
                    for (; c_it < it1; c_it += G) {
                        const uint32_t blk = (c_it - it0) * 8 + w;
                        mbar_wait_or_die(&sm.full[c_slot], c_par, a.status, dead);
                        if (blk < nblk) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch6 + w * 210u;
                            float o0, o1;
                            if (w & 1u) q6k_block<true>(r0 - 2, r0 + 8 * kPitch6 - 2, t, xa6 + blk * xb, xstride, o0, o1);
                            else q6k_block<false>(r0, r0 + 8 * kPitch6, t, xa6 + blk * xb, xstride, o0, o1);
                            const float xs = sm.xs[blk];
                            acc0 = fmaf(xs, o0, acc0);
                            acc1 = fmaf(xs, o1, acc1);
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sm.empty[c_slot]);
                        c_slot += G;
                        if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                    }
                }
                // the unit's partial sums of rows g and g + 8 over this warp's lane columns
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
                const uint32_t buf = kk & 1u;
                mbar_wait_or_die(&sm.red_empty[buf], ((kk >> 1) & 1u) ^ 1u, a.status, dead);
                if (t == 0) {
                    float *pp = sm.red + (buf * kConsumers + warp) * 16;
                    pp[g] = acc0;
                    pp[g + 8] = acc1;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.red_full[buf]);
            }
        }
        it_base += my_units * nseg;
    }
    if (warp == kFinal && lane == 0) trace_max(a.trace, 3);
}

// Consumer groups per CTA: 2 (16 consumer warps, 96 registers each) measured 15 % faster than 1 (8 warps, 168
// registers) on the 8B-shape step; FLB_TC_GROUPS=1 selects the other instantiation for comparison.
int tc_groups() {
    static const int v = getenv("FLB_TC_GROUPS") ? atoi(getenv("FLB_TC_GROUPS")) : 2;
    return v == 1 ? 1 : 2;
}

} // namespace

cudaError_t matvec_tc_init(void) {
    const int smem = 227 * 1024 - 1024;
    cudaError_t e = cudaFuncSetAttribute(matvec_tc_kernel<1, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 3, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(matvec_tc_kernel<2, 3, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    return e;
}

// True when the launch can run on the tensor-core kernel: Q4_K / Q6_K / Q8_0 tensors only, whole 256-column
// blocks, 16-byte aligned rows, no expert indirection and no exchange prologue.
// Q4_K and Q6_K on the integer forms (q4k_block_i8, q6k_block_i8) unless FLB_TC_I8=0; a launch that holds a Q8_0
// tensor stays on the f16 forms (Q8_0 reads the f16 image of the activation).
bool tc_q4_i8() {
    static const bool on = !(getenv("FLB_TC_I8") && getenv("FLB_TC_I8")[0] == '0');
    return on;
}

bool matvec_tc_eligible(const MatvecArgs &a) {
    static const bool off = getenv("FLB_TC") && getenv("FLB_TC")[0] == '0';
    if (off || a.xr_buf || a.cols % 256 != 0 || a.cols < 256) return false;
    if (a.n_tensors < 1 || a.n_tensors > 3) return false;
    if ((((uintptr_t)a.x) & 15u) || (((uintptr_t)a.x2) & 15u) || (((uintptr_t)a.wnorm) & 15u)) return false;
    const int groups = tc_groups();
    if (a.cols / 256 > (uint32_t)(max_blk_per_half_warp(groups) * 2 * (groups * kCW + 1))) return false;
    bool q4 = false, q6 = false, q8 = false;
    for (int i = 0; i < a.n_tensors; ++i) {
        const MatvecTensor &t = a.t[i];
        if (t.fmt != FMT_Q4_K && t.fmt != FMT_Q6_K && t.fmt != FMT_Q8_0) return false;
        if (t.expert_id || t.rows == 0) return false;
        const uint64_t pitch = t.pitch ? t.pitch : row_bytes(t.fmt, a.cols);
        if ((pitch & 15u) || (((uintptr_t)t.w) & 15u) || pitch < row_bytes(t.fmt, a.cols)) return false;
        (t.fmt == FMT_Q6_K ? q6 : q4) = true;   // Q8_0 uses the Q4_K layout of the activation
        q8 = q8 || t.fmt == FMT_Q8_0;
    }
    if (a.swiglu && (a.n_tensors != 2 || a.t[0].rows != a.t[1].rows || a.t[0].fmt != a.t[1].fmt || a.accumulate)) return false;
    const uint32_t slot = q8 ? kSlot8 : q6 ? kSlot6 : kSlot4;
    return tc_head_bytes(2, groups) + tc_x_bytes(a.cols, q4, q6, !q8 && tc_q4_i8()) + 1024 + 2u * slot <= 227 * 1024 - 1024;
}

// One launch of n dependent matvecs (phase i + 1 consumes what phase i writes). n = 1: a plain launch.
// cudaErrorNotSupported when a phase does not qualify or the phases do not fit together; the caller then
// launches them one by one.
cudaError_t launch_matvec_tc_chain(const MatvecArgs *args, int n, int sms, cudaStream_t stream) {
    if (n < 1 || n > 4) return cudaErrorInvalidValue;
    TcArgs k;
    memset(&k, 0, sizeof(k));
    const int groups = tc_groups();
    bool any6 = false, any8 = false;
    size_t xmax = 0;
    uint32_t max_units = 0;
    for (int p = 0; p < n; ++p) {
        const MatvecArgs &a = args[p];
        if (!matvec_tc_eligible(a)) return cudaErrorNotSupported;
        if (p > 0 && (a.trace || a.issue_late)) { /* per-launch diagnostics apply to the first phase only */ }
        TcPhase &ph = k.ph[p];
        bool q4 = false, q6 = false, q8 = false;
        uint32_t units = 0;
        ph.n_tensors = a.n_tensors;
        for (int i = 0; i < a.n_tensors; ++i) {
            const MatvecTensor &t = a.t[i];
            ph.t[i].w = t.w; ph.t[i].y = t.y; ph.t[i].resid = t.resid; ph.t[i].rows = t.rows; ph.t[i].fmt = t.fmt;
            ph.t[i].pitch = t.pitch ? t.pitch : (uint32_t)row_bytes(t.fmt, a.cols);
            ph.t[i].unit0 = units;
            units += (t.rows + 15) / 16;
            if (t.fmt != FMT_Q8_0) {   // the tiled view the stages' boxes are cut from (16 rows; SwiGLU: 8 + 8)
                const uint32_t segb = t.fmt == FMT_Q4_K ? kSeg4 : kSeg6, brows = a.swiglu ? 8 : 16;
                ph.t[i].swz = (t.fmt == FMT_Q4_K && ph.t[i].pitch % 128 == 0) ? 1 : 0;
                const cudaError_t e = ph.t[i].swz ? tensor_map_lines_swz(&ph.t[i].map, t.w, t.rows, ph.t[i].pitch, segb / 128, brows)
                                                  : tensor_map_2d(&ph.t[i].map, 8, t.w, ph.t[i].pitch / 8, t.rows, ph.t[i].pitch,
                                                                  segb / 8, brows, false);
                if (e != cudaSuccess) return e;
            }
            (t.fmt == FMT_Q6_K ? q6 : q4) = true;   // Q8_0 uses the Q4_K layout of the activation
            any8 = any8 || t.fmt == FMT_Q8_0;
            q8 = q8 || t.fmt == FMT_Q8_0;
        }
        if (a.swiglu) units = (a.t[0].rows + 7) / 8;
        ph.x = a.x; ph.x2 = a.x2; ph.wnorm = a.wnorm; ph.eps = a.eps; ph.cols = a.cols; ph.x_mode = a.x_mode;
        ph.accumulate = a.accumulate; ph.swiglu = a.swiglu; ph.total_units = units;
        ph.use_q4 = q4 ? 1 : 0; ph.use_q6 = q6 ? 1 : 0;
        ph.q4_i8 = (!q8 && tc_q4_i8()) ? 1 : 0;
        ph.xn_out = a.xn_out;
        any6 = any6 || q6;
        xmax = std::max(xmax, tc_x_bytes(a.cols, q4, q6, ph.q4_i8 != 0));
        max_units = std::max(max_units, units);
    }
    k.n_phases = n;
    k.status = args[0].status;
    k.trace = args[0].trace;
    static const bool hints = !(getenv("FLB_TC_L2HINT") && getenv("FLB_TC_L2HINT")[0] == '0');
    k.l2_hints = hints ? 1 : 0;
    k.slot_bytes = any8 ? kSlot8 : any6 ? kSlot6 : kSlot4;
    const size_t limit = 227 * 1024 - 1024;
    uint32_t nslots = 2;
    auto total = [&](uint32_t ns) {
        const size_t ring_off = (tc_head_bytes(ns, groups) + xmax + 1023) & ~(size_t)1023;   // the swizzle pattern repeats every 1024 bytes
        return ring_off + (size_t)ns * k.slot_bytes;
    };
    if (total(nslots) > limit) return cudaErrorNotSupported;
    while (nslots < 32 && total(nslots + 1) <= limit) ++nslots;
    k.nslots = nslots;
    k.ring_off = (uint32_t)((tc_head_bytes(nslots, groups) + xmax + 1023) & ~(size_t)1023);
    const size_t smem = total(nslots);
    uint32_t grid = max_units < (uint32_t)sms ? max_units : (uint32_t)sms;
    if (n > 1) {
        // the barrier needs every CTA resident: one CTA per SM (the shared memory of a CTA is more than half an SM's)
        if (smem <= 114 * 1024) return cudaErrorNotSupported;
        if (!args[0].grid_bar) return cudaErrorInvalidValue;
        k.bar = reinterpret_cast<GridBar *>(args[0].grid_bar);
    }
    if (groups == 2) {
        const dim3 block((2 * kCW + 2) * 32);
        const bool pdl = args[0].pdl != 0;
        static const bool generic = getenv("FLB_TC_GENERIC") && getenv("FLB_TC_GENERIC")[0] == '1';   // A/B: the run-time form for every launch
        const TcPhase &p0 = k.ph[0];
        // the specialised instances: one phase, integer forms, plain or RMSNorm prologue, no copy of the activation asked for
        const bool special = n == 1 && p0.q4_i8 && !generic && p0.x_mode != MV_X_SILU_MUL && p0.xn_out == nullptr;
        const int f = special ? (p0.use_q4 ? 1 : 0) | (p0.use_q6 ? 2 : 0) : 0;
        const bool one = p0.cols / 256 <= 2u * (2 * kCW + 1);   // every half-warp of the prologue converts at most one block
        if (f == 1) return one ? launch_kernel(matvec_tc_kernel<2, 1, 1>, dim3(grid), block, smem, stream, pdl, k)
                               : launch_kernel(matvec_tc_kernel<2, 1, 2>, dim3(grid), block, smem, stream, pdl, k);
        // Q6_K only: the two-block instance for every width (the one-block instance spills in its consume loop: with 18
        // warps a thread can have 96 registers, five warps share a quarter of the register file)
        if (f == 2) return launch_kernel(matvec_tc_kernel<2, 2, 2>, dim3(grid), block, smem, stream, pdl, k);
        if (f == 3) return one ? launch_kernel(matvec_tc_kernel<2, 3, 1>, dim3(grid), block, smem, stream, pdl, k)
                               : launch_kernel(matvec_tc_kernel<2, 3, 2>, dim3(grid), block, smem, stream, pdl, k);
        return launch_kernel(matvec_tc_kernel<2, 0, 0>, dim3(grid), block, smem, stream, pdl, k);
    }
    return launch_kernel(matvec_tc_kernel<1, 0, 0>, dim3(grid), dim3((kCW + 2) * 32), smem, stream, args[0].pdl != 0, k);
}

cudaError_t launch_matvec_tc(const MatvecArgs &a, int sms, cudaStream_t stream) {
    return launch_matvec_tc_chain(&a, 1, sms, stream);
}

} // namespace flb
