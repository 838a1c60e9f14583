// Several activation columns in one pass over a k-quant tensor: Y[p][r] (+)= dot(W[r], X[p]) for p < P <= 8,
// the STREAM_DOT semantics of Task::nx (include/fastllm/fastllm.h:87-96; the reference's GPU form is
// gdot_i8k_q4_K_mc, src/runtime/kernels_gpu.h:682-740, Q4_K only). Used for draft-verification batches,
// prompt chunks and the tokens that share an expert of a mixture-of-experts block.
//
// The pipeline is the one of the single-column tensor-core kernel (matvec_tc.cu): a unit is 16 rows, a stage is
// the same 2048-column segment of the unit's rows (one bulk copy per row into a padded shared-memory row), a
// producer warp keeps a ring of stages full, consumer warp w owns super-block w of the segment, a finalizer warp
// adds the warps' partial sums in warp order and writes Y. What differs is the use of mma.sync.m16n8k16:
//   * the 8 columns of the B operand are 4 activation columns ("tokens"), each as an f16 (hi, lo) pair, so
//     every product of the instruction is used; two instructions serve 8 tokens from the same A registers;
//   * the 16 k-slots of an instruction are 16 consecutive weights of ONE scale group of a row (half a Q4_K
//     sub-block, a whole Q6_K one): lane column t unpacks word t of the group. The accumulator a lane reads
//     back, C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1], is then the complete 16-weight dot product of rows g
//     and g + 8 with token t of the group of four, and the scale of the group is applied in f32;
//   * the activations are converted once, by a small kernel of their own, into exactly the register layout of
//     the B operand (per 256-column block and group of four tokens 4096 bytes of f16 pairs, then the tokens'
//     sub-block sums and power-of-two block scales); the matmul kernel brings that image into shared memory with
//     bulk copies, a chunk of at most 16 blocks (4096 columns) at a time. With more columns than a chunk the
//     kernel walks the chunks one after the other (all units of the CTA per chunk) and the finalizer keeps
//     the units' running sums in shared memory.
// Every weight byte still crosses HBM once per pass, whatever P is; a pass over 8 tokens costs about what a
// single-column pass costs.
// For the experts of a mixture-of-experts block the columns of a call are a device-side list: the number of
// valid columns is read from device memory (a call with none returns at once and reads no weights), the
// conversion gathers the listed tokens (optionally as SiLU(x) * x2, the input of a down projection) and the
// finalizer scatters the results to the listed output rows.
#include "common.cuh"
#include "kernels.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace flb {

namespace {

constexpr int kCW = 8;
constexpr uint32_t kSeg4 = 8 * 144, kSeg6 = 8 * 210;
// A stage arrives as one tiled TMA box of 16 rows x the segment, so the row pitch in shared memory is the segment's
// size. Q6_K: 420 words = 4 mod 32: the 32-bit loads of lanes (g, t) are conflict free as they are. Q4_K: 288 words =
// 0 mod 32: the rows are fetched as lines of 128 bytes with the 128-byte swizzle (tensor_map_lines_swz), which
// spreads the same 16-byte chunk of 8 consecutive rows over 8 bank groups; rows whose pitch in memory is not a
// multiple of 128 bytes (columns not a multiple of 2048) use the plain box and pay the conflicts.
constexpr uint32_t kPitch4 = kSeg4, kPitch6 = kSeg6;
constexpr uint32_t slot_round(uint32_t b) { return (b + 1023u) & ~1023u; }   // the swizzle pattern is tied to the address
constexpr uint32_t kSlot4 = slot_round(16 * kPitch4), kSlot6 = slot_round(16 * kPitch6);
constexpr uint32_t kFragBytes = 4096;                    // B fragments of one (block, token group)
constexpr uint32_t kXqBlk = kFragBytes + 128 + 16;       // + sub-block sums [4 tokens][8] + block scales [4]
constexpr uint32_t kMaxChunkBlks = 16;                   // blocks of activation resident at a time, at most
constexpr uint32_t kMaxChunkUnits = 16;                  // units per CTA when the columns span several chunks

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
__device__ __forceinline__ float ldsf(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
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
// Byte offset o of a Q4_K row as the stage holds it: as it is, or in the swizzled 128-byte lines.
__device__ __forceinline__ uint32_t q4_row_off(uint32_t o, uint32_t g, bool swz) {
    return swz ? (o & ~127u) + ((((o >> 4) ^ (g + (o >> 7))) & 7u) << 4) + (o & 15u) : o;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t h, __half2 off) {
    const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&h), off);
    return *reinterpret_cast<const uint32_t *>(&r);
}
template <int K>
__device__ __forceinline__ float u8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K)) - 8388608.0f;
}
__device__ __noinline__ bool mbar_wait_slow(uint64_t *bar, uint32_t parity, uint32_t *status) {
    return mbar_wait_bounded(bar, parity, status);
}
// A warp whose wait ran out once waits for nothing any more (its results are void, the status word says so).
__device__ __forceinline__ void mbar_wait_or_die(uint64_t *bar, uint32_t parity, uint32_t *status, bool &dead) {
    if (dead || mbar_try_wait(bar, parity)) return;
    dead = !mbar_wait_slow(bar, parity, status);
}

// ---- activations -> the B operand's register image ----------------------------------------------------------
// Combo m of a block = one tensor-core instruction's 16 columns. Q4_K: m = column / 16 (chunk c, nibble kind,
// half of the sub-block). Q6_K: m = ((hf * 2 + hq) * 4 + gq) for columns 128 hf + 32 gq + 16 hq + [0, 16).
// Within a combo lane column t' holds columns 4 t' + {0, 2} (register b0) and 4 t' + {1, 3} (register b1); lane
// = 4 * (2 p' + h) + t' for token p' of the group and part h (0 = hi, 1 = lo). Byte offset in the fragment
// image: (m / 2) * 512 + lane * 16 + (m & 1) * 8, so that a lane's 128-bit load fetches two combos and a warp's
// load is one contiguous 512 bytes.
// grid (nblk, ntg), 64 threads: half-warp p' converts the block's 256 columns of token 4 tg + p'.
// Column p of the call is row col_idx[col_off + p] of x (col_idx == nullptr: row p); columns at or past *cnt - col_off
// (cnt == nullptr: P) are zeros. x2 != nullptr: the value is SiLU(x) * x2 (fl_op_silu_mul, src/runtime/decode_params.h:267-272).
__global__ void __launch_bounds__(64) act_convert_nx_kernel(const float *__restrict__ x, const float *__restrict__ x2, uint32_t xstride,
                                                            uint32_t P, int fmt, uint8_t *__restrict__ xq, uint32_t ntg,
                                                            const uint32_t *__restrict__ cnt, uint32_t col_off,
                                                            const uint32_t *__restrict__ col_idx) {
    const uint32_t blk = blockIdx.x, tg = blockIdx.y;
    const uint32_t pp = threadIdx.x >> 4, hl = threadIdx.x & 15u, p = 4 * tg + pp;
    // launched as a programmatic dependent: the launch itself overlaps the tail of the kernel before, whose output
    // (x, the column list) is read only after it has completed
    griddep_launch_dependents();
    griddep_wait();
    uint32_t n_valid = P;
    if (cnt) { const uint32_t c = *cnt; n_valid = c > col_off ? min(c - col_off, P) : 0u; }
    if (n_valid == 0) return;   // the matmul of this call returns at entry too
    float v[16];
    if (p < n_valid) {
        const size_t row = col_idx ? col_idx[col_off + p] : p;
        const float4 *src = reinterpret_cast<const float4 *>(x + row * xstride + blk * 256 + hl * 16);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float4 u = src[k];
            v[4 * k] = u.x; v[4 * k + 1] = u.y; v[4 * k + 2] = u.z; v[4 * k + 3] = u.w;
        }
        if (x2) {
            const float4 *src2 = reinterpret_cast<const float4 *>(x2 + row * xstride + blk * 256 + hl * 16);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 u = src2[k];
                v[4 * k] = (v[4 * k] / (1.0f + expf(-v[4 * k]))) * u.x;
                v[4 * k + 1] = (v[4 * k + 1] / (1.0f + expf(-v[4 * k + 1]))) * u.y;
                v[4 * k + 2] = (v[4 * k + 2] / (1.0f + expf(-v[4 * k + 2]))) * u.z;
                v[4 * k + 3] = (v[4 * k + 3] / (1.0f + expf(-v[4 * k + 3]))) * u.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 13;
    e = amax > 0.f ? max(-126, min(e, 114)) : 0;
    const float inv_s = __uint_as_float((uint32_t)(127 - e) << 23);
    uint8_t *base = xq + ((size_t)blk * ntg + tg) * kXqBlk;
    uint32_t m;
    if (fmt == FMT_Q4_K) m = hl;
    else m = (((hl >> 3) * 2 + (hl & 1u)) * 4) + ((hl >> 1) & 3u);
    float sum = 0.f;
#pragma unroll
    for (int tq = 0; tq < 4; ++tq) {
        __half hh[4], ll[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const float s = v[4 * tq + b] * inv_s;
            hh[b] = __float2half_rn(s);
            ll[b] = __float2half_rn(s - __half2float(hh[b]));
            sum += __half2float(hh[b]) + __half2float(ll[b]);
        }
        const uint32_t off = (m >> 1) * 512u + (m & 1u) * 8u + tq * 16u;
        uint2 hi, lo;
        hi.x = (uint32_t)__half_as_ushort(hh[0]) | ((uint32_t)__half_as_ushort(hh[2]) << 16);
        hi.y = (uint32_t)__half_as_ushort(hh[1]) | ((uint32_t)__half_as_ushort(hh[3]) << 16);
        lo.x = (uint32_t)__half_as_ushort(ll[0]) | ((uint32_t)__half_as_ushort(ll[2]) << 16);
        lo.y = (uint32_t)__half_as_ushort(ll[1]) | ((uint32_t)__half_as_ushort(ll[3]) << 16);
        *reinterpret_cast<uint2 *>(base + off + (4 * (2 * pp)) * 16u) = hi;        // lane = 4 * (2 p' + 0) + tq
        *reinterpret_cast<uint2 *>(base + off + (4 * (2 * pp + 1)) * 16u) = lo;    // lane = 4 * (2 p' + 1) + tq
    }
    const float sum32 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    if ((hl & 1u) == 0) reinterpret_cast<float *>(base + kFragBytes)[pp * 8 + (hl >> 1)] = sum32;   // [token][sub-block]
    if (hl == 0) reinterpret_cast<float *>(base + kFragBytes + 128)[pp] = __uint_as_float((uint32_t)(127 + e) << 23);
}

struct NxArgs {
    CUtensorMap map;               // the tiled view a stage's box is cut from
    const uint32_t *cnt;           // optional: number of listed columns on the device
    const uint32_t *out_idx;       // optional: output row block (in units of ystride) of listed column col_off + p
    uint32_t col_off, swz;
    const uint8_t *w;
    const uint8_t *xq;
    float *y;
    uint32_t rows, pitch, cols, ystride, P, ntg;
    int fmt, accumulate;
    uint32_t nslots, slot_bytes, ring_off, x_off, uacc_off, chunk_blks;   // chunk_blks: 8 or 16 blocks of activation resident at a time
    uint32_t *status;
};

__host__ __device__ inline size_t nx_head_bytes(uint32_t nslots, int groups) {
    size_t n = (size_t)nslots * 16 + 64;                     // stage barriers; reduction barriers; activation barriers
    n += (size_t)2 * groups * kCW * 128 * 4;                // red [2][warps][16 rows][8 tokens]
    return (n + 127) & ~(size_t)127;
}

// ---- per-block math: rows g (r0) and g + 8 (r1), tokens t and t + 4 -----------------------------------------
// out[row][tg] in units of the tokens' block scales.
// r0: row g of the stage (row g + 8 is 8 pitches further: the same swizzle, 72 lines on); ow[c][i]: offset in the row
// of word 4 i + t of chunk c of this warp's block, oh: of the block's header (q4_row_off).
template <int NTG>
__device__ __forceinline__ void q4k_block_nx(uint32_t r0, const uint32_t (&ow)[4][2], uint32_t oh, uint32_t t, uint32_t xaddr,
                                             uint32_t lane, float (&out)[2][NTG]) {
    const uint32_t r1 = r0 + 8 * kPitch4;
    // all loads first
    uint32_t w0[4][2], w1[4][2];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            w0[c][i] = lds32(r0 + ow[c][i]);
            w1[c][i] = lds32(r1 + ow[c][i]);
        }
    const uint4 h0 = lds128(r0 + oh), h1 = lds128(r1 + oh);
    float sums[NTG][8];   // sub-block sums of token t (+ 4 tg)
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg) {
        const uint32_t sa = xaddr + tg * kXqBlk + kFragBytes + t * 32;
        const uint4 s0 = lds128(sa), s1 = lds128(sa + 16);
        sums[tg][0] = __uint_as_float(s0.x); sums[tg][1] = __uint_as_float(s0.y); sums[tg][2] = __uint_as_float(s0.z); sums[tg][3] = __uint_as_float(s0.w);
        sums[tg][4] = __uint_as_float(s1.x); sums[tg][5] = __uint_as_float(s1.y); sums[tg][6] = __uint_as_float(s1.z); sums[tg][7] = __uint_as_float(s1.w);
    }
    // the eight 6-bit scales and mins of both rows (packing: fl_q4k_scale_min, src/runtime/quants.h:121-129)
    uint32_t scw[2][2], mnw[2][2];   // [row][sub-blocks 0..3 | 4..7], one byte each
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 hdr = r ? h1 : h0;
        scw[r][0] = hdr.y & 0x3F3F3F3Fu;
        mnw[r][0] = hdr.z & 0x3F3F3F3Fu;
        scw[r][1] = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        mnw[r][1] = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    }
    float accq[2][NTG], accm[2][NTG];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int tg = 0; tg < NTG; ++tg) accq[r][tg] = accm[r][tg] = 0.f;
    // the mins against the sub-block sums first: the sums' registers are free again before the unpacking starts
#pragma unroll
    for (int sb = 0; sb < 8; ++sb)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t mw = mnw[r][sb >> 2];
            const float mnf = (sb & 3) == 0 ? u8f<0>(mw) : (sb & 3) == 1 ? u8f<1>(mw) : (sb & 3) == 2 ? u8f<2>(mw) : u8f<3>(mw);
#pragma unroll
            for (int tg = 0; tg < NTG; ++tg) accm[r][tg] = fmaf(mnf, sums[tg][sb], accm[r][tg]);
        }
    const uint32_t ML = 0x000F000Fu, KL = 0x64006400u, MH = 0x00F000F0u, KH = 0x54005400u;
    const __half2 oL = __floats2half2_rn(1024.f, 1024.f), oH = __floats2half2_rn(64.f, 64.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        // A registers of the chunk's four instructions: (low nibbles, i = 0, 1), (high nibbles, i = 0, 1)
        uint32_t aL[2][4], aH[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t W0 = w0[c][i], W1 = w1[c][i], V0 = W0 >> 8, V1 = W1 >> 8;
            aL[i][0] = hsub2_u32(and_or(W0, ML, KL), oL); aL[i][1] = hsub2_u32(and_or(W1, ML, KL), oL);
            aL[i][2] = hsub2_u32(and_or(V0, ML, KL), oL); aL[i][3] = hsub2_u32(and_or(V1, ML, KL), oL);
            aH[i][0] = hsub2_u32(and_or(W0, MH, KH), oH); aH[i][1] = hsub2_u32(and_or(W1, MH, KH), oH);
            aH[i][2] = hsub2_u32(and_or(V0, MH, KH), oH); aH[i][3] = hsub2_u32(and_or(V1, MH, KH), oH);
        }
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const int sb = 2 * c + sub;
            // scale of sub-block sb for both rows, as floats
            float scf[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t sw = scw[r][sb >> 2];
                scf[r] = (sb & 3) == 0 ? u8f<0>(sw) : (sb & 3) == 1 ? u8f<1>(sw) : (sb & 3) == 2 ? u8f<2>(sw) : u8f<3>(sw);
            }
#pragma unroll
            for (int tg = 0; tg < NTG; ++tg) {
                // combos m = 2 sb, 2 sb + 1 (i = 0, 1) sit in one 16-byte piece: q = sb
                const uint4 bx = lds128(xaddr + tg * kXqBlk + sb * 512 + lane * 16);
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
                if (sub == 0) {
                    mma16816(cc, aL[0][0], aL[0][1], aL[0][2], aL[0][3], bx.x, bx.y);
                    mma16816(cc, aL[1][0], aL[1][1], aL[1][2], aL[1][3], bx.z, bx.w);
                } else {
                    mma16816(cc, aH[0][0], aH[0][1], aH[0][2], aH[0][3], bx.x, bx.y);
                    mma16816(cc, aH[1][0], aH[1][1], aH[1][2], aH[1][3], bx.z, bx.w);
                }
                accq[0][tg] = fmaf(scf[0], cc[0] + cc[1], accq[0][tg]);
                accq[1][tg] = fmaf(scf[1], cc[2] + cc[3], accq[1][tg]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint4 hdr = r ? h1 : h0;
        const float d = h2f_bits((uint16_t)(hdr.x & 0xFFFFu)), dmin = h2f_bits((uint16_t)(hdr.x >> 16));
#pragma unroll
        for (int tg = 0; tg < NTG; ++tg) out[r][tg] = d * accq[r][tg] - dmin * accm[r][tg];
    }
}

// Q6_K (q = nibble | two high bits << 4, value d * sc * (q - 32); fl_dot_row_q6_K, src/runtime/quants.h:194-230): an
// instruction covers the 16 columns of one int8 scale; lane column t unpacks bytes 4 t .. 4 t + 3 of the 16-byte runs.
// ODD: the block starts 2 bytes past a word boundary (r0, r1 are the aligned addresses 2 bytes in front of it).
template <int NTG, bool ODD>
__device__ __forceinline__ void q6k_block_nx(uint32_t r0, uint32_t r1, uint32_t t, uint32_t xaddr, uint32_t lane, float (&out)[2][NTG]) {
    uint32_t wa[2][4], wb[2][4], wh[2][4];   // [row][(hf, hq)]
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
        const uint32_t hf = hh >> 1, hq = hh & 1;
        const uint32_t oa = 64 * hf + 16 * hq + 4 * t, oh = 128 + 32 * hf + 16 * hq + 4 * t;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t rb = r ? r1 : r0;
            if (ODD) {
                wa[r][hh] = __byte_perm(lds32(rb + oa), lds32(rb + oa + 4), 0x5432u);
                wb[r][hh] = __byte_perm(lds32(rb + oa + 32), lds32(rb + oa + 36), 0x5432u);
                wh[r][hh] = __byte_perm(lds32(rb + oh), lds32(rb + oh + 4), 0x5432u);
            } else {
                wa[r][hh] = lds32(rb + oa);
                wb[r][hh] = lds32(rb + oa + 32);
                wh[r][hh] = lds32(rb + oh);
            }
        }
    }
    // the 16 int8 scales of both rows as (s + 128) bytes, d at byte 208
    uint32_t sw[2][4];
    float dd[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t rb = r ? r1 : r0;
        if (ODD) {
            uint32_t s[5];
#pragma unroll
            for (int k = 0; k < 5; ++k) s[k] = lds32(rb + 192 + 4 * k);
#pragma unroll
            for (int k = 0; k < 4; ++k) sw[r][k] = __byte_perm(s[k], s[k + 1], 0x5432u) ^ 0x80808080u;
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) sw[r][k] = lds32(rb + 192 + 4 * k) ^ 0x80808080u;
        }
        dd[r] = h2f_bits((uint16_t)lds16(rb + (ODD ? 2u : 0u) + 208));
    }
    float acc[2][NTG];
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int tg = 0; tg < NTG; ++tg) acc[r][tg] = 0.f;
    const __half2 off = __floats2half2_rn(1056.f, 1056.f);
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
        const int hf = hh >> 1, hq = hh & 1;
        uint32_t q[2][4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t a = wa[r][hh], b = wb[r][hh], h = wh[r][hh];
            q[r][0] = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
            q[r][1] = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
            q[r][2] = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
            q[r][3] = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int gq = 0; gq < 4; ++gq) {
            const uint32_t a0 = hsub2_u32(__byte_perm(q[0][gq], 0x64646464u, 0x4240u), off), a1 = hsub2_u32(__byte_perm(q[1][gq], 0x64646464u, 0x4240u), off);
            const uint32_t a2 = hsub2_u32(__byte_perm(q[0][gq], 0x64646464u, 0x4341u), off), a3 = hsub2_u32(__byte_perm(q[1][gq], 0x64646464u, 0x4341u), off);
            // scale index 8 hf + 2 gq + hq: byte (2 gq + hq) of word (2 hf + (gq >> 1)) ... as one index into 16 bytes
            const int si = 8 * hf + 2 * gq + hq;
            float scf[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const uint32_t w = sw[r][si >> 2];
                scf[r] = ((si & 3) == 0 ? u8f<0>(w) : (si & 3) == 1 ? u8f<1>(w) : (si & 3) == 2 ? u8f<2>(w) : u8f<3>(w)) - 128.f;
            }
            const int m = hh * 4 + gq;   // combo: 16-byte piece m / 2, half m & 1
#pragma unroll
            for (int tg = 0; tg < NTG; ++tg) {
                const uint4 bx = lds128(xaddr + tg * kXqBlk + (m >> 1) * 512 + lane * 16);
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
                if (m & 1) mma16816(cc, a0, a1, a2, a3, bx.z, bx.w);
                else mma16816(cc, a0, a1, a2, a3, bx.x, bx.y);
                acc[0][tg] = fmaf(scf[0], cc[0] + cc[1], acc[0][tg]);
                acc[1][tg] = fmaf(scf[1], cc[2] + cc[3], acc[1][tg]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
        for (int tg = 0; tg < NTG; ++tg) out[r][tg] = dd[r] * acc[r][tg];
}

// Warps: G groups of 8 consumers (group i takes stages i, i + G, ... of the CTA's stage sequence), the producer, the finalizer.
template <int NTG, int G>
__global__ void __launch_bounds__((G * kCW + 2) * 32) matmul_tc_nx_kernel(const __grid_constant__ NxArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr uint32_t kConsumers = G * kCW, kProducer = kConsumers, kFinal = kConsumers + 1;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t S = a.nslots;
    uint64_t *full = (uint64_t *)smem_raw, *empty = full + S;
    uint64_t *red_full = empty + S, *red_empty = red_full + 2, *x_full = red_empty + 2, *x_empty = x_full + 1;
    float *red = (float *)(smem_raw + S * 16 + 64);
    const uint32_t nblk = a.cols / 256, nseg = (nblk + 7) / 8;
    const uint32_t kChunkBlks = a.chunk_blks;
    const uint32_t nchunk = (nblk + kChunkBlks - 1) / kChunkBlks;
    const uint32_t units = (a.rows + 15) / 16;
    const uint32_t my_units = blockIdx.x < units ? (units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    // Launched as a programmatic dependent. With a device-side column list the list decides whether any weight is read at
    // all, so everything waits for the kernels before; without one the producer starts streaming the weights (constants)
    // at once and only the finalizer, which fetches the converted activations and touches y, waits.
    griddep_launch_dependents();
    if (a.cnt) griddep_wait();
    uint32_t n_valid = a.P;   // listed columns of this call
    if (a.cnt) { const uint32_t c = *a.cnt; n_valid = c > a.col_off ? min(c - a.col_off, a.P) : 0u; }
    if (n_valid == 0) return;   // nothing routed here: no weights are read
    if (tid == 0) {
        for (uint32_t s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kCW); }
        for (int i = 0; i < 2; ++i) { mbar_init(&red_full[i], kConsumers); mbar_init(&red_empty[i], 1); }
        mbar_init(x_full, 1);
        mbar_init(x_empty, kConsumers);
        fence_barrier_init();
    }
    __syncthreads();
    const uint32_t ring = smem_u32(smem_raw) + a.ring_off, xs_addr = smem_u32(smem_raw) + a.x_off;
    const uint32_t segb = a.fmt == FMT_Q4_K ? kSeg4 : kSeg6;

    if (warp == kProducer) {
        uint32_t slot = 0, par = 1;
        for (uint32_t ch = 0; ch < nchunk; ++ch) {
            const uint32_t seg0 = ch * (kChunkBlks / 8), seg1 = min(seg0 + kChunkBlks / 8, nseg);
            for (uint32_t k = 0; k < my_units; ++k) {
                const uint32_t u = blockIdx.x + k * gridDim.x;
                for (uint32_t seg = seg0; seg < seg1; ++seg) {
                    const uint32_t off = seg * segb;
                    if (!mbar_wait_bounded(&empty[slot], par, a.status)) return;
                    fence_proxy_async_smem();
                    if (lane == 0) {
                        // one box of 16 rows x the segment; rows past the end of the tensor and blocks past the end of a
                        // row arrive as zeros and count as bytes all the same
                        mbar_arrive_expect_tx(&full[slot], 16 * segb);
                        if (a.swz) tma_box3(ring + slot * a.slot_bytes, &a.map, off / 128, 16 * u, &full[slot]);
                        else tma_box2(ring + slot * a.slot_bytes, &a.map, off / 8, 16 * u, &full[slot]);
                    }
                    if (++slot == S) { slot = 0; par ^= 1u; }
                }
            }
        }
        return;
    }

    if (warp == kFinal) {
        // ---- finalizer: 16 rows x 8 tokens per unit; lane <-> outputs 4 lane .. 4 lane + 3 (row = o / 8, token = o % 8) ----
        float *uacc = (float *)(smem_raw + a.uacc_off);   // running sums of the units while the chunks go by
        uint32_t kk = 0;
        if (!a.cnt) griddep_wait();   // the converted activations and y come from the kernels before
        for (uint32_t ch = 0; ch < nchunk; ++ch) {
            {   // the chunk's activation image: one bulk copy per block (lanes in parallel), after the consumers left the last one
                const uint32_t b0 = ch * kChunkBlks, nb = min(kChunkBlks, nblk - b0);
                if (!mbar_wait_bounded(x_empty, (ch & 1u) ^ 1u, a.status)) return;
                fence_proxy_async_smem();
                const uint32_t blk_bytes = a.ntg * kXqBlk;
                if (lane == 0) mbar_arrive_expect_tx(x_full, nb * blk_bytes);
                __syncwarp();
                if (lane < nb) bulk_g2s_addr(xs_addr + lane * blk_bytes, a.xq + (size_t)(b0 + lane) * blk_bytes, blk_bytes, x_full);
            }
            for (uint32_t k = 0; k < my_units; ++k, ++kk) {
                const uint32_t u = blockIdx.x + k * gridDim.x, buf = kk & 1u;
                if (!mbar_wait_bounded(&red_full[buf], (kk >> 1) & 1u, a.status)) return;
                float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (uint32_t w = 0; w < kConsumers; ++w) {
                    const float4 p = *reinterpret_cast<const float4 *>(red + (buf * kConsumers + w) * 128 + lane * 4);
                    v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_empty[buf]);
                if (nchunk > 1) {
                    float4 *ua = reinterpret_cast<float4 *>(uacc + k * 128 + lane * 4);
                    if (ch > 0) { const float4 p = *ua; v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w; }
                    if (ch + 1 < nchunk) { *ua = make_float4(v[0], v[1], v[2], v[3]); continue; }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t o = lane * 4 + i, row = 16 * u + (o >> 3), tok = o & 7u;
                    if (row < a.rows && tok < n_valid) {
                        const size_t orow = a.out_idx ? a.out_idx[a.col_off + tok] : tok;
                        float *dst = a.y + orow * a.ystride + row;
                        *dst = a.accumulate ? *dst + v[i] : v[i];
                    }
                }
            }
        }
        return;
    }

    // ---- consumers ----
    {
        const uint32_t w = warp % kCW, g = lane >> 2, t = lane & 3u;
        uint32_t ow[4][2];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 2; ++i) ow[c][i] = q4_row_off(w * 144u + 16u + 32u * c + 16u * i + 4u * t, g, a.swz != 0);
        const uint32_t oh = q4_row_off(w * 144u, g, a.swz != 0);
        // this group's next stage (index over the CTA's whole stage sequence), its ring slot and parity
        uint32_t c_it = warp / kCW, c_slot = c_it % S, c_par = 0, kk = 0, it0 = 0;
        bool dead = false;
        for (uint32_t ch = 0; ch < nchunk; ++ch) {
            const uint32_t seg0 = ch * (kChunkBlks / 8), seg1 = min(seg0 + kChunkBlks / 8, nseg);
            mbar_wait_or_die(x_full, ch & 1u, a.status, dead);
            for (uint32_t k = 0; k < my_units; ++k, ++kk) {
                float acc[2][NTG];
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int tg = 0; tg < NTG; ++tg) acc[r][tg] = 0.f;
                const uint32_t it1 = it0 + (seg1 - seg0);
                for (; c_it < it1; c_it += G) {
                    const uint32_t blk = (seg0 + (c_it - it0)) * 8 + w;
                    mbar_wait_or_die(&full[c_slot], c_par, a.status, dead);
                    if (blk < nblk) {
                        const uint32_t xaddr = xs_addr + (blk - ch * kChunkBlks) * (NTG * kXqBlk);
                        float o[2][NTG];
                        if (a.fmt == FMT_Q4_K) {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch4;
                            q4k_block_nx<NTG>(r0, ow, oh, t, xaddr, lane, o);
                        } else {
                            const uint32_t r0 = ring + c_slot * a.slot_bytes + g * kPitch6 + w * 210u;
                            if (w & 1u) q6k_block_nx<NTG, true>(r0 - 2, r0 + 8 * kPitch6 - 2, t, xaddr, lane, o);
                            else q6k_block_nx<NTG, false>(r0, r0 + 8 * kPitch6, t, xaddr, lane, o);
                        }
#pragma unroll
                        for (int tg = 0; tg < NTG; ++tg) {
                            const float xs = ldsf(xaddr + tg * kXqBlk + kFragBytes + 128 + t * 4);   // block scale of token 4 tg + t
                            acc[0][tg] = fmaf(xs, o[0][tg], acc[0][tg]);
                            acc[1][tg] = fmaf(xs, o[1][tg], acc[1][tg]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[c_slot]);
                    c_slot += G;
                    if (c_slot >= S) { c_slot -= S; c_par ^= 1u; }
                }
                it0 = it1;
                // this warp's share of the unit: rows g, g + 8 x tokens t, t + 4 (complete over the warp's columns)
                const uint32_t buf = kk & 1u;
                mbar_wait_or_die(&red_empty[buf], ((kk >> 1) & 1u) ^ 1u, a.status, dead);
                float *pp = red + (buf * kConsumers + warp) * 128;
#pragma unroll
                for (int tg = 0; tg < NTG; ++tg) {
                    pp[g * 8 + 4 * tg + t] = acc[0][tg];
                    pp[(g + 8) * 8 + 4 * tg + t] = acc[1][tg];
                }
                if (NTG == 1) { pp[g * 8 + 4 + t] = 0.f; pp[(g + 8) * 8 + 4 + t] = 0.f; }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_full[buf]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(x_empty);   // done with this chunk of the activation
        }
    }
}

} // namespace

// Consumer groups per CTA (FLB_NX_GROUPS=1 selects the single-group instantiation for comparison).
static int nx_groups() {
    static const int v = getenv("FLB_NX_GROUPS") ? atoi(getenv("FLB_NX_GROUPS")) : 2;
    return v == 1 ? 1 : 2;
}

cudaError_t matmul_tc_nx_init(void) {
    const void *ks[] = {(const void *)matmul_tc_nx_kernel<1, 1>, (const void *)matmul_tc_nx_kernel<2, 1>,
                        (const void *)matmul_tc_nx_kernel<1, 2>, (const void *)matmul_tc_nx_kernel<2, 2>};
    for (const void *k : ks) {
        const cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// Bytes of device scratch the converted activations of one call need (cols <= 18432, up to 8 columns).
size_t matmul_tc_nx_scratch_bytes(uint32_t cols, uint32_t P) {
    return (size_t)(cols / 256) * ((P + 3) / 4) * kXqBlk;
}

// Y[c.out row of column p][r] (+)= dot(W[r], column p), P <= 8 columns, Q4_K or Q6_K, cols a multiple of 256, rows
// 16-byte pitched. xq: scratch of matmul_tc_nx_scratch_bytes(cols, P). cudaErrorNotSupported for other shapes.
cudaError_t launch_matmul_tc_nx(const NxCall &c, uint8_t *xq, uint32_t *status, int sms, cudaStream_t stream) {
    static const bool off = getenv("FLB_TC_NX") && getenv("FLB_TC_NX")[0] == '0';
    const int fmt = c.fmt;
    const uint32_t rows = c.rows, cols = c.cols, P = c.P;
    if (off || (fmt != FMT_Q4_K && fmt != FMT_Q6_K) || cols % 256 != 0 || cols < 256 || P == 0 || P > 8 || rows == 0) return cudaErrorNotSupported;
    const uint32_t rb = (uint32_t)row_bytes(fmt, cols);
    const uint32_t pitch = c.pitch ? c.pitch : rb;
    if ((pitch & 15u) || pitch < rb || (((uintptr_t)c.w) & 15u) || (((uintptr_t)c.x) & 15u) || (((uintptr_t)c.x2) & 15u) || (c.xstride & 3u) || !xq)
        return cudaErrorNotSupported;
    const uint32_t nblk = cols / 256, ntg = (P + 3) / 4;
    const uint32_t units = (rows + 15) / 16;
    const uint32_t grid = units < (uint32_t)sms ? units : (uint32_t)sms;
    // a chunk of 16 blocks of 8 tokens leaves room for two Q6_K stages only: 8 blocks then
    const uint32_t kChunkBlks = (ntg == 2 && fmt == FMT_Q6_K && nblk > 8) ? 8u : kMaxChunkBlks;
    const uint32_t nchunk = (nblk + kChunkBlks - 1) / kChunkBlks;
    const uint32_t my_units_max = (units + grid - 1) / grid;
    if (nchunk > 1 && my_units_max > kMaxChunkUnits) return cudaErrorNotSupported;
    NxArgs k;
    memset(&k, 0, sizeof(k));
    const uint32_t segb = fmt == FMT_Q4_K ? kSeg4 : kSeg6;
    k.swz = (fmt == FMT_Q4_K && pitch % 128 == 0) ? 1 : 0;
    cudaError_t e = k.swz ? tensor_map_lines_swz(&k.map, c.w, rows, pitch, segb / 128, 16)
                          : tensor_map_2d(&k.map, 8, c.w, pitch / 8, rows, pitch, segb / 8, 16, false);
    if (e != cudaSuccess) return e;
    if (!c.skip_convert) {
        e = launch_kernel(act_convert_nx_kernel, dim3(nblk, ntg), dim3(64), 0, stream, c.pdl != 0, c.x, c.x2, c.xstride, P, fmt, xq, ntg,
                          c.cnt, c.col_off, c.col_idx);
        if (e != cudaSuccess) return e;
    }
    k.w = (const uint8_t *)c.w; k.xq = xq; k.y = c.y; k.rows = rows; k.pitch = pitch; k.cols = cols; k.ystride = c.ystride; k.P = P; k.ntg = ntg;
    k.fmt = fmt; k.accumulate = c.accumulate; k.status = status; k.chunk_blks = kChunkBlks;
    k.cnt = c.cnt; k.col_off = c.col_off; k.out_idx = c.out_idx;
    k.slot_bytes = fmt == FMT_Q4_K ? kSlot4 : kSlot6;
    const size_t limit = 227 * 1024 - 1024;
    const int groups = nx_groups();
    const size_t xbytes = (size_t)std::min(nblk, kChunkBlks) * ntg * kXqBlk;
    const size_t uacc = nchunk > 1 ? (size_t)my_units_max * 128 * 4 : 0;
    auto layout = [&](uint32_t ns, size_t &x_off, size_t &uacc_off, size_t &ring_off) {
        x_off = nx_head_bytes(ns, groups);
        uacc_off = (x_off + xbytes + 15) & ~(size_t)15;
        ring_off = (uacc_off + uacc + 1023) & ~(size_t)1023;
        return ring_off + (size_t)ns * k.slot_bytes;
    };
    size_t xo, uo, ro;
    uint32_t nslots = 2;
    if (layout(nslots, xo, uo, ro) > limit) return cudaErrorNotSupported;
    while (nslots < 32 && layout(nslots + 1, xo, uo, ro) <= limit) ++nslots;
    const size_t smem = layout(nslots, xo, uo, ro);
    k.nslots = nslots; k.x_off = (uint32_t)xo; k.uacc_off = (uint32_t)uo; k.ring_off = (uint32_t)ro;
    const dim3 block((groups * kCW + 2) * 32);
    const bool pdl = c.pdl != 0;
    if (groups == 2) {
        if (ntg == 1) return launch_kernel(matmul_tc_nx_kernel<1, 2>, dim3(grid), block, smem, stream, pdl, k);
        return launch_kernel(matmul_tc_nx_kernel<2, 2>, dim3(grid), block, smem, stream, pdl, k);
    }
    if (ntg == 1) return launch_kernel(matmul_tc_nx_kernel<1, 1>, dim3(grid), block, smem, stream, pdl, k);
    return launch_kernel(matmul_tc_nx_kernel<2, 1>, dim3(grid), block, smem, stream, pdl, k);
}

} // namespace flb
