// Q4_K dequantize-matmul for up to 8 activation columns on the Blackwell tensor cores proper: tcgen05.mma with the
// accumulator in tensor memory (replaces the nx-column STREAM_DOT of the reference, include/fastllm/fastllm.h:87-96,
// src/runtime/kernels_gpu.h:682-740 gdot_i8k_q4_K_mc, and the add_dot_m call sites of src/model/decoder.cpp:482-528).
//
// Why this form: with mma.sync (matvec_tc.cu, matvec_tc_nx.cu) every lane has to bring its weights into a register
// fragment, feed the instruction, read the accumulators back and scale them: about 490-620 warp instructions per
// 16 rows x 256 columns, of which 160 are the unpack itself. Here the CUDA cores only unpack: a thread turns 32 packed
// bytes of ONE row into 64 f16 values q * sc (the 6-bit sub-block scale folded in exactly by one fused multiply-add
// per pair) and stores them into the A tile in shared memory; the contraction over k, the sum across the row and the
// accumulation over the super-block happen in the tensor core, which reads A and B from shared memory and keeps
// D (128 rows x 16 columns, f32) in tensor memory.
//
//   * tile: 128 rows x a range of super-blocks (split-K: a work item is (row tile, k range); the partial results of a
//     row tile are added in k order by the last item to finish, through a ticket, so the result does not depend on timing);
//   * B operand: the activation as f16 (hi, lo) pairs, 2 columns of D per token (22 significant bits per element, exact
//     products), prepared once per call by act_convert_umma_kernel in the 128-byte-swizzled K-major layout and streamed
//     beside the weights (it is the same for every CTA and comes from L2);
//   * per super-block: D = sum over the 4 chunks of 64 columns of A_chunk B_chunk (16 instructions of K = 16), then the
//     epilogue warps read D from tensor memory and add xs * (d * D - dmin * sum_sb m_sb S_sb) in f32, d / dmin / mins
//     being the row's own header, xs the block scale and S_sb the sub-block sums of the activation;
//   * warps: 16 unpack (4 groups of 128 threads: group c takes the 32-byte chunk c of every row), 4 epilogue (one per
//     32 lanes of tensor memory), 1 TMA producer, 1 MMA issuer (one elected thread).
// Every wait is bounded; a wait that runs out sets the status word and an abort flag all roles watch, the launch then
// drains, frees its tensor memory and returns.
#include "common.cuh"
#include "kernels.h"

#include <cuda.h>
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace flb {

namespace {

constexpr uint32_t kRows = 128;                       // rows of a tile = lanes of tensor memory
constexpr uint32_t kUnpackWarps = 16, kEpiWarp0 = 16, kProducerWarp = 20, kMmaWarp = 21, kThreads = 22 * 32;
constexpr uint32_t kRawW = kRows * 144;               // packed Q4_K bytes of a stage: 128 rows x one super-block
constexpr uint32_t kBChunk = 2048;                    // B tile of one 64-column chunk: 16 rows (8 tokens x hi, lo) x 128 B
constexpr uint32_t kBBytes = 4 * kBChunk;
constexpr uint32_t kSideFloats = 8 * 9;               // per token: 8 sub-block sums and the block scale
constexpr uint32_t kXuBlk = kBBytes + 512;            // one super-block of the converted activation in global memory
constexpr uint32_t kStage = ((kRawW + kXuBlk + 1023u) / 1024u) * 1024u;
constexpr uint32_t kATile = kRows * 128;              // 128 rows x 64 f16
constexpr uint32_t kNA = 5, kNS = 5;                  // A tiles and raw stages in flight
constexpr uint32_t kHdrBuf = kRows * 16 + 512;        // per accumulator buffer: the rows' headers and the side data
constexpr uint32_t kTmemCols = 32;                    // two accumulators of 16 columns

struct UmArgs {
    CUtensorMap map;                  // [rows][pitch / 8] 8-byte elements, box 18 x 128
    const uint8_t *xu;                // converted activation, kXuBlk bytes per super-block
    float *y;
    uint32_t ystride, rows, nblk, P;
    uint32_t n_tiles, splits, blk_per_split;
    int accumulate;
    const uint32_t *cnt, *out_idx;
    uint32_t col_off;
    float *scratch;                   // [n_tiles * splits][128][8] partial results (splits > 1)
    uint32_t *tickets;                // [n_tiles][4 epilogue warps], zero between launches
    uint32_t *status;
};

struct UmSmem {
    uint8_t *a;          // [kNA][kATile], 1024-aligned
    uint8_t *stage;      // [kNS][kStage]
    uint8_t *hdr;        // [2][kHdrBuf]
    uint64_t *raw_full, *raw_empty;   // [kNS]
    uint64_t *a_full, *a_empty;       // [kNA]
    uint64_t *acc_full, *acc_empty;   // [2]
    uint64_t *hdr_full;               // [2]: the rows' headers of the accumulator's super-block are in place
    uint32_t *tmem_slot, *abort_flag;
};
constexpr size_t kUmSmemBytes = (size_t)kNA * kATile + (size_t)kNS * kStage + 2 * kHdrBuf + (2 * kNS + 2 * kNA + 6) * 8 + 64;

__device__ __forceinline__ UmSmem um_carve(uint8_t *base) {
    UmSmem s;
    s.a = base;
    s.stage = base + kNA * kATile;
    s.hdr = s.stage + kNS * kStage;
    uint64_t *b = reinterpret_cast<uint64_t *>(s.hdr + 2 * kHdrBuf);
    s.raw_full = b; s.raw_empty = b + kNS;
    s.a_full = b + 2 * kNS; s.a_empty = b + 2 * kNS + kNA;
    s.acc_full = b + 2 * kNS + 2 * kNA; s.acc_empty = s.acc_full + 2;
    s.hdr_full = s.acc_empty + 2;
    s.tmem_slot = reinterpret_cast<uint32_t *>(s.hdr_full + 2);
    s.abort_flag = s.tmem_slot + 1;
    return s;
}

// Bounded wait that also gives up as soon as another thread of the CTA has given up.
__device__ __noinline__ bool um_wait_slow(uint64_t *bar, uint32_t parity, uint32_t *status, volatile uint32_t *abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > 1000000000ull) {
            atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
            *abort_flag = 1u;
            return false;
        }
    }
}
__device__ __forceinline__ bool um_wait(uint64_t *bar, uint32_t parity, uint32_t *status, uint32_t *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    return um_wait_slow(bar, parity, status, abort_flag);
}
__device__ __forceinline__ void um_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint4 um_lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void um_sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint32_t um_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// x * s + o for both halves, one rounding (the exact result q * sc is representable, so there is none)
__device__ __forceinline__ uint32_t um_hfma2(uint32_t x, __half2 s, __half2 o) {
    const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&x), s, o);
    return *reinterpret_cast<const uint32_t *>(&r);
}
// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups `sbo` bytes apart.
__device__ __forceinline__ uint64_t um_desc(uint32_t saddr, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = 16.
constexpr uint32_t kIdesc = (1u << 4) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void um_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
                 : "memory");
}
// Arrives on the barrier once every tensor-core instruction this thread issued before has completed.
__device__ __forceinline__ void um_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void um_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void um_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
template <int K>
__device__ __forceinline__ float um_u8f(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | K)) - 8388608.0f;
}

// ---- the activation as the B operand --------------------------------------------------------------------------
// One CTA per 256-column block, 128 threads = 8 tokens x 16 lanes; lane hl of a token holds columns 16 hl .. 16 hl + 15.
// Per block kXuBlk bytes: four chunk tiles of 16 rows x 128 bytes (row 2 p: the hi parts of token p, row 2 p + 1: the lo
// parts; 16-byte piece j of a row stored at j ^ (row & 7): the 128-byte swizzle), then per token 8 sub-block sums and
// the block scale 2^e (x = 2^e (hi + lo)). Position k of a chunk's K axis holds column pi(k) of the chunk, the order in
// which the unpack produces the weights: pi(8 j + e) = 4 j + {0, 2, 1, 3, 32, 34, 33, 35}[e].
__global__ void __launch_bounds__(128) act_convert_umma_kernel(const float *__restrict__ x, const float *__restrict__ x2, uint32_t xstride,
                                                               uint32_t P, uint8_t *__restrict__ xu, const uint32_t *__restrict__ cnt,
                                                               uint32_t col_off, const uint32_t *__restrict__ col_idx) {
    const uint32_t blk = blockIdx.x, p = threadIdx.x >> 4, hl = threadIdx.x & 15u;
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
        if (x2) {   // SiLU(x) * x2 (fl_op_silu_mul, src/runtime/decode_params.h:267-272)
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
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));   // over the token's 16 lanes
    // block scale 2^e with amax / 2^e in [2^13, 2^14); e clamped so that 2^e and 2^-e are normal floats
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 13;
    e = amax > 0.f ? max(-126, min(e, 114)) : 0;
    const float inv_s = __uint_as_float((uint32_t)(127 - e) << 23);
    uint8_t *base = xu + (size_t)blk * kXuBlk;
    // columns 16 hl + i: chunk hl / 4, nibble half (hl / 2) & 1, 16-byte piece j = 4 (hl & 1) + i / 4
    uint8_t *tile = base + (hl >> 2) * kBChunk;
    const uint32_t half = (hl >> 1) & 1u;
    float sum = 0.f;
#pragma unroll
    for (int g4 = 0; g4 < 4; ++g4) {
        __half hh[4], ll[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const float s = v[4 * g4 + t] * inv_s;
            hh[t] = __float2half_rn(s);
            ll[t] = __float2half_rn(s - __half2float(hh[t]));
            sum += __half2float(hh[t]) + __half2float(ll[t]);
        }
        const uint32_t j = 4 * (hl & 1u) + g4;
        uint2 hi, lo;   // K order within the piece: columns t = 0, 2, 1, 3
        hi.x = (uint32_t)__half_as_ushort(hh[0]) | ((uint32_t)__half_as_ushort(hh[2]) << 16);
        hi.y = (uint32_t)__half_as_ushort(hh[1]) | ((uint32_t)__half_as_ushort(hh[3]) << 16);
        lo.x = (uint32_t)__half_as_ushort(ll[0]) | ((uint32_t)__half_as_ushort(ll[2]) << 16);
        lo.y = (uint32_t)__half_as_ushort(ll[1]) | ((uint32_t)__half_as_ushort(ll[3]) << 16);
        const uint32_t r_hi = 2 * p, r_lo = 2 * p + 1;
        *reinterpret_cast<uint2 *>(tile + r_hi * 128 + ((j ^ (r_hi & 7u)) << 4) + half * 8) = hi;
        *reinterpret_cast<uint2 *>(tile + r_lo * 128 + ((j ^ (r_lo & 7u)) << 4) + half * 8) = lo;
    }
    const float sum32 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
    float *side = reinterpret_cast<float *>(base + kBBytes);
    if ((hl & 1u) == 0) side[p * 9 + (hl >> 1)] = sum32;
    if (hl == 0) side[p * 9 + 8] = __uint_as_float((uint32_t)(127 + e) << 23);
}

// ---- the kernel -----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) matmul_umma_kernel(const __grid_constant__ UmArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint32_t n_valid = a.P;
    if (a.cnt) { const uint32_t c = *a.cnt; n_valid = c > a.col_off ? min(c - a.col_off, a.P) : 0u; }
    if (n_valid == 0) return;   // no column of this call exists (uniform over the grid)
    const UmSmem sm = um_carve(smem_raw);
    if (tid == 0) {
        for (uint32_t i = 0; i < kNS; ++i) { mbar_init(&sm.raw_full[i], 1); mbar_init(&sm.raw_empty[i], kUnpackWarps + 1); }
        for (uint32_t i = 0; i < kNA; ++i) { mbar_init(&sm.a_full[i], 4); mbar_init(&sm.a_empty[i], 1); }
        for (uint32_t i = 0; i < 2; ++i) { mbar_init(&sm.acc_full[i], 1); mbar_init(&sm.acc_empty[i], 4); mbar_init(&sm.hdr_full[i], 4); }
        *sm.abort_flag = 0u;
        fence_barrier_init();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    um_fence_before();
    __syncthreads();
    um_fence_after();
    const uint32_t tbase = *sm.tmem_slot;
    const uint32_t n_items = a.n_tiles * a.splits;
    const uint32_t a_base = smem_u32(sm.a), st_base = smem_u32(sm.stage), hdr_base = smem_u32(sm.hdr);
    bool dead = false;

    if (warp == kProducerWarp) {
        if (lane == 0) {
            uint32_t q = 0;   // super-blocks of this CTA so far
            for (uint32_t it = blockIdx.x; it < n_items && !dead; it += gridDim.x) {
                const uint32_t tile = it / a.splits, split = it % a.splits;
                const uint32_t b0 = split * a.blk_per_split, b1 = min(a.nblk, b0 + a.blk_per_split);
                for (uint32_t blk = b0; blk < b1; ++blk, ++q) {
                    const uint32_t st = q % kNS, use = q / kNS;
                    if (!um_wait(&sm.raw_empty[st], (use & 1u) ^ 1u, a.status, sm.abort_flag)) { dead = true; break; }
                    fence_proxy_async_smem();
                    const uint32_t dst = st_base + st * kStage;
                    mbar_arrive_expect_tx(&sm.raw_full[st], kRawW + kXuBlk);
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                                 "l"(&a.map), "r"(blk * 18u), "r"(tile * kRows), "r"(smem_u32(&sm.raw_full[st]))
                                 : "memory");
                    bulk_g2s_addr(dst + kRawW, a.xu + (size_t)blk * kXuBlk, kXuBlk, &sm.raw_full[st]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            uint32_t q = 0;
            for (uint32_t it = blockIdx.x; it < n_items && !dead; it += gridDim.x) {
                const uint32_t split = it % a.splits;
                const uint32_t b0 = split * a.blk_per_split, b1 = min(a.nblk, b0 + a.blk_per_split);
                for (uint32_t blk = b0; blk < b1 && !dead; ++blk, ++q) {
                    const uint32_t st = q % kNS, ab = q & 1u;
                    if (!um_wait(&sm.raw_full[st], (q / kNS) & 1u, a.status, sm.abort_flag)) { dead = true; break; }
                    if (!um_wait(&sm.acc_empty[ab], ((q >> 1) & 1u) ^ 1u, a.status, sm.abort_flag)) { dead = true; break; }
                    const uint32_t d_tmem = tbase + ab * 16u;
                    const uint32_t b_tile = st_base + st * kStage + kRawW;
                    for (uint32_t c = 0; c < 4; ++c) {
                        const uint32_t n = 4 * q + c, slot = n % kNA;
                        if (!um_wait(&sm.a_full[slot], (n / kNA) & 1u, a.status, sm.abort_flag)) { dead = true; break; }
                        um_fence_after();
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk)
                            um_mma(d_tmem, um_desc(a_base + slot * kATile + kk * 32u, 1024u), um_desc(b_tile + c * kBChunk + kk * 32u, 1024u),
                                   (c | kk) != 0u ? 1u : 0u);
                        um_commit(&sm.a_empty[slot]);
                    }
                    if (dead) break;
                    um_commit(&sm.acc_full[ab]);
                    um_commit(&sm.raw_empty[st]);   // the B tile of the stage has been read
                }
            }
        }
    } else if (warp < kUnpackWarps) {
        // ---- unpack: thread = (row, 32-byte chunk c); A[row][k] = q * sc as f16 ----
        const uint32_t c = warp >> 2, row = (warp & 3u) * 32u + lane;
        const uint32_t ML = 0x000F000Fu, KL = 0x64006400u, MH = 0x00F000F0u, KH = 0x54005400u;
        uint32_t q = 0;
        for (uint32_t it = blockIdx.x; it < n_items && !dead; it += gridDim.x) {
            const uint32_t split = it % a.splits;
            const uint32_t b0 = split * a.blk_per_split, b1 = min(a.nblk, b0 + a.blk_per_split);
            for (uint32_t blk = b0; blk < b1; ++blk, ++q) {
                const uint32_t st = q % kNS, ab = q & 1u;
                if (!um_wait(&sm.raw_full[st], (q / kNS) & 1u, a.status, sm.abort_flag)) { dead = true; break; }
                const uint32_t raw = st_base + st * kStage + row * 144u;
                const uint4 hdr = um_lds128(raw);
                const uint4 w0 = um_lds128(raw + 16u + 32u * c), w1 = um_lds128(raw + 32u + 32u * c);
                if (c == 0) {
                    // the row's d | dmin and its eight mins for the epilogue, and the block's side data
                    if (!um_wait(&sm.acc_empty[ab], ((q >> 1) & 1u) ^ 1u, a.status, sm.abort_flag)) { dead = true; break; }
                    const uint32_t mn_lo = hdr.z & 0x3F3F3F3Fu, mn_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
                    um_sts128(hdr_base + ab * kHdrBuf + row * 16u, hdr.x, mn_lo, mn_hi, 0u);
                    if (row < kSideFloats) {
                        uint32_t v;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(st_base + st * kStage + kRawW + kBBytes + row * 4u));
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(hdr_base + ab * kHdrBuf + kRows * 16u + row * 4u), "r"(v) : "memory");
                    }
                    __syncwarp();
                    if (lane == 0) um_arrive(&sm.hdr_full[ab]);
                }
                // 6-bit scales of sub-blocks 2c (low nibbles) and 2c + 1 (high nibbles): fl_q4k_scale_min, src/runtime/quants.h:121-129
                uint32_t scb;   // bytes 0, 1: the two scales
                if (c < 2) scb = (hdr.y >> (16u * c)) & 0x3F3Fu;
                else scb = (((hdr.w >> (16u * (c - 2))) & 0x0F0Fu) | (((hdr.y >> (16u * (c - 2))) >> 2) & 0x3030u));
                // as f16 pairs (sc, sc): the byte under 0x64 is 1024 + sc; the offsets -1024 sc and -64 sc are exact too
                const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
                const uint32_t sLb = __byte_perm(scb, 0x64646464u, 0x4040u), sHb = __byte_perm(scb, 0x64646464u, 0x4141u);
                const __half2 sL = __hsub2(*reinterpret_cast<const __half2 *>(&sLb), k1024), sH = __hsub2(*reinterpret_cast<const __half2 *>(&sHb), k1024);
                const __half2 oL = __hmul2(sL, __floats2half2_rn(-1024.f, -1024.f)), oH = __hmul2(sH, __floats2half2_rn(-64.f, -64.f));
                const uint32_t n = 4 * q + c, slot = n % kNA;
                if (!um_wait(&sm.a_empty[slot], ((n / kNA) & 1u) ^ 1u, a.status, sm.abort_flag)) { dead = true; break; }
                const uint32_t arow = a_base + slot * kATile + row * 128u, sw = row & 7u;
#pragma unroll
                for (uint32_t j = 0; j < 8; ++j) {
                    const uint32_t W = j < 4 ? (j == 0 ? w0.x : j == 1 ? w0.y : j == 2 ? w0.z : w0.w) : (j == 4 ? w1.x : j == 5 ? w1.y : j == 6 ? w1.z : w1.w);
                    const uint32_t V = W >> 8;
                    // bytes 0, 2 | bytes 1, 3 of the word, low nibbles then high nibbles: columns 4j + {0, 2, 1, 3} and 32 + the same
                    um_sts128(arow + ((j ^ sw) << 4), um_hfma2(um_and_or(W, ML, KL), sL, oL), um_hfma2(um_and_or(V, ML, KL), sL, oL),
                              um_hfma2(um_and_or(W, MH, KH), sH, oH), um_hfma2(um_and_or(V, MH, KH), sH, oH));
                }
                fence_proxy_async_smem();   // the tensor core reads the tile through the async proxy
                __syncwarp();
                if (lane == 0) {
                    um_arrive(&sm.a_full[slot]);
                    um_arrive(&sm.raw_empty[st]);
                }
            }
        }
    } else {
        // ---- epilogue: warp e reads lanes 32 e .. 32 e + 31 of tensor memory (rows of the tile) ----
        const uint32_t ew = warp - kEpiWarp0, row = ew * 32u + lane;
        uint32_t q = 0;
        for (uint32_t it = blockIdx.x; it < n_items; it += gridDim.x) {
            const uint32_t tile = it / a.splits, split = it % a.splits;
            const uint32_t b0 = split * a.blk_per_split, b1 = min(a.nblk, b0 + a.blk_per_split);
            float acc[8];
#pragma unroll
            for (int p = 0; p < 8; ++p) acc[p] = 0.f;
            for (uint32_t blk = b0; blk < b1 && !dead; ++blk, ++q) {
                const uint32_t ab = q & 1u;
                if (!um_wait(&sm.acc_full[ab], (q >> 1) & 1u, a.status, sm.abort_flag)) { dead = true; break; }
                if (!um_wait(&sm.hdr_full[ab], (q >> 1) & 1u, a.status, sm.abort_flag)) { dead = true; break; }
                um_fence_after();
                uint32_t d[16];
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
                               "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
                             : "r"(tbase + ((ew * 32u) << 16) + ab * 16u));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                um_fence_before();
                const uint32_t hb = hdr_base + ab * kHdrBuf;
                const uint4 h = um_lds128(hb + row * 16u);
                const float dd = h2f_bits((uint16_t)(h.x & 0xFFFFu)), dmin = h2f_bits((uint16_t)(h.x >> 16));
                float mn[8];
                mn[0] = um_u8f<0>(h.y); mn[1] = um_u8f<1>(h.y); mn[2] = um_u8f<2>(h.y); mn[3] = um_u8f<3>(h.y);
                mn[4] = um_u8f<0>(h.z); mn[5] = um_u8f<1>(h.z); mn[6] = um_u8f<2>(h.z); mn[7] = um_u8f<3>(h.z);
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    if ((uint32_t)p < n_valid) {   // uniform
                        const uint32_t sa = hb + kRows * 16u + p * 36u;
                        float m = 0.f;
#pragma unroll
                        for (int sb = 0; sb < 8; ++sb) {
                            float s;
                            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(s) : "r"(sa + sb * 4u));
                            m = fmaf(mn[sb], s, m);
                        }
                        float xs;
                        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xs) : "r"(sa + 32u));
                        const float qv = __uint_as_float(d[2 * p]) + __uint_as_float(d[2 * p + 1]);
                        acc[p] = fmaf(xs, dd * qv - dmin * m, acc[p]);
                    }
                }
                __syncwarp();
                if (lane == 0) um_arrive(&sm.acc_empty[ab]);
            }
            if (dead) break;
            // ---- the item's rows: straight to y, or to the scratch and through the ticket of the row tile ----
            const uint32_t grow = tile * kRows + row;
            if (a.splits > 1) {
                // every epilogue warp settles its own 32 rows: no barrier between warps, so a warp that gave up cannot
                // leave another one waiting
                float *part = a.scratch + ((size_t)it * kRows + row) * 8;
                *reinterpret_cast<float4 *>(part) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4 *>(part + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
                __threadfence();
                __syncwarp();
                uint32_t last = 0;
                if (lane == 0) {
                    const uint32_t t = atomicAdd(&a.tickets[tile * 4 + ew], 1u);
                    last = t == a.splits - 1u ? 1u : 0u;
                    if (last) a.tickets[tile * 4 + ew] = 0u;   // every other item of the tile has arrived: ready for the next launch
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (!last) continue;
                __threadfence();
#pragma unroll
                for (int p = 0; p < 8; ++p) acc[p] = 0.f;
                for (uint32_t s = 0; s < a.splits; ++s) {   // in k order, whatever order the items finished in
                    const float *src = a.scratch + ((size_t)(tile * a.splits + s) * kRows + row) * 8;
                    const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(src)), u1 = __ldcg(reinterpret_cast<const float4 *>(src + 4));
                    acc[0] += u0.x; acc[1] += u0.y; acc[2] += u0.z; acc[3] += u0.w;
                    acc[4] += u1.x; acc[5] += u1.y; acc[6] += u1.z; acc[7] += u1.w;
                }
            }
            if (grow < a.rows) {
#pragma unroll
                for (int p = 0; p < 8; ++p) {
                    if ((uint32_t)p < n_valid) {
                        const size_t ob = a.out_idx ? a.out_idx[a.col_off + p] : (uint32_t)p;
                        float *dst = a.y + ob * a.ystride + grow;
                        *dst = a.accumulate ? *dst + acc[p] : acc[p];
                    }
                }
            }
        }
    }
    // every thread comes here, whatever happened; then the tensor memory goes back
    um_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        um_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(kTmemCols) : "memory");
    }
}

// Off unless FLB_UMMA=1 (read at every call, so that one process can run both kernels): on the shapes of the decode
// step the 128-row tile makes the weight stream fetch 144-byte pieces of 128 different rows per stage, two 128-byte
// lines each, and the TMA unit's rate of about one line per 6.5 cycles then caps the stream at 2.7 TB/s; measured on
// the gate|up shape with 8 columns: 56 us per pass against 37 us for the mma.sync kernel (37 us already with the
// unpack, the tensor-core instructions and the epilogue all switched off).
bool umma_on() {
    const char *v = getenv("FLB_UMMA");
    return v && v[0] == '1';
}

} // namespace

size_t matmul_umma_xu_bytes(uint32_t cols) { return (size_t)(cols / 256) * kXuBlk; }
size_t matmul_umma_scratch_bytes(void) { return (size_t)16 << 20; }
size_t matmul_umma_ticket_count(void) { return 4 * 4096; }

cudaError_t matmul_umma_init(void) {
    return cudaFuncSetAttribute(matmul_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmSmemBytes + 1024);
}

// One pass over a Q4_K tensor for up to 8 columns. cudaErrorNotSupported when the shape does not qualify (the caller
// then takes the mma.sync kernel).
cudaError_t launch_matmul_umma(const NxCall &c, uint8_t *xu, float *scratch, uint32_t *tickets, uint32_t *status, int sms,
                               cudaStream_t stream) {
    if (!umma_on() || c.fmt != FMT_Q4_K || c.P < 1 || c.P > 8 || c.cols % 256 != 0 || c.cols < 256 || c.rows == 0) return cudaErrorNotSupported;
    const uint32_t pitch = c.pitch ? c.pitch : (uint32_t)row_bytes(c.fmt, c.cols);
    if ((pitch & 15u) || (((uintptr_t)c.w) & 15u) || (((uintptr_t)c.x) & 15u) || (c.xstride & 3u) || (((uintptr_t)c.x2) & 15u)) return cudaErrorNotSupported;
    UmArgs k;
    memset(&k, 0, sizeof(k));
    const uint32_t nblk = c.cols / 256, n_tiles = (c.rows + kRows - 1) / kRows;
    if ((size_t)n_tiles * 4 > matmul_umma_ticket_count()) return cudaErrorNotSupported;
    // split-K: the number of k ranges that gives the shortest schedule (waves of items x super-blocks per item), each
    // range at least 2 super-blocks, the partial results within the scratch
    uint32_t best_s = 1, best_cost = 0xFFFFFFFFu;
    for (uint32_t s = 1; s <= nblk && s <= 16; ++s) {
        const uint32_t bps = (nblk + s - 1) / s, s_eff = (nblk + bps - 1) / bps;
        if (s_eff != s || (s > 1 && bps < 2)) continue;
        if (s > 1 && (size_t)n_tiles * s * kRows * 8 * 4 > matmul_umma_scratch_bytes()) continue;
        const uint32_t waves = (n_tiles * s + (uint32_t)sms - 1) / (uint32_t)sms;
        const uint32_t cost = waves * (bps + 1) + (s > 1 ? 1u : 0u);   // + 1: the item's own start and end
        if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    k.splits = best_s;
    k.blk_per_split = (nblk + best_s - 1) / best_s;
    k.n_tiles = n_tiles; k.nblk = nblk; k.rows = c.rows; k.P = c.P;
    cudaError_t e = tensor_map_2d(&k.map, 8, c.w, pitch / 8, c.rows, pitch, 18, kRows, false);
    if (e != cudaSuccess) return e;
    if (!c.skip_convert) {
        act_convert_umma_kernel<<<nblk, 128, 0, stream>>>(c.x, c.x2, c.xstride, c.P, xu, c.cnt, c.col_off, c.col_idx);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    k.xu = xu; k.y = c.y; k.ystride = c.ystride; k.accumulate = c.accumulate;
    k.cnt = c.cnt; k.out_idx = c.out_idx; k.col_off = c.col_off;
    k.scratch = scratch; k.tickets = tickets; k.status = status;
    const uint32_t n_items = n_tiles * best_s;
    const uint32_t grid = n_items < (uint32_t)sms ? n_items : (uint32_t)sms;
    return launch_kernel(matmul_umma_kernel, dim3(grid), dim3(kThreads), kUmSmemBytes + 1024, stream, false, k);
}

} // namespace flb
