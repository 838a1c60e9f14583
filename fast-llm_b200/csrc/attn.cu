// Single-token (decode) grouped-query attention over an f16 KV cache, split
// along the sequence with an in-kernel log-sum-exp combine. Semantics follow the
// reference's one-head operator fl_op_attn_head
// (src/runtime/decode_params.h:183-232): scores = scale * (q . k_j) over keys
// 0..pos, softmax, context = sum softmax_j * v_j, all in f32; the reference has
// no GPU attention kernel (it runs the operator on one thread,
// src/runtime/gpu_exec.cu:84-88), no GQA and no f16 cache, so layout and
// parallelisation here are new.
//
// Cache layout in HBM: [batch][n_kv_head][kv_stride][128] f16 for K and for V:
// the 64-position tile a CTA needs is one contiguous 16 KB range, fetched with a
// 1-D bulk copy (TMA engine) into a 3-stage shared-memory ring.
//
// Grid = (n_splits, n_kv_head, batch), 256 threads. A CTA serves the 4 query
// heads of its KV head, so every K/V byte is read from HBM once per group.
//   scores : 8 lanes per position x 16 dims each (32 positions per pass), 4 heads
//            per lane, shuffle reduce over the 8 lanes;
//   softmax: warp h owns head h; online (running max / sum), exp in f32;
//   context: 16 lanes per position x 8 dims, 16 positions in flight, 4 heads;
// Each CTA writes (max, sum, context[128]) per head to scratch and takes a
// ticket; the CTA that draws the last ticket of its (batch, kv head) rescales
// and sums the partials in split order (deterministic) and writes the output.
// No CTA ever waits for another one.
#include "common.cuh"
#include "kernels.h"

namespace flb {

namespace {

constexpr int kD = 128;              // head dimension
constexpr int kGroup = 4;            // query heads per KV head handled by one CTA
constexpr int kTile = 64;            // positions per stage
constexpr int kStages = 3;
constexpr int kAttnThreads = 256;
constexpr int kPosPerPass = kAttnThreads / 8;    // scores: 8 lanes per position
constexpr int kPosGroups = kAttnThreads / 16;    // context: 16 lanes per position
constexpr uint32_t kTileBytes = kTile * kD * 2;   // 16 KB
constexpr int kPartStride = kD + 4;  // o[128], m, l, pad (keeps o 16-byte aligned)

struct AttnSmem {
    __half k[kStages][kTile][kD];
    __half v[kStages][kTile][kD];
    float s[kGroup][kTile];          // scaled scores of the current tile
    float p[kTile][kGroup];          // exp(s - m) of the current tile
    float alpha[kGroup];
    uint64_t full[kStages];
    uint32_t is_last;
};

__global__ void __launch_bounds__(kAttnThreads, 2) attn_decode_kernel(const AttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    AttnSmem &sm = *reinterpret_cast<AttnSmem *>(smem_raw);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
    const uint32_t group = a.n_q_head / a.n_kv_head;   // == kGroup (checked on the host)
    if (tid == 0) trace_min(a.trace, 0);
    griddep_wait();   // *pos, q and the appended K/V row come from the previous kernels
    if (tid == 0) trace_min(a.trace, 1);
    const uint32_t kv_len = a.pos ? (uint32_t)(*a.pos) + 1u : a.kv_len;

    const uint32_t tiles_total = (kv_len + kTile - 1) / kTile;
    const uint32_t tps = (tiles_total + a.n_splits - 1) / a.n_splits;
    const uint32_t t0 = split * tps;
    const uint32_t t1 = min(t0 + tps, tiles_total);
    const uint32_t n_tiles = t1 > t0 ? t1 - t0 : 0;

    const __half *kbase = a.k + (uint64_t)b * a.batch_stride + (uint64_t)hkv * a.kv_stride * kD;
    const __half *vbase = a.v + (uint64_t)b * a.batch_stride + (uint64_t)hkv * a.kv_stride * kD;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&sm.full[s], 1);
        sm.is_last = 0;
    }
    fence_barrier_init();
    griddep_launch_dependents();
    __syncthreads();

    auto issue = [&](uint32_t i) {   // thread 0 only: tile t0 + i into slot i % kStages
        const uint32_t slot = i % kStages, p0 = (t0 + i) * kTile;
        const uint32_t n = min((uint32_t)kTile, kv_len - p0);
        mbar_arrive_expect_tx(&sm.full[slot], 2 * n * kD * 2);
        bulk_g2s(&sm.k[slot][0][0], kbase + (uint64_t)p0 * kD, n * kD * 2, &sm.full[slot]);
        bulk_g2s(&sm.v[slot][0][0], vbase + (uint64_t)p0 * kD, n * kD * 2, &sm.full[slot]);
    };
    if (tid == 0)
        for (uint32_t i = 0; i < (uint32_t)kStages && i < n_tiles; ++i) issue(i);

    // q: this thread's 16 dims of the 4 heads: dims 8*ds .. 8*ds+7 and 64+8*ds ..
    // 64+8*ds+7, so that the 8 lanes of a position read 128 contiguous bytes of its
    // K row per load (no shared-memory bank conflicts).
    const uint32_t pp = tid >> 3, ds = tid & 7u;
    const float *qg = a.q + ((uint64_t)b * a.n_q_head + (uint64_t)hkv * group) * kD + ds * 8;
    float q[kGroup][16];
#pragma unroll
    for (int h = 0; h < kGroup; ++h)
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const float4 t = *reinterpret_cast<const float4 *>(qg + h * kD + (i & 7) + (i >> 3) * 64);
            q[h][i] = t.x; q[h][i + 1] = t.y; q[h][i + 2] = t.z; q[h][i + 3] = t.w;
        }

    // context accumulators: 8 dims x 4 heads; positions pg, pg+8, ...
    const uint32_t pg = tid >> 4, dseg = tid & 15u;
    float o[kGroup][8];
#pragma unroll
    for (int h = 0; h < kGroup; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) o[h][i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;   // warp `warp` tracks head `warp`

    for (uint32_t it = 0; it < n_tiles; ++it) {
        const uint32_t slot = it % kStages;
        const uint32_t p0 = (t0 + it) * kTile;
        const uint32_t n = min((uint32_t)kTile, kv_len - p0);
        if (!mbar_wait_bounded(&sm.full[slot], (it / kStages) & 1u, a.status)) return;

        // ---- scores ----
#pragma unroll
        for (int pass = 0; pass < kTile / kPosPerPass; ++pass) {
            const uint32_t p = pass * kPosPerPass + pp;
            float acc[kGroup] = {0.f, 0.f, 0.f, 0.f};
            if (p < n) {
                const uint4 r0 = *reinterpret_cast<const uint4 *>(&sm.k[slot][p][ds * 8]);
                const uint4 r1 = *reinterpret_cast<const uint4 *>(&sm.k[slot][p][64 + ds * 8]);
                const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 kf = __half22float2(*reinterpret_cast<const __half2 *>(&rw[i]));
#pragma unroll
                    for (int h = 0; h < kGroup; ++h) {
                        acc[h] = fmaf(q[h][2 * i], kf.x, acc[h]);
                        acc[h] = fmaf(q[h][2 * i + 1], kf.y, acc[h]);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < kGroup; ++h) {
                acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 1);
                acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 2);
                acc[h] += __shfl_xor_sync(0xffffffffu, acc[h], 4);
            }
            if (ds < kGroup) {
                const float v = ds == 0 ? acc[0] : ds == 1 ? acc[1] : ds == 2 ? acc[2] : acc[3];
                sm.s[ds][p] = p < n ? v * a.scale : -INFINITY;
            }
        }
        __syncthreads();

        // ---- online softmax: warp h <-> head h (warps 0..3) ----
        if (warp < kGroup) {
            const float s0 = sm.s[warp][lane], s1 = sm.s[warp][lane + 32];
            const float m_new = fmaxf(m_run, warp_max(fmaxf(s0, s1)));
            const float e0 = expf(s0 - m_new), e1 = expf(s1 - m_new);
            const float al = expf(m_run - m_new);
            sm.p[lane][warp] = e0;
            sm.p[lane + 32][warp] = e1;
            l_run = l_run * al + warp_sum(e0 + e1);
            m_run = m_new;
            if (lane == 0) sm.alpha[warp] = al;
        }
        __syncthreads();

        // ---- context ----
        {
            const float4 al = *reinterpret_cast<const float4 *>(sm.alpha);
            const float alv[kGroup] = {al.x, al.y, al.z, al.w};
#pragma unroll
            for (int h = 0; h < kGroup; ++h)
#pragma unroll
                for (int i = 0; i < 8; ++i) o[h][i] *= alv[h];
#pragma unroll
            for (int j = 0; j < kTile / kPosGroups; ++j) {
                const uint32_t p = j * kPosGroups + pg;
                if (p < n) {
                    const uint4 r = *reinterpret_cast<const uint4 *>(&sm.v[slot][p][dseg * 8]);
                    const float4 w = *reinterpret_cast<const float4 *>(&sm.p[p][0]);
                    const float wv[kGroup] = {w.x, w.y, w.z, w.w};
                    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 vf = __half22float2(*reinterpret_cast<const __half2 *>(&rw[i]));
#pragma unroll
                        for (int h = 0; h < kGroup; ++h) {
                            o[h][2 * i] = fmaf(wv[h], vf.x, o[h][2 * i]);
                            o[h][2 * i + 1] = fmaf(wv[h], vf.y, o[h][2 * i + 1]);
                        }
                    }
                }
            }
        }
        __syncthreads();   // tile fully consumed: s/p reusable, slot reusable
        if (tid == 0 && it + kStages < n_tiles) {
            fence_proxy_async_smem();
            issue(it + kStages);
        }
    }

    // ---- reduce the 8 position groups, write this split's partial ----
    float *red = reinterpret_cast<float *>(&sm.k[0][0][0]);   // [kPosGroups][kGroup][kD] floats = 32 KB, ring is idle now
#pragma unroll
    for (int h = 0; h < kGroup; ++h)
#pragma unroll
        for (int i = 0; i < 8; ++i) red[(pg * kGroup + h) * kD + dseg * 8 + i] = o[h][i];
    __syncthreads();
    if (warp < kGroup) {
        const uint32_t h = warp;   // head within the group
        float *part = a.part + (((uint64_t)b * a.n_q_head + (uint64_t)hkv * group + h) * a.n_splits + split) * kPartStride;
#pragma unroll
        for (int k = 0; k < kD / 32; ++k) {
            const uint32_t d = lane + 32 * k;
            float t = 0.f;
#pragma unroll
            for (int g = 0; g < kPosGroups; ++g) t += red[(g * kGroup + h) * kD + d];
            part[d] = t;
        }
        if (lane == 0) { part[kD] = m_run; part[kD + 1] = l_run; }
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

    // ---- combine: warps h and h+4 <-> head h. Every lane first derives the global
    // maximum and the rescaled sum from all splits' (m, l); warp h then accumulates
    // the context of the even splits and warp h+4 of the odd ones (each lane 4
    // dims, 16 loads in flight), and the two halves are added in a fixed order. ----
    {
        const uint32_t h = warp & 3u, half = warp >> 2;
        const uint64_t hq = (uint64_t)b * a.n_q_head + (uint64_t)hkv * group + h;
        const float *part = a.part + hq * a.n_splits * kPartStride;
        const uint32_t S = a.n_splits;
        const float m0 = lane < S ? __ldcg(part + (uint64_t)lane * kPartStride + kD) : -INFINITY;
        const float m1 = lane + 32 < S ? __ldcg(part + (uint64_t)(lane + 32) * kPartStride + kD) : -INFINITY;
        const float l0 = lane < S ? __ldcg(part + (uint64_t)lane * kPartStride + kD + 1) : 0.f;
        const float l1 = lane + 32 < S ? __ldcg(part + (uint64_t)(lane + 32) * kPartStride + kD + 1) : 0.f;
        const float mx = warp_max(fmaxf(m0, m1));
        const float w0 = m0 == -INFINITY ? 0.f : expf(m0 - mx);
        const float w1 = m1 == -INFINITY ? 0.f : expf(m1 - mx);
        const float L = warp_sum(l0 * w0 + l1 * w1);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = half; s0 < S; s0 += 32) {
            float4 o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
                o[j] = s0 + 2 * j < S ? __ldcg(reinterpret_cast<const float4 *>(part + (uint64_t)(s0 + 2 * j) * kPartStride) + lane)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint32_t s = s0 + 2 * j;
                const float w = __shfl_sync(0xffffffffu, s < 32 ? w0 : w1, s & 31u);
                acc.x = fmaf(o[j].x, w, acc.x); acc.y = fmaf(o[j].y, w, acc.y);
                acc.z = fmaf(o[j].z, w, acc.z); acc.w = fmaf(o[j].w, w, acc.w);
            }
        }
        float4 *xch = reinterpret_cast<float4 *>(&sm.v[0][0][0]);   // the V ring is idle now
        if (half == 1) xch[h * 32 + lane] = acc;
        __syncthreads();
        if (half == 0) {
            const float4 other = xch[h * 32 + lane];
            const float inv = 1.0f / L;
            acc.x = (acc.x + other.x) * inv; acc.y = (acc.y + other.y) * inv;
            acc.z = (acc.z + other.z) * inv; acc.w = (acc.w + other.w) * inv;
            reinterpret_cast<float4 *>(a.out + hq * kD)[lane] = acc;
        }
    }
    if (tid == 0) {
        a.tickets[b * a.n_kv_head + hkv] = 0;   // ready for the next launch
        trace_max(a.trace, 3);
    }
}

} // namespace

cudaError_t attn_init(void) {
    return cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnSmem));
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
    if (records > kStaticMaxRecords || (uint64_t)a.n_kv_head * a.batch > kStaticMaxTickets)
        return cudaErrorMemoryAllocation;   // the caller turns this into its size message
    if (!g_static_ptr[device]) {
        float *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_attn_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_ptr[device] = ptr;
    }
    float *ptr = g_static_ptr[device];
    a.part = ptr;
    a.tickets = reinterpret_cast<uint32_t *>(ptr + kStaticPartFloats);
    const cudaError_t e = cudaMemsetAsync(a.tickets, 0, (size_t)a.n_kv_head * a.batch * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    return launch_attn_decode(a, stream);
}

size_t attn_static_max_records(void) { return kStaticMaxRecords; }
uint32_t attn_static_max_tickets(void) { return kStaticMaxTickets; }

cudaError_t launch_attn_decode(const AttnArgs &a, cudaStream_t stream) {
    if (a.n_kv_head == 0 || a.n_q_head != a.n_kv_head * kGroup || a.n_splits == 0 || a.batch == 0)
        return cudaErrorInvalidValue;
    if (a.pos == nullptr && a.kv_len == 0) return cudaErrorInvalidValue;
    const dim3 grid(a.n_splits, a.n_kv_head, a.batch);
    return launch_kernel(attn_decode_kernel, grid, dim3(kAttnThreads), sizeof(AttnSmem), stream, a.pdl != 0, a);
}

} // namespace flb
