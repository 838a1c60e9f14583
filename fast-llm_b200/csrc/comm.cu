// Exchange steps of the tensor-parallel decode step (one process per GPU, up to
// 8 GPUs of one NVSwitch domain). The reference has no multi-GPU path; the
// partition follows the decode graph: Q/K/V, gate/up and the head are split by
// output rows (KV heads), O and down by input columns, so a layer needs two
// sums of a hidden-size vector over the ranks and the step one exchange of the
// per-rank (best, index, runner-up) of the logits.
//
// One-shot push all-reduce over peer memory. Every rank owns a communication
// buffer that all ranks map (CUDA IPC):
//     recv [2 slots][kMaxRanks][kMaxVec] f32    partial vectors, written by the owners of the rows
//     flags[2 slots][kMaxRanks][kChunks] u32    "chunk c of rank r has landed", holds the epoch
//     top  [2 slots][kMaxRanks][4] f32          per-rank argmax records
//     tflag[2 slots][kMaxRanks] u32
// A launch with epoch e (per rank one counter per chunk, bumped by the CTA that
// owns the chunk in every exchange launch, so identical on all ranks because they
// run the same launch sequence) uses slot e & 1. CTA c pushes chunk c of its partial vector into every rank's recv
// (plain stores over NVLink) and, after a CTA barrier, publishes flag = e at each
// destination with a system-scope release store (which orders the CTA's data
// stores before the flag); then it waits until the
// flags of all ranks for its chunk in its OWN buffer equal e, and adds the G
// partials in rank order (so every rank computes bit-identical sums) plus the
// residual. Two slots are enough: a rank can only push epoch e+2 after it has
// seen every rank's flag of epoch e+1, which a rank publishes after it has
// finished reading epoch e.
//
// Waits are bounded (about one second of %globaltimer); on expiry the kernel
// records ST_PEER_TIMEOUT in the status word and returns without writing its
// output. No multimem / NVLS and no TMA are used here: plain peer stores and
// local loads only, so a rank that dies leaves the others with a time-out, not
// a fault.
#include "common.cuh"
#include "kernels.h"

namespace flb {

namespace {

__device__ __forceinline__ float *recv_of(uint8_t *base, uint32_t slot, uint32_t rank) {
    return reinterpret_cast<float *>(base) + ((size_t)slot * kCommMaxRanks + rank) * kCommMaxVec;
}
__device__ __forceinline__ uint32_t *flag_of(uint8_t *base, uint32_t slot, uint32_t rank, uint32_t chunk) {
    return reinterpret_cast<uint32_t *>(base + kCommFlagsOff) + ((size_t)slot * kCommMaxRanks + rank) * kCommChunks + chunk;
}
__device__ __forceinline__ float *top_of(uint8_t *base, uint32_t slot, uint32_t rank) {
    return reinterpret_cast<float *>(base + kCommTopOff) + ((size_t)slot * kCommMaxRanks + rank) * 4;
}
__device__ __forceinline__ uint32_t *tflag_of(uint8_t *base, uint32_t slot, uint32_t rank) {
    return reinterpret_cast<uint32_t *>(base + kCommTFlagOff) + (size_t)slot * kCommMaxRanks + rank;
}

// Epoch of this launch for the calling CTA: its own counter + 1, stored back at once
// (only this CTA of this stream's exchange launches ever touches the counter).
__device__ __forceinline__ uint32_t next_epoch(uint32_t *ctr) {
    __shared__ uint32_t e_s;
    if (threadIdx.x == 0) {
        e_s = *ctr + 1u;
        *ctr = e_s;
    }
    __syncthreads();
    return e_s;
}

// out[i] = resid[i] + sum over ranks of their `in`[i], i < n (n a multiple of 4 * kCommChunks).
// grid = kCommChunks, block = n / (4 * kCommChunks) threads.
__global__ void __launch_bounds__(1024) allreduce_resid_kernel(const AllReduceArgs a) {
    griddep_launch_dependents();
    griddep_wait();
    __shared__ uint32_t ok_s;
    const uint32_t tid = threadIdx.x, chunk = blockIdx.x;
    const uint32_t i = (chunk * blockDim.x + tid) * 4;
    const float4 mine = *reinterpret_cast<const float4 *>(a.in + i);
    if (tid == 0) ok_s = 1u;
    const uint32_t e = next_epoch(a.st.epoch + chunk), slot = e & 1u;
    for (uint32_t k = 0; k < a.world; ++k) {
        const uint32_t p = (a.rank + k) % a.world;   // own buffer first, then the ring of peers
        *reinterpret_cast<float4 *>(recv_of(a.peers[p], slot, a.rank) + i) = mine;
    }
    __syncthreads();
    if (tid < a.world) {
        st_release_sys(flag_of(a.peers[tid], slot, a.rank, chunk), e);
        if (!wait_flag(flag_of(a.peers[a.rank], slot, tid, chunk), e, a.status, a.wait_ns)) ok_s = 0u;
    }
    __syncthreads();
    if (ok_s) {
        float4 acc = a.resid ? *reinterpret_cast<const float4 *>(a.resid + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t r = 0; r < a.world; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(recv_of(a.peers[a.rank], slot, r) + i));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4 *>(a.out + i) = acc;
    }
}

// The first half of the all-reduce alone: push this rank's chunk to every rank and publish the flags.
// The kernel that consumes the sum (the next matvec's prologue) waits for the flags and adds.
__global__ void __launch_bounds__(1024) allreduce_push_kernel(const AllReduceArgs a) {
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t tid = threadIdx.x, chunk = blockIdx.x;
    const uint32_t i = (chunk * blockDim.x + tid) * 4;
    const float4 mine = *reinterpret_cast<const float4 *>(a.in + i);
    const uint32_t e = next_epoch(a.st.epoch + chunk), slot = e & 1u;
    for (uint32_t k = 0; k < a.world; ++k) {
        const uint32_t p = (a.rank + k) % a.world;
        *reinterpret_cast<float4 *>(recv_of(a.peers[p], slot, a.rank) + i) = mine;
    }
    __syncthreads();
    if (tid < a.world) st_release_sys(flag_of(a.peers[tid], slot, a.rank, chunk), e);
}

struct Top { float b; uint32_t i; float s; };
__device__ __forceinline__ Top top_merge(const Top &x, const Top &y) {
    const bool y_wins = y.b > x.b || (y.b == x.b && y.i < x.i);
    Top r;
    if (y_wins) { r.b = y.b; r.i = y.i; r.s = fmaxf(x.b, fmaxf(x.s, y.s)); }
    else { r.b = x.b; r.i = x.i; r.s = fmaxf(y.b, fmaxf(x.s, y.s)); }
    return r;
}

// Every rank holds the (best, index, runner-up) of its slice of the logits
// (top3 = {best, index bits, runner-up}; index local to the slice). All ranks
// exchange them and merge in rank order with the reference's tie rule (lowest
// global index wins, src/model/decoder.cpp:1253-1264): identical token on all ranks.
__global__ void __launch_bounds__(32) argmax_exchange_kernel(const TopExchangeArgs a) {
    griddep_launch_dependents();
    griddep_wait();
    const uint32_t tid = threadIdx.x;
    const uint32_t e = next_epoch(a.st.epoch + kCommChunks), slot = e & 1u;   // its own counter, after the chunks'
    bool ok = true;
    if (tid < a.world) {
        float4 rec;
        rec.x = a.top3[0];
        rec.y = __uint_as_float(__float_as_uint(a.top3[1]) + a.index_base);
        rec.z = a.top3[2];
        rec.w = 0.f;
        *reinterpret_cast<float4 *>(top_of(a.peers[tid], slot, a.rank)) = rec;
        st_release_sys(tflag_of(a.peers[tid], slot, a.rank), e);
        ok = wait_flag(tflag_of(a.peers[a.rank], slot, tid), e, a.status, a.wait_ns);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok && tid == 0) {
        Top r{-INFINITY, 0xFFFFFFFFu, -INFINITY};
        for (uint32_t k = 0; k < a.world; ++k) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(top_of(a.peers[a.rank], slot, k)));
            Top u{v.x, __float_as_uint(v.y), v.z};
            r = top_merge(r, u);
        }
        *a.out_idx = (int32_t)r.i;
        *a.out_margin = r.b - r.s;
    }
}

// Merge of the ranks' attention records (sequence-parallel attention). Record i of rank r: context
// o_r[128] normalised over the rank's own keys, m_r = max score, l_r = sum exp(score - m_r). With
// M = max_r m_r and w_r = l_r * exp(m_r - M): out = sum_r w_r o_r / sum_r w_r, ranks in ascending
// order (identical bits on every rank). CTA c handles records c, c + kLseChunks, ...; one warp per
// record, lane <-> 4 dims. Same push / flag / bounded wait protocol as the all-reduce above.
__global__ void __launch_bounds__(128) lse_combine_kernel(const LseCombineArgs a) {
    __shared__ uint32_t ok_s;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, chunk = blockIdx.x;
    if (tid == 0) ok_s = 1u;
    const uint32_t e = next_epoch(a.epoch + chunk), slot = e & 1u;
    const size_t rec_floats = 132;
    const size_t slot_floats = (size_t)a.world * a.max_records * rec_floats;
    auto rec_of = [&](uint8_t *base, uint32_t r, uint32_t i) {
        return reinterpret_cast<float *>(base) + (size_t)slot * slot_floats + ((size_t)r * a.max_records + i) * rec_floats;
    };
    auto flag_of2 = [&](uint8_t *base, uint32_t r) {
        return reinterpret_cast<uint32_t *>(base + 2 * slot_floats * 4) + ((size_t)slot * a.world + r) * kLseChunks + chunk;
    };
    for (uint32_t i = chunk + warp * kLseChunks; i < a.n; i += kLseChunks * 4) {
        const float4 o = *reinterpret_cast<const float4 *>(a.out_local + (size_t)i * 128 + lane * 4);
        const float2 ml = a.lse_local[i];
        for (uint32_t k = 0; k < a.world; ++k) {
            const uint32_t p = (a.rank + k) % a.world;
            float *dst = rec_of(a.peers[p], a.rank, i);
            *reinterpret_cast<float4 *>(dst + lane * 4) = o;
            if (lane == 0) *reinterpret_cast<float2 *>(dst + 128) = ml;
        }
    }
    __syncthreads();
    if (tid < a.world) {
        st_release_sys(flag_of2(a.peers[tid], a.rank), e);
        if (!wait_flag(flag_of2(a.peers[a.rank], tid), e, a.status, a.wait_ns)) ok_s = 0u;
    }
    __syncthreads();
    if (!ok_s) return;
    for (uint32_t i = chunk + warp * kLseChunks; i < a.n; i += kLseChunks * 4) {
        float M = -INFINITY;
        for (uint32_t r = 0; r < a.world; ++r) M = fmaxf(M, __ldcg(rec_of(a.peers[a.rank], r, i) + 128));
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float W = 0.f;
        for (uint32_t r = 0; r < a.world; ++r) {
            const float *rec = rec_of(a.peers[a.rank], r, i);
            const float m = __ldcg(rec + 128), l = __ldcg(rec + 129);
            const float w = (m == -INFINITY || l == 0.f) ? 0.f : l * expf(m - M);
            const float4 o = __ldcg(reinterpret_cast<const float4 *>(rec) + lane);
            if (w != 0.f) {   // a rank without keys contributes nothing (its context may be undefined)
                acc.x = fmaf(o.x, w, acc.x); acc.y = fmaf(o.y, w, acc.y);
                acc.z = fmaf(o.z, w, acc.z); acc.w = fmaf(o.w, w, acc.w);
            }
            W += w;
        }
        const float inv = 1.0f / W;
        *reinterpret_cast<float4 *>(a.out + (size_t)i * 128 + lane * 4) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    }
}

} // namespace

size_t lse_buffer_bytes(uint32_t max_records) {
    return (size_t)2 * kCommMaxRanks * max_records * 132 * 4 + (size_t)2 * kCommMaxRanks * kLseChunks * 4;
}

cudaError_t launch_lse_combine(const LseCombineArgs &a, cudaStream_t stream) {
    if (a.world < 1 || a.world > kCommMaxRanks || a.rank >= a.world || a.n == 0 || a.n > a.max_records)
        return cudaErrorInvalidValue;
    lse_combine_kernel<<<kLseChunks, 128, 0, stream>>>(a);
    return cudaGetLastError();
}

size_t comm_buffer_bytes(void) { return kCommBytes; }

cudaError_t launch_allreduce_resid(const AllReduceArgs &a, cudaStream_t stream, bool pdl) {
    if (a.world < 1 || a.world > kCommMaxRanks || a.rank >= a.world || a.n == 0 || a.n > kCommMaxVec ||
        a.n % (4 * kCommChunks) != 0 || a.n / (4 * kCommChunks) > 1024)
        return cudaErrorInvalidValue;
    return launch_kernel(allreduce_resid_kernel, dim3(kCommChunks), dim3(a.n / (4 * kCommChunks)), 0, stream, pdl, a);
}

cudaError_t launch_allreduce_push(const AllReduceArgs &a, cudaStream_t stream, bool pdl) {
    if (a.world < 1 || a.world > kCommMaxRanks || a.rank >= a.world || a.n == 0 || a.n > kCommMaxVec ||
        a.n % (4 * kCommChunks) != 0 || a.n / (4 * kCommChunks) > 1024)
        return cudaErrorInvalidValue;
    return launch_kernel(allreduce_push_kernel, dim3(kCommChunks), dim3(a.n / (4 * kCommChunks)), 0, stream, pdl, a);
}

cudaError_t launch_argmax_exchange(const TopExchangeArgs &a, cudaStream_t stream, bool pdl) {
    if (a.world < 1 || a.world > kCommMaxRanks || a.rank >= a.world) return cudaErrorInvalidValue;
    return launch_kernel(argmax_exchange_kernel, dim3(1), dim3(32), 0, stream, pdl, a);
}

} // namespace flb
