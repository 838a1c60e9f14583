// Shared device helpers for the sm_100a decode kernels: mbarrier + bulk-copy
// (TMA) wrappers with bounded waits, warp reductions, the kernel status word.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace flb {

// Format ids: identical to fastllm::Fmt (include/fastllm/fastllm.h:56-57).
enum : int { FMT_F32 = 0, FMT_Q8_0 = 1, FMT_Q5_0 = 2, FMT_Q4_K = 3, FMT_Q6_K = 4 };

// Kernel status word values (written to the context's device status word; the
// first error wins, later launches keep running).
enum : uint32_t {
    ST_OK = 0,
    ST_WAIT_TIMEOUT = 1,   // a bounded mbarrier wait gave up
    ST_PEER_TIMEOUT = 2,   // a bounded wait for another rank's flag gave up
};

__host__ __device__ inline uint32_t blk_elems(int fmt) {
    return fmt == FMT_F32 ? 1u : (fmt == FMT_Q8_0 || fmt == FMT_Q5_0) ? 32u : 256u;
}
__host__ __device__ inline uint32_t blk_bytes(int fmt) {
    switch (fmt) {
    case FMT_F32: return 4;
    case FMT_Q8_0: return 34;
    case FMT_Q5_0: return 22;
    case FMT_Q4_K: return 144;
    default: return 210;
    }
}
__host__ __device__ inline uint64_t row_bytes(int fmt, uint32_t cols) {
    return (uint64_t)(cols / blk_elems(fmt)) * blk_bytes(fmt);
}

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes mbarrier initialisation visible to the async (TMA) proxy.
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders this thread's generic-proxy shared-memory accesses before later
// async-proxy (bulk copy) accesses to the same locations.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for phase `parity` of an mbarrier for at most about one second. On
// timeout it records ST_WAIT_TIMEOUT in *status and returns false; the caller
// must then stop using the pipeline and return.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (globaltimer_ns() - t0 > 1000000000ull) {
            atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
            return false;
        }
    }
}

// 1-D bulk copy global -> shared through the TMA engine. dst, src 16-byte
// aligned, bytes a multiple of 16; completion is signalled on `bar` as
// transaction bytes.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Same, with the destination given as a 32-bit shared address.
__device__ __forceinline__ void bulk_g2s_addr(uint32_t dst_smem_addr, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem_addr),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Hint: pull [src, src+bytes) into L2 (16-byte aligned, multiple of 16).
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// Programmatic dependent launch. launch_dependents lets the next kernel of the
// stream start its independent preamble (barrier set-up, weight prefetch) while
// this one is still running; wait blocks until the previous kernel has completed
// and its writes are visible. Both are no-ops for a kernel launched without the
// programmatic-serialization attribute.
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Optional per-launch timeline (diagnostics): rec[0] = earliest kernel entry,
// rec[1] = earliest point after the dependency wait, rec[2] = latest end of the
// prologue, rec[3] = latest exit, as %globaltimer nanoseconds. rec[0..1] must be
// pre-set to all ones, rec[2..3] to zero. One thread per CTA calls these.
__device__ __forceinline__ void trace_min(unsigned long long *rec, int i) {
    if (rec) atomicMin(rec + i, (unsigned long long)globaltimer_ns());
}
__device__ __forceinline__ void trace_max(unsigned long long *rec, int i) {
    if (rec) atomicMax(rec + i, (unsigned long long)globaltimer_ns());
}

// Release / acquire fences at GPU scope (cheaper than the sequentially
// consistent __threadfence()).
__device__ __forceinline__ void fence_acq_rel_gpu() {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

// System-scope release store / acquire load (flags that another GPU reads or writes).
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Spins until *flag == want; false (and ST_PEER_TIMEOUT in the status word) after limit_ns of
// %globaltimer (0 = the default of one second). The caller returns without touching its output.
constexpr uint64_t kDefaultWaitNs = 1000000000ull;
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t want, uint32_t *status, uint64_t limit_ns = 0) {
    if (ld_acquire_sys(flag) == want) return true;
    if (limit_ns == 0) limit_ns = kDefaultWaitNs;
    const uint64_t t0 = globaltimer_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if (ld_acquire_sys(flag) == want) return true;
        if (globaltimer_ns() - t0 > limit_ns) {
            atomicCAS(status, ST_OK, ST_PEER_TIMEOUT);
            return false;
        }
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float h2f_bits(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

#endif // __CUDACC__

// Launch helper: optional programmatic dependent launch (the kernel must call
// griddep_wait() before it touches anything the previous kernel wrote).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

} // namespace flb
