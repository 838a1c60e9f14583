// C ABI of the decode hot path (include/fl_b200.h): context, memory helpers,
// single operators, the task-level entry. The decoder lives in decoder.cu.
#include "capi_internal.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <array>
#include <vector>

namespace flb {

static thread_local char g_err[512] = "";

int set_err(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_err(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return FL_B200_OK;
    return set_err(FL_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

} // namespace flb

using namespace flb;

#define CK(call)                                                       \
    do {                                                               \
        cudaError_t e_ = (call);                                       \
        if (e_ != cudaSuccess) return cuda_err(e_, #call);             \
    } while (0)

int flb::grow_attn_part(fl_b200_ctx *c, size_t bytes) {
    if (c->attn_part_cap >= bytes) return FL_B200_OK;
    CK(cudaSetDevice(c->device));
    float *p = nullptr;
    CK(cudaMalloc(&p, bytes));
    if (c->attn_part) c->retired.push_back(c->attn_part);   // a captured plan may still write through it
    c->attn_part = p;
    c->attn_part_cap = bytes;
    return FL_B200_OK;
}

extern "C" {

int fl_b200_abi_version(void) { return FL_B200_ABI_VERSION; }
const char *fl_b200_last_error(void) { return g_err; }

int fl_b200_create(int device, fl_b200_ctx **out) {
    if (!out) return set_err(FL_B200_ERR_ARG, "fl_b200_create: out is null");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return set_err(FL_B200_ERR_CUDA, "fl_b200_create: no CUDA device (%s); this library has no CPU path",
                       cudaGetErrorString(e));
    if (device < 0 || device >= n) return set_err(FL_B200_ERR_ARG, "fl_b200_create: device %d of %d", device, n);
    CK(cudaSetDevice(device));
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return set_err(FL_B200_ERR_CUDA, "fl_b200_create: device %d is sm_%d%d; kernels are built for sm_100a only",
                       device, prop.major, prop.minor);
    fl_b200_ctx *c = new fl_b200_ctx();
    c->device = device;
    c->sms = prop.multiProcessorCount;
    CK(cudaStreamCreate(&c->stream));
    CK(cudaEventCreate(&c->ev0));
    CK(cudaEventCreate(&c->ev1));
    CK(cudaMalloc(&c->status, 256));
    CK(cudaMemset(c->status, 0, 256));
    c->argmax_ticket = c->status + 1;
    c->grid_bar = c->status + 16;        // two words of the zeroed 256-byte block
    c->attn_tickets_cap = 1024;
    CK(cudaMalloc(&c->attn_tickets, c->attn_tickets_cap * sizeof(uint32_t)));
    CK(cudaMemset(c->attn_tickets, 0, c->attn_tickets_cap * sizeof(uint32_t)));
    CK(cudaMalloc(&c->argmax_scratch, (size_t)3 * 1024 * sizeof(float)));
    CK(cudaMalloc(&c->small, 64));
    CK(matvec_init());
    CK(matvec_tc_init());
    CK(matmul_tc_nx_init());
    CK(cudaMalloc(&c->xq, matmul_tc_nx_scratch_bytes(18432, 8)));   // the widest activation the kernels take, 8 columns
    CK(matmul_umma_init());
    CK(cudaMalloc(&c->xu, matmul_umma_xu_bytes(18432)));
    CK(cudaMalloc(&c->um_scratch, matmul_umma_scratch_bytes()));
    CK(cudaMalloc(&c->um_tickets, matmul_umma_ticket_count() * sizeof(uint32_t)));
    CK(cudaMemset(c->um_tickets, 0, matmul_umma_ticket_count() * sizeof(uint32_t)));
    CK(attn_init());
    *out = c;
    return FL_B200_OK;
}

void fl_b200_destroy(fl_b200_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    cudaFree(c->attn_part);
    cudaFree(c->xq);
    cudaFree(c->xu); cudaFree(c->um_scratch); cudaFree(c->um_tickets);
    for (void *p : c->retired) cudaFree(p);
    cudaFree(c->attn_tickets);
    cudaFree(c->argmax_scratch);
    cudaFree(c->small);
    cudaFree(c->status);
    cudaFree(c->stage);
    cudaEventDestroy(c->ev0);
    cudaEventDestroy(c->ev1);
    cudaStreamDestroy(c->stream);
    delete c;
}

int fl_b200_sync(fl_b200_ctx *c) {
    CK(cudaStreamSynchronize(c->stream));
    return FL_B200_OK;
}

int fl_b200_device_status(fl_b200_ctx *c, uint32_t *out) {
    uint32_t v = 0;
    CK(cudaMemcpyAsync(&v, c->status, 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    if (v != 0) {
        CK(cudaMemsetAsync(c->status, 0, 4, c->stream));
        CK(cudaMemsetAsync(c->grid_bar, 0, 8, c->stream));   // a launch that gave up may have left arrivals behind
    }
    if (out) *out = v;
    return FL_B200_OK;
}

int fl_b200_set_wait_limit(fl_b200_ctx *c, uint64_t nanoseconds) {
    if (!c) return set_err(FL_B200_ERR_ARG, "set_wait_limit: null context");
    c->wait_limit_ns = nanoseconds;
    return FL_B200_OK;
}

int fl_b200_sm_count(fl_b200_ctx *c) { return c->sms; }
void *fl_b200_stream(fl_b200_ctx *c) { return (void *)c->stream; }

int fl_b200_malloc(fl_b200_ctx *c, size_t bytes, void **out) {
    CK(cudaSetDevice(c->device));
    CK(cudaMalloc(out, bytes ? bytes : 1));
    return FL_B200_OK;
}
int fl_b200_free(fl_b200_ctx *c, void *p) {
    CK(cudaSetDevice(c->device));
    CK(cudaFree(p));
    return FL_B200_OK;
}
int fl_b200_upload(fl_b200_ctx *c, void *dst, const void *src, size_t bytes) {
    CK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, c->stream));   // src: host or device
    CK(cudaStreamSynchronize(c->stream));
    return FL_B200_OK;
}
int fl_b200_download(fl_b200_ctx *c, void *dst, const void *src, size_t bytes) {
    CK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return FL_B200_OK;
}
// CUDA IPC: lets the ranks of a tensor-parallel group (one process per GPU) map
// each other's exchange buffers. The handle is the 64-byte cudaIpcMemHandle_t.
int fl_b200_ipc_export(fl_b200_ctx *c, const void *dev_ptr, uint8_t handle_out[64]) {
    if (!c || !dev_ptr || !handle_out) return set_err(FL_B200_ERR_ARG, "ipc_export: null");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    CK(cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    CK(cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)));
    memcpy(handle_out, &h, 64);
    return FL_B200_OK;
}

int fl_b200_ipc_open(fl_b200_ctx *c, const uint8_t handle[64], void **dev_ptr_out) {
    if (!c || !handle || !dev_ptr_out) return set_err(FL_B200_ERR_ARG, "ipc_open: null");
    CK(cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    CK(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
    return FL_B200_OK;
}

int fl_b200_ipc_close(fl_b200_ctx *c, void *dev_ptr) {
    if (!c || !dev_ptr) return set_err(FL_B200_ERR_ARG, "ipc_close: null");
    CK(cudaSetDevice(c->device));
    CK(cudaIpcCloseMemHandle(dev_ptr));
    return FL_B200_OK;
}

int fl_b200_memset(fl_b200_ctx *c, void *dst, int value, size_t bytes) {
    CK(cudaMemsetAsync(dst, value, bytes, c->stream));
    return FL_B200_OK;
}

int fl_b200_timer_start(fl_b200_ctx *c) {
    CK(cudaEventRecord(c->ev0, c->stream));
    return FL_B200_OK;
}
int fl_b200_timer_stop(fl_b200_ctx *c, float *ms) {
    CK(cudaEventRecord(c->ev1, c->stream));
    CK(cudaEventSynchronize(c->ev1));
    CK(cudaEventElapsedTime(ms, c->ev0, c->ev1));
    return FL_B200_OK;
}

int fl_b200_dequant(fl_b200_ctx *c, int fmt, const void *w, uint64_t rows, uint32_t cols, float *out) {
    if (!w || !out) return set_err(FL_B200_ERR_ARG, "dequant: null pointer");
    if (fmt < FL_B200_F32 || fmt > FL_B200_Q6_K) return set_err(FL_B200_ERR_ARG, "dequant: format %d", fmt);
    if (cols % blk_elems(fmt) != 0 || cols % 4 != 0)
        return set_err(FL_B200_ERR_ARG, "dequant: cols %u not a multiple of the %u-element block", cols, blk_elems(fmt));
    if (((uintptr_t)out & 15u) != 0) return set_err(FL_B200_ERR_ARG, "dequant: out must be 16-byte aligned");
    if (fmt == FL_B200_Q4_K && ((uintptr_t)w & 3u) != 0) return set_err(FL_B200_ERR_ARG, "dequant: Q4_K weights must be 4-byte aligned");
    if (((uintptr_t)w & 1u) != 0) return set_err(FL_B200_ERR_ARG, "dequant: weights must be 2-byte aligned");
    return cuda_err(launch_dequant(fmt, w, rows, cols, out, c->sms, c->stream), "dequant launch");
}

static int check_matvec(int fmt, const void *w, uint32_t rows, uint32_t cols, const void *x, const void *y) {
    if (!w || !x || !y) return set_err(FL_B200_ERR_ARG, "matvec: null pointer");
    if (fmt < FL_B200_F32 || fmt > FL_B200_Q6_K) return set_err(FL_B200_ERR_ARG, "matvec: format %d", fmt);
    if (rows == 0 || cols == 0) return set_err(FL_B200_ERR_ARG, "matvec: empty shape %u x %u", rows, cols);
    // Graph::freeze rule (src/runtime/graph.cpp:88-89)
    if (cols % blk_elems(fmt) != 0)
        return set_err(FL_B200_ERR_ARG, "matvec: cols %u not a multiple of the format block size %u", cols, blk_elems(fmt));
    if (((uintptr_t)w & 1u) != 0 || (fmt == FL_B200_F32 && ((uintptr_t)w & 3u) != 0))
        return set_err(FL_B200_ERR_ARG, "matvec: misaligned weights");
    return FL_B200_OK;
}

} // extern "C"

// y[p * ystride + r] (+)= dot(W[r], x + p * xstride) for p < nx on the context's stream (declared in
// capi_internal.h: the decoder's batch pass uses it too).
int flb::matmul(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols, const float *x,
                uint32_t nx, uint32_t xstride, float *y, uint32_t ystride, int accumulate, uint32_t pitch,
                const uint32_t *expert_id, uint64_t expert_stride, int pdl, const float *x2, int same_columns) {
    if (int rc = check_matvec(fmt, w, rows, cols, x, y)) return rc;
    if (pitch != 0 && pitch < row_bytes(fmt, cols))
        return set_err(FL_B200_ERR_ARG, "matvec: row pitch %u smaller than the packed row (%llu bytes)", pitch,
                       (unsigned long long)row_bytes(fmt, cols));
    if (nx == 0) nx = 1;
    if (pitch == row_bytes(fmt, cols)) pitch = 0;   // packed rows
    uint32_t first_single = 0;   // columns from here on go through the one-column kernel
    if (nx >= 2 && (fmt == FL_B200_Q4_K || fmt == FL_B200_Q6_K) && !expert_id && cols <= 18432) {
        // verify batches, prompt chunks: up to 8 columns per pass over the weights on the tensor cores, either format
        for (uint32_t p0 = 0; p0 < nx; p0 += 8) {
            const uint32_t nt = nx - p0 < 8 ? nx - p0 : 8;
            if (nt < 2 && p0 > 0) break;   // a last single column goes to the one-column kernel
            NxCall nc{};
            nc.fmt = fmt; nc.w = w; nc.rows = rows; nc.cols = cols; nc.pitch = pitch;
            nc.x = x + (size_t)p0 * xstride; nc.P = nt; nc.xstride = xstride;
            if (x2) nc.x2 = x2 + (size_t)p0 * xstride;
            nc.skip_convert = (same_columns && nx <= 8) ? 1 : 0;   // with more than 8 columns the scratch holds the last chunk only
            nc.y = y + (size_t)p0 * ystride; nc.ystride = ystride; nc.accumulate = accumulate;
            nc.pdl = pdl;
            // Q4_K: tcgen05 with the accumulator in tensor memory; what it does not take goes to the mma.sync kernel
            cudaError_t e = launch_matmul_umma(nc, c->xu, c->um_scratch, c->um_tickets, c->status, c->sms, c->stream);
            if (e == cudaErrorNotSupported) {
                if (fmt == FL_B200_Q4_K) nc.skip_convert = 0;   // the other kernel's scratch does not hold these columns
                e = launch_matmul_tc_nx(nc, c->xq, c->status, c->sms, c->stream);
            }
            if (e == cudaErrorNotSupported) break;   // the shape does not qualify (same answer for every chunk)
            if (e != cudaSuccess) return cuda_err(e, "multi-column matmul launch");
            first_single = p0 + nt;
        }
    }
    for (uint32_t p = first_single; p < nx; ++p) {
        MatvecArgs a{};
        a.n_tensors = 1;
        a.t[0].w = (const uint8_t *)w;
        a.t[0].y = y + (size_t)p * ystride;
        a.t[0].resid = nullptr;
        a.t[0].rows = rows;
        a.t[0].fmt = fmt;
        a.t[0].pitch = pitch;
        if (expert_id) {
            const uint64_t rb = pitch ? pitch : row_bytes(fmt, cols);
            if (expert_stride == 0 || expert_stride % rb != 0)
                return set_err(FL_B200_ERR_ARG, "matvec: expert stride %llu is not a whole number of %llu-byte rows",
                               (unsigned long long)expert_stride, (unsigned long long)rb);
            a.t[0].expert_id = expert_id;
            a.t[0].expert_rows = (uint32_t)(expert_stride / rb);
        }
        a.x = x + (size_t)p * xstride;
        a.cols = cols;
        a.x_mode = MV_X_PLAIN;
        if (x2) { a.x2 = x2 + (size_t)p * xstride; a.x_mode = MV_X_SILU_MUL; }
        a.accumulate = accumulate;
        a.status = c->status;
        a.pdl = pdl;
        if (int rc = cuda_err(launch_matvec(a, c->sms, c->stream), "matvec launch")) return rc;
    }
    return FL_B200_OK;
}

extern "C" {

int fl_b200_matvec_expert(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols,
                          const uint32_t *expert_id, uint64_t expert_stride, const float *x, uint32_t nx, uint32_t xstride,
                          float *y, uint32_t ystride) {
    if (!expert_id) return set_err(FL_B200_ERR_ARG, "matvec_expert: null expert id pointer");
    return flb::matmul(c, fmt, w, rows, cols, x, nx, xstride, y, ystride, 1, 0, expert_id, expert_stride);
}

int fl_b200_matvec_pitched(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols, uint32_t pitch,
                           const float *x, float *y) {
    return flb::matmul(c, fmt, w, rows, cols, x, 1, 0, y, 0, 0, pitch);
}

int fl_b200_matvec(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols, const float *x,
                   uint32_t nx, uint32_t xstride, float *y, uint32_t ystride) {
    return flb::matmul(c, fmt, w, rows, cols, x, nx, xstride, y, ystride, 1);
}

int fl_b200_matvec_assign(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols,
                          const float *x, float *y) {
    return flb::matmul(c, fmt, w, rows, cols, x, 1, 0, y, 0, 0);
}

static int ensure_stage(fl_b200_ctx *c, size_t bytes) {
    if (c->stage_cap >= bytes) return FL_B200_OK;
    CK(cudaStreamSynchronize(c->stream));
    cudaFree(c->stage);
    c->stage = nullptr;
    c->stage_cap = 0;
    CK(cudaMalloc(&c->stage, bytes));
    c->stage_cap = bytes;
    return FL_B200_OK;
}

int fl_b200_matvec_host(fl_b200_ctx *c, int fmt, const void *w, uint32_t rows, uint32_t cols,
                        const float *x_host, float *y_host) {
    if (!x_host || !y_host) return set_err(FL_B200_ERR_ARG, "matvec_host: null pointer");
    const size_t xb = ((size_t)cols * 4 + 255) & ~(size_t)255, yb = (size_t)rows * 4;
    if (int rc = ensure_stage(c, xb + yb)) return rc;
    float *xd = (float *)c->stage, *yd = (float *)((uint8_t *)c->stage + xb);
    CK(cudaMemcpyAsync(xd, x_host, (size_t)cols * 4, cudaMemcpyHostToDevice, c->stream));
    if (int rc = flb::matmul(c, fmt, w, rows, cols, xd, 1, 0, yd, 0, 0)) return rc;
    CK(cudaMemcpyAsync(y_host, yd, yb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return FL_B200_OK;
}

static int attn_impl(fl_b200_ctx *c, const float *q, const uint16_t *k, const uint16_t *v, uint32_t n_q,
                     uint32_t n_kv, uint32_t d, uint32_t kv_len, uint32_t kv_stride, uint32_t batch, float scale,
                     float *out, const int32_t *pos_dev, bool verify = false, float *lse_out = nullptr) {
    if (!q || !k || !v || !out) return set_err(FL_B200_ERR_ARG, "attn_decode: null pointer");
    if (d != 128) return set_err(FL_B200_ERR_ARG, "attn_decode: head_dim %u (only 128 is built)", d);
    if (n_kv == 0 || n_q != 4 * n_kv)
        return set_err(FL_B200_ERR_ARG, "attn_decode: %u query heads over %u KV heads (only groups of 4 are built)", n_q, n_kv);
    if (batch == 0) return set_err(FL_B200_ERR_ARG, "attn_decode: batch 0");
    if (!pos_dev && (kv_len == 0 || kv_len + (verify ? batch - 1 : 0) > kv_stride))
        return set_err(FL_B200_ERR_ARG, "attn_decode: kv_len %u outside 1..kv_stride %u", kv_len, kv_stride);
    if (((uintptr_t)k & 15u) || ((uintptr_t)v & 15u) || ((uintptr_t)q & 15u))
        return set_err(FL_B200_ERR_ARG, "attn_decode: q, k, v must be 16-byte aligned");
    if ((uint64_t)n_kv * batch > c->attn_tickets_cap)
        return set_err(FL_B200_ERR_ARG, "attn_decode: n_kv_head * batch = %llu exceeds %u", (unsigned long long)n_kv * batch, c->attn_tickets_cap);
    AttnArgs a{};
    a.q = q;
    a.k = (const __half *)k;
    a.v = (const __half *)v;
    a.out = out;
    a.pos = pos_dev;
    a.kv_len = kv_len;
    a.kv_stride = kv_stride;
    a.batch_stride = (uint64_t)n_kv * kv_stride * d;
    a.n_q_head = n_q;
    a.n_kv_head = n_kv;
    a.batch = batch;
    a.n_splits = attn_pick_splits(n_kv, batch, pos_dev ? kv_stride : kv_len + (verify ? batch - 1 : 0), c->sms);
    a.lse_out = reinterpret_cast<float2 *>(lse_out);
    a.kv_len_step = verify ? 1u : 0u;
    a.shared_kv = verify ? 1u : 0u;
    a.scale = scale;
    a.status = c->status;
    const size_t need = attn_part_floats(n_q, batch, a.n_splits) * sizeof(float);
    if (int rc = grow_attn_part(c, need)) return rc;
    a.part = c->attn_part;
    a.tickets = c->attn_tickets;
    if (int rc = cuda_err(attn_make_maps(a), "attn tensor maps")) return rc;
    return cuda_err(launch_attn_decode(a, c->stream), "attn launch");
}

int fl_b200_attn_decode(fl_b200_ctx *c, const float *q, const uint16_t *k, const uint16_t *v, uint32_t n_q,
                        uint32_t n_kv, uint32_t d, uint32_t kv_len, uint32_t kv_stride, uint32_t batch,
                        float scale, float *out) {
    return attn_impl(c, q, k, v, n_q, n_kv, d, kv_len, kv_stride, batch, scale, out, nullptr);
}

// fl_b200_attn_decode without any allocation at call time: the split-KV scratch
// is a fixed array in the library image (attn.cu). Same arguments, same kernel,
// same results as fl_b200_attn_decode.
int fl_b200_attn_decode_static(fl_b200_ctx *c, const float *q, const uint16_t *k, const uint16_t *v, uint32_t n_q,
                               uint32_t n_kv, uint32_t d, uint32_t kv_len, uint32_t kv_stride, uint32_t batch,
                               float scale, float *out) {
    if (!c) return set_err(FL_B200_ERR_ARG, "attn_decode_static: null context");
    if (!q || !k || !v || !out) return set_err(FL_B200_ERR_ARG, "attn_decode_static: null pointer");
    if (d != 128) return set_err(FL_B200_ERR_ARG, "attn_decode_static: head_dim %u (only 128 is built)", d);
    if (n_kv == 0 || n_q != 4 * n_kv)
        return set_err(FL_B200_ERR_ARG, "attn_decode_static: %u query heads over %u KV heads (only groups of 4 are built)", n_q, n_kv);
    if (batch == 0) return set_err(FL_B200_ERR_ARG, "attn_decode_static: batch 0");
    if (kv_len == 0 || kv_len > kv_stride)
        return set_err(FL_B200_ERR_ARG, "attn_decode_static: kv_len %u outside 1..kv_stride %u", kv_len, kv_stride);
    if (((uintptr_t)k & 15u) || ((uintptr_t)v & 15u) || ((uintptr_t)q & 15u))
        return set_err(FL_B200_ERR_ARG, "attn_decode_static: q, k, v must be 16-byte aligned");
    // The scratch array's address is looked up for the CURRENT device: make the context's device current
    // first (a process that holds contexts on several devices may call with another one current).
    CK(cudaSetDevice(c->device));
    AttnArgs a{};
    a.q = q;
    a.k = (const __half *)k;
    a.v = (const __half *)v;
    a.out = out;
    a.pos = nullptr;
    a.kv_len = kv_len;
    a.kv_stride = kv_stride;
    a.batch_stride = (uint64_t)n_kv * kv_stride * d;
    a.n_q_head = n_q;
    a.n_kv_head = n_kv;
    a.batch = batch;
    a.n_splits = attn_pick_splits(n_kv, batch, kv_len, c->sms);
    a.scale = scale;
    a.status = c->status;
    size_t records = 0;
    const cudaError_t e = launch_attn_decode_static(a, c->device, c->stream, &records);
    if (e == cudaErrorMemoryAllocation)
        return set_err(FL_B200_ERR_ARG,
                       "attn_decode_static: needs %zu scratch records (n_q_head * batch * splits) and %llu counters; "
                       "the fixed scratch holds %zu records and %u counters - use fl_b200_attn_decode",
                       records, (unsigned long long)n_kv * batch, attn_static_max_records(), attn_static_max_tickets());
    return cuda_err(e, "attn_decode_static launch");
}

// Draft verification (causal within the draft): query b of `n_draft` attends keys 0 .. base_len + b - 1 of
// ONE shared cache, i.e. fl_op_attn_head called once per draft position with pos = base_len - 1 + b.
int fl_b200_attn_verify(fl_b200_ctx *c, const float *q, const uint16_t *k, const uint16_t *v, uint32_t n_q,
                        uint32_t n_kv, uint32_t d, uint32_t base_len, uint32_t kv_stride, uint32_t n_draft,
                        float scale, float *out) {
    if (!c) return set_err(FL_B200_ERR_ARG, "attn_verify: null context");
    return attn_impl(c, q, k, v, n_q, n_kv, d, base_len, kv_stride, n_draft, scale, out, nullptr, true);
}

// ---- sequence-parallel attention: every rank attends its slice of the keys, then the ranks' records merge ----
int fl_b200_attn_decode_lse(fl_b200_ctx *c, const float *q, const uint16_t *k, const uint16_t *v, uint32_t n_q,
                            uint32_t n_kv, uint32_t d, uint32_t kv_len, uint32_t kv_stride, uint32_t batch,
                            float scale, float *out, float *lse_out) {
    if (!c || !lse_out) return set_err(FL_B200_ERR_ARG, "attn_decode_lse: null");
    if (((uintptr_t)lse_out & 7u) != 0) return set_err(FL_B200_ERR_ARG, "attn_decode_lse: lse_out must be 8-byte aligned");
    return attn_impl(c, q, k, v, n_q, n_kv, d, kv_len, kv_stride, batch, scale, out, nullptr, false, lse_out);
}

struct fl_b200_seqpar {
    fl_b200_ctx *ctx = nullptr;
    uint32_t rank = 0, world = 1, max_records = 0;
    uint8_t *buf = nullptr;
    uint8_t *peers[kCommMaxRanks] = {};
    bool peers_set = false;
    uint32_t *epoch = nullptr;
};

int fl_b200_seqpar_create(fl_b200_ctx *c, uint32_t rank, uint32_t world, uint32_t max_records, fl_b200_seqpar **out) {
    if (!c || !out) return set_err(FL_B200_ERR_ARG, "seqpar_create: null");
    if (world == 0 || world > kCommMaxRanks || rank >= world || max_records == 0 || max_records > (1u << 16))
        return set_err(FL_B200_ERR_ARG, "seqpar_create: rank %u of %u, %u records", rank, world, max_records);
    fl_b200_seqpar *h = new fl_b200_seqpar();
    h->ctx = c; h->rank = rank; h->world = world; h->max_records = max_records;
    CK(cudaSetDevice(c->device));
    CK(cudaMalloc(&h->buf, lse_buffer_bytes(max_records)));
    CK(cudaMemsetAsync(h->buf, 0, lse_buffer_bytes(max_records), c->stream));
    CK(cudaMalloc(&h->epoch, kLseChunks * 4));
    CK(cudaMemsetAsync(h->epoch, 0, kLseChunks * 4, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    *out = h;
    return FL_B200_OK;
}

void fl_b200_seqpar_destroy(fl_b200_seqpar *h) {
    if (!h) return;
    cudaSetDevice(h->ctx->device);
    cudaStreamSynchronize(h->ctx->stream);
    cudaFree(h->buf);
    cudaFree(h->epoch);
    delete h;
}

int fl_b200_seqpar_comm(fl_b200_seqpar *h, void **buf, size_t *bytes) {
    if (!h || !buf || !bytes) return set_err(FL_B200_ERR_ARG, "seqpar_comm: null");
    *buf = h->buf;
    *bytes = lse_buffer_bytes(h->max_records);
    return FL_B200_OK;
}

int fl_b200_seqpar_set_peers(fl_b200_seqpar *h, void *const *bufs, uint32_t n) {
    if (!h || !bufs || n != h->world) return set_err(FL_B200_ERR_ARG, "seqpar_set_peers: need %u buffers", h ? h->world : 0);
    for (uint32_t p = 0; p < n; ++p) {
        if (!bufs[p]) return set_err(FL_B200_ERR_ARG, "seqpar_set_peers: buffer of rank %u is null", p);
        h->peers[p] = (uint8_t *)bufs[p];
    }
    if (h->peers[h->rank] != h->buf) return set_err(FL_B200_ERR_ARG, "seqpar_set_peers: entry %u must be this rank's own buffer", h->rank);
    h->peers_set = true;
    return FL_B200_OK;
}

int fl_b200_seqpar_combine(fl_b200_seqpar *h, const float *out_local, const float *lse_local, uint32_t n, float *out) {
    if (!h || !out_local || !lse_local || !out) return set_err(FL_B200_ERR_ARG, "seqpar_combine: null");
    if (!h->peers_set) return set_err(FL_B200_ERR_STATE, "seqpar_combine: set the peers first");
    if (n == 0 || n > h->max_records) return set_err(FL_B200_ERR_ARG, "seqpar_combine: %u records (at most %u)", n, h->max_records);
    LseCombineArgs a{};
    for (uint32_t p = 0; p < h->world; ++p) a.peers[p] = h->peers[p];
    a.out_local = out_local; a.lse_local = reinterpret_cast<const float2 *>(lse_local); a.out = out;
    a.n = n; a.max_records = h->max_records; a.rank = h->rank; a.world = h->world;
    a.epoch = h->epoch; a.status = h->ctx->status; a.wait_ns = h->ctx->wait_limit_ns;
    return cuda_err(launch_lse_combine(a, h->ctx->stream), "lse combine launch");
}

int fl_b200_attn_decode_host(fl_b200_ctx *c, const float *q_host, const uint16_t *k, const uint16_t *v,
                             uint32_t n_q, uint32_t n_kv, uint32_t d, uint32_t kv_len, uint32_t kv_stride,
                             uint32_t batch, float scale, float *out_host) {
    if (!q_host || !out_host) return set_err(FL_B200_ERR_ARG, "attn_decode_host: null pointer");
    const size_t qb = (size_t)batch * n_q * d * 4;
    if (int rc = ensure_stage(c, 2 * qb + 512)) return rc;
    float *qd = (float *)c->stage, *od = (float *)((uint8_t *)c->stage + ((qb + 255) & ~(size_t)255));
    CK(cudaMemcpyAsync(qd, q_host, qb, cudaMemcpyHostToDevice, c->stream));
    if (int rc = attn_impl(c, qd, k, v, n_q, n_kv, d, kv_len, kv_stride, batch, scale, od, nullptr)) return rc;
    CK(cudaMemcpyAsync(out_host, od, qb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return FL_B200_OK;
}

int fl_b200_rmsnorm(fl_b200_ctx *c, const float *x, const float *w, float *y, float eps, uint32_t n) {
    if (!x || !w || !y || n == 0) return set_err(FL_B200_ERR_ARG, "rmsnorm: bad argument");
    return cuda_err(launch_rmsnorm(x, w, y, eps, n, c->stream), "rmsnorm launch");
}
int fl_b200_add2(fl_b200_ctx *c, const float *a, const float *b, float *y, uint32_t n) {
    if (!a || !b || !y || n == 0) return set_err(FL_B200_ERR_ARG, "add2: bad argument");
    return cuda_err(launch_add2(a, b, y, n, c->stream), "add2 launch");
}
int fl_b200_silu_mul(fl_b200_ctx *c, const float *g, const float *u, float *h, uint32_t n) {
    if (!g || !u || !h || n == 0) return set_err(FL_B200_ERR_ARG, "silu_mul: bad argument");
    return cuda_err(launch_silu_mul(g, u, h, n, c->stream), "silu_mul launch");
}

int fl_b200_router_sel(fl_b200_ctx *c, const float *logits, uint32_t *ids, float *gates, uint32_t n_expert,
                       uint32_t top_k, uint32_t norm, float scale) {
    if (!c || !logits || !ids || !gates) return set_err(FL_B200_ERR_ARG, "router_sel: null pointer");
    if (n_expert == 0 || n_expert > 256 || top_k == 0 || top_k > n_expert)
        return set_err(FL_B200_ERR_ARG, "router_sel: %u experts (1..256), top_k %u", n_expert, top_k);
    return cuda_err(launch_router_sel(logits, ids, gates, 1, n_expert, top_k, norm, scale, c->stream), "router_sel launch");
}

int fl_b200_wmerge(fl_b200_ctx *c, const float *parts, const float *gates, const float *add1, const float *add2,
                   float *y, float scale, uint32_t n_parts, uint32_t n, uint32_t n_full) {
    if (!c || !parts || !y || n == 0 || n_parts == 0) return set_err(FL_B200_ERR_ARG, "wmerge: bad argument");
    return cuda_err(launch_wmerge(parts, gates, add1, add2, y, scale, n_parts, n, n_full, c->stream), "wmerge launch");
}

int fl_b200_rope_kv_append(fl_b200_ctx *c, float *q, const float *k, const float *v, uint16_t *kc,
                           uint16_t *vc, const int32_t *pos, uint32_t n_q, uint32_t n_kv, uint32_t d,
                           uint32_t kv_stride, float freq_base) {
    if (!k || !v || !kc || !vc || !pos) return set_err(FL_B200_ERR_ARG, "rope_kv_append: null pointer");
    if (d == 0 || (d & 1u)) return set_err(FL_B200_ERR_ARG, "rope_kv_append: head_dim %u must be even", d);
    RopeAppendArgs a{};
    a.q = q;
    a.k = k;
    a.v = v;
    a.kcache = (__half *)kc;
    a.vcache = (__half *)vc;
    a.pos = pos;
    a.n_q_head = n_q;
    a.n_kv_head = n_kv;
    a.head_dim = d;
    a.kv_stride = kv_stride;
    // Same expression, same libm as the reference's host path
    // (src/runtime/decode_params.h:125).
    a.theta_scale = powf(freq_base, -2.0f / (float)d);
    return cuda_err(launch_rope_append(a, c->stream), "rope_append launch");
}

int fl_b200_argmax(fl_b200_ctx *c, const float *lg, uint32_t n, int32_t *idx, float *margin) {
    if (!lg || !idx || !margin || n == 0) return set_err(FL_B200_ERR_ARG, "argmax: bad argument");
    return cuda_err(launch_argmax(lg, n, idx, margin, c->argmax_scratch, c->argmax_ticket, c->sms, c->stream),
                    "argmax launch");
}

// Host buffers for one parameter block: large enough for every POD below.
constexpr size_t kAuxMax = 128;
static_assert(sizeof(fl_b200_router_p) <= kAuxMax && sizeof(fl_b200_wmerge_p) <= kAuxMax && sizeof(fl_b200_rmsnorm_p) <= kAuxMax &&
              sizeof(fl_b200_add2_p) <= kAuxMax && sizeof(fl_b200_silu_mul_p) <= kAuxMax &&
              sizeof(fl_b200_attn_gqa_f16_p) <= kAuxMax && sizeof(fl_b200_rope_kv_append_f16_p) <= kAuxMax, "parameter block buffer");

// Size of the parameter block behind Task::aux for a kind (0: none / not a parameter block).
static size_t aux_bytes(int kind) {
    switch (kind) {
    case FL_B200_ROUTER_SEL: return sizeof(fl_b200_router_p);
    case FL_B200_WMERGE: return sizeof(fl_b200_wmerge_p);
    case FL_B200_RMSNORM: return sizeof(fl_b200_rmsnorm_p);
    case FL_B200_ADD2: return sizeof(fl_b200_add2_p);
    case FL_B200_SILU_MUL: return sizeof(fl_b200_silu_mul_p);
    case FL_B200_ATTN_GQA_F16: return sizeof(fl_b200_attn_gqa_f16_p);
    case FL_B200_ROPE_KV_APPEND_F16: return sizeof(fl_b200_rope_kv_append_f16_p);
    default: return 0;
    }
}

// Launches one task on the context's stream. aux_host: host copy of the task's parameter block
// (fetched here, with a stream synchronisation, when null).
static int launch_task(fl_b200_ctx *c, const fl_b200_task *t, const void *aux_host) {
    if (!t) return set_err(FL_B200_ERR_ARG, "exec_task: null task");
    alignas(8) uint8_t local[kAuxMax];
    const size_t ab = aux_bytes(t->kind);
    if (ab) {
        if (!t->aux) return set_err(FL_B200_ERR_ARG, "exec_task: decode op without aux param block");
        if (!aux_host) {
            CK(cudaMemcpyAsync(local, t->aux, ab, cudaMemcpyDefault, c->stream));
            CK(cudaStreamSynchronize(c->stream));
            aux_host = local;
        }
    }
    switch (t->kind) {
    case FL_B200_SIGNAL: return FL_B200_OK;
    case FL_B200_STREAM_DOT: {
        // Graph::freeze rule (src/runtime/graph.cpp:90-91)
        if (t->w_bytes != (uint64_t)t->rows * row_bytes(t->fmt, t->cols))
            return set_err(FL_B200_ERR_ARG, "exec_task: STREAM_DOT w_bytes mismatch");
        return fl_b200_matvec(c, t->fmt, t->w, t->rows, t->cols, (const float *)t->x, t->nx ? t->nx : 1, t->xstride,
                              (float *)t->y, t->ystride);
    }
    case FL_B200_STREAM_DOT_IDX: {
        // aux -> router-written expert id (read on the device at run time), aux2 = expert stride in bytes
        if (!t->aux) return set_err(FL_B200_ERR_ARG, "exec_task: STREAM_DOT_IDX without the expert id pointer");
        if (t->w_bytes != (uint64_t)t->rows * row_bytes(t->fmt, t->cols))
            return set_err(FL_B200_ERR_ARG, "exec_task: STREAM_DOT_IDX w_bytes mismatch");
        return fl_b200_matvec_expert(c, t->fmt, t->w, t->rows, t->cols, (const uint32_t *)t->aux, t->aux2,
                                     (const float *)t->x, t->nx ? t->nx : 1, t->xstride, (float *)t->y, t->ystride);
    }
    case FL_B200_ROUTER_SEL: {
        const fl_b200_router_p &p = *(const fl_b200_router_p *)aux_host;
        return fl_b200_router_sel(c, p.logits, p.ids, p.gates, p.n_expert, p.top_k, p.norm, p.scale);
    }
    case FL_B200_WMERGE: {
        const fl_b200_wmerge_p &p = *(const fl_b200_wmerge_p *)aux_host;
        return fl_b200_wmerge(c, p.parts, p.gates, p.add1, p.add2, p.y, p.scale, p.n_parts, p.n, p.n_full);
    }
    case FL_B200_RMSNORM: {
        const fl_b200_rmsnorm_p &p = *(const fl_b200_rmsnorm_p *)aux_host;
        return fl_b200_rmsnorm(c, p.x, p.wnorm, p.y, p.eps, p.n);
    }
    case FL_B200_ADD2: {
        const fl_b200_add2_p &p = *(const fl_b200_add2_p *)aux_host;
        return fl_b200_add2(c, p.a, p.b, p.y, p.n);
    }
    case FL_B200_SILU_MUL: {
        const fl_b200_silu_mul_p &p = *(const fl_b200_silu_mul_p *)aux_host;
        return fl_b200_silu_mul(c, p.gate, p.up, p.h, p.n);
    }
    case FL_B200_ATTN_GQA_F16: {
        const fl_b200_attn_gqa_f16_p &p = *(const fl_b200_attn_gqa_f16_p *)aux_host;
        return attn_impl(c, p.q, p.kcache, p.vcache, p.n_q_head, p.n_kv_head, p.head_dim, 0, p.kv_stride, 1,
                         p.scale, p.out, p.pos);
    }
    case FL_B200_ROPE_KV_APPEND_F16: {
        const fl_b200_rope_kv_append_f16_p &p = *(const fl_b200_rope_kv_append_f16_p *)aux_host;
        return fl_b200_rope_kv_append(c, p.q, p.k, p.v, p.kcache, p.vcache, p.pos, p.n_q_head, p.n_kv_head,
                                      p.head_dim, p.kv_stride, p.freq_base);
    }
    default:
        return set_err(FL_B200_ERR_ARG, "exec_task: task kind %d has no device implementation in this library", (int)t->kind);
    }
}

int fl_b200_exec_task(fl_b200_ctx *c, const fl_b200_task *t) { return launch_task(c, t, nullptr); }

// ---- a frozen task table as one CUDA graph -------------------------------------------------------
// The counterpart of Graph::freeze + Runtime::run for the GPU side (src/runtime/graph.cpp:48-148,
// src/runtime/runtime.cpp:178-292): the table is validated with the reference's rules, ordered by
// dependency level, row tiles of one weight tensor are merged back into one matvec launch (the
// reference cuts a tensor into 192..1024-row tiles for its CPU/GPU work queues,
// src/model/decoder.cpp:713-717; here a launch covers the GPU whatever its size), and the launches
// are recorded once as a CUDA graph that fl_b200_plan_run replays.
struct fl_b200_plan {
    fl_b200_ctx *ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint32_t n_tasks = 0, n_launches = 0, n_merged = 0;
};

int fl_b200_plan_create(fl_b200_ctx *c, const fl_b200_task *tasks, uint32_t n, fl_b200_plan **out) {
    if (!c || !tasks || !out || n == 0) return set_err(FL_B200_ERR_ARG, "plan_create: null / empty");
    *out = nullptr;
    // --- Graph::freeze: Kahn's algorithm (cycle check), exactly one sink, which must be SIGNAL ---
    std::vector<int32_t> deps(n);
    std::vector<uint32_t> level(n, 0), order;
    std::vector<uint32_t> ready;
    for (uint32_t i = 0; i < n; ++i) {
        if (tasks[i].n_consumers > 6) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: consumer fan-out exceeded", i);
        deps[i] = tasks[i].dep_init;
        if (deps[i] == 0) ready.push_back(i);
    }
    uint32_t seen = 0, sinks = 0, terminal = 0;
    while (!ready.empty()) {
        const uint32_t id = ready.back();
        ready.pop_back();
        ++seen;
        order.push_back(id);
        const fl_b200_task &t = tasks[id];
        if (t.n_consumers == 0) { ++sinks; terminal = id; }
        for (uint16_t k = 0; k < t.n_consumers; ++k) {
            const uint32_t cns = t.consumers[k];
            if (cns >= n || cns == id) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: bad edge to %u", id, cns);
            if (level[cns] < level[id] + 1) level[cns] = level[id] + 1;
            if (--deps[cns] == 0) ready.push_back(cns);
        }
    }
    if (seen != n) return set_err(FL_B200_ERR_ARG, "plan_create: cycle in graph (or dep_init does not match the edges)");
    if (sinks != 1) return set_err(FL_B200_ERR_ARG, "plan_create: graph must have exactly one sink (terminal SIGNAL), found %u", sinks);
    if (tasks[terminal].kind != FL_B200_SIGNAL) return set_err(FL_B200_ERR_ARG, "plan_create: terminal must be SIGNAL");
    for (uint32_t i = 0; i < n; ++i) {
        const fl_b200_task &t = tasks[i];
        if (t.kind != FL_B200_STREAM_DOT && t.kind != FL_B200_STREAM_DOT_IDX) {
            if (t.kind > FL_B200_ROPE_KV_APPEND_F16) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: unknown task kind %d", i, (int)t.kind);
            if (t.kind >= FL_B200_RMSNORM && t.aux == nullptr) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: decode op without aux param block", i);
            continue;
        }
        if (t.kind == FL_B200_STREAM_DOT_IDX && (t.aux == nullptr || t.aux2 == 0))
            return set_err(FL_B200_ERR_ARG, "plan_create: task %u: STREAM_DOT_IDX without id slot / stride", i);
        if (t.fmt > FL_B200_Q6_K) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: weight format %d has no device kernel", i, (int)t.fmt);
        if (t.cols % blk_elems(t.fmt) != 0) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: STREAM_DOT cols not a multiple of the format block size", i);
        if (t.w_bytes != (uint64_t)t.rows * row_bytes(t.fmt, t.cols)) return set_err(FL_B200_ERR_ARG, "plan_create: task %u: STREAM_DOT w_bytes mismatch", i);
    }
    // --- parameter blocks to the host (one synchronisation), attention scratch sized before the capture ---
    std::vector<std::array<uint8_t, kAuxMax>> aux(n);
    CK(cudaSetDevice(c->device));
    for (uint32_t i = 0; i < n; ++i) {
        const size_t ab = aux_bytes(tasks[i].kind);
        if (ab) CK(cudaMemcpyAsync(aux[i].data(), tasks[i].aux, ab, cudaMemcpyDefault, c->stream));
    }
    CK(cudaStreamSynchronize(c->stream));
    for (uint32_t i = 0; i < n; ++i)
        if (tasks[i].kind == FL_B200_ATTN_GQA_F16) {
            const fl_b200_attn_gqa_f16_p &p = *(const fl_b200_attn_gqa_f16_p *)aux[i].data();
            if (p.n_kv_head == 0 || p.n_q_head != 4 * p.n_kv_head || p.head_dim != 128)
                return set_err(FL_B200_ERR_ARG, "plan_create: task %u: attention shape %u/%u x %u is not built", i, p.n_q_head, p.n_kv_head, p.head_dim);
            const uint32_t splits = attn_pick_splits(p.n_kv_head, 1, p.kv_stride, c->sms);
            const size_t need = attn_part_floats(p.n_q_head, 1, splits) * sizeof(float);
            if (int rc = grow_attn_part(c, need)) return rc;
        }
    // --- launch list: by dependency level; within a level, STREAM_DOT tiles of one tensor merge ---
    std::vector<uint32_t> by_level(order);
    std::stable_sort(by_level.begin(), by_level.end(), [&](uint32_t a, uint32_t b) {
        if (level[a] != level[b]) return level[a] < level[b];
        const fl_b200_task &x = tasks[a], &y = tasks[b];
        const bool dx = x.kind == FL_B200_STREAM_DOT, dy = y.kind == FL_B200_STREAM_DOT;
        if (dx != dy) return dx;                      // dots first
        if (!dx) return false;
        if (x.x != y.x) return x.x < y.x;
        return x.w < y.w;                             // tiles of one tensor next to each other, ascending
    });
    std::vector<fl_b200_task> launches;
    std::vector<uint32_t> src;                        // the task a launch takes its parameter block from
    uint32_t merged = 0;
    for (uint32_t id : by_level) {
        const fl_b200_task &t = tasks[id];
        if (t.kind == FL_B200_SIGNAL) continue;
        if (t.kind == FL_B200_STREAM_DOT && !launches.empty()) {
            fl_b200_task &p = launches.back();
            const uint32_t pnx = p.nx ? p.nx : 1, tnx = t.nx ? t.nx : 1;
            if (p.kind == FL_B200_STREAM_DOT && level[src.back()] == level[id] && p.fmt == t.fmt && p.cols == t.cols &&
                p.x == t.x && pnx == tnx && p.xstride == t.xstride && p.ystride == t.ystride &&
                (const uint8_t *)p.w + p.w_bytes == (const uint8_t *)t.w && (const float *)p.y + p.rows == (const float *)t.y &&
                (pnx == 1 || p.ystride >= p.rows + t.rows)) {
                p.rows += t.rows;
                p.w_bytes += t.w_bytes;
                ++merged;
                continue;
            }
        }
        launches.push_back(t);
        src.push_back(id);
    }
    // --- record ---
    fl_b200_plan *pl = new fl_b200_plan();
    pl->ctx = c;
    pl->n_tasks = n;
    pl->n_launches = (uint32_t)launches.size();
    pl->n_merged = merged;
    cudaStream_t s = c->stream;
    cudaError_t e = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) { delete pl; return cuda_err(e, "cudaStreamBeginCapture"); }
    int rc = FL_B200_OK;
    for (size_t i = 0; i < launches.size() && rc == FL_B200_OK; ++i) rc = launch_task(c, &launches[i], aux[src[i]].data());
    cudaGraph_t g = nullptr;
    e = cudaStreamEndCapture(s, &g);
    if (rc != FL_B200_OK || e != cudaSuccess) {
        if (g) cudaGraphDestroy(g);
        delete pl;
        return rc != FL_B200_OK ? rc : cuda_err(e, "cudaStreamEndCapture");
    }
    pl->graph = g;
    e = cudaGraphInstantiate(&pl->exec, g, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(g); delete pl; return cuda_err(e, "cudaGraphInstantiate"); }
    *out = pl;
    return FL_B200_OK;
}

// One run of the table (asynchronous on the context's stream; fl_b200_sync waits). STREAM_DOT accumulates:
// the caller zeroes the y slots per run like the reference does (src/model/decoder.cpp:1206-1208).
int fl_b200_plan_run(fl_b200_plan *p) {
    if (!p) return set_err(FL_B200_ERR_ARG, "plan_run: null");
    return cuda_err(cudaGraphLaunch(p->exec, p->ctx->stream), "cudaGraphLaunch");
}

int fl_b200_plan_info(fl_b200_plan *p, uint32_t *n_tasks, uint32_t *n_launches, uint32_t *n_merged) {
    if (!p) return set_err(FL_B200_ERR_ARG, "plan_info: null");
    if (n_tasks) *n_tasks = p->n_tasks;
    if (n_launches) *n_launches = p->n_launches;
    if (n_merged) *n_merged = p->n_merged;
    return FL_B200_OK;
}

void fl_b200_plan_destroy(fl_b200_plan *p) {
    if (!p) return;
    cudaSetDevice(p->ctx->device);
    cudaStreamSynchronize(p->ctx->stream);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    delete p;
}

} // extern "C"
