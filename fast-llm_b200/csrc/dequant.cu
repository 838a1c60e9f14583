// Bulk dequantiser: packed GGUF blocks -> f32, bit-exact with the reference's
// dequant_chunk (src/runtime/kernels.h:162-242). The reference rounds every
// multiply and subtract separately (it builds with contraction off), so the
// kernels use __fmul_rn / __fsub_rn, which the compiler never fuses.
//
// One thread produces four consecutive elements (one float4 store); the packed
// bytes it needs are one aligned 32-bit word for Q4_K and two 16-bit halves
// for the formats whose blocks are only 2-byte aligned (Q6_K 210 B, Q8_0 34 B,
// Q5_0 22 B). The kernel is bound by its 4 B/element output stream.
#include "common.cuh"
#include "kernels.h"

namespace flb {

__device__ __forceinline__ uint32_t ld_u32_2(const uint8_t *p) {  // 2-byte aligned
    const uint16_t *h = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}

__device__ __forceinline__ void q4k_scale_min(const uint8_t *s, int j, uint32_t &sc, uint32_t &mn) {
    if (j < 4) {
        sc = s[j] & 63u;
        mn = s[j + 4] & 63u;
    } else {
        sc = (s[j + 4] & 0x0Fu) | ((uint32_t)(s[j - 4] >> 6) << 4);
        mn = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ w, float *__restrict__ out,
                                                      uint64_t n4, const int32_t *__restrict__ sel,
                                                      uint64_t sel_stride) {
    griddep_launch_dependents();
    griddep_wait();
    // Row gather (embedding lookup): start at row *sel of a table whose rows are
    // sel_stride bytes apart.
    if (sel != nullptr) w += (uint64_t)(*sel) * sel_stride;
    for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n4;
         t += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t e = t * 4;
        float4 r;
        if (FMT == FMT_Q4_K) {
            const uint8_t *b = w + (e >> 8) * 144;
            const uint32_t i = (uint32_t)e & 255u;
            const uint32_t c = i >> 6, hi = (i >> 5) & 1u, l = i & 31u;
            const float d = h2f_bits(*reinterpret_cast<const uint16_t *>(b));
            const float dmin = h2f_bits(*reinterpret_cast<const uint16_t *>(b + 2));
            uint32_t sc, mn;
            q4k_scale_min(b + 4, (int)(2 * c + hi), sc, mn);
            const float ds = __fmul_rn(d, (float)sc), ms = __fmul_rn(dmin, (float)mn);
            uint32_t q = *reinterpret_cast<const uint32_t *>(b + 16 + 32 * c + l);
            q = hi ? (q >> 4) : q;
            r.x = __fsub_rn(__fmul_rn(ds, (float)(q & 15u)), ms);
            r.y = __fsub_rn(__fmul_rn(ds, (float)((q >> 8) & 15u)), ms);
            r.z = __fsub_rn(__fmul_rn(ds, (float)((q >> 16) & 15u)), ms);
            r.w = __fsub_rn(__fmul_rn(ds, (float)((q >> 24) & 15u)), ms);
        } else if (FMT == FMT_Q6_K) {
            const uint8_t *b = w + (e >> 8) * 210;
            const uint32_t i = (uint32_t)e & 255u;
            const uint32_t hf = i >> 7, g = (i >> 5) & 3u, l = i & 31u;
            const float d = h2f_bits(*reinterpret_cast<const uint16_t *>(b + 208));
            const int sc = (int)(int8_t)b[192 + 8 * hf + 2 * g + (l >> 4)];
            const float ds = __fmul_rn(d, (float)sc);
            uint32_t lo = ld_u32_2(b + 64 * hf + 32 * (g & 1u) + l);
            const uint32_t hb = ld_u32_2(b + 128 + 32 * hf + l) >> (2 * g);
            lo = g < 2 ? lo : (lo >> 4);
            const uint32_t q = (lo & 0x0F0F0F0Fu) | ((hb & 0x03030303u) << 4);
            r.x = __fmul_rn(ds, (float)((int)(q & 63u) - 32));
            r.y = __fmul_rn(ds, (float)((int)((q >> 8) & 63u) - 32));
            r.z = __fmul_rn(ds, (float)((int)((q >> 16) & 63u) - 32));
            r.w = __fmul_rn(ds, (float)((int)((q >> 24) & 63u) - 32));
        } else if (FMT == FMT_Q8_0) {
            const uint8_t *b = w + (e >> 5) * 34;
            const uint32_t l = (uint32_t)e & 31u;
            const float d = h2f_bits(*reinterpret_cast<const uint16_t *>(b));
            const uint32_t q = ld_u32_2(b + 2 + l);
            r.x = __fmul_rn(d, (float)(int)(int8_t)(q & 255u));
            r.y = __fmul_rn(d, (float)(int)(int8_t)((q >> 8) & 255u));
            r.z = __fmul_rn(d, (float)(int)(int8_t)((q >> 16) & 255u));
            r.w = __fmul_rn(d, (float)(int)(int8_t)(q >> 24));
        } else if (FMT == FMT_Q5_0) {
            const uint8_t *b = w + (e >> 5) * 22;
            const uint32_t l = (uint32_t)e & 31u;   // 0..28 step 4; 16..31 are high nibbles
            const float d = h2f_bits(*reinterpret_cast<const uint16_t *>(b));
            const uint32_t qh = ld_u32_2(b + 2);
            const uint32_t j = l & 15u;
            uint32_t q = ld_u32_2(b + 6 + j);
            q = l < 16 ? q : (q >> 4);
            const uint32_t fb = qh >> l;            // fifth bits of elements l..l+3
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int qq = (int)(((q >> (8 * k)) & 15u) | (((fb >> k) & 1u) << 4)) - 16;
                v[k] = __fmul_rn(d, (float)qq);
            }
            r = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            r = *reinterpret_cast<const float4 *>(w + e * 4);
        }
        *reinterpret_cast<float4 *>(out + e) = r;
    }
}

cudaError_t launch_dequant(int fmt, const void *w, uint64_t rows, uint32_t cols, float *out, int sms,
                           cudaStream_t stream) {
    const uint64_t n4 = rows * (uint64_t)cols / 4;
    if (n4 == 0) return cudaSuccess;
    const uint64_t want = (n4 + 255) / 256;
    const int grid = (int)(want < (uint64_t)sms * 8 ? want : (uint64_t)sms * 8);
    const uint8_t *wp = static_cast<const uint8_t *>(w);
    switch (fmt) {
    case FMT_F32: dequant_kernel<FMT_F32><<<grid, 256, 0, stream>>>(wp, out, n4, nullptr, 0); break;
    case FMT_Q8_0: dequant_kernel<FMT_Q8_0><<<grid, 256, 0, stream>>>(wp, out, n4, nullptr, 0); break;
    case FMT_Q5_0: dequant_kernel<FMT_Q5_0><<<grid, 256, 0, stream>>>(wp, out, n4, nullptr, 0); break;
    case FMT_Q4_K: dequant_kernel<FMT_Q4_K><<<grid, 256, 0, stream>>>(wp, out, n4, nullptr, 0); break;
    case FMT_Q6_K: dequant_kernel<FMT_Q6_K><<<grid, 256, 0, stream>>>(wp, out, n4, nullptr, 0); break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// Embedding lookup: out[0..cols) = dequant(row *token of the table), the device
// version of the host step in Decoder::step_batch (src/model/decoder.cpp:1194-1201).
cudaError_t launch_embed(int fmt, const void *table, const int32_t *token, uint32_t cols, float *out,
                         cudaStream_t stream, bool pdl) {
    const uint64_t n4 = cols / 4;
    const int grid = (int)((n4 + 255) / 256);
    const uint8_t *wp = static_cast<const uint8_t *>(table);
    const uint64_t rb = row_bytes(fmt, cols);
    switch (fmt) {
    case FMT_F32: return launch_kernel(dequant_kernel<FMT_F32>, dim3(grid), dim3(256), 0, stream, pdl, wp, out, n4, token, rb);
    case FMT_Q8_0: return launch_kernel(dequant_kernel<FMT_Q8_0>, dim3(grid), dim3(256), 0, stream, pdl, wp, out, n4, token, rb);
    case FMT_Q5_0: return launch_kernel(dequant_kernel<FMT_Q5_0>, dim3(grid), dim3(256), 0, stream, pdl, wp, out, n4, token, rb);
    case FMT_Q4_K: return launch_kernel(dequant_kernel<FMT_Q4_K>, dim3(grid), dim3(256), 0, stream, pdl, wp, out, n4, token, rb);
    case FMT_Q6_K: return launch_kernel(dequant_kernel<FMT_Q6_K>, dim3(grid), dim3(256), 0, stream, pdl, wp, out, n4, token, rb);
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

} // namespace flb
