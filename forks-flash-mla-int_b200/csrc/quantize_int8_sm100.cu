// int8_ds_mla row quantizer for sm_100a.
//
// Bit-exact with quantize_int8_ds_mla_rows (flash_mla/int8_sparse_mla.py:15-26 of the
// reference): scale = max(amax|x|, 1e-12f) / 127.0f and q = clamp(rint(x / scale), -127, 127),
// evaluated in IEEE fp32 with true division (__fdiv_rn) and round-half-even (rintf).
// This translation unit must NOT be built with --use_fast_math.
//
// HBM-bound: one warp per 512-element row, 16-byte loads, one pass (the row stays in
// registers between the amax reduction and the quantisation), 1024 + 512 + 4 bytes per bf16 row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "smla_internal.h"

namespace smla {
namespace {

template <typename T> struct Vec16;   // 16 bytes of T -> floats
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void unpack(const uint4 &v, float *f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};
template <> struct Vec16<__half> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void unpack(const uint4 &v, float *f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            const float2 p = __half22float2(h);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
};
template <> struct Vec16<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void unpack(const uint4 &v, float *f) {
        f[0] = __uint_as_float(v.x);
        f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z);
        f[3] = __uint_as_float(v.w);
    }
};

constexpr int kWarpsPerBlock = 8;

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quantize_int8_rows_kernel(const T *__restrict__ x, int64_t rows, int64_t row_stride,
                          int8_t *__restrict__ q, float *__restrict__ scale) {
    constexpr int E = Vec16<T>::kElems;          // elements per 16-byte vector
    constexpr int V = 512 / (32 * E);            // vectors per lane (2 for 16-bit, 4 for fp32)
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;

    const uint4 *src = reinterpret_cast<const uint4 *>(x + row * row_stride);
    float f[V * E];
    float amax = 0.0f;
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const uint4 raw = __ldg(src + v * 32 + lane);     // vector v covers elements [(v*32+lane)*E, +E)
        Vec16<T>::unpack(raw, f + v * E);
#pragma unroll
        for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(f[v * E + i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));

    const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f);
    if (lane == 0) scale[row] = s;

    int8_t *dst = q + row * 512;
#pragma unroll
    for (int v = 0; v < V; ++v) {
        uint32_t packed[E / 4];
#pragma unroll
        for (int w = 0; w < E / 4; ++w) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                float r = rintf(__fdiv_rn(f[v * E + 4 * w + b], s));
                r = fminf(fmaxf(r, -127.0f), 127.0f);
                word |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xFFu) << (8 * b);
            }
            packed[w] = word;
        }
        if constexpr (E == 8) {
            *reinterpret_cast<uint2 *>(dst + (v * 32 + lane) * E) = make_uint2(packed[0], packed[1]);
        } else {
            *reinterpret_cast<uint32_t *>(dst + (v * 32 + lane) * E) = packed[0];
        }
    }
}

}  // namespace

int launch_quantize_int8_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, int8_t *q,
                              float *scale, cudaStream_t stream) {
    if (rows == 0) return SMLA_OK;
    if (!x || !q || !scale || rows < 0) return SMLA_EINVAL;
    const int64_t elem = (x_dtype == 2) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || ((x_row_stride * elem) & 15) ||
        (reinterpret_cast<uintptr_t>(q) & 7u))
        return SMLA_EALIGN;
    const int64_t blocks64 = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks64 > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    const dim3 grid(static_cast<unsigned>(blocks64)), block(kWarpsPerBlock * 32);
    switch (x_dtype) {
        case 0:
            quantize_int8_rows_kernel<<<grid, block, 0, stream>>>(static_cast<const __nv_bfloat16 *>(x), rows,
                                                                  x_row_stride, q, scale);
            break;
        case 1:
            quantize_int8_rows_kernel<<<grid, block, 0, stream>>>(static_cast<const __half *>(x), rows,
                                                                  x_row_stride, q, scale);
            break;
        case 2:
            quantize_int8_rows_kernel<<<grid, block, 0, stream>>>(static_cast<const float *>(x), rows,
                                                                  x_row_stride, q, scale);
            break;
        default:
            return SMLA_EINVAL;
    }
    return static_cast<int>(cudaGetLastError());
}

}  // namespace smla
