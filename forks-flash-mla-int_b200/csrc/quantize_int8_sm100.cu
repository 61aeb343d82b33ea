// int8_ds_mla row quantizer for sm_100a.
//
// Bit-exact with quantize_int8_ds_mla_rows (flash_mla/int8_sparse_mla.py:15-26 of the
// reference): scale = max(amax|x|, 1e-12f) / 127.0f and q = clamp(rint(x / scale), -127, 127),
// as evaluated in IEEE fp32 with true division and round-half-even (row_codec.cuh shows how the
// codes are obtained without a division per element).  This translation unit must NOT be built with
// --use_fast_math.
//
// HBM-bound: one warp per 512-element row, one 256-bit load and one 16-byte store per lane, one pass
// (the row stays in registers between the amax reduction and the quantisation): 1024 + 512 + 4 bytes
// per bf16 row.  The grid is sized to the SMs and every warp walks rows with the next row's loads in
// flight while it works on the current one.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "row_codec.cuh"
#include "smla_internal.h"

namespace smla {
namespace {

using rowcodec::Lane16;
constexpr int kWarpsPerBlock = 8;

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quantize_int8_rows_kernel(const uint8_t *__restrict__ x, int64_t rows, int64_t row_bytes, int wide,
                          int8_t *__restrict__ q, float *__restrict__ scale) {
    constexpr int V = Lane16<T>::kVecs;
    const int lane = threadIdx.x & 31;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
    int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    uint4 raw[V];
    Lane16<T>::load(x + row * row_bytes, lane, wide != 0, raw);
    while (true) {
        const int64_t next = row + stride;
        uint4 raw_next[V];
        if (next < rows) Lane16<T>::load(x + next * row_bytes, lane, wide != 0, raw_next);

        float f[16];
        Lane16<T>::unpack(raw, f);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
        amax = rowcodec::warp_max(amax);
        const float s = __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f);
        uint32_t w[4];
        rowcodec::int8_codes16(f, s, w);
        *reinterpret_cast<uint4 *>(q + row * 512 + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        if (lane == 0) scale[row] = s;

        if (next >= rows) break;
#pragma unroll
        for (int v = 0; v < V; ++v) raw[v] = raw_next[v];
        row = next;
    }
}

}  // namespace

// Blocks for a grid-stride row kernel of 8 warps per block: enough to fill every SM at the kernel's
// occupancy, never more than one row per warp needs.
int row_kernel_blocks(const void *kernel, int64_t rows, unsigned *blocks) {
    int dev = 0, sms = 0, per_sm = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kWarpsPerBlock * 32, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int64_t need = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const int64_t fill = static_cast<int64_t>(sms) * (per_sm > 0 ? per_sm : 1);
    *blocks = static_cast<unsigned>(need < fill ? need : fill);
    return SMLA_OK;
}

int launch_quantize_int8_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, int8_t *q,
                              float *scale, cudaStream_t stream) {
    if (rows == 0) return SMLA_OK;
    if (!x || !q || !scale || rows < 0 || x_dtype < 0 || x_dtype > 2) return SMLA_EINVAL;
    const int64_t row_bytes = x_row_stride * ((x_dtype == 2) ? 4 : 2);
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (row_bytes & 15) || (reinterpret_cast<uintptr_t>(q) & 15u))
        return SMLA_EALIGN;
    const int wide = !(reinterpret_cast<uintptr_t>(x) & 31u) && !(row_bytes & 31);
    const void *kernel = x_dtype == 0   ? reinterpret_cast<const void *>(&quantize_int8_rows_kernel<__nv_bfloat16>)
                         : x_dtype == 1 ? reinterpret_cast<const void *>(&quantize_int8_rows_kernel<__half>)
                                        : reinterpret_cast<const void *>(&quantize_int8_rows_kernel<float>);
    unsigned blocks = 0;
    if (const int rc = row_kernel_blocks(kernel, rows, &blocks)) return rc;
    const uint8_t *xb = static_cast<const uint8_t *>(x);
    void *args[] = {&xb, &rows, const_cast<int64_t *>(&row_bytes), const_cast<int *>(&wide), &q, &scale};
    return static_cast<int>(cudaLaunchKernel(kernel, dim3(blocks), dim3(kWarpsPerBlock * 32), args, 0, stream));
}

}  // namespace smla
