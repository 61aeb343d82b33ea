// Writers of the two paged sparse-MLA cache formats for sm_100a: encode a batch of new latent rows
// and scatter them to their slots in one pass.
//
// The reference ships no device writer; its tests and benchmarks build caches with torch composites
// (tests/test_sparse_mla_decode_sm86.py:14-44 for fp8_ds_mla, tests/test_sparse_mla_prefill_int8_adversarial.py:5-12,35-60
// for the 528-byte int8_ds_mla token of the serving engine's writer).  The bytes written here are
// those formats:
//   int8_ds_mla  token = 512 int8 | fp32 scale | 12 zero bytes; scale and codes as in
//                quantize_int8_ds_mla_rows (flash_mla/int8_sparse_mla.py:15-26) or, scale_rule 1,
//                scale = max(amax / 127, 1e-12) as in the test's _quantize_rows;
//   fp8_ds_mla   block = [bs x 576 data][bs x 8 scales]; data = 448 e4m3 codes of x / 2^e + 64 bf16,
//                scales = 7 x (e + 127) + 127, e the smallest exponent with amax <= 448 * 2^e per 64 dims
//                (clamped to [-120, 120], 0 for an all-zero group), found exactly from the fp32 bits.
// Everything is evaluated in IEEE fp32 with true division; this file must NOT be built with
// --use_fast_math.
//
// HBM-bound: one warp per row, each lane owns 16 consecutive elements (one 256-bit load for 16-bit
// inputs, two for fp32) and stores its 16 output bytes with one 16-byte store; per bf16 row the
// kernel moves 1024 + 528 (int8) or 1024 + 584 (fp8) bytes plus the slot index.  The grid is sized
// to the SMs; a warp walks rows with the next row's loads (and slot) in flight while it encodes the
// current one.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "row_codec.cuh"
#include "smla_internal.h"

namespace smla {

int row_kernel_blocks(const void *kernel, int64_t rows, unsigned *blocks);   // quantize_int8_sm100.cu

namespace {

using rowcodec::Lane16;
constexpr int kWarpsPerBlock = 8;

struct WriterArgs {
    const uint8_t *x;          // rows of 512 elements
    int64_t rows;
    int64_t x_row_bytes;
    const void *slots;         // int32 or int64 [rows]
    int slots_i64;
    uint8_t *cache;
    int64_t block_stride;      // bytes
    int64_t pos_stride;        // bytes between the tokens of a block (int8 format)
    uint32_t block_size;
    int block_shift;           // log2(block_size) when it is a power of two, else -1
    int64_t num_slots;         // num_blocks * block_size, below 2^31
    int scale_rule;            // int8 format: 0 = max(amax, 1e-12) / 127, 1 = max(amax / 127, 1e-12)
    int wide;                  // rows are 32-byte aligned: 256-bit loads
    int st16;                  // fp8 format: blocks are 16-byte aligned (else 8-byte stores)
};

__device__ __forceinline__ void store16(uint8_t *p, const uint4 &v, bool st16) {
    if (st16) {
        *reinterpret_cast<uint4 *>(p) = v;
    } else {
        *reinterpret_cast<uint2 *>(p) = make_uint2(v.x, v.y);
        *reinterpret_cast<uint2 *>(p + 8) = make_uint2(v.z, v.w);
    }
}

// slot -> (block, position); 32-bit arithmetic (a 64-bit division costs as much as encoding the row).
__device__ __forceinline__ void split_slot(const WriterArgs &a, int64_t slot, uint32_t &blk, uint32_t &pos) {
    const uint32_t s32 = static_cast<uint32_t>(slot);
    if (a.block_shift >= 0) {
        blk = s32 >> a.block_shift;
        pos = s32 & (a.block_size - 1u);
    } else {
        blk = s32 / a.block_size;
        pos = s32 - blk * a.block_size;
    }
}

__device__ __forceinline__ int64_t slot_of(const WriterArgs &a, int64_t row) {
    return a.slots_i64 ? __ldg(static_cast<const int64_t *>(a.slots) + row)
                       : static_cast<int64_t>(__ldg(static_cast<const int32_t *>(a.slots) + row));
}

// One row, already in registers as fp32, to its int8_ds_mla token.
__device__ __forceinline__ void encode_int8(const WriterArgs &a, const float *f, int64_t slot, int lane) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = rowcodec::warp_max(amax);
    const float s = a.scale_rule == 0 ? __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f)
                                      : fmaxf(__fdiv_rn(amax, 127.0f), 1e-12f);
    uint32_t w[4];
    rowcodec::int8_codes16(f, s, w);
    uint32_t blk, pos;
    split_slot(a, slot, blk, pos);
    uint8_t *tok = a.cache + blk * a.block_stride + pos * a.pos_stride;
    *reinterpret_cast<uint4 *>(tok + lane * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    if (lane == 0) *reinterpret_cast<uint4 *>(tok + 512) = make_uint4(__float_as_uint(s), 0u, 0u, 0u);
}

// Smallest e with amax <= 448 * 2^e, from the bits of amax = 1.f * 2^(E - 127) and 448 = 1.75 * 2^8:
// e = E - 135 when 1.f <= 1.75, else E - 134 (subnormal amax lands far below the clamp either way).
__device__ __forceinline__ int ue8m0_exponent(float amax) {
    const uint32_t u = __float_as_uint(amax);
    if (u == 0u) return 0;
    const int e = static_cast<int>(u >> 23) - 135 + ((u & 0x7FFFFFu) > 0x600000u ? 1 : 0);
    return max(-120, min(120, e));
}

__device__ __forceinline__ uint32_t pack_bf16_rn(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);   // .x = a in the low half
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);   // a in the low byte
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

// One row to its fp8_ds_mla token: four lanes share a group of 64 dims; groups 0..6 are NoPE, lanes
// 28..31 hold the RoPE tail (bf16 inputs round to themselves).
__device__ __forceinline__ void encode_fp8(const WriterArgs &a, const float *f, int64_t slot, int lane) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const int e = ue8m0_exponent(amax);
    uint32_t sc_lo = 0, sc_hi = 127u << 24;                // the 8 scale bytes, assembled in every lane
#pragma unroll
    for (int g = 0; g < 7; ++g) {
        const uint32_t byte = static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, 4 * g) + 127);
        if (g < 4) sc_lo |= byte << (8 * g);
        else sc_hi |= byte << (8 * (g - 4));
    }
    uint32_t blk, pos;
    split_slot(a, slot, blk, pos);
    uint8_t *block = a.cache + blk * a.block_stride;
    uint8_t *tok = block + pos * 576u;
    if (lane < 28) {
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);     // 2^-e, exact
        uint4 w;
        w.x = pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
        w.y = pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
        w.z = pack_e4m3x4(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
        w.w = pack_e4m3x4(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
        store16(tok + lane * 16, w, a.st16 != 0);
    } else {
        const uint4 r0 = make_uint4(pack_bf16_rn(f[0], f[1]), pack_bf16_rn(f[2], f[3]), pack_bf16_rn(f[4], f[5]),
                                    pack_bf16_rn(f[6], f[7]));
        const uint4 r1 = make_uint4(pack_bf16_rn(f[8], f[9]), pack_bf16_rn(f[10], f[11]), pack_bf16_rn(f[12], f[13]),
                                    pack_bf16_rn(f[14], f[15]));
        store16(tok + 448 + (lane - 28) * 32, r0, a.st16 != 0);
        store16(tok + 448 + (lane - 28) * 32 + 16, r1, a.st16 != 0);
    }
    if (lane == 0)
        *reinterpret_cast<uint2 *>(block + static_cast<int64_t>(a.block_size) * 576 + pos * 8) = make_uint2(sc_lo, sc_hi);
}

template <typename T, bool FP8>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) write_ds_mla_cache_kernel(const WriterArgs a) {
    constexpr int V = Lane16<T>::kVecs;
    const int lane = threadIdx.x & 31;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
    int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    uint4 raw[V];
    int64_t slot = slot_of(a, row);
    Lane16<T>::load(a.x + row * a.x_row_bytes, lane, a.wide != 0, raw);
    while (true) {
        const int64_t next = row + stride;
        uint4 raw_next[V];
        int64_t slot_next = -1;
        if (next < a.rows) {
            slot_next = slot_of(a, next);
            Lane16<T>::load(a.x + next * a.x_row_bytes, lane, a.wide != 0, raw_next);
        }
        if (slot >= 0 && slot < a.num_slots) {             // padding rows of a batch carry slot -1
            float f[16];
            Lane16<T>::unpack(raw, f);
            if constexpr (FP8) encode_fp8(a, f, slot, lane);
            else encode_int8(a, f, slot, lane);
        }
        if (next >= a.rows) break;
#pragma unroll
        for (int v = 0; v < V; ++v) raw[v] = raw_next[v];
        slot = slot_next;
        row = next;
    }
}

int check_common(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, const void *slots, void *cache,
                 int64_t num_blocks, int block_size, WriterArgs &a) {
    if (!x || !slots || !cache || rows < 0 || num_blocks <= 0 || block_size <= 0 || x_dtype < 0 || x_dtype > 2)
        return SMLA_EINVAL;
    const int64_t elem = (x_dtype == 2) ? 4 : 2;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || ((x_row_stride * elem) & 15) ||
        (reinterpret_cast<uintptr_t>(cache) & 15u))
        return SMLA_EALIGN;
    a.x = static_cast<const uint8_t *>(x);
    a.rows = rows;
    a.x_row_bytes = x_row_stride * elem;
    a.slots = slots;
    a.cache = static_cast<uint8_t *>(cache);
    if (num_blocks * block_size > 0x7FFFFFFFll) return SMLA_ETOOBIG;     // more tokens than any device holds
    a.block_size = static_cast<uint32_t>(block_size);
    a.block_shift = (block_size & (block_size - 1)) ? -1 : __builtin_ctz(static_cast<unsigned>(block_size));
    a.num_slots = num_blocks * block_size;
    a.wide = !(reinterpret_cast<uintptr_t>(x) & 31u) && !(a.x_row_bytes & 31);
    return SMLA_OK;
}

template <bool FP8>
int dispatch(int x_dtype, const WriterArgs &a, cudaStream_t stream) {
    const void *kernel =
        x_dtype == 0   ? reinterpret_cast<const void *>(&write_ds_mla_cache_kernel<__nv_bfloat16, FP8>)
        : x_dtype == 1 ? reinterpret_cast<const void *>(&write_ds_mla_cache_kernel<__half, FP8>)
                       : reinterpret_cast<const void *>(&write_ds_mla_cache_kernel<float, FP8>);
    unsigned blocks = 0;
    if (const int rc = row_kernel_blocks(kernel, a.rows, &blocks)) return rc;
    void *args[] = {const_cast<WriterArgs *>(&a)};
    return static_cast<int>(cudaLaunchKernel(kernel, dim3(blocks), dim3(kWarpsPerBlock * 32), args, 0, stream));
}

}  // namespace

int launch_write_int8_ds_mla(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, const void *slots,
                             int slots_i64, void *cache, int64_t num_blocks, int block_size, int64_t block_stride,
                             int64_t pos_stride, int scale_rule, cudaStream_t stream) {
    if (rows == 0) return SMLA_OK;
    WriterArgs a{};
    if (const int rc = check_common(x, x_dtype, rows, x_row_stride, slots, cache, num_blocks, block_size, a)) return rc;
    if (scale_rule != 0 && scale_rule != 1) return SMLA_EINVAL;
    if (pos_stride < 528 || block_stride < pos_stride * block_size) return SMLA_EINVAL;
    if ((pos_stride & 15) || (block_stride & 15)) return SMLA_EALIGN;
    a.slots_i64 = slots_i64;
    a.block_stride = block_stride;
    a.pos_stride = pos_stride;
    a.scale_rule = scale_rule;
    return dispatch<false>(x_dtype, a, stream);
}

int launch_write_fp8_ds_mla(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, const void *slots,
                            int slots_i64, void *cache, int64_t num_blocks, int block_size, int64_t block_stride,
                            cudaStream_t stream) {
    if (rows == 0) return SMLA_OK;
    WriterArgs a{};
    if (const int rc = check_common(x, x_dtype, rows, x_row_stride, slots, cache, num_blocks, block_size, a)) return rc;
    if (block_stride < 584ll * block_size) return SMLA_EINVAL;
    // 16-byte stores into the data area where every block starts on a 16-byte boundary (an even
    // block_size does that for dense blocks), 8-byte stores otherwise and for the scale records.
    if (block_stride & 7) return SMLA_EALIGN;
    a.st16 = !(block_stride & 15);
    a.slots_i64 = slots_i64;
    a.block_stride = block_stride;
    a.pos_stride = 576;
    return dispatch<true>(x_dtype, a, stream);
}

}  // namespace smla
