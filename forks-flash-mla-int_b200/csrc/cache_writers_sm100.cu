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
// kernel moves 1024 + 528 (int8) or 1024 + 584 (fp8) bytes plus the slot index.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "smla_internal.h"

namespace smla {
namespace {

constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void ldg_nc_v8(const void *p, uint4 &lo, uint4 &hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
}
__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// 32 bytes at p: one 256-bit request when p is 32-byte aligned (warp-uniform), else two of 128 bits.
__device__ __forceinline__ void load32(const uint8_t *p, bool wide, uint4 &lo, uint4 &hi) {
    if (wide) {
        ldg_nc_v8(p, lo, hi);
    } else {
        lo = ldg_nc_v4(p);
        hi = ldg_nc_v4(p + 16);
    }
}

// The 16 consecutive elements [16 * lane, 16 * lane + 16) of a row as floats; `bits` keeps the raw
// 16-bit patterns of a 16-bit input (the fp8 writer copies bf16 RoPE values through unchanged).
template <typename T> struct Lane16;
template <> struct Lane16<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, float *f, uint4 *bits) {
        load32(row + lane * 32, wide, bits[0], bits[1]);
        const uint32_t w[8] = {bits[0].x, bits[0].y, bits[0].z, bits[0].w, bits[1].x, bits[1].y, bits[1].z, bits[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    // bf16 patterns of the 16 elements: unchanged.
    static __device__ __forceinline__ void to_bf16(const float *, const uint4 *bits, uint4 *out) {
        out[0] = bits[0];
        out[1] = bits[1];
    }
};
__device__ __forceinline__ uint32_t pack_bf16_rn(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);   // .x = a in the low half
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ void floats_to_bf16(const float *f, uint4 *out) {
    out[0] = make_uint4(pack_bf16_rn(f[0], f[1]), pack_bf16_rn(f[2], f[3]), pack_bf16_rn(f[4], f[5]),
                        pack_bf16_rn(f[6], f[7]));
    out[1] = make_uint4(pack_bf16_rn(f[8], f[9]), pack_bf16_rn(f[10], f[11]), pack_bf16_rn(f[12], f[13]),
                        pack_bf16_rn(f[14], f[15]));
}
template <> struct Lane16<__half> {
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, float *f, uint4 *bits) {
        load32(row + lane * 32, wide, bits[0], bits[1]);
        const uint32_t w[8] = {bits[0].x, bits[0].y, bits[0].z, bits[0].w, bits[1].x, bits[1].y, bits[1].z, bits[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    static __device__ __forceinline__ void to_bf16(const float *f, const uint4 *, uint4 *out) { floats_to_bf16(f, out); }
};
template <> struct Lane16<float> {
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, float *f, uint4 *) {
        uint4 v[4];
        load32(row + lane * 64, wide, v[0], v[1]);
        load32(row + lane * 64 + 32, wide, v[2], v[3]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[4 * i] = __uint_as_float(v[i].x);
            f[4 * i + 1] = __uint_as_float(v[i].y);
            f[4 * i + 2] = __uint_as_float(v[i].z);
            f[4 * i + 3] = __uint_as_float(v[i].w);
        }
    }
    static __device__ __forceinline__ void to_bf16(const float *f, const uint4 *, uint4 *out) { floats_to_bf16(f, out); }
};

struct WriterArgs {
    const uint8_t *x;          // rows of 512 elements
    int64_t rows;
    int64_t x_row_bytes;
    const void *slots;         // int32 or int64 [rows]
    int slots_i64;
    uint8_t *cache;
    int64_t block_stride;      // bytes
    int64_t pos_stride;        // bytes between the tokens of a block (int8 format)
    int block_size;
    int64_t num_slots;         // num_blocks * block_size
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

__device__ __forceinline__ int64_t slot_of(const WriterArgs &a, int64_t row) {
    return a.slots_i64 ? static_cast<const int64_t *>(a.slots)[row]
                       : static_cast<int64_t>(static_cast<const int32_t *>(a.slots)[row]);
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) write_int8_ds_mla_kernel(const WriterArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const int64_t slot = slot_of(a, row);
    if (slot < 0 || slot >= a.num_slots) return;          // padding rows of a batch carry slot -1

    float f[16];
    uint4 bits[2];
    Lane16<T>::load(a.x + row * a.x_row_bytes, lane, a.wide != 0, f, bits);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = a.scale_rule == 0 ? __fdiv_rn(fmaxf(amax, 1e-12f), 127.0f)
                                      : fmaxf(__fdiv_rn(amax, 127.0f), 1e-12f);

    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float r = rintf(__fdiv_rn(f[4 * j + b], s));
            r = fminf(fmaxf(r, -127.0f), 127.0f);
            word |= (static_cast<uint32_t>(static_cast<int>(r)) & 0xFFu) << (8 * b);
        }
        w[j] = word;
    }
    uint8_t *tok = a.cache + (slot / a.block_size) * a.block_stride + (slot % a.block_size) * a.pos_stride;
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

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) write_fp8_ds_mla_kernel(const WriterArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const int64_t slot = slot_of(a, row);
    if (slot < 0 || slot >= a.num_slots) return;

    float f[16];
    uint4 bits[2];
    Lane16<T>::load(a.x + row * a.x_row_bytes, lane, a.wide != 0, f, bits);
    // Four lanes share a group of 64 dims: groups 0..6 are NoPE, lanes 28..31 hold the RoPE tail.
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const int e = ue8m0_exponent(amax);
    uint32_t sc_lo = 0, sc_hi = 0;                         // the 8 scale bytes, assembled in every lane
#pragma unroll
    for (int g = 0; g < 7; ++g) {
        const uint32_t byte = static_cast<uint32_t>(__shfl_sync(0xffffffffu, e, 4 * g) + 127);
        if (g < 4) sc_lo |= byte << (8 * g);
        else sc_hi |= byte << (8 * (g - 4));
    }
    sc_hi |= 127u << 24;

    const int64_t blk = slot / a.block_size;
    const int pos = static_cast<int>(slot % a.block_size);
    uint8_t *block = a.cache + blk * a.block_stride;
    uint8_t *tok = block + static_cast<int64_t>(pos) * 576;
    if (lane < 28) {
        const float inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);     // 2^-e, exact
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t code = __nv_cvt_float_to_fp8(f[4 * j + b] * inv, __NV_SATFINITE, __NV_E4M3);
                word |= code << (8 * b);
            }
            w[j] = word;
        }
        store16(tok + lane * 16, make_uint4(w[0], w[1], w[2], w[3]), a.st16 != 0);
    } else {
        uint4 r[2];
        Lane16<T>::to_bf16(f, bits, r);
        store16(tok + 448 + (lane - 28) * 32, r[0], a.st16 != 0);
        store16(tok + 448 + (lane - 28) * 32 + 16, r[1], a.st16 != 0);
    }
    if (lane == 0)
        *reinterpret_cast<uint2 *>(block + static_cast<int64_t>(a.block_size) * 576 + pos * 8) = make_uint2(sc_lo, sc_hi);
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
    a.block_size = block_size;
    a.num_slots = num_blocks * block_size;
    a.wide = !(reinterpret_cast<uintptr_t>(x) & 31u) && !(a.x_row_bytes & 31);
    return SMLA_OK;
}

template <template <typename> class Launcher>
int dispatch(int x_dtype, const WriterArgs &a, cudaStream_t stream) {
    const int64_t blocks64 = (a.rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (blocks64 > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    const dim3 grid(static_cast<unsigned>(blocks64)), block(kWarpsPerBlock * 32);
    switch (x_dtype) {
        case 0: Launcher<__nv_bfloat16>::run(grid, block, stream, a); break;
        case 1: Launcher<__half>::run(grid, block, stream, a); break;
        default: Launcher<float>::run(grid, block, stream, a); break;
    }
    return static_cast<int>(cudaGetLastError());
}
template <typename T> struct LaunchInt8 {
    static void run(dim3 g, dim3 b, cudaStream_t s, const WriterArgs &a) { write_int8_ds_mla_kernel<T><<<g, b, 0, s>>>(a); }
};
template <typename T> struct LaunchFp8 {
    static void run(dim3 g, dim3 b, cudaStream_t s, const WriterArgs &a) { write_fp8_ds_mla_kernel<T><<<g, b, 0, s>>>(a); }
};

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
    return dispatch<LaunchInt8>(x_dtype, a, stream);
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
    return dispatch<LaunchFp8>(x_dtype, a, stream);
}

}  // namespace smla
