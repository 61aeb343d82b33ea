// Row loaders and the int8_ds_mla code computation shared by the row quantizer and the cache writers.
//
// A warp owns a 512-element row; lane l owns the 16 consecutive elements [16 l, 16 l + 16): one
// 256-bit load for 16-bit inputs (two for fp32) and one 16-byte store of the 16 output bytes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace smla {
namespace rowcodec {

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
// 32 bytes at p: one 256-bit request when p is 32-byte aligned (warp-uniform choice), else two of 128 bits.
__device__ __forceinline__ void load32(const uint8_t *p, bool wide, uint4 &lo, uint4 &hi) {
    if (wide) {
        ldg_nc_v8(p, lo, hi);
    } else {
        lo = ldg_nc_v4(p);
        hi = ldg_nc_v4(p + 16);
    }
}

// The raw bytes of a lane's 16 elements (kept in flight while the previous row is processed) and
// their conversion to fp32.
template <typename T> struct Lane16;
template <> struct Lane16<__nv_bfloat16> {
    static constexpr int kVecs = 2;
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, uint4 *raw) {
        load32(row + lane * 32, wide, raw[0], raw[1]);
    }
    static __device__ __forceinline__ void unpack(const uint4 *raw, float *f) {
        const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
};
template <> struct Lane16<__half> {
    static constexpr int kVecs = 2;
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, uint4 *raw) {
        load32(row + lane * 32, wide, raw[0], raw[1]);
    }
    static __device__ __forceinline__ void unpack(const uint4 *raw, float *f) {
        const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
};
template <> struct Lane16<float> {
    static constexpr int kVecs = 4;
    static __device__ __forceinline__ void load(const uint8_t *row, int lane, bool wide, uint4 *raw) {
        load32(row + lane * 64, wide, raw[0], raw[1]);
        load32(row + lane * 64 + 32, wide, raw[2], raw[3]);
    }
    static __device__ __forceinline__ void unpack(const uint4 *raw, float *f) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[4 * i] = __uint_as_float(raw[i].x);
            f[4 * i + 1] = __uint_as_float(raw[i].y);
            f[4 * i + 2] = __uint_as_float(raw[i].z);
            f[4 * i + 3] = __uint_as_float(raw[i].w);
        }
    }
};

// Maximum over the warp of a NON-NEGATIVE float: the bit patterns order like the values, so one
// integer warp reduction does it.
__device__ __forceinline__ float warp_max(float v) {
    return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
}

__device__ __forceinline__ uint32_t pack_low_bytes(const uint32_t *y) {   // byte i of the result = low byte of y[i]
    const uint32_t lo = __byte_perm(y[0], y[1], 0x0040);
    const uint32_t hi = __byte_perm(y[2], y[3], 0x0040);
    return __byte_perm(lo, hi, 0x5410);
}

// The 16 codes clamp(rint(f[i] / s), -127, 127) of a lane, packed four to a word, BIT-EXACT with IEEE
// fp32 division followed by round-half-even -- without a division instruction sequence per element.
//
// s is the row scale (amax / 127 up to rounding, at least 7.8e-15), so |f / s| <= 127 (1 + 2^-23) and
// the clamp never acts: rint alone gives +-127 at the ends.  Rounding is one addition of 1.5 * 2^23
// (round-half-even by the adder), which leaves the code in the low byte of the sum.
//
// Far from a tie.  q0 = f * RN(1 / s) is within |f / s| (2^-23 + 2^-48) < 2^-16 of the true quotient
// t, and RN(t) within half an ulp (<= 2^-18 below 128).  When q0 lies at least 2^-15 away from every
// half-integer, t, RN(t) and q0 sit strictly between the same two half-integers: rint(q0) is the code.
//
// Near a tie (about 1 % of the elements of bf16 rows, whose quotients are ratios of 8-bit
// significands) the correctly rounded quotient itself is needed.  One Newton step
// q1 = q0 + (f - q0 s) / s lands on it or next to it, and the residual e = f - q1 s, which one FMA
// delivers EXACTLY when q1 is within an ulp of t, proves which: t - q1 = e / s, so RN(t) = q1 if and
// only if |e| < (ulp(q1) / 2) s (q1 not a power of two; a quotient is never a midpoint).  Anything
// else -- the proof failing, |q1| = 0.5 -- sends the lane to true divisions; that path is there for
// rigour and practically never runs.
// Packed fp32 pairs (sm_100 has two-wide fp32 add / mul / fma on 64-bit register pairs).
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void split_f32x2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ void int8_codes16(const float *f, float s, uint32_t *w) {
    constexpr float kMagic = 12582912.0f;                     // 1.5 * 2^23
    constexpr float kTie = 0.5f - 0x1p-15f;
    const float r = __frcp_rn(s);
    const uint64_t rr = f32x2(r, r), magic2 = f32x2(kMagic, kMagic), neg_magic2 = f32x2(-kMagic, -kMagic),
                   neg_one2 = f32x2(-1.0f, -1.0f);
    bool unsure = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t y[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // two elements at a time: q0 = x r, sum = q0 + magic, back = sum - magic = rint(q0), d = q0 - back
            const uint64_t q2 = mul_f32x2(f32x2(f[4 * j + 2 * h], f[4 * j + 2 * h + 1]), rr);
            const uint64_t sum2 = add_f32x2(q2, magic2);
            const uint64_t d2 = fma_f32x2(add_f32x2(sum2, neg_magic2), neg_one2, q2);
            float q0[2], sum[2], d[2];
            split_f32x2(q2, q0[0], q0[1]);
            split_f32x2(sum2, sum[0], sum[1]);
            split_f32x2(d2, d[0], d[1]);
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const bool near_tie = fabsf(d[b]) > kTie;
                if (__any_sync(0xffffffffu, near_tie)) {      // warp-uniform: skipped for most elements
                    if (near_tie) {
                        const float x = f[4 * j + 2 * h + b];
                        const float q1 = __fmaf_rn(__fmaf_rn(-q0[b], s, x), r, q0[b]);
                        const float e = __fmaf_rn(-q1, s, x);
                        const float half_ulp_s = s * __uint_as_float((__float_as_uint(q1) & 0x7F800000u) - (24u << 23));
                        unsure |= !(fabsf(e) < half_ulp_s) || fabsf(q1) == 0.5f;
                        sum[b] = __fadd_rn(q1, kMagic);
                    }
                }
                y[2 * h + b] = __float_as_uint(sum[b]);
            }
        }
        w[j] = pack_low_bytes(y);
    }
    if (unsure) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t y[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float c = fminf(fmaxf(__fdiv_rn(f[4 * j + b], s), -127.0f), 127.0f);
                y[b] = __float_as_uint(__fadd_rn(c, kMagic));
            }
            w[j] = pack_low_bytes(y);
        }
    }
}

}  // namespace rowcodec
}  // namespace smla
