// Sparse MLA attention (decode and prefill) for sm_100a: gather + dequant + QK^T + online
// softmax + PV in one kernel, tensor-core work on tcgen05.mma with TMEM accumulators.
//
// Replaces, for both cache formats, the reference's selection-dequant pre-pass, split-KV
// mma.sync decode kernel and fused prefill kernel (csrc/flash_sparse_mla_decode_sm80.cu:129-191,
// 443-738; csrc/flash_sparse_mla_prefill_fused_sm80.cu:50-86,154-457) and their combine kernel
// (csrc/flash_sparse_mla_decode_sm80.cu:382-439).  Semantics follow the reference's fp32 oracle
// (tests/test_sparse_mla_prefill_adversarial.py:25-53): invalid slot ids are zero rows that stay
// in the softmax, positions >= lens are excluded, attn_sink joins the denominator once.
//
// Orientation.  One CTA owns one (token, block of <= 64 heads[, split]).  The selected rows are
// the MMA M dimension, 128 per tile:
//     S^T[128 rows, N heads]   = K_tile[128, 512] . Q[N, 512]^T         (A, B both K-major)
//     O^T[512 dims, N heads]  += K_tile^T[512, 128] . P^T[128, N]       (A, B both MN-major)
// so a 64-head block still fills the 128-lane datapath, and the SAME shared-memory K tile
// serves both products: it is stored as 8x16-byte core matrices (8 rows x 8 dims) which a
// no-swizzle descriptor can walk row-group-first (K-major) or dim-group-first (MN-major).
//
// Roles (640 threads): warps 0-3 softmax/epilogue (thread 0 also issues every MMA); warps 4-19
// gather: each owns 8 rows of the tile, loads the raw bytes of its rows for the NEXT tile into
// registers (16-byte loads), and converts them chunk by chunk (128 dims) into the single K
// buffer as soon as the previous tile's PV releases that chunk.
//
// Every spin is time-bounded; a wait that runs out sets a bit in the device status word and the
// CTA leaves through the normal teardown.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "sm100_ptx.cuh"
#include "smla_internal.h"

namespace smla {

__device__ int g_device_status = 0;

#ifdef SMLA_TRACE   // developer timing trace of CTA 0 (never defined in the product build)
__device__ unsigned long long g_trace[32 * 16];
#define SMLA_MARK(tile, k)                                                              \
    do {                                                                                \
        if (blockIdx.x == 0 && blockIdx.y == 0 && (tile) < 32) g_trace[(tile) * 16 + (k)] = clock64(); \
    } while (0)
#else
#define SMLA_MARK(tile, k) do {} while (0)
#endif

namespace {

constexpr int kD = 512;
constexpr int kTileRows = 128;
constexpr int kSoftmaxThreads = 128;
constexpr int kGatherWarps = 16;
constexpr int kThreads = kSoftmaxThreads + kGatherWarps * 32;  // 640
constexpr int kNumWarps = kThreads / 32;
constexpr int kCoreBytes = 128;             // one 8x16B core matrix
constexpr int kRowGroupBytes = 64 * kCoreBytes;  // 8 rows x 512 dims of bf16
constexpr int kKBytes = 16 * kRowGroupBytes;     // 128 rows
constexpr int kTmemCols = 512;
constexpr int kTmemOCol = 64;               // O^T chunks start here; S^T at column 0
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units: the running max may lag by up to 2^8
constexpr int kSoftmaxBar = 1;
// Register rebalancing.  setmaxnreg.inc blocks (without any time limit) until the registers it asks
// for have been released INSIDE THE SAME CTA, so the two role budgets must fit the pool the CTA was
// launched with: 640 threads x 96 registers (the cap __launch_bounds__(640, 1) gives ptxas).
constexpr int kLaunchRegs = 96;
constexpr int kSoftmaxRegs = 224;
constexpr int kGatherRegs = 64;
static_assert(kSoftmaxThreads * kSoftmaxRegs + kGatherWarps * 32 * kGatherRegs <= kThreads * kLaunchRegs,
              "role register budgets exceed the CTA's launch-time register pool: setmaxnreg.inc would never return");
static_assert(kThreads * kLaunchRegs <= 65536 && kLaunchRegs == ((65536 / kThreads) / 8) * 8, "launch register cap");

struct StreamDev {
    const uint8_t *cache;
    const float *scale;
    const int *indices;
    const int *lens;
    long long idx_stride, block_stride, pos_stride, scale_block_stride, scale_pos_stride;
    int topk, num_slots, block_size, vec16;
};

struct KernelArgs {
    const __nv_bfloat16 *q;
    long long q_ts, q_hs;
    __nv_bfloat16 *out;
    long long o_ts, o_hs;
    const float *sink;
    float *part_o;   // fp32 [T, H, S, 512] un-normalised partial outputs (S > 1)
    float *part_ml;  // fp32 [T, H, S, 2]   {reference max (log2 units), denominator}
    StreamDev swa, extra;
    int T, H, head_blocks, num_splits;
    float scale_log2;
};

template <int NPAD>
struct Smem {
    static constexpr int kQ = 0;                         // Q tile, core(hg, dg) at hg*8192 + dg*128
    static constexpr int kK = kQ + NPAD * 1024;          // K tile, core(rg, dg) at rg*8192 + dg*128
    static constexpr int kP = kK + kKBytes;              // P^T,   core(hg, rg) at hg*2048 + rg*128
    static constexpr int kRed = kP + NPAD * 256;         // [4][NPAD] floats
    static constexpr int kM = kRed + 4 * NPAD * 4;       // running reference max per head
    static constexpr int kAlpha = kM + NPAD * 4;         // rescale factor / final 1/l per head
    static constexpr int kBars = kAlpha + NPAD * 4;      // ready[4], free[4], s, o
    static constexpr int kTmemPtr = kBars + 10 * 8;
    static constexpr int kAbort = kTmemPtr + 4;
    static constexpr int kTotal = kAbort + 4 + 8;
};

// ------------------------------------------------------------------ small device helpers
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ldg_nc_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_nc_v2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_nc_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
// 16 bytes of a cache row.  fp8 rows are at least 8-byte aligned, int8 rows at least 4.
template <int FMT>
__device__ __forceinline__ uint4 load16(const uint8_t *p, bool vec16) {
    if (vec16) return ldg_nc_v4(p);
    if constexpr (FMT == SMLA_FP8_DS_MLA) {
        const uint2 a = ldg_nc_v2(p), b = ldg_nc_v2(p + 8);
        return make_uint4(a.x, a.y, b.x, b.y);
    } else {
        return make_uint4(ldg_nc_u32(p), ldg_nc_u32(p + 4), ldg_nc_u32(p + 8), ldg_nc_u32(p + 12));
    }
}

// 4 int8 -> 4 x bf16_rn(float(v) * scale).  float(v) is built exactly with the 2^23 magic.
__device__ __forceinline__ void cvt_i8x4(uint32_t w, float s, uint32_t &lo, uint32_t &hi) {
    const uint32_t x = w ^ 0x80808080u;
    const float f0 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)) - 8388736.0f) * s;
    const float f1 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)) - 8388736.0f) * s;
    const float f2 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)) - 8388736.0f) * s;
    const float f3 = (__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)) - 8388736.0f) * s;
    lo = pack_bf16x2(f0, f1);
    hi = pack_bf16x2(f2, f3);
}
// 4 e4m3 -> 4 x bf16(e4m3 * 2^(ue8m0 - 127)); exact (power-of-two scaling of a 4-bit significand).
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, float mult, uint32_t &lo, uint32_t &hi) {
    const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xFFFFu), __NV_E4M3);
    const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
    const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&a));
    const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&b));
    lo = pack_bf16x2(fa.x * mult, fa.y * mult);
    hi = pack_bf16x2(fb.x * mult, fb.y * mult);
}

// Column reduction across the 32 lanes of a warp: every lane holds L values (one per column);
// each step trades half of them with the lane `MASK` away, so 62 shuffles reduce 64 columns.
// Result: N=64 -> out[0..1] are columns 2*lane, 2*lane+1; N=32 -> out[0] is column lane;
// N=16 -> out[0] is column lane>>1 (held by both lanes of a pair).
template <int L, int MASK, bool IS_MAX>
struct ColReduce {
    static __device__ __forceinline__ float op(float a, float b) { return IS_MAX ? fmaxf(a, b) : a + b; }
    static __device__ __forceinline__ void run(const float *v, int lane, float *out) {
        if constexpr (MASK == 0) {
#pragma unroll
            for (int i = 0; i < L; ++i) out[i] = v[i];
        } else if constexpr (L > 1) {
            const bool up = (lane & MASK) != 0;
            float nv[L / 2];
#pragma unroll
            for (int i = 0; i < L / 2; ++i) {
                const float keep = up ? v[i + L / 2] : v[i];
                const float send = up ? v[i] : v[i + L / 2];
                nv[i] = op(keep, __shfl_xor_sync(0xffffffffu, send, MASK));
            }
            ColReduce<L / 2, MASK / 2, IS_MAX>::run(nv, lane, out);
        } else {
            float nv[1] = {op(v[0], __shfl_xor_sync(0xffffffffu, v[0], MASK))};
            ColReduce<1, MASK / 2, IS_MAX>::run(nv, lane, out);
        }
    }
};
template <int NPAD>
__device__ __forceinline__ void store_col_partials(float *red_row, const float *r, int lane) {
    if constexpr (NPAD == 64) {
        *reinterpret_cast<float2 *>(red_row + 2 * lane) = make_float2(r[0], r[1]);
    } else if constexpr (NPAD == 32) {
        red_row[lane] = r[0];
    } else {
        if ((lane & 1) == 0) red_row[lane >> 1] = r[0];
    }
}

template <int N> struct TmemIO;
template <> struct TmemIO<16> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[16]) { tmem_ld_x16(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[16]) { tmem_st_x16(a, r); }
};
template <> struct TmemIO<32> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[32]) { tmem_ld_x32(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[32]) { tmem_st_x32(a, r); }
};
template <> struct TmemIO<64> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[64]) { tmem_ld_x64(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[64]) { tmem_st_x64(a, r); }
};

__device__ __forceinline__ void give_up(volatile int *abort_flag, int bit) {
    *abort_flag = 1;
    atomicOr(&g_device_status, bit);
}

// ------------------------------------------------------------------ gather role (warps 4..19)
template <int FMT>
struct RowRef {
    const uint8_t *ptr;   // first data byte of the row (unused when !ok)
    uint32_t sc0, sc1;    // fp8: the 8 UE8M0 bytes; int8: sc0 = fp32 scale bits
    bool ok, vec16;
};

__device__ __forceinline__ int load_slot_id(const KernelArgs &a, int t, int ns, int n, int g) {
    if (g < ns) return __ldg(a.swa.indices + static_cast<long long>(t) * a.swa.idx_stride + g);
    if (g < n) return __ldg(a.extra.indices + static_cast<long long>(t) * a.extra.idx_stride + (g - ns));
    return -1;
}

template <int FMT>
__device__ __forceinline__ RowRef<FMT> make_row_ref(const KernelArgs &a, int ns, int n, int g, int id) {
    RowRef<FMT> r;
    r.ptr = nullptr;
    r.sc0 = 0u;
    r.sc1 = 0u;
    r.ok = false;
    r.vec16 = true;
    if (g >= n) return r;
    const StreamDev &s = (g < ns) ? a.swa : a.extra;
    if (static_cast<unsigned>(id) >= static_cast<unsigned>(s.num_slots)) return r;
    const int b = id / s.block_size;
    const int i = id - b * s.block_size;
    const uint8_t *blk = s.cache + static_cast<long long>(b) * s.block_stride;
    r.ok = true;
    r.vec16 = s.vec16 != 0;
    if constexpr (FMT == SMLA_FP8_DS_MLA) {
        r.ptr = blk + static_cast<long long>(i) * 576;
        const uint2 sc = ldg_nc_v2(blk + static_cast<long long>(s.block_size) * 576 + static_cast<long long>(i) * 8);
        r.sc0 = sc.x;
        r.sc1 = sc.y;
    } else {
        r.ptr = blk + static_cast<long long>(i) * s.pos_stride;
        r.sc0 = __float_as_uint(__ldg(s.scale + static_cast<long long>(b) * s.scale_block_stride +
                                      static_cast<long long>(i) * s.scale_pos_stride));
    }
    return r;
}

// Register-chunk schedule: lane (row = lane & 7, quarter = lane >> 3) loads 16-byte piece
// 4*j + quarter of its row in step j.  int8: 8 steps (512 B); fp8: 9 steps (448 B e4m3 + 128 B rope).
// K-buffer chunk c (dims 128c..128c+127) is fed by steps {2c, 2c+1}, plus step 8 for fp8 chunk 3.
template <int FMT> struct Steps { static constexpr int kCount = (FMT == SMLA_FP8_DS_MLA) ? 9 : 8; };

template <int FMT>
__device__ __forceinline__ void load_step(const RowRef<FMT> &r, int j, int quarter, uint4 &dst) {
    if (r.ok) dst = load16<FMT>(r.ptr + (4 * j + quarter) * 16, r.vec16);
    else dst = make_uint4(0u, 0u, 0u, 0u);
}

template <int FMT>
__device__ __forceinline__ void convert_step(const uint4 &raw, int j, int quarter, uint32_t sc0, uint32_t sc1,
                                             uint32_t k_row_addr /* K + rg*8192 + (lane&7)*16 */) {
    uint32_t o[8];
    if constexpr (FMT == SMLA_INT8_DS_MLA) {
        const float s = __uint_as_float(sc0);
        cvt_i8x4(raw.x, s, o[0], o[1]);
        cvt_i8x4(raw.y, s, o[2], o[3]);
        cvt_i8x4(raw.z, s, o[4], o[5]);
        cvt_i8x4(raw.w, s, o[6], o[7]);
        const uint32_t dg = 2u * (4u * j + quarter);
        st_shared_v4(k_row_addr + dg * kCoreBytes, o[0], o[1], o[2], o[3]);
        st_shared_v4(k_row_addr + (dg + 1u) * kCoreBytes, o[4], o[5], o[6], o[7]);
    } else {
        if (j < 7) {
            const uint32_t byte = (j < 4) ? ((sc0 >> (8 * j)) & 0xFFu) : ((sc1 >> (8 * (j - 4))) & 0xFFu);
            const float mult = __uint_as_float(byte << 23);   // 2^(ue8m0 - 127)
            cvt_e4m3x4(raw.x, mult, o[0], o[1]);
            cvt_e4m3x4(raw.y, mult, o[2], o[3]);
            cvt_e4m3x4(raw.z, mult, o[4], o[5]);
            cvt_e4m3x4(raw.w, mult, o[6], o[7]);
            const uint32_t dg = 2u * (4u * j + quarter);
            st_shared_v4(k_row_addr + dg * kCoreBytes, o[0], o[1], o[2], o[3]);
            st_shared_v4(k_row_addr + (dg + 1u) * kCoreBytes, o[4], o[5], o[6], o[7]);
        } else {
            const uint32_t dg = 56u + 4u * (j - 7) + quarter;   // RoPE tail: already bf16
            st_shared_v4(k_row_addr + dg * kCoreBytes, raw.x, raw.y, raw.z, raw.w);
        }
    }
}

template <int FMT, int NPAD>
__device__ __forceinline__ void gather_role(const KernelArgs &a, uint8_t *smem, int t, int ns, int n, int tile0,
                                            int ntl, int gwarp, int lane) {
    using L = Smem<NPAD>;
    constexpr int J = Steps<FMT>::kCount;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    const int quarter = lane >> 3;
    const int r_in_tile = gwarp * 8 + (lane & 7);
    const uint32_t k_row_addr = smem_u32(smem + L::kK) + gwarp * kRowGroupBytes + (lane & 7) * 16;

    int g = tile0 * kTileRows + r_in_tile;
    RowRef<FMT> cur = make_row_ref<FMT>(a, ns, n, g, load_slot_id(a, t, ns, n, g));
    uint4 raw[J];
#pragma unroll
    for (int j = 0; j < J; ++j) load_step<FMT>(cur, j, quarter, raw[j]);
    int id_next = (ntl > 1) ? load_slot_id(a, t, ns, n, g + kTileRows) : -1;

    for (int it = 0; it < ntl; ++it) {
        const bool has_next = it + 1 < ntl;
        RowRef<FMT> nxt = make_row_ref<FMT>(a, ns, n, has_next ? g + kTileRows : n, id_next);
        if (it + 2 < ntl) id_next = load_slot_id(a, t, ns, n, g + 2 * kTileRows);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (it > 0) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(bars + (4 + c) * 8, (it - 1) & 1, abort_flag) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    if (lane == 0) give_up(abort_flag, kStatusGatherWait);
                    return;
                }
            }
            if (gwarp == 0 && lane == 0 && c == 0) SMLA_MARK(it, 7);
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const bool mine = (j < 8) ? ((j >> 1) == c) : (c == 3);
                if (mine) convert_step<FMT>(raw[j], j, quarter, cur.sc0, cur.sc1, k_row_addr);
            }
            if (gwarp == 0 && lane == 0) SMLA_MARK(it, 8 + c);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + c * 8);
            if (gwarp == 0 && lane == 0 && c == 3) SMLA_MARK(it, 12);
            if (has_next) {
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    const bool mine = (j < 8) ? ((j >> 1) == c) : (c == 3);
                    if (mine) load_step<FMT>(nxt, j, quarter, raw[j]);
                }
            }
        }
        cur = nxt;
        g += kTileRows;
    }
}

// ------------------------------------------------------------------ MMA issue (thread 0)
template <int NPAD>
__device__ __forceinline__ bool issue_qk(uint8_t *smem, uint32_t tmem_base, int it) {
    using L = Smem<NPAD>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    constexpr uint32_t idesc = umma_idesc_bf16(128, NPAD, 0, 0);
    // K-major A (rows x dims) and B (heads x dims): step along M/N = 8 rows = one row group
    // (8192 B), step along K = 8 dims = one core matrix (128 B).
    const uint64_t a0 = umma_desc(smem_u32(smem + L::kK), kCoreBytes, kRowGroupBytes);
    const uint64_t b0 = umma_desc(smem_u32(smem + L::kQ), kCoreBytes, kRowGroupBytes);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        if (!mbar_wait(bars + c * 8, it & 1, abort_flag)) {
            give_up(abort_flag, kStatusMmaWait);
            return false;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint64_t off = static_cast<uint64_t>(((16 * c + 2 * k) * kCoreBytes) >> 4);
            umma_bf16_ss(tmem_base, a0 + off, b0 + off, idesc, (c | k) != 0 ? 1u : 0u);
        }
    }
    umma_commit(bars + 8 * 8);
    return true;
}

template <int NPAD>
__device__ __forceinline__ void issue_pv(uint8_t *smem, uint32_t tmem_base, int it, bool last) {
    using L = Smem<NPAD>;
    const uint32_t bars = smem_u32(smem + L::kBars);
    constexpr uint32_t idesc = umma_idesc_bf16(128, NPAD, 1, 1);
    // MN-major A = K^T chunk (128 dims x 16 rows): M step = next dim group (128 B), K step = next
    // row group (8192 B).  MN-major B = P^T (N heads x 16 rows): N step = next head group
    // (2048 B), K step = next row group (128 B).
    const uint64_t a0 = umma_desc(smem_u32(smem + L::kK), kRowGroupBytes, kCoreBytes);
    const uint64_t b0 = umma_desc(smem_u32(smem + L::kP), kCoreBytes, 2048);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint64_t aoff = static_cast<uint64_t>((c * 16 * kCoreBytes + 2 * k * kRowGroupBytes) >> 4);
            const uint64_t boff = static_cast<uint64_t>((2 * k * kCoreBytes) >> 4);
            umma_bf16_ss(tmem_base + kTmemOCol + c * NPAD, a0 + aoff, b0 + boff, idesc, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bars + (4 + c) * 8);   // chunk c of the K buffer may be refilled
    }
    if (last) umma_commit(bars + 9 * 8);
}

// ------------------------------------------------------------------ softmax / epilogue role (warps 0..3)
template <int FMT, int NPAD>
__device__ __forceinline__ void softmax_role(const KernelArgs &a, uint8_t *smem, uint32_t tmem_base, int t, int h0,
                                             int hvalid, int sp, int n, int tile0, int ntl, int tid) {
    using L = Smem<NPAD>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    float *red = reinterpret_cast<float *>(smem + L::kRed);
    float *m_s = reinterpret_cast<float *>(smem + L::kM);
    float *alpha_s = reinterpret_cast<float *>(smem + L::kAlpha);
    const int lane = tid & 31, wq = tid >> 5;
    const int row = tid;                                     // TMEM lane = row of the tile / dim of an O chunk
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
    const uint32_t p_row_addr = smem_u32(smem + L::kP) + (row >> 3) * kCoreBytes + (row & 7) * 16;
    const bool direct = a.num_splits == 1;

    float lsum[NPAD];
#pragma unroll
    for (int h = 0; h < NPAD; ++h) lsum[h] = 0.0f;

    bool ok = true;
    for (int it = 0; it < ntl && ok; ++it) {
        if (tid == 0) {
            SMLA_MARK(it, 0);
            ok = issue_qk<NPAD>(smem, tmem_base, it);
            SMLA_MARK(it, 1);
        }
        __syncwarp();
        if (!mbar_wait(bars + 8 * 8, it & 1, abort_flag)) {
            give_up(abort_flag, kStatusSoftmaxWait);
            ok = false;
        }
        __syncwarp();
        // Leave together: every softmax thread must see the same decision before the named barriers.
        if (named_bar_or(kSoftmaxBar, kSoftmaxThreads, !ok)) {
            ok = false;
            break;
        }
        tc_fence_after_sync();

        if (tid == 0) SMLA_MARK(it, 2);
        uint32_t sraw[NPAD];
        TmemIO<NPAD>::ld(tmem_lane, sraw);
        float s[NPAD];
        const bool row_valid = (tile0 + it) * kTileRows + row < n;
#pragma unroll
        for (int h = 0; h < NPAD; ++h) s[h] = row_valid ? __uint_as_float(sraw[h]) * a.scale_log2 : -INFINITY;

        {   // per-head max over the 128 rows of the tile
            float r[2];
            ColReduce<NPAD, 16, true>::run(s, lane, r);
            store_col_partials<NPAD>(red + wq * NPAD, r, lane);
        }
        named_bar_sync(kSoftmaxBar, kSoftmaxThreads);
        bool need = false;
        if (tid < NPAD) {
            const float tm = fmaxf(fmaxf(red[tid], red[NPAD + tid]), fmaxf(red[2 * NPAD + tid], red[3 * NPAD + tid]));
            const float m_old = m_s[tid];
            need = tm > m_old + kRescaleThreshold;
            // The reference point is kept INTEGER-valued (log2 units): then 2^(s - m) has the same
            // mantissa whatever m is, so P rounds to bf16 identically in every split and the split
            // count only changes fp32 summation order, not the rounding of the weights.
            const float m_new = need ? ceilf(tm) : m_old;
            alpha_s[tid] = need ? fast_exp2(m_old - m_new) : 1.0f;
            m_s[tid] = m_new;
        }
        const bool rescale = named_bar_or(kSoftmaxBar, kSoftmaxThreads, need);
        if (tid == 0) SMLA_MARK(it, 3);

        if (rescale) {
#pragma unroll
            for (int h = 0; h < NPAD; ++h) lsum[h] *= alpha_s[h];
        }
        // P^T = exp2(S^T - m), rounded to bf16, into the MN-major B-operand layout.
#pragma unroll
        for (int hg = 0; hg < NPAD / 8; ++hg) {
            float p[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                p[i] = fast_exp2(s[hg * 8 + i] - m_s[hg * 8 + i]);
                lsum[hg * 8 + i] += p[i];
            }
            st_shared_v4(p_row_addr + hg * 2048, pack_bf16x2(p[0], p[1]), pack_bf16x2(p[2], p[3]),
                         pack_bf16x2(p[4], p[5]), pack_bf16x2(p[6], p[7]));
        }
        if (rescale && it > 0) {   // O^T[:, h] *= alpha[h]; the previous PV has completed (it precedes this QK)
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[NPAD];
                TmemIO<NPAD>::ld(tmem_lane + kTmemOCol + c * NPAD, o);
#pragma unroll
                for (int h = 0; h < NPAD; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha_s[h]);
                TmemIO<NPAD>::st(tmem_lane + kTmemOCol + c * NPAD, o);
            }
            tmem_st_wait();
        }
        if (tid == 0) SMLA_MARK(it, 4);
        fence_async_smem();
        tc_fence_before_sync();
        named_bar_sync(kSoftmaxBar, kSoftmaxThreads);
        if (tid == 0) {
            tc_fence_after_sync();
            SMLA_MARK(it, 5);
            issue_pv<NPAD>(smem, tmem_base, it, it + 1 == ntl);
            SMLA_MARK(it, 6);
        }
        __syncwarp();
    }
    if (!ok) return;

    // ---- epilogue: O^T / l
    if (!mbar_wait(bars + 9 * 8, 0, abort_flag)) give_up(abort_flag, kStatusEpilogueWait), ok = false;
    __syncwarp();
    if (named_bar_or(kSoftmaxBar, kSoftmaxThreads, !ok)) return;
    tc_fence_after_sync();
    {
        float r[2];
        ColReduce<NPAD, 16, false>::run(lsum, lane, r);
        store_col_partials<NPAD>(red + wq * NPAD, r, lane);
    }
    named_bar_sync(kSoftmaxBar, kSoftmaxThreads);
    if (tid < NPAD) {
        float l = (red[tid] + red[NPAD + tid]) + (red[2 * NPAD + tid] + red[3 * NPAD + tid]);
        if (direct) {
            if (a.sink != nullptr && tid < hvalid) l += fast_exp2(a.sink[h0 + tid] * kLog2e - m_s[tid]);
            alpha_s[tid] = 1.0f / l;
        } else if (tid < hvalid) {
            float *ml = a.part_ml + ((static_cast<long long>(t) * a.H + h0 + tid) * a.num_splits + sp) * 2;
            ml[0] = m_s[tid];
            ml[1] = l;
        }
    }
    named_bar_sync(kSoftmaxBar, kSoftmaxThreads);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        uint32_t o[NPAD];
        TmemIO<NPAD>::ld(tmem_lane + kTmemOCol + c * NPAD, o);
        const int d = c * 128 + row;
        if (direct) {
            __nv_bfloat16 *dst = a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0) * a.o_hs + d;
#pragma unroll
            for (int h = 0; h < NPAD; ++h)
                if (h < hvalid) dst[h * a.o_hs] = __float2bfloat16_rn(__uint_as_float(o[h]) * alpha_s[h]);
        } else {
            float *dst = a.part_o + ((static_cast<long long>(t) * a.H + h0) * a.num_splits + sp) * kD + d;
#pragma unroll
            for (int h = 0; h < NPAD; ++h)
                if (h < hvalid) dst[static_cast<long long>(h) * a.num_splits * kD] = __uint_as_float(o[h]);
        }
    }
    tc_fence_before_sync();
}

// ------------------------------------------------------------------ the kernel
template <int FMT, int NPAD>
__global__ void __launch_bounds__(kThreads, 1) sparse_mla_fwd_kernel(const __grid_constant__ KernelArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    using L = Smem<NPAD>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = blockIdx.x / a.head_blocks, hb = blockIdx.x - t * a.head_blocks, sp = blockIdx.y;
    const int h0 = hb * 64;
    const int hvalid = min(NPAD, a.H - h0);

    const int ns = min(max(__ldg(a.swa.lens + t), 0), a.swa.topk);
    const int ne = (a.extra.cache != nullptr) ? min(max(__ldg(a.extra.lens + t), 0), a.extra.topk) : 0;
    const int n = ns + ne;
    const int ntiles = (n + kTileRows - 1) / kTileRows;
    const int tps = (ntiles + a.num_splits - 1) / a.num_splits;
    const int tile0 = sp * tps;
    const int ntl = min(ntiles, tile0 + tps) - tile0;

    if (ntl <= 0) {   // nothing selected for this (token, split): zeros / an empty partial
        if (a.num_splits == 1) {
            for (int i = tid; i < hvalid * (kD / 8); i += kThreads) {
                const int h = i / (kD / 8), d8 = i - h * (kD / 8);
                *reinterpret_cast<uint4 *>(a.out + static_cast<long long>(t) * a.o_ts +
                                           static_cast<long long>(h0 + h) * a.o_hs + d8 * 8) = make_uint4(0, 0, 0, 0);
            }
        } else if (tid < hvalid) {
            float *ml = a.part_ml + ((static_cast<long long>(t) * a.H + h0 + tid) * a.num_splits + sp) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.0f;
        }
        return;
    }

    // ---- set-up: barriers, TMEM, reference max, Q tile
    if (tid == 0) {
        const uint32_t bars = smem_u32(smem + L::kBars);
        for (int c = 0; c < 4; ++c) mbar_init(bars + c * 8, kGatherWarps);   // K chunk filled
        for (int c = 0; c < 4; ++c) mbar_init(bars + (4 + c) * 8, 1);        // K chunk released by PV
        mbar_init(bars + 8 * 8, 1);                                           // S^T ready
        mbar_init(bars + 9 * 8, 1);                                           // last PV done
        *reinterpret_cast<volatile int *>(smem + L::kAbort) = 0;
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(smem + L::kTmemPtr), kTmemCols);
        tmem_relinquish();
    }
    if (tid < NPAD) {
        float m0 = -INFINITY;
        if (a.num_splits == 1 && a.sink != nullptr && tid < hvalid) m0 = ceilf(a.sink[h0 + tid] * kLog2e);
        reinterpret_cast<float *>(smem + L::kM)[tid] = m0;
    }
    {
        const __nv_bfloat16 *qt = a.q + static_cast<long long>(t) * a.q_ts + static_cast<long long>(h0) * a.q_hs;
        const uint32_t q_addr = smem_u32(smem + L::kQ);
        for (int idx = warp; idx < (NPAD / 8) * 16; idx += kNumWarps) {
            const int hg = idx >> 4, dg = (idx & 15) * 4 + (lane >> 3), h = hg * 8 + (lane & 7);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (h < hvalid) v = __ldg(reinterpret_cast<const uint4 *>(qt + static_cast<long long>(h) * a.q_hs + dg * 8));
            st_shared_v4(q_addr + hg * kRowGroupBytes + dg * kCoreBytes + (lane & 7) * 16, v.x, v.y, v.z, v.w);
        }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);

    if (warp < 4) {
        setmaxnreg_inc<kSoftmaxRegs>();
        softmax_role<FMT, NPAD>(a, smem, tmem_base, t, h0, hvalid, sp, n, tile0, ntl, tid);
    } else {
        setmaxnreg_dec<kGatherRegs>();
        gather_role<FMT, NPAD>(a, smem, t, ns, n, tile0, ntl, warp - 4, lane);
    }

    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ split-KV combine
// One warp per (token, head): out = sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)).
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const float *__restrict__ part_o,
                                                                 const float *__restrict__ part_ml,
                                                                 const float *__restrict__ sink,
                                                                 __nv_bfloat16 *__restrict__ out, long long o_ts,
                                                                 long long o_hs, int T, int H, int S) {
    const int lane = threadIdx.x & 31;
    const long long th = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (th >= static_cast<long long>(T) * H) return;
    const int t = static_cast<int>(th / H), h = static_cast<int>(th - static_cast<long long>(t) * H);
    const float *ml = part_ml + th * S * 2;
    const float sink_l2 = sink ? sink[h] * kLog2e : -INFINITY;
    float M = sink_l2;
    for (int s = 0; s < S; ++s)
        if (ml[2 * s + 1] > 0.0f) M = fmaxf(M, ml[2 * s]);
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    float denom = 0.0f;
    if (M > -INFINITY) {
        denom = fast_exp2(sink_l2 - M);
        for (int s = 0; s < S; ++s) {
            const float l = ml[2 * s + 1];
            if (!(l > 0.0f)) continue;
            const float w = fast_exp2(ml[2 * s] - M);
            denom += w * l;
            const float4 *src = reinterpret_cast<const float4 *>(part_o + (th * S + s) * kD);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const float4 x = __ldg(src + v * 32 + lane);
                acc[4 * v] += w * x.x;
                acc[4 * v + 1] += w * x.y;
                acc[4 * v + 2] += w * x.z;
                acc[4 * v + 3] += w * x.w;
            }
        }
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    __nv_bfloat16 *dst = out + static_cast<long long>(t) * o_ts + static_cast<long long>(h) * o_hs;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const uint2 pk = make_uint2(pack_bf16x2(acc[4 * v] * inv, acc[4 * v + 1] * inv),
                                    pack_bf16x2(acc[4 * v + 2] * inv, acc[4 * v + 3] * inv));
        *reinterpret_cast<uint2 *>(dst + (v * 32 + lane) * 4) = pk;
    }
}

// ------------------------------------------------------------------ host side
int fill_stream(const smla_stream_t &s, int fmt, StreamDev &d) {
    if (!s.cache || !s.indices || !s.lens || s.topk < 0 || s.num_blocks < 0 || s.block_size <= 0) return SMLA_EINVAL;
    d.cache = static_cast<const uint8_t *>(s.cache);
    d.scale = s.scale;
    d.indices = s.indices;
    d.lens = s.lens;
    d.idx_stride = s.indices_stride;
    d.block_stride = s.block_stride;
    d.pos_stride = s.pos_stride;
    d.scale_block_stride = s.scale_block_stride;
    d.scale_pos_stride = s.scale_pos_stride;
    d.topk = s.topk;
    const long long slots = static_cast<long long>(s.num_blocks) * s.block_size;
    if (slots > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    d.num_slots = static_cast<int>(slots);
    d.block_size = s.block_size;
    const uintptr_t base = reinterpret_cast<uintptr_t>(s.cache);
    if (fmt == SMLA_FP8_DS_MLA) {
        if ((base & 7u) || (s.block_stride & 7)) return SMLA_EALIGN;
        d.vec16 = ((base & 15u) == 0 && (s.block_stride & 15) == 0) ? 1 : 0;
    } else {
        if (!s.scale) return SMLA_EINVAL;
        if ((base & 3u) || (s.block_stride & 3) || (s.pos_stride & 3)) return SMLA_EALIGN;
        d.vec16 = ((base & 15u) == 0 && (s.block_stride & 15) == 0 && (s.pos_stride & 15) == 0) ? 1 : 0;
    }
    return SMLA_OK;
}

template <int FMT, int NPAD>
int launch_fwd(const KernelArgs &a, dim3 grid, cudaStream_t stream) {
    constexpr int smem_bytes = Smem<NPAD>::kTotal;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        e = cudaFuncSetAttribute(sparse_mla_fwd_kernel<FMT, NPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    sparse_mla_fwd_kernel<FMT, NPAD><<<grid, kThreads, smem_bytes, stream>>>(a);
    return static_cast<int>(cudaGetLastError());
}

template <int FMT>
int launch_fwd_npad(int npad, const KernelArgs &a, dim3 grid, cudaStream_t stream) {
    switch (npad) {
        case 16: return launch_fwd<FMT, 16>(a, grid, stream);
        case 32: return launch_fwd<FMT, 32>(a, grid, stream);
        default: return launch_fwd<FMT, 64>(a, grid, stream);
    }
}

}  // namespace

int launch_sparse_mla_attention(const smla_attn_params_t &p, int num_splits, void *workspace, cudaStream_t stream) {
    if (p.num_tokens < 0 || p.num_heads <= 0 || !p.q || !p.out) return SMLA_EINVAL;
    if (p.num_tokens == 0) return SMLA_OK;
    if (p.cache_format != SMLA_FP8_DS_MLA && p.cache_format != SMLA_INT8_DS_MLA) return SMLA_EINVAL;
    if ((reinterpret_cast<uintptr_t>(p.q) & 15u) || (p.q_token_stride & 7) || (p.q_head_stride & 7) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15u) || (p.out_token_stride & 7) || (p.out_head_stride & 7))
        return SMLA_EALIGN;

    KernelArgs a = {};
    a.q = static_cast<const __nv_bfloat16 *>(p.q);
    a.q_ts = p.q_token_stride;
    a.q_hs = p.q_head_stride;
    a.out = static_cast<__nv_bfloat16 *>(p.out);
    a.o_ts = p.out_token_stride;
    a.o_hs = p.out_head_stride;
    a.sink = p.attn_sink;
    a.T = p.num_tokens;
    a.H = p.num_heads;
    a.scale_log2 = p.softmax_scale * kLog2e;
    int rc = fill_stream(p.swa, p.cache_format, a.swa);
    if (rc != SMLA_OK) return rc;
    if (p.extra.cache != nullptr) {
        rc = fill_stream(p.extra, p.cache_format, a.extra);
        if (rc != SMLA_OK) return rc;
    }
    const int npad = p.num_heads <= 16 ? 16 : (p.num_heads <= 32 ? 32 : 64);
    a.head_blocks = (p.num_heads + 63) / 64;
    a.num_splits = num_splits < 1 ? 1 : num_splits;
    if (a.num_splits > 1) {
        if (!workspace) return SMLA_EWORKSPACE;
        a.part_o = static_cast<float *>(workspace);
        a.part_ml = a.part_o + static_cast<size_t>(p.num_tokens) * p.num_heads * a.num_splits * kD;
    }
    const long long gx = static_cast<long long>(p.num_tokens) * a.head_blocks;
    if (gx > 0x7FFFFFFFLL || a.num_splits > 65535) return SMLA_ETOOBIG;
    const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(a.num_splits));
    rc = (p.cache_format == SMLA_FP8_DS_MLA) ? launch_fwd_npad<SMLA_FP8_DS_MLA>(npad, a, grid, stream)
                                             : launch_fwd_npad<SMLA_INT8_DS_MLA>(npad, a, grid, stream);
    if (rc != 0) return rc;
    if (a.num_splits > 1) {
        const long long th = static_cast<long long>(p.num_tokens) * p.num_heads;
        sparse_mla_combine_kernel<<<static_cast<unsigned>((th + 3) / 4), 128, 0, stream>>>(
            a.part_o, a.part_ml, a.sink, a.out, a.o_ts, a.o_hs, a.T, a.H, a.num_splits);
        rc = static_cast<int>(cudaGetLastError());
    }
    return rc;
}

#ifdef SMLA_TRACE
extern "C" __attribute__((visibility("default"))) int smla_debug_read_trace(unsigned long long *host_out) {
    cudaDeviceSynchronize();
    return static_cast<int>(cudaMemcpyFromSymbol(host_out, g_trace, sizeof(unsigned long long) * 32 * 16));
}
#endif

int read_and_clear_device_status(int *status_out) {
    int v = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    if (status_out) *status_out = v;
    return static_cast<int>(e);
}

}  // namespace smla
