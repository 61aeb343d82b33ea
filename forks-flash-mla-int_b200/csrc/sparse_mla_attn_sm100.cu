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
// Roles (544 threads, no register rebalancing: setmaxnreg.inc can block without any time limit).
// Warps 0-15 are workers that alternate between two jobs: (1) convert -- warp w owns rows 8w..8w+7
// of the tile, keeps their raw bytes for the NEXT tile in registers (16-byte loads issued a tile
// ahead) and writes them as bf16 into the single K buffer chunk by chunk (128 dims), each chunk as
// soon as the previous tile's PV has released it; (2) softmax -- warp w owns TMEM lanes
// 32*(w%4).. and head columns (N/4)*(w/4)..: S^T -> P^T with a lazily moved, integer-valued
// reference max, running denominators, and the epilogue.  Warp 16 allocates TMEM and its lane 0
// issues every tcgen05.mma.
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
constexpr int kWorkerWarps = 16;                 // gather/dequant + softmax + epilogue
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kMmaWarp = kWorkerWarps;           // one more warp: TMEM allocation and every tcgen05.mma
constexpr int kThreads = kWorkerThreads + 128;   // 640: the MMA warp plus three idle warps (register
                                                 // files are handed out per group of four warps)
// No register rebalancing between the roles: setmaxnreg.inc blocks with no time limit until the
// registers it asks for have been released inside the same CTA, a hang this kernel has no way to
// bound.  Every thread gets the 96 registers __launch_bounds__(640, 1) allows.
constexpr int kNumWarps = kThreads / 32;
constexpr int kCoreBytes = 128;                  // one 8x16B core matrix
constexpr int kRowGroupBytes = 64 * kCoreBytes;  // 8 rows x 512 dims of bf16
constexpr int kKBytes = 16 * kRowGroupBytes;     // 128 rows
constexpr int kTmemCols = 512;
constexpr int kTmemOCol = 64;                    // O^T chunks start here; S^T at column 0
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;        // log2 units: the reference max may lag by up to 2^8
constexpr int kAllWorkersBar = 5;                // named barriers 1..4: the four column-slice groups
// mbarrier slots
constexpr int kBarReady = 0;   // [4] K chunk c holds this tile (16 arrivals: one per worker warp)
constexpr int kBarFree = 4;    // [4] PV of the previous tile has finished reading K chunk c
constexpr int kBarS = 8;       //     S^T of this tile is complete in TMEM
constexpr int kBarP = 9;       //     P^T of this tile is in shared memory (16 arrivals)
constexpr int kBarO = 10;      //     the last PV has completed
static_assert(kBarO + 1 <= 12, "mbarrier slots reserved in Smem");

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
    static constexpr int kBars = kAlpha + NPAD * 4;      // kNumBars mbarriers
    static constexpr int kTmemPtr = kBars + 12 * 8;
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
// After ColReduce<W, 16, .> the value of column c (0 <= c < W <= 16) sits in every lane with
// lane >> kShift == c; the lane whose low kShift bits are zero writes it.
template <int W>
__device__ __forceinline__ void store_col_partial(float *dst_cols, float v, int lane) {
    constexpr int kShift = (W == 16) ? 1 : (W == 8) ? 2 : 3;
    if ((lane & ((1 << kShift) - 1)) == 0) dst_cols[lane >> kShift] = v;
}

template <int N> struct TmemIO;
template <> struct TmemIO<4> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[4]) { tmem_ld_x4(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[4]) { tmem_st_x4(a, r); }
};
template <> struct TmemIO<8> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[8]) { tmem_ld_x8(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[8]) { tmem_st_x8(a, r); }
};
template <> struct TmemIO<16> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[16]) { tmem_ld_x16(a, r); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[16]) { tmem_st_x16(a, r); }
};

__device__ __forceinline__ void give_up(volatile int *abort_flag, int bit) {
    *abort_flag = 1;
    atomicOr(&g_device_status, bit);
}

// ------------------------------------------------------------------ row gather / dequant helpers
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

// Warp-level wait: lane 0 polls, the result is broadcast.  A wait that runs out (or finds the CTA
// already aborted) records `bit` and returns false; callers carry on with garbage instead of leaving,
// so that every named barrier below still sees all of its threads.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int lane, int bit) {
    int ok = 1;
    if (lane == 0) {
        ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
        if (!ok) give_up(abort_flag, bit);
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// ------------------------------------------------------------------ MMA issue (lane 0 of the MMA warp)
template <int NPAD>
__device__ __forceinline__ void mma_role(uint8_t *smem, uint32_t tmem_base, int ntl) {
    using L = Smem<NPAD>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, NPAD, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NPAD, 1, 1);
    // QK^T: K-major A (rows x dims) and B (heads x dims): M/N step = one row group (8192 B), K step =
    // one core matrix (128 B).  PV: MN-major A = K^T chunk (dims x rows): M step = next dim group
    // (128 B), K step = next row group (8192 B); MN-major B = P^T: N step = next head group (2048 B),
    // K step = next row group (128 B).  Only the 14-bit start-address field changes between MMAs, so
    // stepping a descriptor is one 32-bit add: the thread must sustain one MMA per ~50 cycles.
    const uint64_t qa = umma_desc(smem_u32(smem + L::kK), kCoreBytes, kRowGroupBytes);
    const uint64_t qb = umma_desc(smem_u32(smem + L::kQ), kCoreBytes, kRowGroupBytes);
    const uint64_t pa = umma_desc(smem_u32(smem + L::kK), kRowGroupBytes, kCoreBytes);
    const uint64_t pb = umma_desc(smem_u32(smem + L::kP), kCoreBytes, 2048);
    const uint32_t qa_lo = static_cast<uint32_t>(qa), qa_hi = static_cast<uint32_t>(qa >> 32);
    const uint32_t qb_lo = static_cast<uint32_t>(qb), qb_hi = static_cast<uint32_t>(qb >> 32);
    const uint32_t pa_lo = static_cast<uint32_t>(pa), pa_hi = static_cast<uint32_t>(pa >> 32);
    const uint32_t pb_lo = static_cast<uint32_t>(pb), pb_hi = static_cast<uint32_t>(pb >> 32);

    for (int it = 0; it < ntl; ++it) {
        SMLA_MARK(it, 0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (!mbar_wait(bars + (kBarReady + c) * 8, it & 1, abort_flag)) {
                give_up(abort_flag, kStatusMmaWait);
                return;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t off = static_cast<uint32_t>(((16 * c + 2 * k) * kCoreBytes) >> 4);
                umma_bf16_ss_lohi(tmem_base, qa_lo + off, qa_hi, qb_lo + off, qb_hi, idesc_qk, (c | k) != 0 ? 1u : 0u);
            }
        }
        umma_commit(bars + kBarS * 8);
        SMLA_MARK(it, 1);
        if (!mbar_wait(bars + kBarP * 8, it & 1, abort_flag)) {
            give_up(abort_flag, kStatusMmaWait);
            return;
        }
        tc_fence_after_sync();
        SMLA_MARK(it, 5);
        const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t aoff = static_cast<uint32_t>((c * 16 * kCoreBytes + 2 * k * kRowGroupBytes) >> 4);
                const uint32_t boff = static_cast<uint32_t>((2 * k * kCoreBytes) >> 4);
                umma_bf16_ss_lohi(tmem_base + kTmemOCol + c * NPAD, pa_lo + aoff, pa_hi, pb_lo + boff, pb_hi, idesc_pv,
                                  k > 0 ? 1u : acc0);
            }
            umma_commit(bars + (kBarFree + c) * 8);   // chunk c of the K buffer may be refilled
        }
        if (it + 1 == ntl) umma_commit(bars + kBarO * 8);
        SMLA_MARK(it, 6);
    }
}

// ------------------------------------------------------------------ worker warps (0..15)
// Each worker warp alternates between two jobs that never overlap in time for one tile:
//   convert: it owns rows 8w..8w+7 of the tile; raw bytes (already in registers) -> bf16 K chunks;
//   softmax: it owns TMEM lanes 32*(w%4).. (rows of S^T / dims of O^T) and head columns
//            (NPAD/4)*(w/4)..: scores -> P^T, running denominators, rare accumulator rescale.
template <int FMT, int NPAD>
__device__ __forceinline__ void worker_role(const KernelArgs &a, uint8_t *smem, uint32_t tmem_base, int t, int h0,
                                            int hvalid, int sp, int ns, int n, int tile0, int ntl, int warp,
                                            int lane) {
    using L = Smem<NPAD>;
    constexpr int J = Steps<FMT>::kCount;
    constexpr int CW = NPAD / 4;   // head columns per warp in the softmax job
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    float *red = reinterpret_cast<float *>(smem + L::kRed);
    float *m_s = reinterpret_cast<float *>(smem + L::kM);
    float *alpha_s = reinterpret_cast<float *>(smem + L::kAlpha);
    const int tid = warp * 32 + lane;
    const bool direct = a.num_splits == 1;
    const bool tracer = (warp == 0 && lane == 0);
    (void)tracer;

    // convert job
    const int quarter = lane >> 3;
    const uint32_t k_row_addr = smem_u32(smem + L::kK) + warp * kRowGroupBytes + (lane & 7) * 16;
    // softmax job
    const int q = warp & 3, cs = warp >> 2;
    const int row = q * 32 + lane;
    const int col0 = cs * CW;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t p_addr = smem_u32(smem + L::kP) + (col0 >> 3) * 2048 + (row >> 3) * kCoreBytes + (row & 7) * 16 +
                            (col0 & 7) * 2;
    const int group_bar = 1 + cs;

    float lsum[CW];
#pragma unroll
    for (int j = 0; j < CW; ++j) lsum[j] = 0.0f;

    int g = tile0 * kTileRows + warp * 8 + (lane & 7);
    RowRef<FMT> cur = make_row_ref<FMT>(a, ns, n, g, load_slot_id(a, t, ns, n, g));
    uint4 raw[J];
#pragma unroll
    for (int j = 0; j < J; ++j) load_step<FMT>(cur, j, quarter, raw[j]);
    int id_next = (ntl > 1) ? load_slot_id(a, t, ns, n, g + kTileRows) : -1;

    for (int it = 0; it < ntl; ++it) {
        const bool has_next = it + 1 < ntl;
        RowRef<FMT> nxt = make_row_ref<FMT>(a, ns, n, has_next ? g + kTileRows : n, id_next);
        if (it + 2 < ntl) id_next = load_slot_id(a, t, ns, n, g + 2 * kTileRows);

        // ---- convert: raw registers -> K chunks, each as soon as the previous tile's PV released it
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (it > 0) warp_wait(bars + (kBarFree + c) * 8, (it - 1) & 1, abort_flag, lane, kStatusGatherWait);
            if (tracer && c == 0) SMLA_MARK(it, 7);
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const bool mine = (j < 8) ? ((j >> 1) == c) : (c == 3);
                if (mine) convert_step<FMT>(raw[j], j, quarter, cur.sc0, cur.sc1, k_row_addr);
            }
            if (tracer) SMLA_MARK(it, 8 + c);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + (kBarReady + c) * 8);
        }
        if (tracer) SMLA_MARK(it, 12);
        // Raw bytes of the next tile.  Issued only now, after this tile's last conversion fence: a
        // proxy fence also waits for the thread's global loads in flight, so loads issued between
        // the chunks would put a memory latency on every hand-over.  They land while QK^T runs.
        if (has_next) {
#pragma unroll
            for (int j = 0; j < J; ++j) load_step<FMT>(nxt, j, quarter, raw[j]);
        }
        cur = nxt;
        g += kTileRows;

        // ---- softmax of this tile
        warp_wait(bars + kBarS * 8, it & 1, abort_flag, lane, kStatusSoftmaxWait);
        tc_fence_after_sync();
        if (tracer) SMLA_MARK(it, 2);
        // sm = S^T * scale - m, with m read once per tile as float4s (the same for all rows).
        const bool row_valid = (tile0 + it) * kTileRows + row < n;
        float sm[CW];
        uint32_t sraw[CW];
        TmemIO<CW>::ld(tmem_lane + col0, sraw);
#pragma unroll
        for (int j = 0; j < CW; ++j)
            sm[j] = row_valid ? fmaf(__uint_as_float(sraw[j]), a.scale_log2, -m_s[col0 + j]) : -INFINITY;
        // The reference max m is only moved when some score exceeds it by more than the threshold
        // (always on the first tile).  The vote spans the four warps that share these columns.
        bool need = false;
#pragma unroll
        for (int j = 0; j < CW; ++j) need |= sm[j] > kRescaleThreshold;
        if (named_bar_or(group_bar, 128, need)) {
            float s[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j) s[j] = row_valid ? __uint_as_float(sraw[j]) * a.scale_log2 : -INFINITY;
            float r[1];
            ColReduce<CW, 16, true>::run(s, lane, r);
            store_col_partial<CW>(red + q * NPAD + col0, r[0], lane);
            named_bar_sync(group_bar, 128);
            if (q == 0 && lane < CW) {
                const int col = col0 + lane;
                const float tm = fmaxf(fmaxf(red[col], red[NPAD + col]), fmaxf(red[2 * NPAD + col], red[3 * NPAD + col]));
                const float m_old = m_s[col];
                const bool up = tm > m_old + kRescaleThreshold;
                // m stays INTEGER-valued (log2 units): 2^(s - m) then has the same mantissa whatever m
                // is, so P rounds to bf16 identically in every split-KV schedule.
                const float m_new = up ? ceilf(tm) : m_old;
                alpha_s[col] = up ? fast_exp2(m_old - m_new) : 1.0f;
                m_s[col] = m_new;
            }
            named_bar_sync(group_bar, 128);
#pragma unroll
            for (int j = 0; j < CW; ++j) {
                lsum[j] *= alpha_s[col0 + j];
                sm[j] = s[j] - m_s[col0 + j];
            }
            if (it > 0) {   // O^T[:, h] *= alpha[h]; the previous PV completed before this tile's S^T did
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t o[CW];
                    TmemIO<CW>::ld(tmem_lane + kTmemOCol + c * NPAD + col0, o);
#pragma unroll
                    for (int j = 0; j < CW; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha_s[col0 + j]);
                    TmemIO<CW>::st(tmem_lane + kTmemOCol + c * NPAD + col0, o);
                }
                tmem_st_wait();
            }
        }
        if (tracer) SMLA_MARK(it, 3);
        {   // P^T = 2^(S^T - m) rounded to bf16, MN-major B-operand layout (8 heads = 16 bytes per row)
            uint32_t pk[CW / 2];
#pragma unroll
            for (int j = 0; j < CW; j += 2) {
                const float p0 = fast_exp2(sm[j]);
                const float p1 = fast_exp2(sm[j + 1]);
                lsum[j] += p0;
                lsum[j + 1] += p1;
                pk[j / 2] = pack_bf16x2(p0, p1);
            }
            if constexpr (CW == 16) {
                st_shared_v4(p_addr, pk[0], pk[1], pk[2], pk[3]);
                st_shared_v4(p_addr + 2048, pk[4], pk[5], pk[6], pk[7]);
            } else if constexpr (CW == 8) {
                st_shared_v4(p_addr, pk[0], pk[1], pk[2], pk[3]);
            } else {
                asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(p_addr), "r"(pk[0]), "r"(pk[1]) : "memory");
            }
        }
        if (tracer) SMLA_MARK(it, 4);
        fence_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + kBarP * 8);
    }

    // ---- epilogue: O^T / l
    warp_wait(bars + kBarO * 8, 0, abort_flag, lane, kStatusEpilogueWait);
    tc_fence_after_sync();
    {
        float r[1];
        ColReduce<CW, 16, false>::run(lsum, lane, r);
        store_col_partial<CW>(red + q * NPAD + col0, r[0], lane);
    }
    named_bar_sync(kAllWorkersBar, kWorkerThreads);
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
    named_bar_sync(kAllWorkersBar, kWorkerThreads);
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
        uint32_t o[CW];
        TmemIO<CW>::ld(tmem_lane + kTmemOCol + c * NPAD + col0, o);
        const int d = c * 128 + row;
        if (direct) {
            __nv_bfloat16 *dst = a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0 + col0) * a.o_hs + d;
#pragma unroll
            for (int j = 0; j < CW; ++j)
                if (col0 + j < hvalid) dst[j * a.o_hs] = __float2bfloat16_rn(__uint_as_float(o[j]) * alpha_s[col0 + j]);
        } else {
            float *dst = a.part_o + ((static_cast<long long>(t) * a.H + h0 + col0) * a.num_splits + sp) * kD + d;
#pragma unroll
            for (int j = 0; j < CW; ++j)
                if (col0 + j < hvalid) dst[static_cast<long long>(j) * a.num_splits * kD] = __uint_as_float(o[j]);
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
        for (int c = 0; c < 4; ++c) mbar_init(bars + (kBarReady + c) * 8, kWorkerWarps);
        for (int c = 0; c < 4; ++c) mbar_init(bars + (kBarFree + c) * 8, 1);
        mbar_init(bars + kBarS * 8, 1);
        mbar_init(bars + kBarP * 8, kWorkerWarps);
        mbar_init(bars + kBarO * 8, 1);
        *reinterpret_cast<volatile int *>(smem + L::kAbort) = 0;
        mbar_init_fence();
    }
    if (warp == kMmaWarp) {
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

    if (warp < kWorkerWarps) {
        worker_role<FMT, NPAD>(a, smem, tmem_base, t, h0, hvalid, sp, ns, n, tile0, ntl, warp, lane);
    } else {
        if (warp == kMmaWarp && lane == 0) mma_role<NPAD>(smem, tmem_base, ntl);
        __syncwarp();
    }

    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ split-KV combine
// One warp per (token, head): out = sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)).
// Lane s first turns {m_s, l_s} into a weight (S <= 64: two per lane); the partial rows are then
// streamed four splits at a time so that 16 independent 16-byte loads are in flight per lane.
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const float *__restrict__ part_o,
                                                                 const float *__restrict__ part_ml,
                                                                 const float *__restrict__ sink,
                                                                 __nv_bfloat16 *__restrict__ out, long long o_ts,
                                                                 long long o_hs, int T, int H, int S) {
    const int lane = threadIdx.x & 31;
    const long long th = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
    if (th >= static_cast<long long>(T) * H) return;
    const int t = static_cast<int>(th / H), h = static_cast<int>(th - static_cast<long long>(t) * H);
    const float2 *ml = reinterpret_cast<const float2 *>(part_ml + th * S * 2);
    const float sink_l2 = sink ? sink[h] * kLog2e : -INFINITY;
    float2 e0 = make_float2(-INFINITY, 0.0f), e1 = make_float2(-INFINITY, 0.0f);
    if (lane < S) e0 = ml[lane];
    if (lane + 32 < S) e1 = ml[lane + 32];
    float M = sink_l2;
    if (e0.y > 0.0f) M = fmaxf(M, e0.x);
    if (e1.y > 0.0f) M = fmaxf(M, e1.x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    // empty splits (l == 0) get weight 0 and their (unwritten) partial rows are never multiplied in
    const float w0 = (e0.y > 0.0f && M > -INFINITY) ? fast_exp2(e0.x - M) : 0.0f;
    const float w1 = (e1.y > 0.0f && M > -INFINITY) ? fast_exp2(e1.x - M) : 0.0f;
    float denom = w0 * e0.y + w1 * e1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (M > -INFINITY) denom += fast_exp2(sink_l2 - M);

    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    const float4 *base = reinterpret_cast<const float4 *>(part_o + th * S * kD);
    for (int s0 = 0; s0 < S; s0 += 4) {
        float4 x[4][4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int s = s0 + u;
            const float ws = __shfl_sync(0xffffffffu, (s < 32) ? w0 : w1, s & 31);
            w[u] = (s < S) ? ws : 0.0f;
            const float4 *src = base + static_cast<long long>(min(s, S - 1)) * (kD / 4);
#pragma unroll
            for (int v = 0; v < 4; ++v) x[u][v] = __ldg(src + v * 32 + lane);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (w[u] != 0.0f) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    acc[4 * v] += w[u] * x[u][v].x;
                    acc[4 * v + 1] += w[u] * x[u][v].y;
                    acc[4 * v + 2] += w[u] * x[u][v].z;
                    acc[4 * v + 3] += w[u] * x[u][v].w;
                }
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
    if (gx > 0x7FFFFFFFLL || a.num_splits > 64) return SMLA_ETOOBIG;   // the combine kernel keeps two weights per lane
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
