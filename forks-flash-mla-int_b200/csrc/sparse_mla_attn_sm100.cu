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
// Orientation.  The work is a list of items (token, block of <= 64 heads).  The selected rows are
// the MMA M dimension, 128 per tile:
//     S^T[128 rows, N heads]   = K_tile[128, 512] . Q[N, 512]^T         (A, B both K-major)
//     O^T[512 dims, N heads]  += K_tile^T[512, 128] . P^T[128, N]       (A, B both MN-major)
// so a 64-head block still fills the 128-lane datapath, and the SAME shared-memory K tile
// serves both products: it is stored as 8x16-byte core matrices (8 rows x 8 dims) which a
// no-swizzle descriptor can walk row-group-first (K-major) or dim-group-first (MN-major).
//
// Schedule.  The grid is persistent (at most one CTA per SM).  Either whole items are dealt out to
// the CTAs, or -- when there are few items or their lengths differ -- the 128-row tiles of all items
// are cut into equal contiguous ranges, one per CTA; the pieces of an item that was cut are merged
// inside this kernel (by the CTA that holds the item's first tiles, or slice-wise by all CTAs of the
// item) or by a small second kernel; see "work distribution" below.
//
// Roles (640 threads, no register rebalancing).  Warps 0-15 are workers that alternate between two
// jobs: (1) convert -- warp w owns rows 8w..8w+7 of the tile, keeps their raw bytes for the NEXT
// tile in registers (256-bit loads issued a tile ahead) and writes them as bf16 into the single K
// buffer chunk by chunk (128 dims), each chunk as soon as the previous tile's PV has released it;
// (2) softmax -- warp w owns TMEM lanes 32*(w%4).. and head columns (N/4)*(w/4)..: S^T -> P^T with a
// lazily moved reference max, running denominators, and the epilogue.  Warp 16
// allocates TMEM and issues every tcgen05.mma (warp-uniform code, one elected lane); warp 17 fetches
// each item's Q tile (one TMA tensor copy); warp 18 publishes the CTA's segments into a ring in shared
// memory.
//
// Dense paged MLA decode (the path behind flash_mla_with_kvcache: csrc/flash_api.cpp:159-322 of the
// reference) is two more values of the format parameter: bf16 rows of 576 dims found through a block
// table, scores over all 576 dims (the 64 RoPE dims of a tile in a fifth K piece that shares its memory
// with P^T), values = the first 512, log-sum-exp output.  The rows are copied, not converted: by TMA from
// warp 19 into 128-byte-swizzled slabs (kFmtBf16DenseTma), or with cp.async by the workers (kFmtBf16Dense).
//
// Every spin is time-bounded; a wait that runs out sets a bit in the device status word and the
// CTA leaves through the normal teardown.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda.h>            // CUtensorMap and its enums only; the encoder is looked up at run time, libcuda is not linked
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "sm100_ptx.cuh"
#include <algorithm>
#include <atomic>
#include <random>
#include <type_traits>

#include "smla_internal.h"

namespace smla {

__device__ int g_device_status = 0;

namespace {

constexpr int kD = 512;
// Third value of the kernels' FMT parameter: int8_ds_mla rows that are 16-byte aligned inside 32-byte
// aligned blocks (the usual 528-byte tokens), gathered with 256-bit loads (see load_row_pieces).
constexpr int kFmtInt8Wide = 2;
// Fourth value: dense paged MLA (bf16 rows of 576 dims found through a block table; scores over all 576
// dims, values = the first 512).  The 64 RoPE dims of a tile sit in a fifth K chunk that shares its
// shared memory with P^T: they are only read by QK^T, P^T is only written after QK^T has completed.
constexpr int kFmtBf16Dense = 3;
// Fifth value: the same, with the K tile fetched by TMA (a warp of its own issues 2-D boxes of R rows x 64
// dims, R = min(page, 128)) into eight slabs of [128 rows][128 bytes] with the 128-byte swizzle, which the
// tensor pipe reads K-major for QK^T and MN-major for PV.  (cp.async moves 16 bytes per thread and about one
// such request per cycle and SM: measured 8-9k cycles for the 147 KB of a tile.)
constexpr int kFmtBf16DenseTma = 4;
__host__ __device__ constexpr bool is_dense(int fmt) { return fmt == kFmtBf16Dense || fmt == kFmtBf16DenseTma; }
constexpr int kSlabBytes = 128 * 128;            // 128 rows x 64 dims of bf16 (swizzled K tile)
constexpr int kDenseRowBytes = 1152;             // 576 bf16
constexpr int kTileRows = 128;
constexpr int kWorkerWarps = 16;                 // gather/dequant + softmax + epilogue
constexpr int kWorkerThreads = kWorkerWarps * 32;
constexpr int kMmaWarp = kWorkerWarps;           // one more warp: TMEM allocation and every tcgen05.mma
constexpr int kThreads = kWorkerThreads + 128;   // 640: the MMA warp plus three idle warps (register
                                                 // files are handed out per group of four warps)
// No register rebalancing between the roles (setmaxnreg): measured, ptxas spills whatever is live
// above the lower budget at the release point and the worker code gains nothing.  Every thread has
// the 96 registers __launch_bounds__(640, 1) allows.
constexpr int kNumWarps = kThreads / 32;
constexpr int kCoreBytes = 128;                  // one 8x16B core matrix
constexpr int kRowGroupBytes = 64 * kCoreBytes;  // 8 rows x 512 dims of bf16
constexpr int kKBytes = 16 * kRowGroupBytes;     // 128 rows
constexpr int kTmemCols = 512;
constexpr int kTmemOCol = 64;                    // O^T chunks start here; S^T at column 0
constexpr float kLog2e = 1.4426950408889634f;
// The softmax reference m (log2 units) is the running maximum AS IT WAS WHEN m WAS LAST MOVED: it is left
// alone until a score exceeds it by kRescaleThreshold, and then set to the new maximum itself, not to a
// rounded value.  Two things follow.  (1) The row that holds the maximum gets P = 2^0 = 1, which bf16
// holds exactly: where one row dominates -- the x50 outlier rows of the int8 workloads, |K| up to 200 --
// the output carries no rounding error of that row's weight.  With an integer-valued reference (tried
// first, because P then rounds identically however the rows are cut into segments) every weight was
// rounded, and small elements of such rows were up to four times further from the fp32 oracle than the
// reference's own kernels; a CPU emulation of both rules reproduces the factor.  (2) Ordinary data never
// moves m after a segment's first tile (scores within a few units of each other); outlier rows move it
// in most tiles either way (13 of 20 tiles with a 100-unit window, 18 of 20 with this one), and each
// move rescales the accumulators, which stalls the tile pipeline.  The bound on the threshold: a rescale
// factor 2^(m_old - m_new), or a merge weight 2^(m_i - M), multiplies terms that still matter (within
// 2^-24 of the largest) only when its exponent is above -(kRescaleThreshold + kRefHeadroom + 24), which
// has to stay a normal fp32 number (2^-126).
constexpr float kRescaleThreshold = 8.0f;
constexpr float kRefHeadroom = 0.0f;
// What the exact weight of the top row is worth grows with |K| of that row, and large rows show as large
// scores: above kBigScore (log2 units; ordinary N(0,1) data stays below 10) the reference follows the
// running maximum exactly, below it the threshold applies.  Per head: m moves when s - m > move_threshold(m).
constexpr float kBigScore = 32.0f;
__device__ __forceinline__ float move_threshold(float m) { return fminf(fmaxf(kBigScore - m, 0.0f), kRescaleThreshold); }
static_assert(kRescaleThreshold + kRefHeadroom + 24.0f <= 126.0f, "rescale factors must stay normal fp32 numbers");
constexpr int kAllWorkersBar = 5;                // named barriers 1..4: the four column-slice groups
// mbarrier slots
constexpr int kBarReady = 0;   // [4] K chunk c holds this tile (16 arrivals: one per worker warp)
constexpr int kBarFree = 4;    // [4] PV of the previous tile has finished reading K chunk c
constexpr int kBarS = 8;       //     S^T of this tile is complete in TMEM
constexpr int kBarP = 9;       //     P^T of this tile is in shared memory (16 arrivals)
constexpr int kBarO = 10;      //     the last PV of a segment has completed
constexpr int kBarOFree = 11;  //     the segment's epilogue has read O^T (16 arrivals)
constexpr int kBarQ = 12;      //     the segment's Q tile is in shared memory (TMA: 1 arrival + bytes; else 2 warps)
constexpr int kBarLand = 13;   // [4] dense, K by TMA: the boxes of K chunk c have landed (1 arrival + bytes)
constexpr int kBarLandAlt = 17;//     the same for chunk 0 of odd tiles where chunk 0 has two buffers (Smem::kAltBytes)
static_assert(kBarLandAlt + 1 <= 18, "mbarrier slots reserved in Smem");
constexpr int kQLoadWarps = 2;                   // warps 17 and 19 (cp.async fallback; with TMA warp 17 alone)

struct StreamDev {
    const uint8_t *cache;
    const float *scale;
    const int *indices;
    const int *lens;
    long long idx_stride, block_stride, pos_stride, scale_block_stride, scale_pos_stride;
    int topk, num_slots, block_size;
    int block_shift;   // log2(block_size) when it is a power of two, else -1
    int vec;   // widest aligned load of a row piece: 2 = 32 bytes, 1 = 16 bytes, 0 = 8 (fp8) / 4 (int8) bytes
};

struct KernelArgs {
    const __nv_bfloat16 *q;
    long long q_ts, q_hs;
    __nv_bfloat16 *out;
    long long o_ts, o_hs;
    const float *sink;
    float *part_o;   // fp32 [slot, NPAD, 512] un-normalised partial outputs (balanced schedule)
    float *part_ml;  // fp32 [slot, NPAD, 2]   {reference max (log2 units), denominator}
    int *desc;       // int4 [CTA] merge descriptors {item, segments, first slot, heads} or {-1} (combine kernel)
    unsigned long long *flags;    // [slot] launch tag once the slot's partial is complete (fused merge)
    unsigned long long tag;       // unique per launch
    int fused_merge;              // 0: combine kernel; 1: the CTA that holds an item's first tiles merges the
                                  // other partials in its own epilogue; 2: every CTA of an item merges a
                                  // slice of its heads at the end of its run
    StreamDev swa, extra;
    int T, H, head_blocks, balanced;
    float scale_log2;
    int q_tma;            // the Q tile is fetched with one TMA tensor copy through q_map (else cp.async)
    CUtensorMap q_map;    // 5-D view of q: {8 dims, 8 heads, 64 (dense: 72) dim groups, H/8 head groups, T}; dense with K by TMA: 3-D {dims, heads, T}
    // dense paged MLA only (dense_sq > 0): token t is query position t % dense_sq of sequence t / dense_sq;
    // swa.indices is the block table, swa.lens the sequences' lengths; with `causal` query position i sees
    // the first len - (dense_sq - 1 - i) rows.  lse[(b * H + h) * dense_sq + i], natural log, may be null.
    float *lse;
    int dense_sq, causal;
    int dense_dims;       // 576, or 512 (no RoPE dims: the fifth K chunk and the last eight Q groups are zero-filled)
    CUtensorMap k_map;    // kFmtBf16DenseTma: 3-D view {576 dims, page rows, pages} of the cache, box {64, k_box_rows, 1}
    int k_box_rows;
    // Dense paged MLA with several query positions and few heads (fold_sq * fold_h <= 64): the positions of a
    // sequence are folded into the head dimension, column i * fold_h + h = (query position i, head h), so that
    // one item reads the sequence's rows once for all positions.  T, H, q_ts, o_ts describe the folded problem
    // (dense_sq == 1); with fold_causal the columns of position i see fold_sq - 1 - i rows less.
    int fold_sq, fold_h, fold_causal;
    int hb_major;         // items are ordered head block first (item = hb * T + t) instead of token first: see schedule_and_launch
};

template <int NPAD, bool DENSE = false>
struct Smem {
    static constexpr int kQDimGroups = DENSE ? 72 : 64;  // 16-byte pieces of a Q row
    static constexpr int kQRowGroup = kQDimGroups * kCoreBytes;   // 8 heads of Q
    static constexpr int kQBytes = (NPAD / 8) * kQRowGroup;
    static constexpr int kQ = 0;                         // Q tile, core(hg, dg) at hg*kQRowGroup + dg*128
    static constexpr int kK = kQ + kQBytes;              // K tile, core(rg, dg) at rg*8192 + dg*128
    static constexpr int kP = kK + kKBytes;              // P^T,   core(hg, rg) at hg*2048 + rg*128; dense: also
                                                         // the tile's RoPE dims, core(rg, dg) at rg*1024 + dg*128
    static constexpr int kPBytes = DENSE ? 16384 : NPAD * 256;
    static constexpr int kRed = kP + kPBytes;            // [4][NPAD] floats
    static constexpr int kM = kRed + 4 * NPAD * 4;       // running reference max per head
    static constexpr int kAlpha = kM + NPAD * 4;         // rescale factor / final 1/l per head
    static constexpr int kShift = kAlpha + NPAD * 4;     // m_old - m_new of the last reference move
    static constexpr int kThr = kShift + NPAD * 4;       // how far a score may exceed m before m moves (move_threshold)
    static constexpr int kBars = kThr + NPAD * 4;        // kNumBars mbarriers
    static constexpr int kTmemPtr = kBars + 18 * 8;
    static constexpr int kAbort = kTmemPtr + 4;
    static constexpr int kSched = kAbort + 4 + 8;        // 160 ints: work distribution (scan scratch, iterator, segment ring)
    // Epilogue staging, 8 KB per column-slice group.  With 64 heads only 16 KB are left, so groups 0
    // and 1 stage in the P buffer (idle between a segment's last PV and the next softmax).
    static constexpr int kStage = kSched + 640;
    static constexpr int kStageBytes = DENSE ? 0 : (NPAD == 64) ? 16384 : 32768;   // dense: output stored from registers
    static constexpr int kTotal = kStage + kStageBytes;
    // Dense, K by TMA, at most 32 heads: a second buffer for K chunk 0, used by the odd tiles, so that the
    // next tile's first 128 dims are fetched while this tile is scored (not part of kTotal: only that format asks for it).
    static constexpr int kAlt = (kTotal + 1023) & ~1023;
    static constexpr int kAltBytes = (DENSE && NPAD <= 32) ? 2 * kSlabBytes : 0;
    static constexpr int kTotalTma = kAltBytes > 0 ? kAlt + kAltBytes : kTotal;
    static_assert(kTotal <= 232448 && kTotalTma <= 232448, "more than 227 KB of shared memory");
};

// ------------------------------------------------------------------ small device helpers
constexpr float kLn2 = 0.6931471805599453f;
// Where the log-sum-exp of (token t, head h) goes (dense paged MLA: [sequence, head, query position]).
__device__ __forceinline__ float *lse_ptr(const KernelArgs &a, int t, int h) {
    if (a.fold_sq > 1) {      // folded query positions: column h = position * fold_h + head, token t = sequence
        const int i = h / a.fold_h;
        return a.lse + (static_cast<long long>(t) * a.fold_h + (h - i * a.fold_h)) * a.fold_sq + i;
    }
    const int b = t / a.dense_sq, i = t - b * a.dense_sq;
    return a.lse + (static_cast<long long>(b) * a.H + h) * a.dense_sq + i;
}
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
// 32 bytes in one request (sm_100: 256-bit global loads); p must be 32-byte aligned.
__device__ __forceinline__ void ldg_nc_v8(const void *p, uint4 &lo, uint4 &hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(p));
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
// Two-wide fp32 arithmetic on 64-bit register pairs (sm_100): half the issue slots of the scalar form.
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16x2(uint64_t v) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
    return pack_bf16x2(lo, hi);
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
__device__ __forceinline__ void cvt_i8x4(uint32_t w, float s, uint32_t &lo, uint32_t &hi) {
    const uint32_t x = w ^ 0x80808080u;
    const uint64_t ss = f32x2(s, s), bias = f32x2(-8388736.0f, -8388736.0f);
    const uint64_t a = f32x2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)),
                             __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541)));
    const uint64_t b = f32x2(__uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)),
                             __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543)));
    lo = pack_bf16x2(mul_f32x2(add_f32x2(a, bias), ss));
    hi = pack_bf16x2(mul_f32x2(add_f32x2(b, bias), ss));
}
// 4 e4m3 -> 4 x bf16(e4m3 * 2^(ue8m0 - 127)); exact (power-of-two scaling of a 4-bit significand).
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, float mult, uint32_t &lo, uint32_t &hi) {
    const __half2_raw a = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xFFFFu), __NV_E4M3);
    const __half2_raw b = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
    const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&a));
    const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&b));
    const uint64_t mm = f32x2(mult, mult);
    lo = pack_bf16x2(mul_f32x2(f32x2(fa.x, fa.y), mm));
    hi = pack_bf16x2(mul_f32x2(f32x2(fb.x, fb.y), mm));
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
    static __device__ __forceinline__ void ld2(uint32_t a, uint32_t b, uint32_t (&r)[4], uint32_t (&t)[4]) { tmem_ld_x4_pair(a, b, r, t); }
    static __device__ __forceinline__ void st(uint32_t a, const uint32_t (&r)[4]) { tmem_st_x4(a, r); }
};
template <> struct TmemIO<8> {
    static __device__ __forceinline__ void ld(uint32_t a, uint32_t (&r)[8]) { tmem_ld_x8(a, r); }
    static __device__ __forceinline__ void ld2(uint32_t a, uint32_t b, uint32_t (&r)[8], uint32_t (&t)[8]) { tmem_ld_x8_pair(a, b, r, t); }
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
    bool ok;
    bool odd;  // kFmtInt8Wide: the row starts 16 bytes past a 32-byte boundary
    int vec;   // see StreamDev::vec
};

// Dense paged MLA: row g of a sequence is position g % block_size of the page its block table names.
__device__ __forceinline__ int load_dense_slot_id(const KernelArgs &a, int t, int n, int g) {
    if (g >= n) return -1;
    const int b = a.dense_sq == 1 ? t : t / a.dense_sq;
    const int page_i = a.swa.block_shift >= 0 ? (g >> a.swa.block_shift) : g / a.swa.block_size;
    const int page = __ldg(a.swa.indices + static_cast<long long>(b) * a.swa.idx_stride + page_i);
    return page < 0 ? -1 : page * a.swa.block_size + (g - page_i * a.swa.block_size);
}

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
    r.odd = false;
    r.vec = 2;
    if (g >= n) return r;
    const StreamDev &s = (g < ns) ? a.swa : a.extra;
    if (static_cast<unsigned>(id) >= static_cast<unsigned>(s.num_slots)) return r;
    // id is a valid slot here (0 <= id < num_slots); paged caches use power-of-two blocks as a rule
    const int b = s.block_shift >= 0 ? (id >> s.block_shift) : id / s.block_size;
    const int i = id - b * s.block_size;
    const uint8_t *blk = s.cache + static_cast<long long>(b) * s.block_stride;
    r.ok = true;
    r.vec = s.vec;
    if constexpr (is_dense(FMT)) {
        r.ptr = blk + static_cast<long long>(i) * s.pos_stride;
    } else if constexpr (FMT == SMLA_FP8_DS_MLA) {
        r.ptr = blk + static_cast<long long>(i) * 576;
        const uint2 sc = ldg_nc_v2(blk + static_cast<long long>(s.block_size) * 576 + static_cast<long long>(i) * 8);
        r.sc0 = sc.x;
        r.sc1 = sc.y;
    } else {
        r.ptr = blk + static_cast<long long>(i) * s.pos_stride;
        if constexpr (FMT == kFmtInt8Wide) r.odd = ((reinterpret_cast<uintptr_t>(r.ptr) >> 4) & 1u) != 0;
        r.sc0 = __float_as_uint(__ldg(s.scale + static_cast<long long>(b) * s.scale_block_stride +
                                      static_cast<long long>(i) * s.scale_pos_stride));
    }
    return r;
}

// Register-chunk schedule: a row is cut into 16-byte pieces (fp8: 28 pieces of e4m3 + 8 of bf16 RoPE;
// int8: 32 pieces).  Lane (row = lane & 7, quarter = lane >> 3) holds in raw[j] the piece
//   piece16(j, quarter) = 8 * (j / 2) + 2 * quarter + (j & 1)   for j < 8,   32 + quarter for j = 8
// for fp8 (the "wide" order): raw[2c], raw[2c+1] are 32 contiguous bytes of K-buffer chunk c (dims
// 128c..128c+127) and are fetched by ONE 256-bit load when the rows are 32-byte aligned: 5 load
// instructions per lane and tile instead of 9 (int8 rows: see kFmtInt8Wide).  The count matters more than the bytes: while the tensor pipe
// streams operands, every load instruction takes ~20 cycles of issue (measured: twice as many loads
// for the same bytes cost 18 % of the kernel).
template <int FMT> struct Steps { static constexpr int kCount = is_dense(FMT) ? 1 : (FMT == SMLA_INT8_DS_MLA) ? 8 : 9; };

// The order is fixed per cache format at compile time (a run-time choice cost the int8 kernel 10 %):
// fp8 rows use the wide order (their 576-byte pitch keeps them 32-byte aligned whenever the cache is;
// otherwise the 32 bytes are fetched by narrower loads).  int8 rows, whose usual 528-byte pitch is only
// 16-byte aligned, keep piece 4j + quarter: the four lanes of a row then read 64 contiguous bytes per
// instruction (whole sectors), and chunk c is still raw[2c], raw[2c+1].
template <int FMT>
__device__ __forceinline__ int piece16(int j, int quarter) {
    if (j >= 8) return 32 + quarter;
    return (FMT == SMLA_FP8_DS_MLA) ? 8 * (j >> 1) + 2 * quarter + (j & 1) : 4 * j + quarter;
}

template <int FMT>
__device__ __forceinline__ void load_row_pieces(const RowRef<FMT> &r, int quarter, uint4 (&raw)[Steps<FMT>::kCount],
                                                int row_bytes = kDenseRowBytes) {
    constexpr int J = Steps<FMT>::kCount;
    // Invalid rows are zero rows; the choice is made per load (a select, no divergent branch).
    if constexpr (is_dense(FMT)) {
        // bf16 rows go to the K buffer with cp.async when the buffer is free (no registers could hold
        // 288 bytes per thread a tile ahead); a tile ahead they are only pulled into L2.
        raw[0] = make_uint4(0u, 0u, 0u, 0u);
        if (r.ok && quarter == 0)      // one bulk prefetch per row (1152 bytes)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(r.ptr), "r"(row_bytes) : "memory");
    } else if constexpr (FMT == kFmtInt8Wide) {
        // 512 data bytes from a 16-byte aligned address: an even row is 16 aligned 32-byte windows; an
        // odd row is fetched from 16 bytes earlier (the tail of the token before it, readable), so
        // that its windows are aligned too: raw[2c] is then piece 8c + 2q - 1 and raw[2c + 1] piece
        // 8c + 2q, and the last piece, 31, comes with one 16-byte load in lane quarter 0.
        const uint8_t *base = r.ptr - (r.odd ? 16 : 0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (r.ok) ldg_nc_v8(base + 128 * c + 32 * quarter, raw[2 * c], raw[2 * c + 1]);
            else raw[2 * c] = raw[2 * c + 1] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (r.ok && r.odd && quarter == 0) raw[8] = ldg_nc_v4(r.ptr + 496);
        else raw[8] = make_uint4(0u, 0u, 0u, 0u);
    } else if (FMT == SMLA_FP8_DS_MLA && r.vec == 2) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (r.ok) ldg_nc_v8(r.ptr + 128 * c + 32 * quarter, raw[2 * c], raw[2 * c + 1]);
            else raw[2 * c] = raw[2 * c + 1] = make_uint4(0u, 0u, 0u, 0u);
        }
        if (r.ok) raw[J - 1] = ldg_nc_v4(r.ptr + 512 + 16 * quarter);
        else raw[J - 1] = make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            if (r.ok) raw[j] = load16<FMT>(r.ptr + piece16<FMT>(j, quarter) * 16, r.vec >= 1);
            else raw[j] = make_uint4(0u, 0u, 0u, 0u);
        }
    }
}

// 16 int8 values (piece p16 of the row) -> bf16(value * scale), two core-matrix rows of the K buffer.
__device__ __forceinline__ void convert_int8_piece(const uint4 &raw, uint32_t p16, float s, uint32_t k_row_addr) {
    uint32_t o[8];
    cvt_i8x4(raw.x, s, o[0], o[1]);
    cvt_i8x4(raw.y, s, o[2], o[3]);
    cvt_i8x4(raw.z, s, o[4], o[5]);
    cvt_i8x4(raw.w, s, o[6], o[7]);
    const uint32_t dg = 2u * p16;
    st_shared_v4(k_row_addr + dg * kCoreBytes, o[0], o[1], o[2], o[3]);
    st_shared_v4(k_row_addr + (dg + 1u) * kCoreBytes, o[4], o[5], o[6], o[7]);
}

template <int FMT>
__device__ __forceinline__ void convert_step(const uint4 &raw, int j, int quarter, uint32_t sc0, uint32_t sc1,
                                             uint32_t k_row_addr /* K + rg*8192 + (lane&7)*16 */) {
    uint32_t o[8];
    const uint32_t p16 = static_cast<uint32_t>(piece16<FMT>(j, quarter));
    if constexpr (FMT == SMLA_INT8_DS_MLA) {
        convert_int8_piece(raw, p16, __uint_as_float(sc0), k_row_addr);
    } else {
        if (p16 < 28u) {     // 16 e4m3 values of scale tile p16 / 4
            const uint32_t tile = p16 >> 2;
            const uint32_t byte = ((tile < 4u ? sc0 : sc1) >> (8u * (tile & 3u))) & 0xFFu;
            const float mult = __uint_as_float(byte << 23);   // 2^(ue8m0 - 127)
            cvt_e4m3x4(raw.x, mult, o[0], o[1]);
            cvt_e4m3x4(raw.y, mult, o[2], o[3]);
            cvt_e4m3x4(raw.z, mult, o[4], o[5]);
            cvt_e4m3x4(raw.w, mult, o[6], o[7]);
            const uint32_t dg = 2u * p16;
            st_shared_v4(k_row_addr + dg * kCoreBytes, o[0], o[1], o[2], o[3]);
            st_shared_v4(k_row_addr + (dg + 1u) * kCoreBytes, o[4], o[5], o[6], o[7]);
        } else {             // RoPE tail: already bf16, 8 dims per piece
            const uint32_t dg = 56u + (p16 - 28u);
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

// ------------------------------------------------------------------ work distribution
// The grid is persistent: `gridDim.x` CTAs (at most one per SM) share the launch's work, which is the
// list of items (token t, block of 64 heads hb), item = t * head_blocks + hb (or hb * T + t: `hb_major`), each made of
// ceil(rows(t) / 128) tiles.  Two ways of sharing it:
//   whole items (balanced == 0): CTA c takes items c, c + P, c + 2P, ...; every output is final.
//   balanced tiles (balanced == 1): the tiles of all items, in item order, are cut into P equal
//     contiguous ranges.  A CTA's range starts and ends inside items, so its first and last segment
//     may be partial: those go to scratch slots 2c and 2c + 1 as un-normalised fp32 partials and a
//     second kernel merges them; the items in between are final.  This is what keeps all SMs busy
//     when there are fewer items than SMs or the items differ in length (ragged lens).
// Items without rows count as one tile so that somebody owns (and zeroes) their output.
struct Seg {
    int t, hb;       // item
    int n, ns;       // selected rows of the token: total, and of the swa stream
    int tile0, ntl;  // tiles of the item this segment covers (ntl == 0: the item has no rows)
    int slot;        // scratch slot of a partial segment
    bool complete;   // the segment is the whole item: write the final output
    bool owns_first; // partial segment holding the item's first tile: it writes the merge descriptor
    long long gfirst; // global tile index of the item's first tile (balanced mode)
    int ntS;         // scheduled tiles of the item (max(1, tiles))
};

// DENSE is a template parameter throughout the scheduling code so that the sparse kernels carry none of the
// dense bookkeeping (measured: as run-time branches it cost the sparse decode 1-2 %).
template <bool DENSE>
__device__ __forceinline__ void token_rows(const KernelArgs &a, int t, int &ns, int &n) {
    if constexpr (DENSE) {     // dense paged MLA: all rows of the sequence, minus what the causal mask hides
        const int b = t / a.dense_sq, i = t - b * a.dense_sq;
        // lengths are clamped to what the block table row can name (swa.topk rows), as the sparse lens are to topk
        ns = n = max(min(__ldg(a.swa.lens + b), a.swa.topk) - (a.causal ? a.dense_sq - 1 - i : 0), 0);
    } else {
        ns = min(max(__ldg(a.swa.lens + t), 0), a.swa.topk);
        const int ne = (a.extra.cache != nullptr) ? min(max(__ldg(a.extra.lens + t), 0), a.extra.topk) : 0;
        n = ns + ne;
    }
}
__device__ __forceinline__ int sched_tiles(int n) { return max(1, (n + kTileRows - 1) / kTileRows); }

// Position u in the order the schedule walks the tokens -> token.  Identity, except for dense paged MLA with
// several query positions per sequence: there the tokens are walked query position first (all sequences at
// position 0, then at position 1, ...), so that the positions of one sequence, which read the same rows, are
// handled by different CTAs at the same time and share the rows through L2 instead of reading them from HBM
// one after the other.
template <bool DENSE>
__device__ __forceinline__ int tok_of(const KernelArgs &a, int u) {
    if (!DENSE || a.dense_sq <= 1) return u;
    const int B = a.T / a.dense_sq, i = u / B;
    return (u - i * B) * a.dense_sq + i;
}

struct SegIter {
    int t, hb;          // next item (t: position in the walking order, see tok_of)
    int off;            // first tile of that item still to do (balanced mode)
    long long gpos;     // global tile index of (t, hb, off) (balanced mode)
    long long rem;      // tiles left in this CTA's range (balanced mode)
    int item, stride;   // whole-item mode
    bool first;

};

template <bool DENSE>
__device__ __forceinline__ bool iter_next(const KernelArgs &a, SegIter &it, Seg &s) {
    {
        const bool hb_major = DENSE && a.hb_major != 0;
        int &t = it.t, &hb = it.hb, &off = it.off, &item = it.item;
        const int stride = it.stride;
        long long &gpos = it.gpos, &rem = it.rem;
        bool &first = it.first;
        if (!a.balanced) {
            if (item >= a.T * a.head_blocks) return false;
            if (hb_major) {
                s.hb = item / a.T;
                s.t = tok_of<DENSE>(a, item - s.hb * a.T);
            } else {
                const int u = item / a.head_blocks;
                s.hb = item - u * a.head_blocks;
                s.t = tok_of<DENSE>(a, u);
            }
            token_rows<DENSE>(a, s.t, s.ns, s.n);
            s.tile0 = 0;
            s.ntl = (s.n + kTileRows - 1) / kTileRows;
            s.ntS = max(1, s.ntl);
            s.slot = 0;
            s.complete = true;
            s.owns_first = false;
            s.gfirst = 0;
            item += stride;
            return true;
        }
        if (rem <= 0) return false;
        s.t = tok_of<DENSE>(a, t);
        s.hb = hb;
        token_rows<DENSE>(a, s.t, s.ns, s.n);
        const int nt = (s.n + kTileRows - 1) / kTileRows;
        s.ntS = max(1, nt);
        const int take = static_cast<int>(min(static_cast<long long>(s.ntS - off), rem));
        s.tile0 = off;
        s.ntl = nt == 0 ? 0 : take;
        s.complete = (off == 0 && take == s.ntS);
        s.owns_first = (!s.complete && off == 0);
        s.slot = 2 * static_cast<int>(blockIdx.x) + (first ? 0 : 1);
        s.gfirst = gpos - off;
        first = false;
        rem -= take;
        gpos += take;
        off = 0;
        if (hb_major) {
            if (++t == a.T) {
                t = 0;
                ++hb;
            }
        } else if (++hb == a.head_blocks) {
            hb = 0;
            ++t;
        }
        return true;
    }
}

// First tile of CTA c when W tiles are shared by P CTAs, and the CTA a given tile falls to.
__device__ __forceinline__ long long range_begin(long long c, long long W, long long P) { return c * W / P; }
__device__ __forceinline__ int cta_of_tile(long long x, long long W, long long P) {
    return static_cast<int>(((x + 1) * P + W - 1) / W - 1);
}

// Every thread of the CTA calls this; returns false when the CTA has nothing to do.  `scratch` is a
// shared-memory array of at least 24 ints.  `W_out` / `P_out`: total scheduled tiles and the number
// of CTAs that share them (needed later for the merge descriptors).
template <bool DENSE>
__device__ bool make_schedule(const KernelArgs &a, int *scratch, SegIter &it, long long &W_out, int &P_out) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool hb_major = DENSE && a.hb_major != 0;
    it.first = true;
    it.off = 0;
    it.gpos = 0;
    it.rem = 0;
    it.t = it.hb = 0;
    it.item = blockIdx.x;
    it.stride = gridDim.x;
    W_out = 0;
    P_out = gridDim.x;
    if (!a.balanced) return it.item < a.T * a.head_blocks;

    long long *wsum = reinterpret_cast<long long *>(scratch);          // [kNumWarps] then results
    int *found = scratch + 2 * kNumWarps;                               // {t, excl_lo, excl_hi, scheduled tiles}
    if (a.T <= kThreads) {
        // The usual case (the balanced schedule is chosen for few items): one token per thread, one
        // scan gives the total and every token's first global tile at once.
        int ns = 0, n = 0;
        if (tid < a.T) token_rows<DENSE>(a, tok_of<DENSE>(a, tid), ns, n);
        const int ntS = sched_tiles(n);
        const int per_token = hb_major ? 1 : a.head_blocks;      // items of a token that are neighbours in the order
        const long long v = tid < a.T ? static_cast<long long>(ntS) * per_token : 0;
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        long long before = 0, W1 = 0;
        for (int w = 0; w < kNumWarps; ++w) {
            if (w < warp) before += wsum[w];
            W1 += wsum[w];
        }
        const long long W = hb_major ? W1 * a.head_blocks : W1;
        const long long P = min(static_cast<long long>(gridDim.x), W);
        W_out = W;
        P_out = static_cast<int>(P);
        if (static_cast<long long>(blockIdx.x) >= P) return false;      // uniform
        const long long lo = range_begin(blockIdx.x, W, P), hi = range_begin(blockIdx.x + 1, W, P);
        const long long excl = before + incl - v;
        const int hb_lo = hb_major ? static_cast<int>(lo / W1) : 0;   // head block first: W1 tiles per head block
        const long long lo_in = lo - hb_lo * W1;
        if (tid < a.T && excl <= lo_in && lo_in < excl + v) {
            const long long d = lo_in - excl;
            found[0] = tid;
            found[1] = hb_major ? hb_lo : static_cast<int>(d / ntS);  // head block
            found[2] = static_cast<int>(d - (hb_major ? 0ll : static_cast<long long>(found[1]) * ntS));   // first tile inside the item
        }
        __syncthreads();
        it.t = found[0];
        it.hb = found[1];
        it.off = found[2];
        it.gpos = lo;
        it.rem = hi - lo;
        return true;
    }

    // Many tokens: two passes.  Pass 1: W = head_blocks * sum_t max(1, tiles(t))
    long long mine = 0;
    for (int t = tid; t < a.T; t += kThreads) {
        int ns, n;
        token_rows<DENSE>(a, t, ns, n);
        mine += sched_tiles(n);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) wsum[warp] = mine;
    __syncthreads();
    long long W = 0;
    for (int w = 0; w < kNumWarps; ++w) W += wsum[w];
    W *= a.head_blocks;
    __syncthreads();
    const long long P = min(static_cast<long long>(gridDim.x), W);
    W_out = W;
    P_out = static_cast<int>(P);
    if (static_cast<long long>(blockIdx.x) >= P) return false;
    const long long lo = range_begin(blockIdx.x, W, P), hi = range_begin(blockIdx.x + 1, W, P);
    const long long W1 = W / a.head_blocks;
    const int hb_lo = hb_major ? static_cast<int>(lo / W1) : 0;
    const long long lo_in = lo - hb_lo * W1;       // position inside the head block's run of tokens (head block first)
    const int per_token = hb_major ? 1 : a.head_blocks;

    // pass 2: the token whose tiles contain global tile `lo`
    long long run = 0;
    for (int base = 0; base < a.T; base += kThreads) {
        const int t = base + tid;
        long long v = 0;
        if (t < a.T) {
            int ns, n;
            token_rows<DENSE>(a, tok_of<DENSE>(a, t), ns, n);
            v = static_cast<long long>(sched_tiles(n)) * per_token;
        }
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        long long before = run, total = 0;
        for (int w = 0; w < kNumWarps; ++w) {
            if (w < warp) before += wsum[w];
            total += wsum[w];
        }
        const long long excl = before + incl - v;
        if (t < a.T && excl <= lo_in && lo_in < excl + v) {
            found[0] = t;
            found[1] = static_cast<int>(excl & 0xFFFFFFFFll);
            found[2] = static_cast<int>(excl >> 32);
        }
        run += total;
        __syncthreads();
        if (run > lo_in) break;     // uniform: every thread holds the same `run`
    }
    const int t0 = found[0];
    const long long excl0 = (static_cast<long long>(found[2]) << 32) | static_cast<unsigned int>(found[1]);
    int ns, n;
    token_rows<DENSE>(a, tok_of<DENSE>(a, t0), ns, n);
    const int ntS = sched_tiles(n);
    const long long d = lo_in - excl0;
    it.t = t0;
    it.hb = hb_major ? hb_lo : static_cast<int>(d / ntS);
    it.off = static_cast<int>(d - (hb_major ? 0ll : static_cast<long long>(it.hb) * ntS));
    it.gpos = lo;
    it.rem = hi - lo;
    return true;
}

// The segments live in shared memory, not in registers: a ring of five records (segment k in record
// k % 5) filled by the scheduler warp (warp 18, otherwise idle) three segments ahead, the iterator
// state it continues from, and the count of records published so far, which every reader checks
// before it looks at a record (the count is written after a fence, read volatile).  Offsets in ints
// from Smem::kSched:
constexpr int kSchedScan = 0;       // [64]  scratch of make_schedule
constexpr int kSchedIter = 64;      // [12]  t, hb, off, item, stride, first, gpos(2), rem(2), W(2)
constexpr int kSchedP = 76;         // [1]   CTAs sharing the tiles
constexpr int kSchedPub = 77;       // [1]   records published so far
constexpr int kSchedTiles = 78;     // [1]   tiles whose S^T has been scored (written by the MMA thread)
constexpr int kSchedRec = 80;       // [5][12] t, hb, n, ns, tile0, ntl, slot, flags, last CTA of the item
constexpr int kSchedFin = kSchedRec + 60;   // [2][5] this CTA's partial segments: {valid, item, first CTA, last CTA, first CTA's slot}
constexpr int kSchedInts = kSchedFin + 10;
static_assert(kSchedInts <= 160, "Smem::kSched holds 160 ints");
constexpr int kSegValid = 4, kSegOwnsFirst = 2, kSegComplete = 1;

__device__ __forceinline__ void store_iter(int *p, const SegIter &it, long long W) {
    p[0] = it.t, p[1] = it.hb, p[2] = it.off, p[3] = it.item, p[4] = it.stride, p[5] = it.first ? 1 : 0;
    p[6] = static_cast<int>(it.gpos & 0xFFFFFFFFll), p[7] = static_cast<int>(it.gpos >> 32);
    p[8] = static_cast<int>(it.rem & 0xFFFFFFFFll), p[9] = static_cast<int>(it.rem >> 32);
    p[10] = static_cast<int>(W & 0xFFFFFFFFll), p[11] = static_cast<int>(W >> 32);
}
__device__ __forceinline__ void load_iter(const int *p, SegIter &it, long long &W) {
    it.t = p[0], it.hb = p[1], it.off = p[2], it.item = p[3], it.stride = p[4], it.first = p[5] != 0;
    it.gpos = (static_cast<long long>(p[7]) << 32) | static_cast<unsigned int>(p[6]);
    it.rem = (static_cast<long long>(p[9]) << 32) | static_cast<unsigned int>(p[8]);
    W = (static_cast<long long>(p[11]) << 32) | static_cast<unsigned int>(p[10]);
}

// An item without rows: its output is zero (the reference's "no selected slot" case).
template <bool DENSE>
__device__ __forceinline__ void zero_item(const KernelArgs &a, const Seg &s, int tid, int nthreads) {
    const int h0 = s.hb * 64, hv = min(64, a.H - h0);
    if (DENSE && a.lse != nullptr)
        for (int h = tid; h < hv; h += nthreads) *lse_ptr(a, s.t, h0 + h) = -INFINITY;
    for (int i = tid; i < hv * (kD / 8); i += nthreads) {
        const int h = i / (kD / 8), d8 = i - h * (kD / 8);
        *reinterpret_cast<uint4 *>(a.out + static_cast<long long>(s.t) * a.o_ts + static_cast<long long>(h0 + h) * a.o_hs +
                                   d8 * 8) = make_uint4(0, 0, 0, 0);
    }
}

// One warp (all lanes, uniformly): continue the iterator to the next segment that has tiles, zeroing the
// outputs of items without rows on the way, and publish it as segment `k` (records are published in order).
template <bool DENSE>
__device__ __forceinline__ void publish_segment(const KernelArgs &a, int *sched, int k, int lane) {
    const bool hb_major = DENSE && a.hb_major != 0;
    SegIter it;
    long long W;
    load_iter(sched + kSchedIter, it, W);
    const int P = sched[kSchedP];
    Seg s = {};
    bool ok = false;
    while (iter_next<DENSE>(a, it, s)) {
        if (s.ntl > 0) {
            ok = true;
            break;
        }
        zero_item<DENSE>(a, s, lane, 32);
    }
    if (!DENSE && ok && lane < 5) {
        // Warm L2 (and the TLB) with the slot ids of the segment's first tile: nobody has touched that
        // token's index row yet, and the workers need the ids in the last tile of the segment before,
        // to issue the gather.  Records are published three segments ahead, so the lines have arrived by then.
        const int g0 = s.tile0 * kTileRows;
        const int g = min(g0 + lane * 32, min(g0 + kTileRows, s.n) - 1);
        const int *ip = g < s.ns ? a.swa.indices + static_cast<long long>(s.t) * a.swa.idx_stride + g
                                 : a.extra.indices + static_cast<long long>(s.t) * a.extra.idx_stride + (g - s.ns);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(ip));
    }
    {   // warm the lens of the tokens the next calls will ask for (lane i: i + 1 items ahead)
        const long long ahead = a.balanced ? static_cast<long long>(it.t) + lane
                                           : hb_major ? (static_cast<long long>(it.item) + static_cast<long long>(lane) * it.stride) % a.T
                                           : (static_cast<long long>(it.item) + static_cast<long long>(lane) * it.stride) / a.head_blocks;
        if (ahead < a.T) {
            // dense paged MLA: lens are per sequence, a token is (sequence, query position)
            asm volatile("prefetch.global.L1 [%0];" ::"l"(a.swa.lens + (DENSE && a.dense_sq > 1 ? tok_of<DENSE>(a, static_cast<int>(ahead)) / a.dense_sq : ahead)));
            if (a.extra.cache != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.extra.lens + ahead));
        }
    }
    __syncwarp();
    if (lane == 0) {
        store_iter(sched + kSchedIter, it, W);
        int *r = sched + kSchedRec + 12 * (k % 5);
        r[0] = s.t, r[1] = s.hb, r[2] = s.n, r[3] = s.ns, r[4] = s.tile0, r[5] = s.ntl, r[6] = s.slot;
        r[7] = ok ? (kSegValid | (s.owns_first ? kSegOwnsFirst : 0) | (s.complete ? kSegComplete : 0)) : 0;
        r[8] = (ok && s.owns_first) ? cta_of_tile(s.gfirst + s.ntS - 1, W, P) : 0;
        if (ok && !s.complete && a.fused_merge == 2) {   // at most two per CTA: its first segment (slot 2c), its last (2c + 1)
            int *f = sched + kSchedFin + 5 * (s.slot & 1);
            const int c0 = cta_of_tile(s.gfirst, W, P);
            f[1] = s.t * a.head_blocks + s.hb;
            f[2] = c0;
            f[3] = cta_of_tile(s.gfirst + s.ntS - 1, W, P);
            f[4] = range_begin(c0, W, P) == s.gfirst ? 2 * c0 : 2 * c0 + 1;   // the first CTA's segment of the item
            f[0] = 1;
        }
        __threadfence_block();
        reinterpret_cast<volatile int *>(sched)[kSchedPub] = k + 1;
    }
    __syncwarp();
}

// The following warps wait until `count` tiles of this CTA have been scored (QK^T complete, softmax
// done).  Lane 0 polls, the result is broadcast; time-bounded.
__device__ __forceinline__ bool wait_tiles(const int *sched, int count, volatile int *abort_flag, int lane) {
    int ok = 1;
    if (lane == 0) {
        const volatile int *done = reinterpret_cast<const volatile int *>(sched) + kSchedTiles;
        if (*done < count) {
            const uint64_t t0 = globaltimer_ns();
            while (*done < count) {
                __nanosleep(64);
                if (*abort_flag != 0) {
                    ok = 0;
                    break;
                }
                if (globaltimer_ns() - t0 > kWaitLimitNs) {
                    give_up(abort_flag, kStatusSoftmaxWait);
                    ok = 0;
                    break;
                }
            }
        }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// Readers call this before they look at record k.  In practice it never waits (records are three
// segments ahead); the wait is time-bounded like every other one.
__device__ __forceinline__ bool wait_published(const int *sched, int k, volatile int *abort_flag) {
    const volatile int *pub = reinterpret_cast<const volatile int *>(sched) + kSchedPub;
    if (*pub > k) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1;; ++it) {
        if (*pub > k) return true;
        if ((it & 63u) == 0u) {
            if (*abort_flag != 0) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                give_up(abort_flag, kStatusMmaWait);
                return false;
            }
        }
    }
}

// ------------------------------------------------------------------ MMA issue (the MMA warp, all lanes)
// Walks the segments the scheduler warp publishes.  Barrier phases are counted over the CTA's whole
// life: `gt` tiles for the per-tile barriers, `so` segments for the two accumulator barriers.
//
// The whole warp runs this code and only the tcgen05 instructions themselves are predicated on one
// elected lane.  A tcgen05.mma has to be ISSUED, and this warp shares its scheduler with four worker
// warps that are busy with conversion arithmetic for most of a tile.  Measured on the GPU with the
// scheduler's other warps always ready to issue: one lane inside a divergent branch, building each
// descriptor from two 32-bit halves, got one MMA out per 500 cycles; the same loop run warp-uniformly
// (the compiler keeps the descriptor arithmetic on the uniform datapath) one per 90, against 48 for the
// tensor pipe alone (M128 x N64 x K16 with both operands fetched from shared memory).  In this kernel the
// one-lane form issued one MMA per ~75 cycles, so every PV chunk released its part of the K buffer late
// and the conversion of the next tile, which follows those releases, was paced by MMA issue.
template <int NPAD, bool DENSE, bool KTMA>
__device__ __forceinline__ void mma_role(uint8_t *smem, uint32_t tmem_base) {
    using L = Smem<NPAD, DENSE>;
    // Segment k is read from record k % 5 of the ring.  Warp 0 wrote it three segments earlier, before
    // conversions this thread has since waited for, and overwrites it only during segment k + 2.
    const volatile int *ring = reinterpret_cast<const volatile int *>(smem + L::kSched) + kSchedRec;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    const int lane = threadIdx.x & 31;
    const uint32_t go = elect_one();
    constexpr uint32_t idesc_qk = umma_idesc_bf16(128, NPAD, 0, 0);
    constexpr uint32_t idesc_pv = umma_idesc_bf16(128, NPAD, 1, 1);
    // QK^T: K-major A (rows x dims) and B (heads x dims): M/N step = one row group (8192 B), K step =
    // one core matrix (128 B).  PV: MN-major A = K^T chunk (dims x rows): M step = next dim group
    // (128 B), K step = next row group (8192 B); MN-major B = P^T: N step = next head group (2048 B),
    // K step = next row group (128 B).  Only the 14-bit start-address field changes between MMAs.
    const uint64_t qa = umma_desc(smem_u32(smem + L::kK), kCoreBytes, kRowGroupBytes);
    const uint64_t qb = umma_desc(smem_u32(smem + L::kQ), kCoreBytes, L::kQRowGroup);
    const uint64_t ra = umma_desc(smem_u32(smem + L::kP), kCoreBytes, 1024);      // dense: the tile's 64 RoPE dims
    // K by TMA: slabs of [128 rows][128 B] with the 128-byte swizzle (layout type 2).  QK^T reads a slab
    // K-major (eight rows are 1024 B apart, a K step of 16 dims is 32 B inside the row); PV reads the two
    // slabs of a chunk MN-major (the next 64 dims are one slab on, the next eight rows 1024 B, a K step of 16 rows 2048 B).
    constexpr uint64_t kSw128 = 2ull << 61;
    const uint64_t qa_sw = umma_desc(smem_u32(smem + L::kK), 16, 1024) | kSw128;
    // ... and so is Q there: nine slabs of [NPAD heads][128 B], fetched by nine 3-D boxes (qload_role)
    const uint64_t qb_sw = umma_desc(smem_u32(smem + L::kQ), 16, 1024) | kSw128;
    const uint64_t ra_sw = umma_desc(smem_u32(smem + L::kP), 16, 1024) | kSw128;
    const uint64_t pa_sw = umma_desc(smem_u32(smem + L::kK), kSlabBytes, 1024) | kSw128;
    const uint64_t pa = umma_desc(smem_u32(smem + L::kK), kRowGroupBytes, kCoreBytes);
    const uint64_t pb = umma_desc(smem_u32(smem + L::kP), kCoreBytes, 2048);
    constexpr bool kAlt = KTMA && L::kAltBytes > 0;

    int gt = 0;
    for (int so = 0;; ++so) {
        const volatile int *rec = ring + 12 * (so % 5);
        if (!wait_published(reinterpret_cast<const int *>(smem + L::kSched), so, abort_flag)) return;
        if ((rec[7] & kSegValid) == 0) break;
        const int ntl = rec[5];
        for (int it = 0; it < ntl; ++it, ++gt) {
            if (it == 0 && !mbar_wait(bars + kBarQ * 8, so & 1, abort_flag)) {   // this item's Q tile
                if (lane == 0) give_up(abort_flag, kStatusMmaWait);
                return;
            }
            // K by TMA: a full tile needs nothing from the workers, so its chunks are taken as they land; only a
            // last, partial tile waits for the workers, who wipe the rows past the sequence first.  (The workers
            // arrive on the ready barriers for every tile, so both sets of barriers stay in step with `gt`.)
            const bool from_tma = KTMA && (rec[4] + it + 1) * kTileRows <= rec[2];
            // chunk 0 of an odd tile lies in the second buffer (start-address field of the descriptors: bytes / 16)
            const bool odd = kAlt && (gt & 1);
            const uint64_t c0_off = odd ? static_cast<uint64_t>((L::kAlt - L::kK) >> 4) : 0ull;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const bool landed = !(kAlt && c == 0) ? mbar_wait(bars + ((from_tma ? kBarLand : kBarReady) + c) * 8, gt & 1, abort_flag)
                                    : !from_tma       ? mbar_wait(bars + kBarReady * 8, gt & 1, abort_flag)
                                                      : mbar_wait(bars + (odd ? kBarLandAlt : kBarLand) * 8, (gt >> 1) & 1, abort_flag);
                if (!landed) {
                    if (lane == 0) give_up(abort_flag, kStatusMmaWait);
                    return;
                }
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t off = static_cast<uint64_t>(((16 * c + 2 * k) * kCoreBytes) >> 4);
                    if constexpr (KTMA) {
                        const uint64_t aoff = static_cast<uint64_t>(((2 * c + (k >> 2)) * kSlabBytes + (k & 3) * 32) >> 4);
                        const uint64_t qoff = static_cast<uint64_t>(((2 * c + (k >> 2)) * (NPAD * 128) + (k & 3) * 32) >> 4);
                        umma_bf16_ss_pred(tmem_base, qa_sw + aoff + (c == 0 ? c0_off : 0ull), qb_sw + qoff, idesc_qk, (c | k) != 0 ? 1u : 0u, go);
                    } else {
                        umma_bf16_ss_pred(tmem_base, qa + off, qb + off, idesc_qk, (c | k) != 0 ? 1u : 0u, go);
                    }
                }
                if constexpr (DENSE) {
                    if (c == 3) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t aoff = static_cast<uint64_t>((2 * k * kCoreBytes) >> 4);
                            const uint64_t boff = static_cast<uint64_t>(((64 + 2 * k) * kCoreBytes) >> 4);
                            if constexpr (KTMA) umma_bf16_ss_pred(tmem_base, ra_sw + static_cast<uint64_t>((k * 32) >> 4),
                                                                  qb_sw + static_cast<uint64_t>((8 * (NPAD * 128) + k * 32) >> 4), idesc_qk, 1u, go);
                            else umma_bf16_ss_pred(tmem_base, ra + aoff, qb + boff, idesc_qk, 1u, go);
                        }
                    }
                }
            }
            umma_commit_pred(bars + kBarS * 8, go);
            if (!mbar_wait(bars + kBarP * 8, gt & 1, abort_flag)) {
                if (lane == 0) give_up(abort_flag, kStatusMmaWait);
                return;
            }
            // Progress for the warps that only follow (Q loader, scheduler): a count cannot be missed
            // the way an mbarrier phase can by a waiter that falls two phases behind.
            if (lane == 0) reinterpret_cast<volatile int *>(smem + L::kSched)[kSchedTiles] = gt + 1;
            // The first PV of a segment overwrites O^T: the previous segment's epilogue must have read it.
            if (it == 0 && so > 0 && !mbar_wait(bars + kBarOFree * 8, (so - 1) & 1, abort_flag)) {
                if (lane == 0) give_up(abort_flag, kStatusMmaWait);
                return;
            }
            tc_fence_after_sync();
            const uint32_t acc0 = it > 0 ? 1u : 0u;
#pragma unroll
            for (int ci = 0; ci < 4; ++ci) {
                // with two buffers for chunk 0 nothing waits for its release: chunk 1 goes first (chunk 0 still
                // before chunk 3, which is what the K loader relies on)
                const int c = (kAlt && ci < 2) ? 1 - ci : ci;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t aoff = static_cast<uint64_t>((c * 16 * kCoreBytes + 2 * k * kRowGroupBytes) >> 4);
                    const uint64_t boff = static_cast<uint64_t>((2 * k * kCoreBytes) >> 4);
                    if constexpr (KTMA) {
                        const uint64_t soff = static_cast<uint64_t>((2 * c * kSlabBytes + k * 2048) >> 4);
                        umma_bf16_ss_pred(tmem_base + kTmemOCol + c * NPAD, pa_sw + soff + (c == 0 ? c0_off : 0ull), pb + boff, idesc_pv, k > 0 ? 1u : acc0, go);
                    } else {
                        umma_bf16_ss_pred(tmem_base + kTmemOCol + c * NPAD, pa + aoff, pb + boff, idesc_pv, k > 0 ? 1u : acc0, go);
                    }
                }
                umma_commit_pred(bars + (kBarFree + c) * 8, go);   // chunk c of the K buffer may be refilled
            }
            if (it + 1 == ntl) umma_commit_pred(bars + kBarO * 8, go);
        }
    }
}

// ------------------------------------------------------------------ pieces shared by prologue and workers
// Q tile of one item -> shared memory (K-major core matrices), with cp.async so that no registers are
// held and all pieces are in flight at once; heads beyond the item's last one are zero-filled.
// The caller later runs cp_async_wait_all() + fence_async_smem() before the tensor pipe may read it.
template <int NPAD, bool DENSE>
__device__ __forceinline__ void issue_q_tile(const KernelArgs &a, uint8_t *smem, int t, int h0, int hvalid, int warp,
                                             int lane, int nwarps) {
    using L = Smem<NPAD, DENSE>;
    const __nv_bfloat16 *qt = a.q + static_cast<long long>(t) * a.q_ts + static_cast<long long>(h0) * a.q_hs;
    const uint32_t q_addr = smem_u32(smem + L::kQ);
    constexpr int kQuads = L::kQDimGroups / 4;      // groups of four 16-byte pieces per head row
    for (int idx = warp; idx < (NPAD / 8) * kQuads; idx += nwarps) {
        const int hg = idx / kQuads, dg = (idx - hg * kQuads) * 4 + (lane >> 3), h = hg * 8 + (lane & 7);
        const bool ok = h < hvalid && (!DENSE || dg * 8 < a.dense_dims);
        const __nv_bfloat16 *src = qt + static_cast<long long>(ok ? h : 0) * a.q_hs + (ok ? dg : 0) * 8;
        cp_async_16_zfill(q_addr + hg * L::kQRowGroup + dg * kCoreBytes + (lane & 7) * 16, src, ok ? 16u : 0u);
    }
}

__device__ __forceinline__ float initial_ref(const KernelArgs &a, bool complete, int h0, int hl, int hvalid) {
    // A complete item folds the sink into its own denominator, so the sink takes part in the reference.
    // Without a sink the reference starts at 0: it has to be finite (scores are held relative to it)
    // and the first tile replaces it anyway.
    if (complete && a.sink != nullptr && hl < hvalid) return a.sink[h0 + hl] * kLog2e;
    return 0.0f;
}

// ------------------------------------------------------------------ merging one head (one warp)
// out = sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)),  M = max(m_s, sink), over the S
// partial segments whose slots `slot_of(k)` names.  Four segments in flight per lane; partials are read
// past L1 (another SM wrote them).  With `scratch`, the warp is one of `nsub` that share the head: it sums
// segments sub, sub + nsub, ... and leaves its un-normalised sum, M and the denominator in its scratch row
// (kMergeRow floats) for merge_finish.
constexpr int kMergeRow = kD + 4;
template <typename SlotOf>
__device__ __forceinline__ void merge_head(const float *part_o, const float *part_ml, SlotOf slot_of, int S, int npad,
                                           int hl, float sink_l2, __nv_bfloat16 *dst, int lane, float *lse_dst = nullptr,
                                           int sub = 0, int nsub = 1, float *scratch = nullptr) {
    auto ml_of = [&](int k) {
        return __ldcg(reinterpret_cast<const float2 *>(part_ml) + static_cast<long long>(slot_of(k)) * npad + hl);
    };
    float M = sink_l2;
    for (int k = lane; k < S; k += 32) {
        const float2 e = ml_of(k);
        if (e.y > 0.0f) M = fmaxf(M, e.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float denom = 0.0f;
    if (M > -INFINITY) {
        for (int k = lane; k < S; k += 32) {
            const float2 e = ml_of(k);
            if (e.y > 0.0f) denom += fast_exp2(e.x - M) * e.y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) denom += __shfl_xor_sync(0xffffffffu, denom, o);
    if (M > -INFINITY) denom += fast_exp2(sink_l2 - M);

    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
    for (int k0 = sub; k0 < S; k0 += 4 * nsub) {
        float4 x[4][4];
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int k = min(k0 + u * nsub, S - 1);
            const float2 e = ml_of(k);      // the same address in every lane: one broadcast load
            // empty segments (l == 0) get weight 0; their rows are loaded but never multiplied in
            w[u] = (k0 + u * nsub < S && e.y > 0.0f && M > -INFINITY) ? fast_exp2(e.x - M) : 0.0f;
            const float4 *src = reinterpret_cast<const float4 *>(part_o) +
                                (static_cast<long long>(slot_of(k)) * npad + hl) * (kD / 4);
#pragma unroll
            for (int v = 0; v < 4; ++v) x[u][v] = __ldcg(src + v * 32 + lane);
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
    if (scratch != nullptr) {
#pragma unroll
        for (int v = 0; v < 4; ++v)
            reinterpret_cast<float4 *>(scratch)[v * 32 + lane] = make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
        if (lane == 0) {
            scratch[kD] = M;
            scratch[kD + 1] = denom;
        }
        return;
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    if (lse_dst != nullptr && lane == 0) *lse_dst = denom > 0.0f ? (M + log2f(denom)) * kLn2 : -INFINITY;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const uint2 pk = make_uint2(pack_bf16x2(acc[4 * v] * inv, acc[4 * v + 1] * inv),
                                    pack_bf16x2(acc[4 * v + 2] * inv, acc[4 * v + 3] * inv));
        *reinterpret_cast<uint2 *>(dst + (v * 32 + lane) * 4) = pk;
    }
}
// Sum of the `nsub` scratch rows that merge_head left for one head (shared memory) -> output row and lse.
__device__ __forceinline__ void merge_finish(const float *scratch, int nsub, __nv_bfloat16 *dst, int lane, float *lse_dst) {
    const float M = scratch[kD], denom = scratch[kD + 1];
    float4 acc[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) acc[v] = reinterpret_cast<const float4 *>(scratch)[v * 32 + lane];
    for (int i = 1; i < nsub; ++i) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const float4 x = reinterpret_cast<const float4 *>(scratch + i * kMergeRow)[v * 32 + lane];
            acc[v].x += x.x;
            acc[v].y += x.y;
            acc[v].z += x.z;
            acc[v].w += x.w;
        }
    }
    const float inv = denom > 0.0f ? 1.0f / denom : 0.0f;
    if (lse_dst != nullptr && lane == 0) *lse_dst = denom > 0.0f ? (M + log2f(denom)) * kLn2 : -INFINITY;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
        const uint2 pk = make_uint2(pack_bf16x2(acc[v].x * inv, acc[v].y * inv), pack_bf16x2(acc[v].z * inv, acc[v].w * inv));
        *reinterpret_cast<uint2 *>(dst + (v * 32 + lane) * 4) = pk;
    }
}

// ------------------------------------------------------------------ slice merge (worker warps, end of the CTA)
// A few tokens spread over the whole GPU: an item is cut into many segments, one per CTA.  Every segment
// goes to scratch and raises its flag (the launch's tag).  When a CTA has finished all its tiles it
// waits, time-bounded, for the flags of all segments of each item it took part in and merges ITS SHARE
// of the item's heads (CTA j of S: heads [j*H/S, (j+1)*H/S)), so the merge is spread over as many SMs
// as the item was.  Every CTA has raised all its flags before it waits for anybody's: no cycles.
template <int NPAD, bool DENSE>
__device__ __forceinline__ void merge_head_slices(const KernelArgs &a, uint8_t *smem, int tid, int warp, int lane) {
    using L = Smem<NPAD, DENSE>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const volatile int *fin = reinterpret_cast<const volatile int *>(smem + L::kSched) + kSchedFin;
#pragma unroll 1
    for (int e = 0; e < 2; ++e) {
        const volatile int *f = fin + 5 * e;
        if (f[0] == 0) continue;                                // uniform: shared memory, same for every thread
        const int item = f[1], c0 = f[2], c1 = f[3], first_slot = f[4];
        auto slot_of = [&](int k) { return k == 0 ? first_slot : 2 * (c0 + k); };
        const int S = c1 - c0 + 1;
        if (warp == 0) {
            bool ok = true;
            for (int k = lane; k < S; k += 32) {
                const volatile unsigned long long *fl = a.flags + slot_of(k);
                if (*fl != a.tag) {
                    const uint64_t t0 = globaltimer_ns();
                    while (*fl != a.tag) {
                        __nanosleep(100);
                        if (*abort_flag != 0 || globaltimer_ns() - t0 > kWaitLimitNs) {
                            ok = false;
                            break;
                        }
                    }
                }
            }
            if (!__all_sync(0xffffffffu, ok) && lane == 0) give_up(abort_flag, kStatusEpilogueWait);
            __threadfence();
        }
        named_bar_sync(kAllWorkersBar, kWorkerThreads);
        const int t = item / a.head_blocks, h0 = (item - t * a.head_blocks) * 64;
        const int hvalid = min(NPAD, a.H - h0);
        const int j = static_cast<int>(blockIdx.x) - c0;
        const int hbeg = j * hvalid / S, hend = (j + 1) * hvalid / S, nh = hend - hbeg;
        // A long item cut into many segments leaves a CTA one head or none, and one warp would walk all S
        // partials four at a time (74 segments: ~25 us).  The idle warps then share the head's segments and
        // the sums meet in the K buffer, which nobody uses any more (16 rows per partial item of this CTA).
        // (Dense launches only: the sparse formats select at most 20 tiles per token, where one warp per head is as fast.)
        const int nsub = (DENSE && nh > 0 && 2 * nh <= kWorkerWarps && S >= 8) ? min(kWorkerWarps / nh, (S + 3) / 4) : 1;
        if (DENSE && nsub > 1) {
            float *scratch = reinterpret_cast<float *>(smem + L::kK) + (e * kWorkerWarps + warp) * kMergeRow;
            const int g = warp / nsub, hl = hbeg + g;
            if (g < nh) {
                const float sink_l2 = a.sink ? a.sink[h0 + hl] * kLog2e : -INFINITY;
                merge_head(a.part_o, a.part_ml, slot_of, S, NPAD, hl, sink_l2, nullptr, lane, nullptr, warp - g * nsub, nsub, scratch);
            }
            named_bar_sync(kAllWorkersBar, kWorkerThreads);
            if (g < nh && warp == g * nsub)
                merge_finish(scratch, nsub, a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0 + hl) * a.o_hs, lane,
                             (DENSE && a.lse != nullptr) ? lse_ptr(a, t, h0 + hl) : nullptr);
            continue;
        }
        for (int hl = hbeg + warp; hl < hend; hl += kWorkerWarps) {
            const float sink_l2 = a.sink ? a.sink[h0 + hl] * kLog2e : -INFINITY;
            merge_head(a.part_o, a.part_ml, slot_of, S, NPAD, hl, sink_l2,
                       a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0 + hl) * a.o_hs, lane,
                       (DENSE && a.lse != nullptr) ? lse_ptr(a, t, h0 + hl) : nullptr);
        }
    }
}

// ------------------------------------------------------------------ Q-loader warps (17..19)
// Fetching a 64 KB Q tile takes ~4.5k cycles of load issue; done by the worker warps it sat on the
// critical path of every segment boundary.  These three warps have nothing else to do: they follow
// the segments in the ring, wait for every tile's S^T barrier so that they know when the last QK^T of
// a segment has completed (the Q buffer is then free), fetch the next item's Q tile with cp.async
// and hand it to the MMA thread through the Q barrier.
template <int NPAD, bool DENSE, bool QSW = false>
__device__ __forceinline__ void qload_role(const KernelArgs &a, uint8_t *smem, int qwarp, int lane) {
    using L = Smem<NPAD, DENSE>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    const volatile int *ring = reinterpret_cast<const volatile int *>(smem + L::kSched) + kSchedRec;
    int gt = 0;
    for (int so = 0;; ++so) {
        const volatile int *rec = ring + 12 * (so % 5);
        if (!wait_published(reinterpret_cast<const int *>(smem + L::kSched), so, abort_flag)) return;
        if ((rec[7] & kSegValid) == 0) break;
        const int h0 = rec[1] * 64;
        if (a.q_tma) {
            // One tensor copy: box {8, 8, 64, NPAD/8, 1} of the 5-D view lands as [head group][dim group]
            // [head % 8][8 dims], which is the K-major core-matrix layout of the Q operand; head groups
            // beyond H are zero-filled.  The innermost coordinate is 0 (TMA needs it 16-byte aligned).
            // (That copy moves 16 bytes per element: 7-13k cycles per tile, which the first QK^T of every segment
            // waits for.  Dense, K by TMA: the tensor map is 3-D {dims, heads, tokens} instead and nine boxes
            // {64 dims, NPAD heads, 1 token} land as slabs of [head][128 B] with the 128-byte swizzle, the layout
            // the K slabs have; heads beyond H and, with head_dim 512, the ninth slab are zero-filled.)
            if (qwarp == 0 && lane == 0) {
                mbar_arrive_expect_tx(bars + kBarQ * 8, L::kQBytes);
                if constexpr (QSW) {
#pragma unroll
                    for (int sl = 0; sl < 9; ++sl)
                        tma_load_3d(smem_u32(smem + L::kQ) + sl * (NPAD * 128), &a.q_map, bars + kBarQ * 8, sl * 64, h0, rec[0]);
                } else {
                    tma_load_5d(smem_u32(smem + L::kQ), &a.q_map, bars + kBarQ * 8, 0, 0, 0, h0 / 8, rec[0]);
                }
            }
        } else {
            issue_q_tile<NPAD, DENSE>(a, smem, rec[0], h0, min(NPAD, a.H - h0), qwarp, lane, kQLoadWarps);
            cp_async_wait_all();
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + kBarQ * 8);
        }
        gt += rec[5];      // the Q buffer is free again when the segment's last tile has been scored
        if (!wait_tiles(reinterpret_cast<const int *>(smem + L::kSched), gt, abort_flag, lane)) return;
    }
}

// ------------------------------------------------------------------ K loader warp (19; dense paged MLA with TMA)
// Follows the segments; for every tile and K chunk c it waits until the previous tile's PV has released
// the chunk, then fetches the chunk's two slabs (and with chunk 3 the RoPE slab, which shares its memory
// with P^T) for every piece of R rows of the tile that holds rows of the sequence.  Lane p looks up the page
// of piece p in the block table and issues that piece's boxes; completion is counted in bytes on the
// chunk's "landed" barrier.  It is a producer of the tile chain (nothing advances without its boxes), so
// waiting on the free barriers by phase is safe here.  The pieces of the next tile are pulled into L2.
// With at most 32 heads shared memory has room for a second buffer for chunk 0: tiles alternate between the
// two, chunk 0 of the next tile is fetched right after chunk 3 of this one, and a quarter less is left to
// fetch between this tile's PV and the next tile's scores (16 heads, 4096 rows: 146 -> 134 us).
template <int NPAD>
__device__ __forceinline__ void kload_role(const KernelArgs &a, uint8_t *smem, int lane) {
    using L = Smem<NPAD, true>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    const volatile int *ring = reinterpret_cast<const volatile int *>(smem + L::kSched) + kSchedRec;
    const int R = a.k_box_rows, pieces_per_tile = kTileRows / R;
    const uint32_t k_addr = smem_u32(smem + L::kK), rope_addr = smem_u32(smem + L::kP);
    constexpr bool kAlt = L::kAltBytes > 0;      // chunk 0 of odd tiles has its own buffer and barrier
    const int row_bytes = a.dense_dims * 2;
    const bool contiguous_rows = a.swa.pos_stride == row_bytes;
    int gt = 0;
    for (int so = 0;; ++so) {
        const volatile int *rec = ring + 12 * (so % 5);
        if (!wait_published(reinterpret_cast<const int *>(smem + L::kSched), so, abort_flag)) return;
        if ((rec[7] & kSegValid) == 0) break;
        const int t = rec[0], n = rec[2], tile0 = rec[4], ntl = rec[5];
        const int b = a.dense_sq == 1 ? t : t / a.dense_sq;
        const int *table = a.swa.indices + static_cast<long long>(b) * a.swa.idx_stride;
        for (int it = 0; it < ntl; ++it, ++gt) {
            const int g = (tile0 + it) * kTileRows + lane * R;          // first row of this lane's piece
            const bool mine = lane < pieces_per_tile && g < n;
            int page = 0, row_in_page = 0;
            if (mine) {
                const int page_i = a.swa.block_shift >= 0 ? (g >> a.swa.block_shift) : g / a.swa.block_size;
                page = __ldg(table + page_i);
                row_in_page = g - page_i * a.swa.block_size;
            }
            const uint32_t pieces = __popc(__ballot_sync(0xffffffffu, mine));
            const uint32_t dst_row = static_cast<uint32_t>(lane * R) * 128u;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                // Two buffers for chunk 0: the one this tile fills was last read by the tile before the previous one,
                // whose PV had completed (chunk 0 before chunk 3) when chunk 3 of the previous tile was fetched.
                const bool two = kAlt && c == 0, odd = two && (gt & 1);
                if (!two && gt > 0 && !warp_wait(bars + (kBarFree + c) * 8, (gt - 1) & 1, abort_flag, lane, kStatusGatherWait)) return;
                const uint32_t bar = bars + (odd ? kBarLandAlt : kBarLand + c) * 8;
                const uint32_t dst = (odd ? smem_u32(smem + L::kAlt) : k_addr + (2 * c) * kSlabBytes) + dst_row;
                if (lane == 0) mbar_arrive_expect_tx(bar, pieces * static_cast<uint32_t>(R) * 128u * (c == 3 ? 3u : 2u));
                __syncwarp();
                if (mine) {
                    tma_load_3d(dst, &a.k_map, bar, 128 * c, row_in_page, page);
                    tma_load_3d(dst + kSlabBytes, &a.k_map, bar, 128 * c + 64, row_in_page, page);
                    if (c == 3) tma_load_3d(rope_addr + dst_row, &a.k_map, bar, 512, row_in_page, page);
                }
            }
            // The next tile of this segment, into L2 while this one is scored (the K buffer has no room for it yet).
            // One tile ahead is measured best: two ahead cost 9 % at 16 heads, none 13 %.
            const int g2 = g + kTileRows;
            if (contiguous_rows && lane < pieces_per_tile && it + 1 < ntl && g2 < n) {
                const int page_i = a.swa.block_shift >= 0 ? (g2 >> a.swa.block_shift) : g2 / a.swa.block_size;
                const int pg = __ldg(table + page_i);
                if (pg >= 0 && pg < a.swa.num_slots / a.swa.block_size) {
                    const uint8_t *src = a.swa.cache + static_cast<long long>(pg) * a.swa.block_stride +
                                         static_cast<long long>(g2 - page_i * a.swa.block_size) * row_bytes;
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(min(R, n - g2) * row_bytes) : "memory");
                }
            }
        }
    }
}

// ------------------------------------------------------------------ scheduler warp (18)
// Publishes the segment records.  Records 1..4 at once, then record s + 3 when the first tile of
// segment s has been scored: the ring slot it overwrites belonged to segment s - 2, whose last reader
// (its epilogue, run in the first tile of segment s - 1) has finished by then.
template <int NPAD, bool DENSE>
__device__ __forceinline__ void scheduler_role(const KernelArgs &a, uint8_t *smem, int lane) {
    using L = Smem<NPAD, DENSE>;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    const uint32_t bars = smem_u32(smem + L::kBars);
    int *sched = reinterpret_cast<int *>(smem + L::kSched);
    for (int k = 1; k < 5; ++k) publish_segment<DENSE>(a, sched, k, lane);
    int gt = 0;
    for (int s = 0;; ++s) {
        const volatile int *rec = sched + kSchedRec + 12 * (s % 5);
        if ((rec[7] & kSegValid) == 0) break;
        const int ntl = rec[5];
        if (!wait_tiles(sched, gt + 1, abort_flag, lane)) return;      // first tile of segment s scored
        if (s >= 2) publish_segment<DENSE>(a, sched, s + 3, lane);
        gt += ntl;
    }
}

// ------------------------------------------------------------------ worker warps (0..15)
// Each worker warp alternates between two jobs that never overlap in time for one tile:
//   convert: it owns rows 8w..8w+7 of the tile; raw bytes (already in registers) -> bf16 K chunks;
//   softmax: it owns TMEM lanes 32*(w%4).. (rows of S^T / dims of O^T) and head columns
//            (NPAD/4)*(w/4)..: scores -> P^T, running denominators, rare accumulator rescale.
// The raw bytes of the next tile are always in flight, across segment boundaries too.
template <int FMT, int NPAD>
__device__ __forceinline__ void worker_role(const KernelArgs &a, uint8_t *smem, uint32_t tmem_base, int warp, int lane) {
    using L = Smem<NPAD, is_dense(FMT)>;
    constexpr int J = Steps<FMT>::kCount;
    constexpr int CW = NPAD / 4;   // head columns per warp in the softmax job
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kAbort);
    int *sched = reinterpret_cast<int *>(smem + L::kSched);
    const uint32_t bars = smem_u32(smem + L::kBars);
    float *red = reinterpret_cast<float *>(smem + L::kRed);
    float *m_s = reinterpret_cast<float *>(smem + L::kM);
    float *alpha_s = reinterpret_cast<float *>(smem + L::kAlpha);
    float *shift_s = reinterpret_cast<float *>(smem + L::kShift);
    float *thr_s = reinterpret_cast<float *>(smem + L::kThr);
    const int tid = warp * 32 + lane;

    // convert job
    const int quarter = lane >> 3;
    const int my_row = warp * 8 + (lane & 7);
    const uint32_t k_row_addr = smem_u32(smem + L::kK) + warp * kRowGroupBytes + (lane & 7) * 16;
    // softmax job
    const int q = warp & 3, cs = warp >> 2;
    const int row = q * 32 + lane;
    const int col0 = cs * CW;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t p_addr = smem_u32(smem + L::kP) + (col0 >> 3) * 2048 + (row >> 3) * kCoreBytes + (row & 7) * 16 +
                            (col0 & 7) * 2;
    const int group_bar = 1 + cs;

    // Softmax denominator: after every tile the warp reduces its 32 rows, so one register per thread
    // holds the running sum of column col0 + (lane >> kColShift) instead of CW per-row sums.
    constexpr int kColShift = (CW == 16) ? 1 : (CW == 8) ? 2 : 3;
    float lacc = 0.0f;
    int gt = 0;      // tiles done by this CTA (mbarrier phases)

    // ---- epilogue of a finished segment (record `pg`): O^T / l as final output, or the un-normalised
    // partial.  `cg`: the segment whose softmax comes next (its reference max is initialised here), or
    // nullptr.  It runs while the tensor pipe is busy with the next segment's first QK^T, so it must
    // not touch the K or Q buffers: the final output is turned round (a thread holds one dim of CW
    // heads, a row of `out` is one head's 512 dims) through a small staging area per column-slice
    // group, HR heads at a time, so that global stores are 16 bytes per thread and 1 KB per head.
    auto epilogue = [&](auto final_tag, const volatile int *pg, const volatile int *cg, int parity) {
        constexpr bool kFinal = decltype(final_tag)::value;      // the CTA's last epilogue (only there can it own an item)
        constexpr int HR = CW < 8 ? CW : 8;     // heads per staging round
        const int t = pg[0], h0 = pg[1] * 64, slot = pg[6];
        const int hvalid = min(NPAD, a.H - h0);
        // Fused merge: the segment that holds an item's first tiles (always its CTA's last one) takes
        // the item's other partial segments, slots 2(c+1), 2(c+2), ..., into its own output.
        const bool owner = kFinal && a.fused_merge == 1 && (pg[7] & kSegOwnsFirst) != 0;
        const bool direct = (pg[7] & kSegComplete) != 0 || owner;
        const int others = owner ? pg[8] - static_cast<int>(blockIdx.x) : 0;
        float *wk_s = reinterpret_cast<float *>(smem + L::kK);     // [others][NPAD] weights (the K buffer is idle: last segment)
        // What the merge needs from OTHER CTAs does not depend on this CTA's last PV, which is still running
        // when the final epilogue starts: the flags are checked and the first loads are issued before the
        // wait for the accumulators ({max, denominator} of up to four other segments, and the first other
        // segment's rows for the first group of heads), so that their latency overlaps that PV.
        constexpr int kEarly = 4;
        float pv[kFinal ? 4 : 1][HR];
        float2 e_early[kFinal ? kEarly : 1];
        auto load_pv = [&](int r) {
            const float *src = a.part_o + (static_cast<long long>(2 * (blockIdx.x + 1)) * NPAD + col0 + r * HR) * kD + q * 32 + lane;
#pragma unroll
            for (int c = 0; c < (kFinal ? 4 : 1); ++c)
#pragma unroll
                for (int j = 0; j < HR; ++j) pv[c][j] = __ldcg(src + c * 128 + j * kD);
        };
        if constexpr (kFinal) {
            if (owner) {
                if (warp == 0) {
                    // The others wrote their partials at the start of their runs (or, for an item spread over
                    // three or more CTAs, finish about now): wait, time-bounded, for their flags.
                    bool ok = true;
                    for (int k = lane; k < others; k += 32) {
                        const volatile unsigned long long *f = a.flags + 2 * (static_cast<int>(blockIdx.x) + 1 + k);
                        if (*f != a.tag) {
                            const uint64_t t0 = globaltimer_ns();
                            while (*f != a.tag) {
                                __nanosleep(200);
                                if (*abort_flag != 0 || globaltimer_ns() - t0 > kWaitLimitNs) {
                                    ok = false;
                                    break;
                                }
                            }
                        }
                    }
                    if (!__all_sync(0xffffffffu, ok) && lane == 0) give_up(abort_flag, kStatusEpilogueWait);
                    __threadfence();
                }
                named_bar_sync(kAllWorkersBar, kWorkerThreads);
                if (tid < NPAD) {
#pragma unroll
                    for (int k = 0; k < kEarly; ++k)
                        if (k < others)
                            e_early[k] = __ldcg(reinterpret_cast<const float2 *>(a.part_ml) +
                                                static_cast<long long>(2 * (blockIdx.x + 1 + k)) * NPAD + tid);
                }
                if constexpr (!is_dense(FMT)) load_pv(0);
            }
        }
        warp_wait(bars + kBarO * 8, parity, abort_flag, lane, kStatusEpilogueWait);
        tc_fence_after_sync();
        store_col_partial<CW>(red + q * NPAD + col0, lacc, lane);
        lacc = 0.0f;
        named_bar_sync(kAllWorkersBar, kWorkerThreads);
        if (tid < NPAD) {
            float l = (red[tid] + red[NPAD + tid]) + (red[2 * NPAD + tid] + red[3 * NPAD + tid]);
            if (owner) {
                const float sink_l2 = (a.sink != nullptr && tid < hvalid) ? a.sink[h0 + tid] * kLog2e : -INFINITY;
                float M = fmaxf(m_s[tid], sink_l2);
                auto ml_of = [&](int k) {
                    if constexpr (kFinal) {
                        if (k < kEarly) {
                            float2 e = e_early[0];
#pragma unroll
                            for (int u = 1; u < kEarly; ++u)
                                if (k == u) e = e_early[u];
                            return e;
                        }
                    }
                    return __ldcg(reinterpret_cast<const float2 *>(a.part_ml) + static_cast<long long>(2 * (blockIdx.x + 1 + k)) * NPAD + tid);
                };
                for (int k = 0; k < others; ++k) {
                    const float2 e = ml_of(k);
                    if (e.y > 0.0f) M = fmaxf(M, e.x);
                }
                const float w_own = fast_exp2(m_s[tid] - M);
                float denom = w_own * l + fast_exp2(sink_l2 - M);
                for (int k = 0; k < others; ++k) {
                    const float2 e = ml_of(k);
                    const float w = e.y > 0.0f ? fast_exp2(e.x - M) : 0.0f;
                    denom += w * e.y;
                    wk_s[k * NPAD + tid] = w;
                }
                const float inv = (!is_dense(FMT) || denom > 0.0f) ? 1.0f / denom : 0.0f;
                if (is_dense(FMT) && a.lse != nullptr && tid < hvalid) *lse_ptr(a, t, h0 + tid) = (M + log2f(denom)) * kLn2;
                alpha_s[tid] = w_own * inv;
                for (int k = 0; k < others; ++k) wk_s[k * NPAD + tid] *= inv;
            } else if (direct) {
                if (a.sink != nullptr && tid < hvalid) l += fast_exp2(a.sink[h0 + tid] * kLog2e - m_s[tid]);
                if (is_dense(FMT) && a.lse != nullptr && tid < hvalid) *lse_ptr(a, t, h0 + tid) = (m_s[tid] + log2f(l)) * kLn2;
                alpha_s[tid] = (!is_dense(FMT) || l > 0.0f) ? 1.0f / l : 0.0f;
            } else if (tid < hvalid) {
                float *ml = a.part_ml + (static_cast<long long>(slot) * NPAD + tid) * 2;
                ml[0] = m_s[tid];
                ml[1] = l;
            }
            if (cg != nullptr) {   // reference of the segment that follows (read after the barrier)
                const int c_h0 = cg[1] * 64;
                m_s[tid] = initial_ref(a, (cg[7] & kSegComplete) != 0, c_h0, tid, min(NPAD, a.H - c_h0));
                thr_s[tid] = move_threshold(m_s[tid]);
            }
        }
        named_bar_sync(kAllWorkersBar, kWorkerThreads);
        if (direct) {
            if constexpr (is_dense(FMT)) {
                // Dense paged MLA has no staging area (its longer Q rows take the room): a thread holds one dim
                // of HR heads and stores it as it is; the 32 lanes of a warp hold 32 consecutive dims, so each
                // 2-byte store instruction writes one 64-byte segment of a head's output row.
                __nv_bfloat16 *orow = a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0 + col0) * a.o_hs + row;
    #pragma unroll 1
                for (int r = 0; r < CW / HR; ++r) {
    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t o[HR];
                        TmemIO<HR>::ld(tmem_lane + kTmemOCol + c * NPAD + col0 + r * HR, o);
                        float val[HR];
    #pragma unroll
                        for (int j = 0; j < HR; ++j) val[j] = __uint_as_float(o[j]) * alpha_s[col0 + r * HR + j];
                        if constexpr (kFinal) {
                            for (int k = 0; k < others; ++k) {      // un-normalised rows of the item's other segments
                                const float *src = a.part_o + (static_cast<long long>(2 * (blockIdx.x + 1 + k)) * NPAD + col0 + r * HR) * kD +
                                                   c * 128 + row;
    #pragma unroll
                                for (int j = 0; j < HR; ++j) val[j] = fmaf(wk_s[k * NPAD + col0 + r * HR + j], __ldcg(src + j * kD), val[j]);
                            }
                        }
    #pragma unroll
                        for (int j = 0; j < HR; ++j)
                            if (col0 + r * HR + j < hvalid)
                                orow[static_cast<long long>(r * HR + j) * a.o_hs + c * 128] = __float2bfloat16_rn(val[j]);
                    }
                }
        } else {
                const uint32_t stage = (NPAD == 64 && cs < 2) ? smem_u32(smem + L::kP) + cs * 8192
                                                              : smem_u32(smem + L::kStage) + (NPAD == 64 ? cs - 2 : cs) * 8192;
                const int gtid = q * 32 + lane;     // thread of the group; also the dim inside a 128-dim chunk
                __nv_bfloat16 *orow = a.out + static_cast<long long>(t) * a.o_ts + static_cast<long long>(h0 + col0) * a.o_hs;
    #pragma unroll 1
                for (int r = 0; r < CW / HR; ++r) {
                    // Owner: `pv` holds the first other segment's rows of this round for all four chunks (this is
                    // the CTA's last epilogue: the gather registers are free), fetched one group of heads ahead -- the first
                    // before the wait for the accumulators -- so that their latency is never waited for.
                    uint32_t o2[2][HR];      // two chunks per tensor-memory round trip
    #pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if ((c & 1) == 0)
                            TmemIO<HR>::ld2(tmem_lane + kTmemOCol + c * NPAD + col0 + r * HR,
                                            tmem_lane + kTmemOCol + (c + 1) * NPAD + col0 + r * HR, o2[0], o2[1]);
                        const uint32_t (&o)[HR] = o2[c & 1];
                        const uint32_t dst = stage + (c * 128 + gtid) * 2;
                        float val[HR];
    #pragma unroll
                        for (int j = 0; j < HR; ++j) val[j] = __uint_as_float(o[j]) * alpha_s[col0 + r * HR + j];
                        if constexpr (kFinal) {
                            if (owner) {
    #pragma unroll
                                for (int j = 0; j < HR; ++j) val[j] = fmaf(wk_s[col0 + r * HR + j], pv[c][j], val[j]);
                            }
                            for (int k = 1; k < others; ++k) {      // un-normalised rows of the item's further segments
                                const float *src = a.part_o + (static_cast<long long>(2 * (blockIdx.x + 1 + k)) * NPAD + col0 + r * HR) * kD +
                                                   c * 128 + gtid;
    #pragma unroll
                                for (int j = 0; j < HR; ++j) val[j] = fmaf(wk_s[k * NPAD + col0 + r * HR + j], __ldcg(src + j * kD), val[j]);
                            }
                        }
    #pragma unroll
                        for (int j = 0; j < HR; ++j) {
                            const __nv_bfloat16 v = __float2bfloat16_rn(val[j]);
                            asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst + j * 1024), "h"(*reinterpret_cast<const uint16_t *>(&v)) : "memory");
                        }
                    }
                    if constexpr (kFinal) {
                        if (owner && r + 1 < CW / HR) load_pv(r + 1);
                    }
                    named_bar_sync(group_bar, 128);
    #pragma unroll
                    for (int i = 0; i < HR / 2; ++i) {
                        const int h = 2 * i + (gtid >> 6), piece = gtid & 63;
                        uint4 v;
                        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(stage + h * 1024 + piece * 16));
                        if (col0 + r * HR + h < hvalid)
                            *reinterpret_cast<uint4 *>(orow + static_cast<long long>(r * HR + h) * a.o_hs + piece * 8) = v;
                    }
                    named_bar_sync(group_bar, 128);     // the stage may be rewritten
                }
            }
        } else {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t o[CW];
                TmemIO<CW>::ld(tmem_lane + kTmemOCol + c * NPAD + col0, o);
                float *dst = a.part_o + (static_cast<long long>(slot) * NPAD + col0) * kD + c * 128 + row;
#pragma unroll
                for (int j = 0; j < CW; ++j)
                    if (col0 + j < hvalid) dst[static_cast<long long>(j) * kD] = __uint_as_float(o[j]);
            }
        }
        // Groups 0 and 1 staged in the P buffer, which other groups write in the coming softmax.
        named_bar_sync(kAllWorkersBar, kWorkerThreads);
        if (a.fused_merge && !direct && tid == 0) {     // this partial is complete: tell the item's owner
            __threadfence();
            *reinterpret_cast<volatile unsigned long long *>(a.flags + slot) = a.tag;
        }
        if (owner && tid < others) {
            // Every read of the other partials is behind the barrier above: lower their flags again.
            // A launch replayed from a CUDA graph carries the same tag every time, so a flag left up
            // would let the next replay read a partial that has not been rewritten yet.
            *reinterpret_cast<volatile unsigned long long *>(a.flags + 2 * (blockIdx.x + 1 + tid)) = 0ull;
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + kBarOFree * 8);     // the next segment's first PV may overwrite O^T
    };

    uint4 raw[J];
    RowRef<FMT> cur;
    int g;
    {   // raw bytes of the very first tile (segment 0 was published before the roles split)
        const int *r0 = sched + kSchedRec;
        g = r0[4] * kTileRows + my_row;
        if constexpr (FMT == kFmtBf16DenseTma) {
            cur = make_row_ref<FMT>(a, 0, 0, 0, -1);        // the loader warp fetches the rows
        } else {
            cur = make_row_ref<FMT>(a, r0[3], r0[2], g, is_dense(FMT) ? load_dense_slot_id(a, r0[0], r0[2], g)
                                                                     : load_slot_id(a, r0[0], r0[3], r0[2], g));
            load_row_pieces<FMT>(cur, quarter, raw, is_dense(FMT) ? a.dense_dims * 2 : 0);
        }
    }

    for (int k = 0;; ++k) {      // segments
        // Fields of this segment (sg) and the next (ng) are read from shared memory where they are
        // used rather than held in registers across the tile loop.
        const volatile int *sg = sched + kSchedRec + 12 * (k % 5);
        const volatile int *ng = sched + kSchedRec + 12 * ((k + 1) % 5);
        wait_published(sched, k + 1, abort_flag);
        const bool have_next = (ng[7] & kSegValid) != 0;
        if (tid == 0 && !a.fused_merge && (sg[7] & kSegOwnsFirst)) {   // descriptor for the combine kernel: this CTA holds the first tiles of an item that continues elsewhere
            int4 d;
            d.x = sg[0] * a.head_blocks + sg[1];
            d.y = sg[8] - static_cast<int>(blockIdx.x) + 1;     // CTAs (= partial segments) the item spans
            d.z = sg[6];
            d.w = min(NPAD, a.H - sg[1] * 64);
            reinterpret_cast<int4 *>(a.desc)[blockIdx.x] = d;
        }

        int rows_left = sg[2] - sg[4] * kTileRows;      // rows of the item from this tile on
        for (int left = sg[5]; left > 0; --left, ++gt, rows_left -= kTileRows) {
            const bool first_tile = left == sg[5];
            // ---- which tile comes next (possibly the next segment's first), and its slot id
            const bool in_seg = left > 1;
            const bool more = in_seg || have_next;
            const int n_t = in_seg ? sg[0] : ng[0], n_ns = in_seg ? sg[3] : ng[3], n_n = in_seg ? sg[2] : ng[2];
            const int g_next = in_seg ? g + kTileRows : ng[4] * kTileRows + my_row;
            const int id_next = (!more || FMT == kFmtBf16DenseTma) ? -1
                                : is_dense(FMT)                     ? load_dense_slot_id(a, n_t, n_n, g_next)
                                                                    : load_slot_id(a, n_t, n_ns, n_n, g_next);

            if constexpr (FMT == kFmtBf16DenseTma) {
                // ---- K by TMA: the loader warp fills the chunks; the workers only wait for a chunk to land,
                // wipe the rows of a last, partial tile that lie past the sequence (whatever the boxes brought
                // or left there must not reach the tensor pipe: 0 x NaN is NaN) and hand the chunk over.
                const bool wipe = my_row >= rows_left;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const bool odd = L::kAltBytes > 0 && c == 0 && (gt & 1);      // chunk 0 of odd tiles: second buffer
                    if (L::kAltBytes > 0 && c == 0)
                        warp_wait(bars + (odd ? kBarLandAlt : kBarLand) * 8, (gt >> 1) & 1, abort_flag, lane, kStatusGatherWait);
                    else
                        warp_wait(bars + (kBarLand + c) * 8, gt & 1, abort_flag, lane, kStatusGatherWait);
                    if (rows_left < kTileRows) {
                        if (wipe) {
                            const uint32_t sw = static_cast<uint32_t>(my_row & 7);
                            const uint32_t chunk_addr = smem_u32(smem + (odd ? L::kAlt : L::kK + 2 * c * kSlabBytes));
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t piece = 4u * i + quarter;         // 16-byte piece of the chunk's 256 bytes
                                const uint32_t addr = chunk_addr + (piece >> 3) * kSlabBytes + my_row * 128 +
                                                      (((piece & 7u) ^ sw) << 4);
                                st_shared_v4(addr, 0u, 0u, 0u, 0u);
                            }
                            if (c == 3) {
#pragma unroll
                                for (int i = 0; i < 2; ++i)
                                    st_shared_v4(smem_u32(smem + L::kP) + my_row * 128 + (((4u * i + quarter) ^ sw) << 4), 0u, 0u, 0u, 0u);
                            }
                        }
                        fence_async_smem();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bars + (kBarReady + c) * 8);
                }
            } else if constexpr (FMT == kFmtBf16Dense) {
                // ---- bf16 rows: cp.async straight into the K chunks as the previous tile's PV releases them
                // (this thread: four 16-byte pieces of its row per chunk), the RoPE dims with chunk 3 into the buffer
                // they share with P^T, which PV has finished reading by then; handed over as they land.
                const uint8_t *src = cur.ok ? cur.ptr : a.swa.cache;
                const uint32_t nbytes = cur.ok ? 16u : 0u;        // rows outside the sequence are zero-filled
                const uint32_t rope_row_addr = smem_u32(smem + L::kP) + warp * 1024 + (lane & 7) * 16;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (gt > 0) warp_wait(bars + (kBarFree + c) * 8, (gt - 1) & 1, abort_flag, lane, kStatusGatherWait);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int dg = 16 * c + 4 * i + quarter;      // the four lanes of a row: 64 contiguous bytes
                        cp_async_16_zfill(k_row_addr + dg * kCoreBytes, src + dg * 16, nbytes);
                    }
                    if (c == 3) {
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const int dg = 4 * i + quarter;
                            cp_async_16_zfill(rope_row_addr + dg * kCoreBytes, src + (a.dense_dims > 512 ? 1024 + dg * 16 : 0),
                                              a.dense_dims > 512 ? nbytes : 0u);
                        }
                    }
                    cp_async_commit();
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c == 0) cp_async_wait_group<3>();
                    else if (c == 1) cp_async_wait_group<2>();
                    else if (c == 2) cp_async_wait_group<1>();
                    else cp_async_wait_group<0>();
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bars + (kBarReady + c) * 8);
                }
            } else {
            // ---- convert: raw registers -> K chunks, each as soon as the previous tile's PV released it
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (gt > 0) warp_wait(bars + (kBarFree + c) * 8, (gt - 1) & 1, abort_flag, lane, kStatusGatherWait);
                if constexpr (FMT == kFmtInt8Wide) {
                    // chunk c = pieces 8c .. 8c+7 of the row; which registers hold them depends on the
                    // row's alignment (see load_row_pieces)
                    const bool q0 = cur.odd && quarter == 0;
                    const uint4 &next_first = raw[c < 3 ? 2 * c + 2 : 8];
                    const uint4 x = q0 ? next_first : raw[2 * c];
                    const uint32_t px = cur.odd ? (quarter == 0 ? 8u * c + 7u : 8u * c + 2u * quarter - 1u) : 8u * c + 2u * quarter;
                    const uint32_t py = cur.odd ? 8u * c + 2u * quarter : 8u * c + 2u * quarter + 1u;
                    convert_int8_piece(x, px, __uint_as_float(cur.sc0), k_row_addr);
                    convert_int8_piece(raw[2 * c + 1], py, __uint_as_float(cur.sc0), k_row_addr);
                } else {
#pragma unroll
                    for (int j = 0; j < J; ++j) {
                        const bool mine = (j < 8) ? ((j >> 1) == c) : (c == 3);
                        if (mine) convert_step<FMT>(raw[j], j, quarter, cur.sc0, cur.sc1, k_row_addr);
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + (kBarReady + c) * 8);
            }
            }
            // Raw bytes of the next tile.  Issued only now, after this tile's last conversion fence: a
            // proxy fence also waits for the thread's global loads in flight, so loads issued between
            // the chunks would put a memory latency on every hand-over.  They land while QK^T runs.
            // (Measured: sending half of them after the softmax instead made the tile 25 % slower: the
            // issue of a load blocks the warp while the SM's load queue is full.)
            if constexpr (FMT != kFmtBf16DenseTma) {
                cur = make_row_ref<FMT>(a, n_ns, n_n, more ? g_next : n_n, id_next);
                if (more) load_row_pieces<FMT>(cur, quarter, raw, is_dense(FMT) ? a.dense_dims * 2 : 0);
            }
            if constexpr (FMT == kFmtBf16Dense) {
                // Dense rows come from HBM once (no reuse between query tokens as in the sparse workloads):
                // measured, a row asked for one tile ahead arrives 7-8k cycles after its cp.async was issued,
                // so the tile after next is pulled into L2 as well (two tiles of all SMs are 43 MB).
                if (left > 2) {
                    const int g2 = g_next + kTileRows;
                    const RowRef<FMT> ahead = make_row_ref<FMT>(a, sg[3], sg[2], g2, load_dense_slot_id(a, sg[0], sg[2], g2));
                    load_row_pieces<FMT>(ahead, quarter, raw, a.dense_dims * 2);
                }
            }
            g = g_next;

            // ---- the previous segment's epilogue, while the tensor pipe computes this tile's QK^T
            if (first_tile && k > 0) epilogue(std::false_type{}, sched + kSchedRec + 12 * ((k - 1) % 5), sg, (k - 1) & 1);

            // ---- softmax of this tile
            warp_wait(bars + kBarS * 8, gt & 1, abort_flag, lane, kStatusSoftmaxWait);
            tc_fence_after_sync();
            // sm = S^T * scale - m, with m read once per tile (the same for all rows).
            // (dense, folded query positions: the columns of this warp belong to one position, which the causal
            // mask lets see fewer of the sequence's last rows)
            const bool row_valid = row < rows_left - ((is_dense(FMT) && a.fold_causal) ? a.fold_sq - 1 - col0 / a.fold_h : 0);
            float sm[CW];
            bool need = first_tile;
            {
                // The reference max m is only moved when some score exceeds it by more than its threshold
                // (always on a segment's first tile).  The vote spans the four warps that share these
                // columns.  m and the thresholds are read four columns at a time (one broadcast load each).
                uint32_t sraw[CW];
                TmemIO<CW>::ld(tmem_lane + col0, sraw);
#pragma unroll
                for (int v = 0; v < CW / 4; ++v) {
                    const float4 m4 = *reinterpret_cast<const float4 *>(m_s + col0 + 4 * v);
                    const float4 t4 = *reinterpret_cast<const float4 *>(thr_s + col0 + 4 * v);
                    const float mm[4] = {m4.x, m4.y, m4.z, m4.w}, tt[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = 4 * v + u;
                        sm[j] = row_valid ? fmaf(__uint_as_float(sraw[j]), a.scale_log2, -mm[u]) : -INFINITY;
                        need |= sm[j] > tt[u];
                    }
                }
            }
            if (named_bar_or(group_bar, 128, need)) {
                // Scores relative to the OLD reference are kept (not re-read from tensor memory, not held
                // as raw values): s - m_new = (s - m_old) + (m_old - m_new); for the row that sets the new
                // maximum the sum is zero to within 2^-17, far inside the bf16 quantum of P = 1.
                float (&s)[CW] = sm;
                float r[1];
                ColReduce<CW, 16, true>::run(s, lane, r);
                store_col_partial<CW>(red + q * NPAD + col0, r[0], lane);
                named_bar_sync(group_bar, 128);
                if (q == 0 && lane < CW) {
                    const int col = col0 + lane;
                    const float tmr = fmaxf(fmaxf(red[col], red[NPAD + col]), fmaxf(red[2 * NPAD + col], red[3 * NPAD + col]));
                    const float m_old = m_s[col];
                    const float tm = tmr + m_old;     // column maximum, back in absolute log2 units
                    // The first tile sets m outright (only the sink, if it counts here, holds it up);
                    // nothing has been accumulated yet, so there is nothing to rescale.
                    const bool sink_here = (sg[7] & kSegComplete) != 0 && a.sink != nullptr;
                    bool up = first_tile ? (!sink_here || tm > m_old) : tm > m_old + thr_s[col];
                    if (is_dense(FMT) && tm == -INFINITY) up = false;     // folded positions: no row of this tile is visible to the column
                    const float m_new = up ? tm + kRefHeadroom : m_old;
                    alpha_s[col] = (up && !first_tile) ? fast_exp2(m_old - m_new) : 1.0f;
                    shift_s[col] = m_old - m_new;
                    m_s[col] = m_new;
                    thr_s[col] = move_threshold(m_new);
                }
                named_bar_sync(group_bar, 128);
                lacc *= alpha_s[col0 + (lane >> kColShift)];
#pragma unroll
                for (int j = 0; j < CW; ++j) sm[j] += shift_s[col0 + j];
                // O^T[:, h] *= alpha[h]; the previous PV completed before this tile's S^T did.  Only the column
                // slices in which some head moved are touched (the same answer in all four warps of a slice).
                bool moved = false;
#pragma unroll
                for (int j = 0; j < CW; ++j) moved |= alpha_s[col0 + j] != 1.0f;
                if (!first_tile && moved) {
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
            {   // P^T = 2^(S^T - m) rounded to bf16, MN-major B-operand layout (8 heads = 16 bytes per row)
                uint32_t pk[CW / 2];
#pragma unroll
                for (int j = 0; j < CW; j += 2) {
                    pk[j / 2] = pack_bf16x2(fast_exp2(sm[j]), fast_exp2(sm[j + 1]));
                    // The denominator sums the ROUNDED probabilities, the ones PV multiplies: where one
                    // row dominates, out = P~ K / sum P~ then carries no rounding error of P at all,
                    // while P~ K / sum P is off by the rounding of P times |K| (0.4 for the x50 outlier
                    // rows of the int8 workloads, four times what the reference's kernels show).
                    sm[j] = __uint_as_float(pk[j / 2] << 16);
                    sm[j + 1] = __uint_as_float(pk[j / 2] & 0xFFFF0000u);
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
            fence_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + kBarP * 8);
            {   // denominators, after the hand-over: the tensor pipe is already at work on PV
                float r[1];
                ColReduce<CW, 16, false>::run(sm, lane, r);
                lacc += r[0];
            }
        }

        // ---- end of the segment; its epilogue is run inside the next segment's first tile
        if (!have_next) {
            epilogue(std::true_type{}, sg, nullptr, k & 1);
            break;
        }
    }
    if (a.fused_merge == 2) merge_head_slices<NPAD, is_dense(FMT)>(a, smem, tid, warp, lane);
}

// ------------------------------------------------------------------ the kernel
template <int FMT, int NPAD>
__global__ void __launch_bounds__(kThreads, 1) sparse_mla_fwd_kernel(const __grid_constant__ KernelArgs a) {
    extern __shared__ __align__(FMT == kFmtBf16DenseTma ? 1024 : 128) uint8_t smem[];
    using L = Smem<NPAD, is_dense(FMT)>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if constexpr (FMT == kFmtBf16DenseTma) {
        // the swizzled K slabs (written by TMA, read by the tensor pipe) need a 1024-byte aligned base
        if ((smem_u32(smem) & 1023u) != 0u) {
            if (tid == 0) atomicOr(&g_device_status, kStatusSmemLayout);
            return;
        }
    }

    // ---- this CTA's share of the work
    int *sched = reinterpret_cast<int *>(smem + L::kSched);
    if (a.balanced && !a.fused_merge && tid == 0) reinterpret_cast<int4 *>(a.desc)[blockIdx.x] = make_int4(-1, 0, 0, 0);
    if (tid == 0) sched[kSchedFin] = sched[kSchedFin + 5] = 0;
    if (a.sink != nullptr && tid * 32 < a.H) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.sink + tid * 32));
    {
        SegIter iter;
        long long W;
        int P;
        if (!make_schedule<is_dense(FMT)>(a, sched + kSchedScan, iter, W, P)) return;
        if (tid == 0) {
            store_iter(sched + kSchedIter, iter, W);
            sched[kSchedP] = P;
        }
    }
    __syncthreads();
    // ---- set-up, three things side by side: first segment record, barriers, tensor memory
    if (warp == 0) publish_segment<is_dense(FMT)>(a, sched, 0, lane);      // sets the published count to 1
    if (tid == 32) {
        const uint32_t bars = smem_u32(smem + L::kBars);
        for (int c = 0; c < 4; ++c) mbar_init(bars + (kBarReady + c) * 8, kWorkerWarps);
        for (int c = 0; c < 4; ++c) mbar_init(bars + (kBarFree + c) * 8, 1);
        mbar_init(bars + kBarS * 8, 1);
        mbar_init(bars + kBarP * 8, kWorkerWarps);
        mbar_init(bars + kBarO * 8, 1);
        mbar_init(bars + kBarOFree * 8, kWorkerWarps);
        mbar_init(bars + kBarQ * 8, a.q_tma ? 1 : kQLoadWarps);
        if constexpr (FMT == kFmtBf16DenseTma) {
            for (int c = 0; c < 4; ++c) mbar_init(bars + (kBarLand + c) * 8, 1);
            mbar_init(bars + kBarLandAlt * 8, 1);
        }
        *reinterpret_cast<volatile int *>(smem + L::kAbort) = 0;
        sched[kSchedTiles] = 0;
        mbar_init_fence();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem_u32(smem + L::kTmemPtr), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if ((sched[kSchedRec + 7] & kSegValid) == 0) {   // nothing but items without rows
        if (warp == kMmaWarp) tmem_dealloc(*reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr), kTmemCols);
        return;
    }

    // ---- reference max and Q tile of the first segment
    {
        const int *r0 = sched + kSchedRec;
        const int h0 = r0[1] * 64, hvalid = min(NPAD, a.H - h0);
        if (tid < NPAD) {
            const float m0 = initial_ref(a, (r0[7] & kSegComplete) != 0, h0, tid, hvalid);
            reinterpret_cast<float *>(smem + L::kM)[tid] = m0;
            reinterpret_cast<float *>(smem + L::kThr)[tid] = move_threshold(m0);
        }
    }
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(smem + L::kTmemPtr);

    if (warp < kWorkerWarps) {
        worker_role<FMT, NPAD>(a, smem, tmem_base, warp, lane);
    } else if (warp == kMmaWarp) {
        mma_role<NPAD, is_dense(FMT), FMT == kFmtBf16DenseTma>(smem, tmem_base);
    } else if (a.q_tma) {
        // one tensor copy per item needs one thread; the next warp publishes the schedule
        if (warp == kMmaWarp + 1) qload_role<NPAD, is_dense(FMT), FMT == kFmtBf16DenseTma>(a, smem, 0, lane);
        if (warp == kMmaWarp + 2) scheduler_role<NPAD, is_dense(FMT)>(a, smem, lane);
        if constexpr (FMT == kFmtBf16DenseTma) {
            if (warp == kMmaWarp + 3) kload_role<NPAD>(a, smem, lane);
        }
    } else {
        // cp.async fallback for Q: two loader warps, one scheduler warp
        if (warp == kMmaWarp + 2) scheduler_role<NPAD, is_dense(FMT)>(a, smem, lane);
        else qload_role<NPAD, is_dense(FMT)>(a, smem, warp == kMmaWarp + 1 ? 0 : 1, lane);
    }

    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------ merge of partial segments
// Block (c, y): if CTA c of the attention kernel left a descriptor {item, S, first slot, heads}, the
// item's S partial segments sit in slots {first slot, 2(c+1), 2(c+2), ...}.  One warp per head:
//   out = sum_s 2^(m_s - M) O_s / (sum_s 2^(m_s - M) l_s + 2^(sink - M)),  M = max(m_s, sink).
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const float *__restrict__ part_o,
                                                                 const float *__restrict__ part_ml,
                                                                 const int4 *__restrict__ desc,
                                                                 const float *__restrict__ sink,
                                                                 __nv_bfloat16 *__restrict__ out, long long o_ts,
                                                                 long long o_hs, int head_blocks, int npad,
                                                                 float *__restrict__ lse, int num_heads, int dense_sq, int fold_sq, int fold_h) {
    const int lane = threadIdx.x & 31;
    const int c = blockIdx.x;
    const int4 d = desc[c];
    const int hl = blockIdx.y * 4 + (threadIdx.x >> 5);
    if (d.x < 0 || hl >= d.w) return;
    const int t = d.x / head_blocks, h = (d.x - t * head_blocks) * 64 + hl;
    auto slot_of = [&](int k) { return k == 0 ? d.z : 2 * (c + k); };
    float *lse_dst = nullptr;
    if (lse != nullptr) {      // as lse_ptr()
        if (fold_sq > 1) {
            const int i = h / fold_h;
            lse_dst = lse + (static_cast<long long>(t) * fold_h + (h - i * fold_h)) * fold_sq + i;
        } else {
            const int b = t / dense_sq, i = t - b * dense_sq;
            lse_dst = lse + (static_cast<long long>(b) * num_heads + h) * dense_sq + i;
        }
    }
    merge_head(part_o, part_ml, slot_of, d.y, npad, hl, sink ? sink[h] * kLog2e : -INFINITY,
               out + static_cast<long long>(t) * o_ts + static_cast<long long>(h) * o_hs, lane, lse_dst);
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
    d.block_shift = (s.block_size & (s.block_size - 1)) ? -1 : __builtin_ctz(static_cast<unsigned>(s.block_size));
    const uintptr_t base = reinterpret_cast<uintptr_t>(s.cache);
    if (fmt == SMLA_FP8_DS_MLA) {
        if ((base & 7u) || (s.block_stride & 7)) return SMLA_EALIGN;
        d.vec = ((base & 31u) == 0 && (s.block_stride & 31) == 0) ? 2 : ((base & 15u) == 0 && (s.block_stride & 15) == 0) ? 1 : 0;
    } else {
        if (!s.scale) return SMLA_EINVAL;
        if ((base & 3u) || (s.block_stride & 3) || (s.pos_stride & 3)) return SMLA_EALIGN;
        // 2: every row starts on a 16-byte boundary inside 32-byte aligned blocks and is followed by at
        // least 16 readable bytes of its own token (528-byte tokens, or 512-byte rows that are 32-byte
        // aligned): the wide gather (kFmtInt8Wide) applies.
        const bool wide = (base & 31u) == 0 && (s.block_stride & 31) == 0 && (s.pos_stride & 15) == 0 &&
                          ((s.pos_stride & 31) == 0 || s.pos_stride >= 528);
        d.vec = wide ? 2 : ((base & 15u) == 0 && (s.block_stride & 15) == 0 && (s.pos_stride & 15) == 0) ? 1 : 0;
    }
    return SMLA_OK;
}

template <int FMT, int NPAD>
int launch_fwd(const KernelArgs &a, unsigned grid, cudaStream_t stream) {
    constexpr int smem_bytes = FMT == kFmtBf16DenseTma ? Smem<NPAD, true>::kTotalTma : Smem<NPAD, is_dense(FMT)>::kTotal;
    // The opt-in to 227 KB of dynamic shared memory is per device and per kernel instance; hosts that
    // run one thread per GPU come through here concurrently, hence atomics (setting it twice is harmless).
    static std::atomic<bool> attr_done[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    const bool tracked = dev >= 0 && dev < 64;
    if (!tracked || !attr_done[dev].load(std::memory_order_acquire)) {
        e = cudaFuncSetAttribute(sparse_mla_fwd_kernel<FMT, NPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem_bytes);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (tracked) attr_done[dev].store(true, std::memory_order_release);
    }
    sparse_mla_fwd_kernel<FMT, NPAD><<<grid, kThreads, smem_bytes, stream>>>(a);
    return static_cast<int>(cudaGetLastError());
}

template <int FMT>
int launch_fwd_npad(int npad, const KernelArgs &a, unsigned grid, cudaStream_t stream) {
    switch (npad) {
        case 16: return launch_fwd<FMT, 16>(a, grid, stream);
        case 32: return launch_fwd<FMT, 32>(a, grid, stream);
        default: return launch_fwd<FMT, 64>(a, grid, stream);
    }
}

// cuTensorMapEncodeTiled, fetched through the runtime so that libcuda need not be linked.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 5-D view of q [T, H, 512] whose box {8, 8, 64, npad/8, 1} is the Q operand's shared-memory layout.
// False (the kernel then uses cp.async) when H is not a multiple of 8 or the driver refuses the map.
bool make_q_tensor_map(const KernelArgs &a, int npad, int dim_groups, int box_dim_groups, CUtensorMap *map) {
    if (a.H % 8 != 0) return false;
    EncodeTiledFn enc = tensor_map_encoder();
    if (enc == nullptr) return false;
    const cuuint64_t dims[5] = {8, 8, static_cast<cuuint64_t>(dim_groups), static_cast<cuuint64_t>(a.H / 8), static_cast<cuuint64_t>(a.T)};
    const cuuint64_t strides[4] = {static_cast<cuuint64_t>(a.q_hs) * 2, 16, static_cast<cuuint64_t>(a.q_hs) * 16,
                                   static_cast<cuuint64_t>(a.q_ts) * 2};
    const cuuint32_t box[5] = {8, 8, static_cast<cuuint32_t>(box_dim_groups), static_cast<cuuint32_t>(npad / 8), 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<__nv_bfloat16 *>(a.q), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Dense paged MLA with K by TMA: q [T, H, 576] as a 3-D tensor {dims, heads, tokens}.  A box {64 dims, npad heads,
// 1 token} with the 128-byte swizzle is one slab of the Q operand's shared-memory layout in that format.
bool make_q_tensor_map_slabs(const KernelArgs &a, int npad, CUtensorMap *map) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.dense_dims), static_cast<cuuint64_t>(a.H), static_cast<cuuint64_t>(a.T)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.q_hs) * 2, static_cast<cuuint64_t>(a.q_ts) * 2};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(npad), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16 *>(a.q), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Dense paged MLA: the bf16 cache as a 3-D tensor {576 dims, rows of a page, pages}; a box {64 dims, R rows, 1 page}
// with the 128-byte swizzle is R rows of one slab of the K tile.
bool make_k_tensor_map(const KernelArgs &a, int num_blocks, int box_rows, CUtensorMap *map) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (enc == nullptr || num_blocks <= 0) return false;
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(a.dense_dims), static_cast<cuuint64_t>(a.swa.block_size), static_cast<cuuint64_t>(num_blocks)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(a.swa.pos_stride), static_cast<cuuint64_t>(a.swa.block_stride)};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<uint8_t *>(a.swa.cache), dims, strides, box,
                           estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// 64-bit value that no earlier launch of this process has used and that memory left over from
// anything else will not hold: a random start, then steps of an odd constant.
unsigned long long next_launch_tag() {
    static std::atomic<unsigned long long> seq{[] {
        std::random_device rd;
        return (static_cast<unsigned long long>(rd()) << 32) ^ rd() ^ 0x5851F42D4C957F2Dull;
    }()};
    return seq.fetch_add(0x9E3779B97F4A7C15ull) | 1ull;
}

int sm_count_of_current_device(int &count) {
    static std::atomic<int> cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && (count = cached[dev].load(std::memory_order_relaxed)) > 0) return 0;
    e = cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (tracked) cached[dev].store(count, std::memory_order_relaxed);
    return 0;
}

}  // namespace

namespace {
// The part every attention entry point shares: pick the schedule (balanced tiles with as many CTAs as the
// SM count and the workspace allow, else whole items), the merge form, the Q tensor map, and launch.
int schedule_and_launch(KernelArgs &a, int fmt, int num_splits, void *workspace, size_t workspace_capacity,
                        cudaStream_t stream) {
    const int npad = head_pad(a.H);
    a.head_blocks = (a.H + 63) / 64;
    const long long items = static_cast<long long>(a.T) * a.head_blocks;
    if (items > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    // Dense rows come from HBM (no reuse between tokens).  With several head blocks the items are ordered
    // head block first: CTA c and CTA c + P / blocks then walk the same rows at the same time, one head block
    // each, and the second reader finds them in L2 (token first, the blocks of a sequence ran one after
    // the other in one CTA and read its rows from HBM once per block).
    a.hb_major = (is_dense(fmt) && a.head_blocks > 1) ? 1 : 0;
    int sms = 0;
    int rc = sm_count_of_current_device(sms);
    if (rc != 0) return rc;

    long long ctas = 0;
    if (num_splits > 1) {
        if (!workspace) return SMLA_EWORKSPACE;
        if (reinterpret_cast<uintptr_t>(workspace) & 15u) return SMLA_EALIGN;
        const size_t want = smla_attn_workspace_bytes(a.T, a.H, num_splits);
        ctas = balanced_ctas(sms, npad, static_cast<long long>(std::min(want, workspace_capacity)));
    }
    if (ctas >= 2) {
        a.balanced = 1;
        a.part_o = static_cast<float *>(workspace);
        a.part_ml = a.part_o + static_cast<size_t>(2 * ctas) * npad * kD;
        a.desc = reinterpret_cast<int *>(a.part_ml + static_cast<size_t>(2 * ctas) * npad * 2);      // 16 B per CTA
        a.flags = reinterpret_cast<unsigned long long *>(a.desc + 4 * ctas);                         // 16 B per CTA
        a.fused_merge = merge_mode_policy(items, ctas);
        if (a.fused_merge == 2) {
            // The slice merge relies on the tag being new for every execution; a graph replays the same
            // arguments, so a capturing stream gets the combine kernel instead.
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) a.fused_merge = 0;
        }
        a.tag = next_launch_tag();
    } else {
        a.balanced = 0;
        ctas = std::min<long long>(items, sms);
    }
    if (fmt == kFmtBf16DenseTma) {
        a.q_tma = make_q_tensor_map_slabs(a, npad, &a.q_map) ? 1 : 0;
        if (!a.q_tma) fmt = kFmtBf16Dense;      // the K loader is the warp the Q fallback needs
    }
    if (fmt != kFmtBf16DenseTma)
        a.q_tma = make_q_tensor_map(a, npad, is_dense(fmt) ? a.dense_dims / 8 : 64, is_dense(fmt) ? 72 : 64, &a.q_map) ? 1 : 0;
    const unsigned grid = static_cast<unsigned>(ctas);
    const bool int8_wide = fmt == SMLA_INT8_DS_MLA && a.swa.vec == 2 && (a.extra.cache == nullptr || a.extra.vec == 2);
    rc = (fmt == kFmtBf16DenseTma)   ? launch_fwd_npad<kFmtBf16DenseTma>(npad, a, grid, stream)
         : (fmt == kFmtBf16Dense)   ? launch_fwd_npad<kFmtBf16Dense>(npad, a, grid, stream)
         : (fmt == SMLA_FP8_DS_MLA) ? launch_fwd_npad<SMLA_FP8_DS_MLA>(npad, a, grid, stream)
         : int8_wide                ? launch_fwd_npad<kFmtInt8Wide>(npad, a, grid, stream)
                                    : launch_fwd_npad<SMLA_INT8_DS_MLA>(npad, a, grid, stream);
    if (rc != 0) return rc;
    if (a.balanced && !a.fused_merge) {
        sparse_mla_combine_kernel<<<dim3(grid, static_cast<unsigned>((npad + 3) / 4)), 128, 0, stream>>>(
            a.part_o, a.part_ml, reinterpret_cast<const int4 *>(a.desc), a.sink, a.out, a.o_ts, a.o_hs, a.head_blocks,
            npad, a.lse, a.H, a.dense_sq, a.fold_sq, a.fold_h);
        rc = static_cast<int>(cudaGetLastError());
    }
    return rc;
}

}  // namespace

// `num_splits` > 1 with a workspace of smla_attn_workspace_bytes(T, H, num_splits) bytes selects the
// balanced-tiles schedule with as many CTAs as the SM count and the workspace (two partial slots per
// CTA plus one 16-byte descriptor) allow; otherwise whole items are dealt out to the CTAs.
int launch_sparse_mla_attention(const smla_attn_params_t &p, int num_splits, void *workspace, size_t workspace_capacity,
                                cudaStream_t stream) {
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
    return schedule_and_launch(a, p.cache_format, num_splits, workspace, workspace_capacity, stream);
}

// Dense paged MLA decode: every query position of every sequence is an item list entry ("token"), its rows
// are the sequence's first n rows found through the block table; the same persistent kernel, schedules
// and merges as the sparse path, with bf16 rows copied (not converted) into the K buffer.
int launch_dense_mla_attention(const smla_dense_params_t &p, cudaStream_t stream) {
    if (p.batch <= 0 || p.seqlen_q <= 0 || p.num_heads <= 0 || !p.q || !p.out || !p.k_cache || !p.block_table ||
        !p.cache_seqlens || p.page_block_size <= 0 || p.num_blocks < 0)
        return SMLA_EINVAL;
    const long long tokens = static_cast<long long>(p.batch) * p.seqlen_q;
    if (tokens > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    if ((reinterpret_cast<uintptr_t>(p.q) & 15u) || (p.q_token_stride & 7) || (p.q_head_stride & 7) ||
        (reinterpret_cast<uintptr_t>(p.out) & 15u) || (p.out_token_stride & 7) || (p.out_head_stride & 7) ||
        (reinterpret_cast<uintptr_t>(p.k_cache) & 15u) || (p.k_block_stride & 15) || (p.k_row_stride & 15) ||
        p.k_row_stride < (p.head_dim == 512 ? 1024 : kDenseRowBytes))
        return SMLA_EALIGN;
    if (p.head_dim != 0 && p.head_dim != 576 && p.head_dim != 512) return SMLA_EINVAL;
    KernelArgs a = {};
    a.q = static_cast<const __nv_bfloat16 *>(p.q);
    a.q_ts = p.q_token_stride;
    a.q_hs = p.q_head_stride;
    a.out = static_cast<__nv_bfloat16 *>(p.out);
    a.o_ts = p.out_token_stride;
    a.o_hs = p.out_head_stride;
    a.sink = nullptr;
    a.T = static_cast<int>(tokens);
    a.H = p.num_heads;
    a.scale_log2 = p.softmax_scale * kLog2e;
    a.lse = p.softmax_lse;
    a.dense_sq = p.seqlen_q;
    a.dense_dims = p.head_dim == 512 ? 512 : 576;
    a.causal = (p.causal && p.seqlen_q > 1) ? 1 : 0;
    a.swa.cache = static_cast<const uint8_t *>(p.k_cache);
    a.swa.indices = p.block_table;
    a.swa.lens = p.cache_seqlens;
    a.swa.idx_stride = p.block_table_stride;
    a.swa.block_stride = p.k_block_stride;
    a.swa.pos_stride = p.k_row_stride;
    a.swa.topk = static_cast<int>(std::min<long long>(static_cast<long long>(p.max_blocks_per_seq) * p.page_block_size, 0x7FFFFFFFLL));
    const long long slots = static_cast<long long>(p.num_blocks) * p.page_block_size;
    if (slots > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    a.swa.num_slots = static_cast<int>(slots);
    a.swa.block_size = p.page_block_size;
    a.swa.block_shift = (p.page_block_size & (p.page_block_size - 1)) ? -1 : __builtin_ctz(static_cast<unsigned>(p.page_block_size));
    a.swa.vec = 1;
    // Few heads and several query positions: fold the positions into the head dimension (one pass over the rows)
    const long long folded_heads = static_cast<long long>(p.seqlen_q) * p.num_heads;
    if (p.seqlen_q > 1 && folded_heads <= 64 && p.num_heads % (head_pad(static_cast<int>(folded_heads)) / 4) == 0 &&
        p.q_token_stride == p.num_heads * p.q_head_stride && p.out_token_stride == p.num_heads * p.out_head_stride) {
        a.T = p.batch;
        a.H = static_cast<int>(folded_heads);
        a.q_ts = p.q_token_stride * p.seqlen_q;
        a.o_ts = p.out_token_stride * p.seqlen_q;
        a.fold_sq = p.seqlen_q;
        a.fold_h = p.num_heads;
        a.fold_causal = a.causal;
        a.dense_sq = 1;
        a.causal = 0;
    }
    // K by TMA when a 128-row tile is a whole number of pages or a page a whole number of tiles
    int fmt = kFmtBf16Dense;
    const int page = p.page_block_size;
    if (page % 8 == 0 && (page >= 128 ? page % 128 == 0 : 128 % page == 0)) {
        const int box_rows = std::min(page, 128);
        if (make_k_tensor_map(a, p.num_blocks, box_rows, &a.k_map)) {
            a.k_box_rows = box_rows;
            fmt = kFmtBf16DenseTma;
        }
    }
    return schedule_and_launch(a, fmt, p.num_splits, p.workspace, p.workspace_bytes, stream);
}

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

// Device address of the status word on the CURRENT device (no synchronisation).
int device_status_address(int **addr_out) {
    void *ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_device_status);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (addr_out) *addr_out = static_cast<int *>(ptr);
    return SMLA_OK;
}

}  // namespace smla
