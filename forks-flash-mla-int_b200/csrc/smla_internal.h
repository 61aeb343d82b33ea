// Internal declarations shared by the translation units of the sparse-MLA library.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>

#include "sparse_mla_b200.h"

namespace smla {

// Bits of the per-device error word the kernels set when a bounded wait runs out.
enum DeviceStatusBits : int {
    kStatusGatherWait = 1,   // a gather warp gave up waiting for a free K chunk
    kStatusMmaWait = 2,      // the MMA issuer gave up waiting for a filled K chunk
    kStatusSoftmaxWait = 4,  // a softmax warp gave up waiting for the score tile
    kStatusEpilogueWait = 8, // the epilogue gave up waiting for the last PV
    kStatusSmemLayout = 16,  // the dynamic shared memory did not start on a 1024-byte boundary (nothing was computed)
};

int launch_quantize_int8_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, int8_t *q,
                              float *scale, cudaStream_t stream);

int launch_write_int8_ds_mla(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, const void *slots,
                             int slots_i64, void *cache, int64_t num_blocks, int block_size, int64_t block_stride,
                             int64_t pos_stride, int scale_rule, cudaStream_t stream);
int launch_write_fp8_ds_mla(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, const void *slots,
                            int slots_i64, void *cache, int64_t num_blocks, int block_size, int64_t block_stride,
                            cudaStream_t stream);

// `num_splits` as resolved by the caller (1 = whole items, prefill).  `workspace_capacity` = bytes that may
// be used at `workspace`: the balanced schedule gets as many CTAs as fit into the smaller of that and
// smla_attn_workspace_bytes(T, H, num_splits).
int launch_sparse_mla_attention(const smla_attn_params_t &p, int num_splits, void *workspace, size_t workspace_capacity,
                                cudaStream_t stream);
int launch_dense_mla_attention(const smla_dense_params_t &p, cudaStream_t stream);

int read_and_clear_device_status(int *status_out);
int device_status_address(int **addr_out);

// CTAs of the balanced schedule for a workspace of `workspace_bytes` (two partial slots of `npad` heads
// per CTA, 64 bytes of flags and descriptors per SM); fewer than 2 means whole items are dealt out.
inline long long balanced_ctas(int sm_count, int npad, long long workspace_bytes) {
    const long long slot_bytes = static_cast<long long>(npad) * (SMLA_HEAD_DIM + 2) * 4;
    const long long n = (workspace_bytes - 64ll * sm_count) / slot_bytes / 2;
    return n < sm_count ? n : sm_count;
}
// How the partial segments of the balanced schedule are merged (measured on B200, int8, 64 heads):
//   1  at least half as many items as CTAs (an item is cut in two or three): the CTA that holds the
//      item's first tiles merges the rest in its own epilogue (T=128: 91 us against 98 us);
//   2  sixteen or more CTAs per item (T <= 8): every CTA of the item merges a slice of its heads at the
//      end of its run (T=1: 25 against 27 us, T=8: 27 against 30 us);
//   0  in between: a second kernel, one warp per head on all SMs (T=16..64: equal or 1-4 % better).
inline int merge_mode_policy(long long items, long long ctas) {
    if (items * 2 >= ctas) return 1;
    if (items * 16 <= ctas) return 2;
    return 0;
}
inline int head_pad(int num_heads) { return num_heads <= 16 ? 16 : (num_heads <= 32 ? 32 : 64); }

}  // namespace smla
