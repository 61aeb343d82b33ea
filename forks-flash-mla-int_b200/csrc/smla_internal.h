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
};

int launch_quantize_int8_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, int8_t *q,
                              float *scale, cudaStream_t stream);

// `force_single` = never split (prefill).  `split_ws`/`num_splits` as resolved by the caller.
int launch_sparse_mla_attention(const smla_attn_params_t &p, int num_splits, void *workspace, cudaStream_t stream);

int read_and_clear_device_status(int *status_out);

}  // namespace smla
