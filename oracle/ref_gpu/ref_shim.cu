// Test infrastructure, not product: a C entry point around the REFERENCE's own CUDA launchers
// (run_sparse_mla_decode / run_sparse_mla_prefill, csrc/flash_mla.h:125,159-160), so that the
// reference's mma.sync kernels -- compiled for sm_100 from the sources where they lie in the
// reference checkout, never copied -- can be run on the same B200 as a second oracle and as the GPU
// baseline.  It fills the reference's parameter structs the way its binding does
// (csrc/flash_api.cpp:352-405, 458-508, 558-585, 631-672); scratch buffers are passed in by the caller.
#include <cuda_runtime.h>
#include <cstdint>

#include "flash_mla.h"          // the reference's header, found through -I <reference>/csrc
#include "sparse_mla_b200.h"    // only for the plain-C description of the inputs

namespace {
constexpr double kLog2e = 1.4426950408889634;
}

extern "C" __attribute__((visibility("default")))
int ref_sparse_mla_decode(const smla_attn_params_t *s, int num_splits, void *oaccum, float *mlse, int *counter,
                          void *sel_kv, void *stream) {
    Sparse_mla_decode_params p = {};
    const bool int8 = s->cache_format == SMLA_INT8_DS_MLA;
    p.num_tokens = s->num_tokens;
    p.num_heads = s->num_heads;
    p.block_size = s->swa.block_size;
    p.scale_log2 = static_cast<float>(s->softmax_scale * kLog2e);
    p.q_ptr = s->q;
    p.q_token_stride = s->q_token_stride;
    p.q_head_stride = s->q_head_stride;
    p.o_ptr = s->out;
    p.out_token_stride = s->out_token_stride;
    p.out_head_stride = s->out_head_stride;
    p.attn_sink_ptr = s->attn_sink;
    p.swa_cache_ptr = s->swa.cache;
    p.swa_block_stride = s->swa.block_stride;
    p.swa_indices_ptr = s->swa.indices;
    p.swa_lens_ptr = s->swa.lens;
    p.swa_topk = s->swa.topk;
    p.swa_num_blocks = s->swa.num_blocks;
    if (int8) {
        p.swa_scale_ptr = s->swa.scale;
        p.swa_pos_stride = s->swa.pos_stride;
        p.swa_scale_block_stride = s->swa.scale_block_stride;
        p.swa_scale_pos_stride = s->swa.scale_pos_stride;
    }
    if (s->extra.cache) {
        p.extra_cache_ptr = s->extra.cache;
        p.extra_block_stride = s->extra.block_stride;
        p.extra_indices_ptr = s->extra.indices;
        p.extra_lens_ptr = s->extra.lens;
        p.extra_topk = s->extra.topk;
        p.extra_num_blocks = s->extra.num_blocks;
        p.extra_block_size = s->extra.block_size;
        if (int8) {
            p.extra_scale_ptr = s->extra.scale;
            p.extra_pos_stride = s->extra.pos_stride;
            p.extra_scale_block_stride = s->extra.scale_block_stride;
            p.extra_scale_pos_stride = s->extra.scale_pos_stride;
        }
    }
    p.int8_cache = int8;
    p.num_splits = num_splits;
    p.oaccum_ptr = oaccum;
    p.mlse_ptr = mlse;
    p.combine_counter_ptr = counter;
    p.sel_kv_ptr = sel_kv;
    p.sel_width = s->swa.topk + (s->extra.cache ? s->extra.topk : 0);
    run_sparse_mla_decode(p, static_cast<cudaStream_t>(stream));
    return static_cast<int>(cudaGetLastError());
}

extern "C" __attribute__((visibility("default")))
int ref_sparse_mla_prefill(const smla_attn_params_t *s, void *kv_whole_cache_bf16, void *stream) {
    Sparse_mla_prefill_params p = {};
    const bool int8 = s->cache_format == SMLA_INT8_DS_MLA;
    p.num_tokens = s->num_tokens;
    p.num_heads = s->num_heads;
    p.swa_topk = s->swa.topk;
    p.extra_topk = s->extra.cache ? s->extra.topk : 0;
    p.width = p.swa_topk + p.extra_topk;
    p.swa_num_blocks = s->swa.num_blocks;
    p.swa_block_size = s->swa.block_size;
    p.scale_log2 = static_cast<float>(s->softmax_scale * kLog2e);
    p.q_ptr = s->q;
    p.q_token_stride = s->q_token_stride;
    p.q_head_stride = s->q_head_stride;
    p.o_ptr = s->out;
    p.out_token_stride = s->out_token_stride;
    p.out_head_stride = s->out_head_stride;
    p.kv_ptr = int8 ? nullptr : kv_whole_cache_bf16;
    p.attn_sink_ptr = s->attn_sink;
    p.swa_cache_ptr = s->swa.cache;
    p.swa_block_stride = s->swa.block_stride;
    p.swa_indices_ptr = s->swa.indices;
    p.swa_lens_ptr = s->swa.lens;
    if (int8) {
        p.swa_scale_ptr = s->swa.scale;
        p.swa_pos_stride = s->swa.pos_stride;
        p.swa_scale_block_stride = s->swa.scale_block_stride;
        p.swa_scale_pos_stride = s->swa.scale_pos_stride;
    }
    if (s->extra.cache) {
        p.extra_cache_ptr = s->extra.cache;
        p.extra_block_stride = s->extra.block_stride;
        p.extra_indices_ptr = s->extra.indices;
        p.extra_lens_ptr = s->extra.lens;
        p.extra_num_blocks = s->extra.num_blocks;
        p.extra_block_size = s->extra.block_size;
        if (int8) {
            p.extra_scale_ptr = s->extra.scale;
            p.extra_pos_stride = s->extra.pos_stride;
            p.extra_scale_block_stride = s->extra.scale_block_stride;
            p.extra_scale_pos_stride = s->extra.scale_pos_stride;
        }
    }
    p.int8_cache = int8;
    run_sparse_mla_prefill(p, static_cast<cudaStream_t>(stream));
    return static_cast<int>(cudaGetLastError());
}
