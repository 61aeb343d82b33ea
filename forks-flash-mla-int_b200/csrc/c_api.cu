// extern "C" entry points of the sparse-MLA library (declared in include/sparse_mla_b200.h).
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "smla_internal.h"

namespace {

struct DevInfo {
    int major = 0, sm_count = 0;
};
// Per-device facts, looked up once.  Hosts that run one thread per GPU call in concurrently: the two
// words are published with an atomic flag (two threads that both miss simply look the same values up).
std::atomic<int> g_dev_known[64];
int g_dev_major[64], g_dev_sms[64];

int device_info(DevInfo &out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    const bool tracked = dev >= 0 && dev < 64;
    if (tracked && g_dev_known[dev].load(std::memory_order_acquire)) {
        out.major = g_dev_major[dev];
        out.sm_count = g_dev_sms[dev];
        return SMLA_OK;
    }
    e = cudaDeviceGetAttribute(&out.major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaDeviceGetAttribute(&out.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (tracked) {
        g_dev_major[dev] = out.major;
        g_dev_sms[dev] = out.sm_count;
        g_dev_known[dev].store(1, std::memory_order_release);
    }
    return SMLA_OK;
}

int max_width(const smla_attn_params_t &p) { return p.swa.topk + (p.extra.cache ? p.extra.topk : 0); }

}  // namespace

extern "C" {

const char *smla_version(void) { return "sparse_mla_b200 0.1 (sm_100a)"; }

const char *smla_error_string(int code) {
    switch (code) {
        case SMLA_OK: return "ok";
        case SMLA_EINVAL: return "invalid argument (null pointer, bad size or unknown enum)";
        case SMLA_EALIGN: return "unsupported pointer or stride alignment";
        case SMLA_EWORKSPACE: return "split-KV workspace missing or too small";
        case SMLA_EARCH: return "the current device is not compute capability 10.x (B200 / sm_100a)";
        case SMLA_ETOOBIG: return "request exceeds a fixed capacity of this entry point";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}

int smla_choose_num_splits(int sm_count, int num_tokens, int num_heads, int max_width_rows) {
    // The attention kernel is persistent.  With plenty of items (token x block of 64 heads) per SM,
    // whole items dealt out to the CTAs keep every SM busy and nothing needs merging: 1.  Otherwise
    // the tiles of all items are cut into equal ranges, one per CTA; each CTA may then leave two
    // partial segments in scratch.  The value returned sizes that scratch through
    // smla_attn_workspace_bytes(): room for two partial slots per CTA plus the merge descriptors.
    int rows_per_cta = 128;      // a CTA never gets less than this many rows (one 128-row tile)
    if (const char *e = getenv("FLASH_MLA_SLOTS_PER_SPLIT")) {
        const int v = atoi(e);
        if (v > 0) rows_per_cta = ((v + 127) / 128) * 128;
    }
    const int head_blocks = (num_heads + 63) / 64;
    const long long items = static_cast<long long>(std::max(num_tokens, 1)) * head_blocks;
    if (sm_count <= 1 || items >= 4ll * sm_count) return 1;
    const long long pieces = items * std::max(1, (max_width_rows + rows_per_cta - 1) / rows_per_cta);
    const long long ctas = std::min<long long>(sm_count, pieces);
    if (ctas <= 1) return 1;
    const int npad = num_heads <= 16 ? 16 : (num_heads <= 32 ? 32 : 64);
    const long long head_rows = static_cast<long long>(std::max(num_tokens, 1)) * num_heads;
    const long long need = (2 * ctas + 1) * npad;       // head rows of scratch; the extra slot covers the descriptors
    return static_cast<int>(std::max<long long>(2, (need + head_rows - 1) / head_rows));
}

size_t smla_attn_workspace_bytes(int num_tokens, int num_heads, int num_splits) {
    if (num_splits <= 1 || num_tokens <= 0 || num_heads <= 0) return 0;
    return static_cast<size_t>(num_tokens) * num_heads * num_splits * (SMLA_HEAD_DIM + 2) * sizeof(float);
}

int smla_decode_kernel_launches(int sm_count, int num_tokens, int num_heads, int num_splits) {
    if (num_splits <= 1 || num_tokens <= 0 || num_heads <= 0) return 1;
    const long long ctas = smla::balanced_ctas(sm_count, smla::head_pad(num_heads),
                                               static_cast<long long>(smla_attn_workspace_bytes(num_tokens, num_heads, num_splits)));
    if (ctas < 2) return 1;
    const long long items = static_cast<long long>(num_tokens) * ((num_heads + 63) / 64);
    return smla::merge_mode_policy(items, ctas) == 0 ? 2 : 1;
}

int smla_decode_kernel_launches_captured(int sm_count, int num_tokens, int num_heads, int num_splits) {
    if (num_splits <= 1 || num_tokens <= 0 || num_heads <= 0) return 1;
    const long long ctas = smla::balanced_ctas(sm_count, smla::head_pad(num_heads),
                                               static_cast<long long>(smla_attn_workspace_bytes(num_tokens, num_heads, num_splits)));
    if (ctas < 2) return 1;
    const long long items = static_cast<long long>(num_tokens) * ((num_heads + 63) / 64);
    return smla::merge_mode_policy(items, ctas) == 1 ? 1 : 2;     // the slice merge is not used on a capturing stream
}

int smla_decode_plan(int num_tokens, int num_heads, int max_width_rows, int *num_splits, size_t *workspace_bytes) {
    DevInfo d;
    const int rc = device_info(d);
    if (rc != SMLA_OK) return rc;
    if (d.major != 10) return SMLA_EARCH;
    const int s = smla_choose_num_splits(d.sm_count, num_tokens, num_heads, max_width_rows);
    if (num_splits) *num_splits = s;
    if (workspace_bytes) *workspace_bytes = smla_attn_workspace_bytes(num_tokens, num_heads, s);
    return SMLA_OK;
}

int smla_sparse_mla_decode(const smla_attn_params_t *p, void *stream) {
    if (!p) return SMLA_EINVAL;
    DevInfo d;
    int rc = device_info(d);
    if (rc != SMLA_OK) return rc;
    if (d.major != 10) return SMLA_EARCH;
    int splits = p->num_splits;
    if (splits < 0) return SMLA_EINVAL;
    if (splits == 0) {
        splits = smla_choose_num_splits(d.sm_count, p->num_tokens, p->num_heads, max_width(*p));
        // Without scratch the automatic policy degrades to one split instead of failing.
        if (splits > 1 && (!p->workspace ||
                           p->workspace_bytes < smla_attn_workspace_bytes(p->num_tokens, p->num_heads, splits)))
            splits = 1;
    } else if (splits > 1) {
        if (!p->workspace || p->workspace_bytes < smla_attn_workspace_bytes(p->num_tokens, p->num_heads, splits))
            return SMLA_EWORKSPACE;
    }
    return smla::launch_sparse_mla_attention(*p, splits, p->workspace, p->workspace_bytes, static_cast<cudaStream_t>(stream));
}

int smla_dense_mla_decode(const smla_dense_params_t *p, void *stream) {
    if (!p) return SMLA_EINVAL;
    DevInfo d;
    int rc = device_info(d);
    if (rc != SMLA_OK) return rc;
    if (d.major != 10) return SMLA_EARCH;
    if (p->batch <= 0 || p->seqlen_q <= 0 || p->num_heads <= 0 || p->page_block_size <= 0 || p->block_table_stride < 0 ||
        p->max_blocks_per_seq < 0 || p->max_blocks_per_seq > p->block_table_stride)
        return SMLA_EINVAL;
    const long long tokens_ll = static_cast<long long>(p->batch) * p->seqlen_q;
    if (tokens_ll > 0x7FFFFFFFLL) return SMLA_ETOOBIG;
    const int tokens = static_cast<int>(tokens_ll);
    smla_dense_params_t q = *p;
    if (q.num_splits < 0) return SMLA_EINVAL;
    if (q.num_splits == 0) {
        // The sequences' lengths live on the device: the policy sees the longest a block table row allows.
        const long long width = std::min<long long>(static_cast<long long>(p->max_blocks_per_seq) * p->page_block_size, 0x7FFFFFFFLL);
        q.num_splits = smla_choose_num_splits(d.sm_count, tokens, p->num_heads, static_cast<int>(width));
        if (q.num_splits > 1 && (!p->workspace || p->workspace_bytes < smla_attn_workspace_bytes(tokens, p->num_heads, q.num_splits)))
            q.num_splits = 1;
    } else if (q.num_splits > 1) {
        if (!p->workspace || p->workspace_bytes < smla_attn_workspace_bytes(tokens, p->num_heads, q.num_splits))
            return SMLA_EWORKSPACE;
    }
    return smla::launch_dense_mla_attention(q, static_cast<cudaStream_t>(stream));
}

int smla_sparse_mla_prefill(const smla_attn_params_t *p, void *stream) {
    if (!p) return SMLA_EINVAL;
    DevInfo d;
    int rc = device_info(d);
    if (rc != SMLA_OK) return rc;
    if (d.major != 10) return SMLA_EARCH;
    if (max_width(*p) <= 0) return SMLA_EINVAL;   // "prefill requires at least one selected slot"
    return smla::launch_sparse_mla_attention(*p, 1, nullptr, 0, static_cast<cudaStream_t>(stream));
}

int smla_quantize_int8_ds_mla_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride, int8_t *q,
                                   float *scale, void *stream) {
    return smla::launch_quantize_int8_rows(x, x_dtype, rows, x_row_stride, q, scale,
                                           static_cast<cudaStream_t>(stream));
}

int smla_write_int8_ds_mla_cache(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride,
                                 const void *slot_mapping, int slots_are_int64, void *cache, int64_t num_blocks,
                                 int block_size, int64_t block_stride_bytes, int64_t token_stride_bytes, int scale_rule,
                                 void *stream) {
    return smla::launch_write_int8_ds_mla(x, x_dtype, rows, x_row_stride, slot_mapping, slots_are_int64, cache,
                                          num_blocks, block_size, block_stride_bytes, token_stride_bytes, scale_rule,
                                          static_cast<cudaStream_t>(stream));
}

int smla_write_fp8_ds_mla_cache(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride,
                                const void *slot_mapping, int slots_are_int64, void *cache, int64_t num_blocks,
                                int block_size, int64_t block_stride_bytes, void *stream) {
    return smla::launch_write_fp8_ds_mla(x, x_dtype, rows, x_row_stride, slot_mapping, slots_are_int64, cache,
                                         num_blocks, block_size, block_stride_bytes,
                                         static_cast<cudaStream_t>(stream));
}

int smla_read_device_status(int *status_out) { return smla::read_and_clear_device_status(status_out); }

int smla_device_status_address(int **device_address) {
    if (!device_address) return SMLA_EINVAL;
    return smla::device_status_address(device_address);
}

}  // extern "C"
