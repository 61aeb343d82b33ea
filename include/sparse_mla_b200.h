/* sparse_mla_b200.h -- C ABI of the B200 (sm_100a) sparse-MLA library.
 *
 * Plain pointers and sizes only: every pointer is a DEVICE pointer on the device that is
 * current when the function is called, `stream` is a cudaStream_t passed as void*.  All
 * functions are asynchronous on `stream`, never synchronise, never allocate, and return 0 on
 * success, a negative SMLA_E* code for a rejected argument, or a positive cudaError_t when a
 * launch failed.  Inputs are borrowed and never written.
 *
 * Each entry point names the reference interface (AppMana/forks-flash-mla-int, path within
 * that project) it replaces.
 */
#ifndef SPARSE_MLA_B200_H_
#define SPARSE_MLA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMLA_HEAD_DIM 512

#if defined(__GNUC__)
#define SMLA_API __attribute__((visibility("default")))
#else
#define SMLA_API
#endif

enum smla_cache_format {
    SMLA_FP8_DS_MLA = 0,  /* uint8 [nb, bs, 584]: per block [bs x 576 data][bs x 8 scale] */
    SMLA_INT8_DS_MLA = 1  /* int8 [nb, bs, 512] + fp32 scale [nb, bs], runtime strides     */
};

enum smla_error {
    SMLA_OK = 0,
    SMLA_EINVAL = -1,     /* null pointer / non-positive size / unknown enum            */
    SMLA_EALIGN = -2,     /* pointer or stride alignment the kernels cannot gather from */
    SMLA_EWORKSPACE = -3, /* workspace missing or too small for the requested splits    */
    SMLA_EARCH = -4,      /* current device is not compute capability 10.x              */
    SMLA_ETOOBIG = -5     /* request exceeds a fixed capacity of the entry point         */
};

/* One index stream of the selection (the sliding-window "swa" cache or the optional
 * compressed "extra" cache).  Mirrors the per-stream fields of Sparse_mla_decode_params /
 * Sparse_mla_prefill_params (csrc/flash_mla.h:73-115, 127-152). */
typedef struct smla_stream {
    const void *cache;          /* NULL = stream absent (extra only)                         */
    const float *scale;         /* int8_ds_mla: fp32 [nb, bs]; NULL for fp8_ds_mla            */
    const int32_t *indices;     /* int32 [T, topk] slot ids; <0 or >= nb*bs = zero row         */
    const int32_t *lens;        /* int32 [T], rows of `indices` that take part (<= topk)      */
    int64_t indices_stride;     /* elements between consecutive tokens' index rows           */
    int32_t topk;
    int32_t num_blocks;
    int32_t block_size;
    int64_t block_stride;       /* bytes between paged blocks                                 */
    int64_t pos_stride;         /* int8: bytes between tokens of a block (512, 528, ...)       */
    int64_t scale_block_stride; /* int8: elements                                             */
    int64_t scale_pos_stride;   /* int8: elements                                             */
} smla_stream_t;

/* Launch contract of the attention kernels.  Replaces Sparse_mla_decode_params and
 * Sparse_mla_prefill_params (csrc/flash_mla.h:73-115, 127-152); the reference's dense
 * selection scratch (sel_kv_ptr) and whole-cache dequant buffer (kv_ptr) have no
 * counterpart because rows are gathered and dequantised inside the attention kernel. */
typedef struct smla_attn_params {
    int32_t num_tokens;         /* T */
    int32_t num_heads;          /* H */
    int32_t cache_format;       /* enum smla_cache_format, both streams                       */
    float softmax_scale;        /* natural-log units (the library multiplies by log2 e)        */
    const void *q;              /* bf16 [T, H, 512], innermost stride 1, 16-byte aligned rows  */
    int64_t q_token_stride, q_head_stride;     /* elements */
    void *out;                  /* bf16 [T, H, 512] */
    int64_t out_token_stride, out_head_stride; /* elements */
    const float *attn_sink;     /* fp32 [H] natural-log logits, or NULL                        */
    smla_stream_t swa;
    smla_stream_t extra;        /* extra.cache == NULL when absent                            */
    int32_t num_splits;         /* scratch partials per (token, head); 0 = let the library choose */
    void *workspace;            /* 16-byte aligned, >= smla_attn_workspace_bytes(...) when
                                   num_splits > 1, else NULL                                  */
    size_t workspace_bytes;
} smla_attn_params_t;

/* Library version string. */
SMLA_API const char *smla_version(void);

/* Human-readable text for a return code of this library (negative) or of CUDA (positive). */
SMLA_API const char *smla_error_string(int code);

/* Split-KV policy.  The attention kernel is persistent (at most one CTA per SM).  A result of 1 means
 * whole (token, 64-head block) items are dealt out to the CTAs and nothing is merged.  A result
 * S > 1 means the 128-row tiles of all items are cut into equal contiguous ranges, one per CTA (so
 * ragged lens and fewer items than SMs still fill the GPU); a CTA then leaves up to two partial
 * segments in scratch.  They are merged inside the attention kernel -- by the CTA that holds an
 * item's first tiles, in its own epilogue, or, for a few tokens spread over the whole GPU, slice-wise
 * by all CTAs of the item -- and only between ~10 and ~70 items by a second small kernel (see
 * smla_decode_kernel_launches).  S is the scratch the schedule needs, in partials per (token, head):
 * two slots of 64 heads per CTA plus the merge descriptors.  Counterpart of sparse_mla_num_splits
 * (csrc/flash_api.cpp:75-102); the environment variable FLASH_MLA_SLOTS_PER_SPLIT is honoured as the
 * least number of rows a CTA is given (read per call). */
SMLA_API int smla_choose_num_splits(int sm_count, int num_tokens, int num_heads, int max_width);

/* Bytes of split-KV scratch (fp32 partial outputs + {max, denominator} pairs) for `num_splits`
 * partials per (token, head): num_tokens * num_heads * num_splits * (512 + 2) * 4; 0 when
 * num_splits <= 1.  Counterpart of the oaccum/mlse tensors allocated at csrc/flash_api.cpp:388-400.
 * An explicit num_splits smaller than the policy's only lowers the number of CTAs that share the
 * tiles (two slots each); below two CTAs the unsplit schedule is used. */
SMLA_API size_t smla_attn_workspace_bytes(int num_tokens, int num_heads, int num_splits);

/* Split count smla_sparse_mla_decode would pick on the CURRENT device (queries its SM count) and
 * the scratch bytes that count needs; what the reference binding computes inline at
 * csrc/flash_api.cpp:381-405 before it allocates oaccum / mlse. */
SMLA_API int smla_decode_plan(int num_tokens, int num_heads, int max_width, int *num_splits, size_t *workspace_bytes);

/* Kernels one decode call launches on a device with `sm_count` SMs when given `num_splits` and its
 * workspace: 1 (whole items, or the balanced schedule with the merge fused into the attention kernel)
 * or 2 (attention kernel + combine kernel: between ~10 and ~70 items on a 148-SM part).  For accounting
 * (benchmarks); no counterpart in the reference.  On a CAPTURING stream the slice-wise merge (at most
 * ~8 tokens of 64 heads) is replaced by the combine kernel, because a replayed graph repeats the launch
 * tag that merge relies on: smla_decode_kernel_launches_captured gives the kernel-node count of a
 * captured decode call. */
SMLA_API int smla_decode_kernel_launches(int sm_count, int num_tokens, int num_heads, int num_splits);
SMLA_API int smla_decode_kernel_launches_captured(int sm_count, int num_tokens, int num_heads, int num_splits);

/* Sparse MLA decode.  Replaces run_sparse_mla_decode (csrc/flash_mla.h:125,
 * csrc/flash_sparse_mla_decode_sm80.cu:1198-1275) for both cache formats.
 *
 * Waits inside the kernels.  With num_splits > 1 the in-kernel merges make a CTA wait for partial
 * results of OTHER CTAs of the same launch (a 64-bit flag per scratch slot).  Those waits cannot
 * deadlock when the persistent grid is resident -- a CTA only waits for another CTA's FIRST segment,
 * which waits for nothing -- and when part of the grid is not resident (another kernel holds SMs, MPS,
 * a green context) the resident CTAs are a prefix of the grid, of which only the last can be waiting
 * for a CTA that has not started.  Every wait in the kernels is still bounded (one second): a wait
 * that runs out sets a bit in a per-device status word, the CTA leaves through its normal teardown and
 * the affected output rows are NOT valid although the call returned 0 long before.  Callers that share
 * the GPU with long-running kernels should check smla_read_device_status when they next synchronise
 * (it costs a device synchronisation), or use num_splits = 1 (whole items: no CTA waits for another). */
SMLA_API int smla_sparse_mla_decode(const smla_attn_params_t *params, void *stream);

/* Split-KV decode that brings its own scratch: same contract and results as smla_sparse_mla_decode,
 * but `workspace` / `workspace_bytes` are ignored and the partials go to an array of
 * SMLA_STATIC_SCRATCH_BYTES that is part of the library image (each GPU that loads the library holds
 * it until exit).  No counterpart in the reference, whose binding always allocates its partial
 * buffers through torch (csrc/flash_api.cpp:388-405).  It exists for hosts that cannot allocate
 * device memory when a decode step runs: every byte of HBM already belongs to the engine's KV-cache
 * pool, cudaMalloc would synchronise the device inside the latency-critical loop, and it is not
 * allowed during stream capture.  This function calls no allocator of any kind.
 *   - An explicit num_splits whose scratch (smla_attn_workspace_bytes) exceeds
 *     SMLA_STATIC_SCRATCH_BYTES is rejected with SMLA_ETOOBIG and nothing is launched.  With the
 *     automatic choice (num_splits == 0) the array is offered whole: what the kernels touch is two
 *     partial slots per CTA (39 MB on a 148-SM part), however many tokens there are, so the balanced
 *     schedule runs with as many CTAs as fit (all of them on B200).
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, that
 *     device current).  Under CUDA's lazy module loading that first use is also when the driver sets
 *     the array's memory aside: make the first call per device at start-up -- BEFORE the engine claims
 *     the rest of HBM and outside any stream capture -- and expect a positive cudaError_t (out of
 *     memory) from it if the device is already full.
 *   - All calls on a device share the array, which keeps the previous call's contents (nothing in it
 *     needs clearing); calls whose kernels overlap on the GPU race on it. */
#define SMLA_STATIC_SCRATCH_BYTES (64u << 20)
SMLA_API int smla_sparse_mla_decode_static_scratch(const smla_attn_params_t *params, void *stream);

/* Sparse MLA prefill (many query tokens, never split).  Replaces run_sparse_mla_prefill
 * (csrc/flash_mla.h:159-160, csrc/flash_sparse_mla_prefill_fused_sm80.cu:468-506). */
SMLA_API int smla_sparse_mla_prefill(const smla_attn_params_t *params, void *stream);

/* Dense paged MLA decode: every query attends to ALL rows of its sequence's paged bf16 KV cache (one kv
 * head; scores over 576 dims, values = the first 512).  Replaces the path behind flash_mla_with_kvcache:
 * mha_fwd_kvcache_mla (csrc/flash_api.cpp:159-322), Flash_fwd_mla_params (csrc/flash_mla.h:5-49) and
 * run_mha_fwd_splitkv_mla.  Query tokens are (sequence, query position) pairs flattened in that order.
 * No scheduler metadata is needed: the persistent kernel cuts the work itself (get_mla_metadata of the
 * reference has no counterpart here; the binding returns placeholders of the reference's shapes). */
typedef struct smla_dense_params {
    int32_t batch, seqlen_q, num_heads;   /* q [batch, seqlen_q, num_heads, head_dim] bf16                       */
    int32_t causal;                       /* query position i sees the first len - (seqlen_q - 1 - i) rows       */
    int32_t head_dim;                     /* 576 (0 means 576), or 512: scores over 512 dims, no RoPE part       */
    float softmax_scale;
    const void *q;                        /* 16-byte aligned                                                     */
    int64_t q_token_stride, q_head_stride;       /* elements; token = batch index * seqlen_q + query position   */
    void *out;                            /* [batch, seqlen_q, num_heads, 512] bf16                              */
    int64_t out_token_stride, out_head_stride;   /* elements                                                    */
    float *softmax_lse;                   /* [batch, num_heads, seqlen_q] fp32, natural log; may be NULL         */
    const void *k_cache;                  /* [num_blocks, page_block_size, 1, head_dim] bf16, 16-byte aligned    */
    int64_t k_block_stride, k_row_stride; /* bytes, multiples of 16, k_row_stride >= 2 * head_dim                */
    int32_t num_blocks, page_block_size;
    int32_t max_blocks_per_seq;           /* columns of block_table: lengths are clamped to this many pages      */
    const int32_t *block_table;           /* [batch, max_blocks_per_seq] page numbers (negative: zero rows)      */
    int64_t block_table_stride;           /* elements                                                            */
    const int32_t *cache_seqlens;         /* [batch] rows of each sequence                                       */
    int32_t num_splits;                   /* as smla_attn_params_t: 0 = choose, 1 = whole items, > 1 with workspace */
    void *workspace;                      /* smla_attn_workspace_bytes(batch * seqlen_q, num_heads, num_splits)  */
    size_t workspace_bytes;
} smla_dense_params_t;
SMLA_API int smla_dense_mla_decode(const smla_dense_params_t *params, void *stream);

/* int8_ds_mla row quantizer, bit-exact with quantize_int8_ds_mla_rows
 * (flash_mla/int8_sparse_mla.py:15-26): scale = max(amax|x|, 1e-12) / 127 and
 * q = clamp(rint(x / scale), -127, 127) in IEEE fp32.
 *   x: [rows, 512] of `x_dtype` (0 = bf16, 1 = fp16, 2 = fp32), `x_row_stride` elements apart;
 *   q: int8 [rows, 512] contiguous, 16-byte aligned; scale: fp32 [rows]. */
SMLA_API int smla_quantize_int8_ds_mla_rows(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride,
                                   int8_t *q, float *scale, void *stream);

/* Cache writers: encode `rows` new latent rows and scatter them into a paged cache in one kernel,
 * the step that runs right before the attention calls above.  The reference has no device writer
 * (its tests and benchmarks pack caches with torch composites); the bytes written are the formats
 * its kernels read.  Common arguments:
 *   x: [rows, 512] of `x_dtype` (0 = bf16, 1 = fp16, 2 = fp32), `x_row_stride` elements apart,
 *      16-byte aligned rows (32-byte aligned rows take 256-bit loads);
 *   slot_mapping: int32 or int64 [rows] (`slots_are_int64`); row i goes to block slot / block_size,
 *      position slot % block_size; a negative slot, or one >= num_blocks * block_size, skips the row;
 *      two rows with the same slot race;
 *   cache: 16-byte aligned base of `num_blocks` blocks, `block_stride_bytes` apart.
 *
 * int8_ds_mla inline container (tests/test_sparse_mla_prefill_int8_adversarial.py:5-12): a token is
 * 512 int8 + the fp32 row scale at +512 + 12 zero bytes, tokens `token_stride_bytes` (>= 528, multiple of
 * 16) apart.  scale_rule 0: scale and codes bit-exact with quantize_int8_ds_mla_rows
 * (flash_mla/int8_sparse_mla.py:15-26); scale_rule 1: scale = max(amax / 127, 1e-12), the serving
 * engine's writer as restated at tests/test_sparse_mla_prefill_int8_adversarial.py:35-40 (the two differ
 * only for rows with amax < 1.27e-10). */
SMLA_API int smla_write_int8_ds_mla_cache(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride,
                                          const void *slot_mapping, int slots_are_int64, void *cache,
                                          int64_t num_blocks, int block_size, int64_t block_stride_bytes,
                                          int64_t token_stride_bytes, int scale_rule, void *stream);

/* fp8_ds_mla (docs/sparse_mla_decode_sm86_design.md:23-31, tests/test_sparse_mla_decode_sm86.py:14-44): a
 * block is [block_size x 576 data bytes][block_size x 8 scale bytes]; a token's data are 448 e4m3 codes
 * of x / 2^e (round to nearest even, e per 64 dims) and 64 bf16 (the last 64 elements, round to
 * nearest even); its scale record is 7 bytes e + 127 and one byte 127.  e is the smallest exponent
 * with amax <= 448 * 2^e, clamped to [-120, 120], 0 for an all-zero group.  block_stride_bytes >=
 * block_size * 584 and a multiple of 8 (a multiple of 16 takes 16-byte stores). */
SMLA_API int smla_write_fp8_ds_mla_cache(const void *x, int x_dtype, int64_t rows, int64_t x_row_stride,
                                         const void *slot_mapping, int slots_are_int64, void *cache,
                                         int64_t num_blocks, int block_size, int64_t block_stride_bytes,
                                         void *stream);

/* Reads and clears the per-device error word the kernels set when a bounded wait ran out
 * (0 = none).  Synchronises the device; meant for tests and debugging, not for hot paths. */
SMLA_API int smla_read_device_status(int *status_out);

/* Device address of that status word on the current device, for hosts that must not synchronise: copy
 * the 4 bytes asynchronously on the decode stream behind a step (cudaMemcpyAsync to pinned memory) and
 * look at them whenever the stream is next known to have passed that point.  Non-zero = a bounded wait
 * ran out in some launch since the word was last cleared (smla_read_device_status clears it; so does a
 * 4-byte cudaMemsetAsync by the caller).  No synchronisation, no allocation.  No counterpart in the
 * reference, whose kernels have no waits between CTAs. */
SMLA_API int smla_device_status_address(int **device_address);

#ifdef __cplusplus
}
#endif
#endif /* SPARSE_MLA_B200_H_ */
