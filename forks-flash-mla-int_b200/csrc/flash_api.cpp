// torch-stable-ABI host binding of the B200 sparse-MLA library.
//
// Registers the operator schemas of the reference binding for the sparse path
// (csrc/flash_api.cpp:810-838 of AppMana/forks-flash-mla-int):
//   flash_mla::fwd_sparse_decode_mla, fwd_sparse_prefill_mla,
//   flash_mla::fwd_sparse_int8_decode_mla, fwd_sparse_int8_prefill_mla
// plus flash_mla::quantize_int8_ds_mla_rows (a torch composite in the reference,
// flash_mla/int8_sparse_mla.py:15-26; a CUDA kernel here) and the two cache writers
// flash_mla::write_int8_ds_mla_cache / write_fp8_ds_mla_cache (no counterpart in the reference).  Only torch/csrc/stable, the AOTI
// shim and torch/headeronly are used -- no ATen, c10 or pybind -- and every op validates its
// arguments, allocates its output (and split-KV scratch) with torch's allocator on q's device,
// and forwards plain pointers to the C ABI in include/sparse_mla_b200.h on the current stream.
// Nothing here synchronises, so the ops stay CUDA-graph capturable.
#include <Python.h>
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/ops.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/util/Exception.h>

#include <cstdint>
#include <optional>
#include <string>
#include <vector>

#include "sparse_mla_b200.h"

using torch::headeronly::ScalarType;
using torch::stable::Tensor;

namespace {

void *current_stream(int device) {
    void *s = nullptr;
    TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(device, &s));
    return s;
}

void check_rc(int rc, const char *what) {
    STD_TORCH_CHECK(rc == 0, what, " failed: ", smla_error_string(rc), " (code ", rc, ")");
}

bool aligned16(const Tensor &t) { return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0; }

// q / out style [T, H, 512] bf16 tensor the kernels can read with 16-byte loads.
Tensor as_kernel_q(const Tensor &q) {
    if (q.stride(2) == 1 && q.stride(0) % 8 == 0 && q.stride(1) % 8 == 0 && aligned16(q)) return q;
    return torch::stable::contiguous(q);
}

Tensor as_index_rows(const Tensor &idx, const char *name) {
    STD_TORCH_CHECK(idx.dim() == 2, name, " must have shape (num_tokens, topk)");
    STD_TORCH_CHECK(idx.scalar_type() == ScalarType::Int, name, " must be int32");
    if (idx.size(1) <= 1 || idx.stride(1) == 1) return idx;
    return torch::stable::contiguous(idx);
}

struct StreamTensors {   // keeps the (possibly re-laid-out) tensors alive until the launch returns
    std::optional<Tensor> indices, lens;
};

void fill_stream(smla_stream_t &s, StreamTensors &keep, int T, const char *name, const Tensor &cache,
                 const std::optional<Tensor> &scale, const Tensor &indices, const Tensor &lens, bool int8) {
    STD_TORCH_CHECK(cache.is_cuda() && indices.is_cuda() && lens.is_cuda(), name, " tensors must be on CUDA");
    STD_TORCH_CHECK(cache.dim() == 3, name, "_cache must be [num_blocks, block_size, bytes]");
    keep.indices = as_index_rows(indices, name);
    STD_TORCH_CHECK(keep.indices->size(0) == T, name, "_indices must have one row per query token");
    STD_TORCH_CHECK(lens.scalar_type() == ScalarType::Int, name, "_lens must be int32");
    STD_TORCH_CHECK(lens.dim() == 1 && lens.size(0) == T, name, "_lens must have shape (num_tokens,)");
    keep.lens = lens.is_contiguous() ? lens : torch::stable::contiguous(lens);
    s.cache = cache.data_ptr();
    s.indices = static_cast<const int32_t *>(keep.indices->data_ptr());
    s.lens = static_cast<const int32_t *>(keep.lens->data_ptr());
    s.indices_stride = keep.indices->size(0) > 1 ? keep.indices->stride(0) : keep.indices->size(1);
    s.topk = static_cast<int32_t>(keep.indices->size(1));
    s.num_blocks = static_cast<int32_t>(cache.size(0));
    s.block_size = static_cast<int32_t>(cache.size(1));
    s.block_stride = cache.stride(0) * static_cast<int64_t>(cache.element_size());
    if (int8) {
        STD_TORCH_CHECK(cache.scalar_type() == ScalarType::Char, name, "_cache must be int8");
        STD_TORCH_CHECK(cache.size(2) == 512, "int8 cache payload must be 512 bytes/token");
        STD_TORCH_CHECK(cache.stride(2) == 1, name, "_cache rows must be contiguous");
        STD_TORCH_CHECK(scale.has_value(), name, "_scale is required for an int8 cache");
        const Tensor &sc = scale.value();
        STD_TORCH_CHECK(sc.is_cuda(), name, "_scale must be on CUDA");
        STD_TORCH_CHECK(sc.scalar_type() == ScalarType::Float, name, "_scale must be float32");
        STD_TORCH_CHECK(sc.dim() == 2 && sc.size(0) == cache.size(0) && sc.size(1) == cache.size(1), name,
                        "_scale must have shape (num_blocks, block_size)");
        s.scale = static_cast<const float *>(sc.data_ptr());
        s.pos_stride = cache.stride(1);
        s.scale_block_stride = sc.stride(0);
        s.scale_pos_stride = sc.stride(1);
    } else {
        STD_TORCH_CHECK(cache.scalar_type() == ScalarType::Byte, name, "_cache must be uint8");
        STD_TORCH_CHECK(cache.size(2) == 584 && cache.stride(2) == 1 && cache.stride(1) == 584, name,
                        "_cache must be fp8_ds_mla [num_blocks, block_size, 584] with contiguous blocks");
        s.scale = nullptr;
        s.pos_stride = 576;
    }
}

Tensor sparse_mla_forward(const char *what, bool int8, bool prefill, const Tensor &q_in, const Tensor &swa_cache,
                          const std::optional<Tensor> &swa_scale, const Tensor &swa_indices,
                          const Tensor &swa_lens, double scale, const std::optional<Tensor> &attn_sink,
                          const std::optional<Tensor> &extra_cache, const std::optional<Tensor> &extra_scale,
                          const std::optional<Tensor> &extra_indices, const std::optional<Tensor> &extra_lens,
                          const Tensor *out_given = nullptr, const std::optional<Tensor> *ws_given = nullptr) {
    STD_TORCH_CHECK(q_in.is_cuda(), "q must be on CUDA");
    STD_TORCH_CHECK(q_in.dim() == 3, "q must have shape (num_tokens, num_heads, 512)");
    STD_TORCH_CHECK(q_in.size(2) == 512, "head_dim must be 512");
    STD_TORCH_CHECK(q_in.scalar_type() == ScalarType::BFloat16, "q must be bfloat16");
    const int device = q_in.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);

    const Tensor q = as_kernel_q(q_in);
    const int64_t T = q.size(0), H = q.size(1);
    STD_TORCH_CHECK(H >= 1, "q must have at least one head");
    if (out_given) {
        const Tensor &o = *out_given;
        STD_TORCH_CHECK(o.is_cuda() && o.get_device_index() == device && o.scalar_type() == ScalarType::BFloat16 &&
                            o.dim() == 3 && o.size(0) == T && o.size(1) == H && o.size(2) == 512,
                        "out must be a bfloat16 (num_tokens, num_heads, 512) tensor on q's device");
        STD_TORCH_CHECK(o.stride(2) == 1 && o.stride(0) % 8 == 0 && o.stride(1) % 8 == 0 && aligned16(o),
                        "out must have contiguous 16-byte aligned rows");
    }
    Tensor out = out_given ? *out_given : torch::stable::new_empty(q, {T, H, 512});
    if (T == 0) return out;

    smla_attn_params_t p = {};
    p.num_tokens = static_cast<int32_t>(T);
    p.num_heads = static_cast<int32_t>(H);
    p.cache_format = int8 ? SMLA_INT8_DS_MLA : SMLA_FP8_DS_MLA;
    p.softmax_scale = static_cast<float>(scale);
    p.q = q.data_ptr();
    p.q_token_stride = q.stride(0);
    p.q_head_stride = q.stride(1);
    p.out = out.data_ptr();
    p.out_token_stride = out.stride(0);
    p.out_head_stride = out.stride(1);
    std::optional<Tensor> sink_keep;
    if (attn_sink.has_value()) {
        const Tensor &sk = attn_sink.value();
        STD_TORCH_CHECK(sk.is_cuda(), "attn_sink must be on CUDA");
        STD_TORCH_CHECK(sk.scalar_type() == ScalarType::Float, "attn_sink must be float32");
        STD_TORCH_CHECK(sk.dim() == 1 && sk.size(0) == H, "attn_sink must have shape (num_heads,)");
        sink_keep = sk.is_contiguous() ? sk : torch::stable::contiguous(sk);
        p.attn_sink = static_cast<const float *>(sink_keep->data_ptr());
    }
    StreamTensors swa_keep, extra_keep;
    fill_stream(p.swa, swa_keep, static_cast<int>(T), "swa", swa_cache, swa_scale, swa_indices, swa_lens, int8);
    if (extra_cache.has_value()) {
        STD_TORCH_CHECK(extra_indices.has_value() && extra_lens.has_value() && (!int8 || extra_scale.has_value()),
                        int8 ? "extra scale/indices/lens required with extra cache"
                             : "extra indices/lens required with extra cache");
        fill_stream(p.extra, extra_keep, static_cast<int>(T), "extra", extra_cache.value(), extra_scale,
                    extra_indices.value(), extra_lens.value(), int8);
    }
    const int width = p.swa.topk + (extra_cache.has_value() ? p.extra.topk : 0);

    void *stream = current_stream(device);
    int rc;
    std::optional<Tensor> workspace;   // split-KV scratch; freed stream-ordered by torch's allocator
    if (prefill) {
        STD_TORCH_CHECK(width > 0, "prefill requires at least one selected slot");
        rc = smla_sparse_mla_prefill(&p, stream);
    } else {
        int splits = 1;
        size_t ws_bytes = 0;
        check_rc(smla_decode_plan(p.num_tokens, p.num_heads, width, &splits, &ws_bytes), "sparse-MLA decode plan");
        if (ws_given) {            // planned call: the caller's scratch or none at all, nothing is allocated here
            if (splits > 1 && ws_given->has_value()) {
                const Tensor &w = ws_given->value();
                STD_TORCH_CHECK(w.is_cuda() && w.get_device_index() == device && w.is_contiguous() && aligned16(w),
                                "workspace must be a contiguous 16-byte aligned tensor on q's device");
                STD_TORCH_CHECK(static_cast<size_t>(w.numel()) * w.element_size() >= ws_bytes,
                                "workspace is smaller than the plan for this shape needs");
                p.workspace = w.data_ptr();
                p.workspace_bytes = static_cast<size_t>(w.numel()) * w.element_size();
            } else {
                splits = 1;
            }
        } else if (splits > 1) {
            workspace = torch::stable::new_empty(q, {static_cast<int64_t>((ws_bytes + 3) / 4)}, ScalarType::Float);
            p.workspace = workspace->data_ptr();
            p.workspace_bytes = ws_bytes;
        }
        p.num_splits = splits;
        rc = smla_sparse_mla_decode(&p, stream);
    }
    check_rc(rc, what);
    return out;
}

Tensor fwd_sparse_decode_mla(Tensor q, Tensor swa_cache, Tensor swa_indices, Tensor swa_lens, double scale,
                             std::optional<Tensor> attn_sink, std::optional<Tensor> extra_cache,
                             std::optional<Tensor> extra_indices, std::optional<Tensor> extra_lens) {
    return sparse_mla_forward("sparse-MLA fp8 decode", false, false, q, swa_cache, std::nullopt, swa_indices,
                              swa_lens, scale, attn_sink, extra_cache, std::nullopt, extra_indices, extra_lens);
}
Tensor fwd_sparse_prefill_mla(Tensor q, Tensor swa_cache, Tensor swa_indices, Tensor swa_lens, double scale,
                              std::optional<Tensor> attn_sink, std::optional<Tensor> extra_cache,
                              std::optional<Tensor> extra_indices, std::optional<Tensor> extra_lens) {
    return sparse_mla_forward("sparse-MLA fp8 prefill", false, true, q, swa_cache, std::nullopt, swa_indices,
                              swa_lens, scale, attn_sink, extra_cache, std::nullopt, extra_indices, extra_lens);
}
Tensor fwd_sparse_int8_decode_mla(Tensor q, Tensor swa_cache, Tensor swa_scale, Tensor swa_indices,
                                  Tensor swa_lens, double scale, std::optional<Tensor> attn_sink,
                                  std::optional<Tensor> extra_cache, std::optional<Tensor> extra_scale,
                                  std::optional<Tensor> extra_indices, std::optional<Tensor> extra_lens) {
    return sparse_mla_forward("sparse-MLA int8 decode", true, false, q, swa_cache, swa_scale, swa_indices, swa_lens,
                              scale, attn_sink, extra_cache, extra_scale, extra_indices, extra_lens);
}
Tensor fwd_sparse_int8_prefill_mla(Tensor q, Tensor swa_cache, Tensor swa_scale, Tensor swa_indices,
                                   Tensor swa_lens, double scale, std::optional<Tensor> attn_sink,
                                   std::optional<Tensor> extra_cache, std::optional<Tensor> extra_scale,
                                   std::optional<Tensor> extra_indices, std::optional<Tensor> extra_lens) {
    return sparse_mla_forward("sparse-MLA int8 prefill", true, true, q, swa_cache, swa_scale, swa_indices, swa_lens,
                              scale, attn_sink, extra_cache, extra_scale, extra_indices, extra_lens);
}

// Decode into caller-owned `out` with caller-owned split scratch (or none): no allocation in the call.
// The cache format follows the cache dtype (int8 rows + scales, or uint8 fp8_ds_mla blocks).
void fwd_sparse_decode_mla_planned(Tensor q, Tensor swa_cache, std::optional<Tensor> swa_scale, Tensor swa_indices,
                                   Tensor swa_lens, double scale, std::optional<Tensor> attn_sink,
                                   std::optional<Tensor> extra_cache, std::optional<Tensor> extra_scale,
                                   std::optional<Tensor> extra_indices, std::optional<Tensor> extra_lens, Tensor out,
                                   std::optional<Tensor> workspace) {
    const bool int8 = swa_cache.scalar_type() == ScalarType::Char;
    sparse_mla_forward(int8 ? "sparse-MLA int8 decode (planned)" : "sparse-MLA fp8 decode (planned)", int8, false, q,
                       swa_cache, swa_scale, swa_indices, swa_lens, scale, attn_sink, extra_cache, extra_scale,
                       extra_indices, extra_lens, &out, &workspace);
}

// k: [..., 512] bf16 / fp16 / fp32 on CUDA -> (int8 [..., 512], fp32 [...]).
void quantize_int8_ds_mla_rows(const Tensor &k_in, Tensor &q_out, Tensor &scale_out) {
    STD_TORCH_CHECK(k_in.is_cuda(), "k must be on CUDA");
    STD_TORCH_CHECK(k_in.dim() >= 1 && k_in.size(k_in.dim() - 1) == 512, "expected last dim 512");
    int dtype = -1;
    switch (k_in.scalar_type()) {
        case ScalarType::BFloat16: dtype = 0; break;
        case ScalarType::Half: dtype = 1; break;
        case ScalarType::Float: dtype = 2; break;
        default: STD_TORCH_CHECK(false, "k must be bfloat16, float16 or float32");
    }
    const int device = k_in.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    const Tensor k = (k_in.is_contiguous() && aligned16(k_in)) ? k_in : torch::stable::contiguous(k_in);
    const int64_t rows = k.numel() / 512;
    std::vector<int64_t> qs, ss;
    for (int64_t i = 0; i < k.dim(); ++i) qs.push_back(k.size(i));
    for (int64_t i = 0; i + 1 < k.dim(); ++i) ss.push_back(k.size(i));
    q_out = torch::stable::new_empty(k, torch::headeronly::IntHeaderOnlyArrayRef(qs.data(), qs.size()),
                                     ScalarType::Char);
    scale_out = torch::stable::new_empty(k, torch::headeronly::IntHeaderOnlyArrayRef(ss.data(), ss.size()),
                                         ScalarType::Float);
    check_rc(smla_quantize_int8_ds_mla_rows(k.data_ptr(), dtype, rows, 512, static_cast<int8_t *>(q_out.data_ptr()),
                                            static_cast<float *>(scale_out.data_ptr()), current_stream(device)),
             "int8_ds_mla row quantizer");
}

// Cache writers: latent [N, 512] (bf16 / fp16 / fp32), slot_mapping int32 / int64 [N], cache uint8
// [num_blocks, block_size, 528 or 584] written in place.  The reference has no such op; the schemas
// follow the (rows, slot_mapping, cache) shape of a serving engine's cache-write call.
void write_ds_mla_cache(const char *what, bool fp8, const Tensor &latent_in, const Tensor &slots_in, const Tensor &cache,
                        int64_t scale_rule) {
    STD_TORCH_CHECK(latent_in.is_cuda() && slots_in.is_cuda() && cache.is_cuda(), what, ": tensors must be on CUDA");
    STD_TORCH_CHECK(latent_in.dim() == 2 && latent_in.size(1) == 512, what, ": latent must be [rows, 512]");
    STD_TORCH_CHECK(slots_in.dim() == 1 && slots_in.size(0) == latent_in.size(0), what, ": slot_mapping must be [rows]");
    const int64_t token_bytes = fp8 ? 584 : 528;
    STD_TORCH_CHECK(cache.dim() == 3 && cache.size(2) == token_bytes && cache.element_size() == 1 &&
                        cache.stride(2) == 1 && cache.stride(1) == token_bytes && aligned16(cache),
                    what, ": cache must be a 16-byte aligned byte tensor [num_blocks, block_size, ", token_bytes,
                    "] with dense blocks");
    int dtype = -1;
    switch (latent_in.scalar_type()) {
        case ScalarType::BFloat16: dtype = 0; break;
        case ScalarType::Half: dtype = 1; break;
        case ScalarType::Float: dtype = 2; break;
        default: STD_TORCH_CHECK(false, what, ": latent must be bfloat16, float16 or float32");
    }
    const bool i64 = slots_in.scalar_type() == ScalarType::Long;
    STD_TORCH_CHECK(i64 || slots_in.scalar_type() == ScalarType::Int, what, ": slot_mapping must be int32 or int64");
    const int device = latent_in.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);
    const int64_t elem = dtype == 2 ? 4 : 2;
    const bool usable = latent_in.stride(1) == 1 && (latent_in.stride(0) * elem) % 16 == 0 && aligned16(latent_in);
    const Tensor latent = usable ? latent_in : torch::stable::contiguous(latent_in);
    const Tensor slots = slots_in.is_contiguous() ? slots_in : torch::stable::contiguous(slots_in);
    const int64_t rows = latent.size(0);
    const int64_t row_stride = rows > 1 ? latent.stride(0) : 512;
    const int64_t block_stride = cache.size(0) > 1 ? cache.stride(0) : cache.size(1) * token_bytes;
    if (fp8) {
        check_rc(smla_write_fp8_ds_mla_cache(latent.data_ptr(), dtype, rows, row_stride, slots.data_ptr(), i64,
                                             cache.data_ptr(), cache.size(0), static_cast<int>(cache.size(1)),
                                             block_stride, current_stream(device)),
                 what);
    } else {
        check_rc(smla_write_int8_ds_mla_cache(latent.data_ptr(), dtype, rows, row_stride, slots.data_ptr(), i64,
                                              cache.data_ptr(), cache.size(0), static_cast<int>(cache.size(1)),
                                              block_stride, token_bytes, static_cast<int>(scale_rule),
                                              current_stream(device)),
                 what);
    }
}

// ------------------------------------------------------------------ dense paged MLA
// fwd_kvcache_mla / get_mla_metadata of the reference (csrc/flash_api.cpp:110-157, 159-322; schemas at
// :811-814).  The persistent kernel cuts the work itself from the sequence lengths on the device, so the
// metadata tensors are placeholders of the reference's dtypes that fwd_kvcache_mla accepts and ignores.
void get_mla_metadata(const Tensor &seqlens_k, Tensor &tile_scheduler_metadata, Tensor &num_splits) {
    STD_TORCH_CHECK(seqlens_k.scalar_type() == ScalarType::Int, "seqlens_k must have dtype int32");
    STD_TORCH_CHECK(seqlens_k.dim() == 1, "seqlens_k must have shape (batch_size,)");
    tile_scheduler_metadata = torch::stable::new_zeros(seqlens_k, {1, 8});
    num_splits = torch::stable::new_zeros(seqlens_k, {seqlens_k.size(0) + 1});
}

void fwd_kvcache_mla(const Tensor &q_in, const Tensor &kcache, const std::optional<Tensor> &vcache, int64_t head_size_v,
                     const Tensor &seqlens_k, const Tensor &block_table_in, double softmax_scale, bool is_causal,
                     Tensor &out, Tensor &softmax_lse) {
    STD_TORCH_CHECK(q_in.is_cuda() && kcache.is_cuda() && seqlens_k.is_cuda() && block_table_in.is_cuda(),
                    "q, kcache, seqlens_k and block_table must be on CUDA");
    STD_TORCH_CHECK(q_in.dim() == 4, "q must have shape (batch_size, seqlen_q, num_heads, head_size)");
    STD_TORCH_CHECK(q_in.scalar_type() == ScalarType::BFloat16 && kcache.scalar_type() == ScalarType::BFloat16,
                    "query and key must be bfloat16");
    const int64_t D = q_in.size(3);
    STD_TORCH_CHECK((D == 576 || D == 512) && head_size_v == 512, "head_size must be 576 or 512 with head_size_v 512");
    STD_TORCH_CHECK(kcache.dim() == 4 && kcache.size(2) == 1 && kcache.size(3) == D,
                    "kcache must have shape (num_blocks, page_block_size, 1, head_size)");
    STD_TORCH_CHECK(kcache.stride(3) == 1, "Input tensor must have contiguous last dimension");
    if (vcache.has_value())
        STD_TORCH_CHECK(vcache->data_ptr() == kcache.data_ptr(), "vcache must be a view of kcache (or None)");
    STD_TORCH_CHECK(block_table_in.scalar_type() == ScalarType::Int && block_table_in.dim() == 2,
                    "block_table must be an int32 (batch_size, max_num_blocks_per_seq) tensor");
    STD_TORCH_CHECK(seqlens_k.scalar_type() == ScalarType::Int, "seqlens_k must have dtype int32");
    const int64_t B = q_in.size(0), SQ = q_in.size(1), H = q_in.size(2);
    STD_TORCH_CHECK(B > 0, "batch size must be postive");
    STD_TORCH_CHECK(seqlens_k.dim() == 1 && seqlens_k.size(0) == B && block_table_in.size(0) == B,
                    "seqlens_k / block_table do not match the batch size");
    const int device = q_in.get_device_index();
    torch::stable::accelerator::DeviceGuard guard(device);

    // Tokens are (sequence, query position) pairs: q is read as [B * SQ, H, head_size].
    const bool q_ok = q_in.stride(3) == 1 && q_in.stride(0) == SQ * q_in.stride(1) && q_in.stride(1) % 8 == 0 &&
                      q_in.stride(2) % 8 == 0 && aligned16(q_in);
    const Tensor q = q_ok ? q_in : torch::stable::contiguous(q_in);
    const Tensor block_table = block_table_in.stride(1) == 1 ? block_table_in : torch::stable::contiguous(block_table_in);
    const Tensor lens = seqlens_k.is_contiguous() ? seqlens_k : torch::stable::contiguous(seqlens_k);
    out = torch::stable::new_empty(q, {B, SQ, H, 512});
    softmax_lse = torch::stable::new_empty(q, {B, H, SQ}, ScalarType::Float);

    smla_dense_params_t p = {};
    p.batch = static_cast<int32_t>(B);
    p.seqlen_q = static_cast<int32_t>(SQ);
    p.num_heads = static_cast<int32_t>(H);
    p.causal = is_causal ? 1 : 0;
    p.head_dim = static_cast<int32_t>(D);
    p.softmax_scale = static_cast<float>(softmax_scale);
    p.q = q.data_ptr();
    p.q_token_stride = q.stride(1);
    p.q_head_stride = q.stride(2);
    p.out = out.data_ptr();
    p.out_token_stride = out.stride(1);
    p.out_head_stride = out.stride(2);
    p.softmax_lse = static_cast<float *>(softmax_lse.data_ptr());
    p.k_cache = kcache.data_ptr();
    p.k_block_stride = kcache.stride(0) * 2;
    p.k_row_stride = kcache.stride(1) * 2;
    p.num_blocks = static_cast<int32_t>(kcache.size(0));
    p.page_block_size = static_cast<int32_t>(kcache.size(1));
    p.block_table = static_cast<const int32_t *>(block_table.data_ptr());
    p.block_table_stride = block_table.stride(0);
    p.max_blocks_per_seq = static_cast<int32_t>(std::min<int64_t>(block_table.size(1), 0x7FFFFFFF));
    p.cache_seqlens = static_cast<const int32_t *>(lens.data_ptr());

    const int64_t width = std::min<int64_t>(block_table.size(1) * kcache.size(1), 0x7FFFFFFF);
    int splits = 1;
    size_t ws_bytes = 0;
    check_rc(smla_decode_plan(static_cast<int>(B * SQ), p.num_heads, static_cast<int>(width), &splits, &ws_bytes),
             "dense MLA decode plan");
    std::optional<Tensor> workspace;
    if (splits > 1) {
        workspace = torch::stable::new_empty(q, {static_cast<int64_t>((ws_bytes + 3) / 4)}, ScalarType::Float);
        p.workspace = workspace->data_ptr();
        p.workspace_bytes = ws_bytes;
    }
    p.num_splits = splits;
    check_rc(smla_dense_mla_decode(&p, current_stream(device)), "dense MLA decode");
}

// ------------------------------------------------------------------ boxed shims
using torch::stable::detail::from;
using torch::stable::detail::to;

template <bool PREFILL>
void boxed_fp8(StableIValue *stack, uint64_t, uint64_t) {
    auto q = to<Tensor>(stack[0]);
    auto swa_cache = to<Tensor>(stack[1]);
    auto swa_indices = to<Tensor>(stack[2]);
    auto swa_lens = to<Tensor>(stack[3]);
    auto scale = to<double>(stack[4]);
    auto attn_sink = to<std::optional<Tensor>>(stack[5]);
    auto extra_cache = to<std::optional<Tensor>>(stack[6]);
    auto extra_indices = to<std::optional<Tensor>>(stack[7]);
    auto extra_lens = to<std::optional<Tensor>>(stack[8]);
    Tensor res = PREFILL ? fwd_sparse_prefill_mla(q, swa_cache, swa_indices, swa_lens, scale, attn_sink, extra_cache,
                                                  extra_indices, extra_lens)
                         : fwd_sparse_decode_mla(q, swa_cache, swa_indices, swa_lens, scale, attn_sink, extra_cache,
                                                 extra_indices, extra_lens);
    stack[0] = from(res);
}

template <bool PREFILL>
void boxed_int8(StableIValue *stack, uint64_t, uint64_t) {
    auto q = to<Tensor>(stack[0]);
    auto swa_cache = to<Tensor>(stack[1]);
    auto swa_scale = to<Tensor>(stack[2]);
    auto swa_indices = to<Tensor>(stack[3]);
    auto swa_lens = to<Tensor>(stack[4]);
    auto scale = to<double>(stack[5]);
    auto attn_sink = to<std::optional<Tensor>>(stack[6]);
    auto extra_cache = to<std::optional<Tensor>>(stack[7]);
    auto extra_scale = to<std::optional<Tensor>>(stack[8]);
    auto extra_indices = to<std::optional<Tensor>>(stack[9]);
    auto extra_lens = to<std::optional<Tensor>>(stack[10]);
    Tensor res = PREFILL ? fwd_sparse_int8_prefill_mla(q, swa_cache, swa_scale, swa_indices, swa_lens, scale,
                                                       attn_sink, extra_cache, extra_scale, extra_indices, extra_lens)
                         : fwd_sparse_int8_decode_mla(q, swa_cache, swa_scale, swa_indices, swa_lens, scale,
                                                      attn_sink, extra_cache, extra_scale, extra_indices, extra_lens);
    stack[0] = from(res);
}

void boxed_quantize(StableIValue *stack, uint64_t, uint64_t) {
    auto k = to<Tensor>(stack[0]);
    Tensor q, s;
    quantize_int8_ds_mla_rows(k, q, s);
    stack[0] = from(q);
    stack[1] = from(s);
}

void boxed_get_mla_metadata(StableIValue *stack, uint64_t, uint64_t) {
    Tensor meta, splits;
    get_mla_metadata(to<Tensor>(stack[0]), meta, splits);
    stack[0] = from(meta);
    stack[1] = from(splits);
}

void boxed_fwd_kvcache_mla(StableIValue *stack, uint64_t, uint64_t) {
    Tensor out, lse;
    fwd_kvcache_mla(to<Tensor>(stack[0]), to<Tensor>(stack[1]), to<std::optional<Tensor>>(stack[2]), to<int64_t>(stack[3]),
                    to<Tensor>(stack[4]), to<Tensor>(stack[5]), to<double>(stack[6]), to<bool>(stack[7]), out, lse);
    stack[0] = from(out);
    stack[1] = from(lse);
}

void boxed_decode_planned(StableIValue *stack, uint64_t, uint64_t) {
    fwd_sparse_decode_mla_planned(to<Tensor>(stack[0]), to<Tensor>(stack[1]), to<std::optional<Tensor>>(stack[2]),
                                  to<Tensor>(stack[3]), to<Tensor>(stack[4]), to<double>(stack[5]),
                                  to<std::optional<Tensor>>(stack[6]), to<std::optional<Tensor>>(stack[7]),
                                  to<std::optional<Tensor>>(stack[8]), to<std::optional<Tensor>>(stack[9]),
                                  to<std::optional<Tensor>>(stack[10]), to<Tensor>(stack[11]),
                                  to<std::optional<Tensor>>(stack[12]));
}

void boxed_write_int8(StableIValue *stack, uint64_t, uint64_t) {
    write_ds_mla_cache("int8_ds_mla cache writer", false, to<Tensor>(stack[0]), to<Tensor>(stack[1]),
                       to<Tensor>(stack[2]), to<int64_t>(stack[3]));
}

void boxed_write_fp8(StableIValue *stack, uint64_t, uint64_t) {
    write_ds_mla_cache("fp8_ds_mla cache writer", true, to<Tensor>(stack[0]), to<Tensor>(stack[1]),
                       to<Tensor>(stack[2]), 0);
}

}  // namespace

STABLE_TORCH_LIBRARY(flash_mla, m) {
    m.def("fwd_sparse_decode_mla(Tensor q, Tensor swa_cache, Tensor swa_indices, Tensor swa_lens, "
          "float scale, Tensor? attn_sink, Tensor? extra_cache, Tensor? extra_indices, "
          "Tensor? extra_lens) -> Tensor");
    m.def("fwd_sparse_prefill_mla(Tensor q, Tensor swa_cache, Tensor swa_indices, Tensor swa_lens, "
          "float scale, Tensor? attn_sink, Tensor? extra_cache, Tensor? extra_indices, "
          "Tensor? extra_lens) -> Tensor");
    m.def("fwd_sparse_int8_prefill_mla(Tensor q, Tensor swa_cache, Tensor swa_scale, "
          "Tensor swa_indices, Tensor swa_lens, float scale, Tensor? attn_sink, "
          "Tensor? extra_cache, Tensor? extra_scale, Tensor? extra_indices, Tensor? extra_lens) -> Tensor");
    m.def("fwd_sparse_int8_decode_mla(Tensor q, Tensor swa_cache, Tensor swa_scale, "
          "Tensor swa_indices, Tensor swa_lens, float scale, Tensor? attn_sink, "
          "Tensor? extra_cache, Tensor? extra_scale, Tensor? extra_indices, Tensor? extra_lens) -> Tensor");
    m.def("quantize_int8_ds_mla_rows(Tensor k) -> (Tensor, Tensor)");
    m.def("get_mla_metadata(Tensor seqlens_k, int num_heads_per_head_k, int num_heads_k) -> (Tensor, Tensor)");
    m.def("fwd_kvcache_mla(Tensor q, Tensor kcache, Tensor? vcache, int head_size_v, Tensor seqlens_k, "
          "Tensor block_table, float softmax_scale, bool is_causal, Tensor tile_scheduler_metadata, "
          "Tensor num_splits, bool warp_spec) -> (Tensor, Tensor)");
    m.def("fwd_sparse_decode_mla_planned(Tensor q, Tensor swa_cache, Tensor? swa_scale, Tensor swa_indices, "
          "Tensor swa_lens, float scale, Tensor? attn_sink, Tensor? extra_cache, Tensor? extra_scale, "
          "Tensor? extra_indices, Tensor? extra_lens, Tensor(a!) out, Tensor? workspace) -> ()");
    m.def("write_int8_ds_mla_cache(Tensor latent, Tensor slot_mapping, Tensor(a!) cache, int scale_rule) -> ()");
    m.def("write_fp8_ds_mla_cache(Tensor latent, Tensor slot_mapping, Tensor(a!) cache) -> ()");
}

STABLE_TORCH_LIBRARY_IMPL(flash_mla, CUDA, m) {
    m.impl("fwd_sparse_decode_mla", &boxed_fp8<false>);
    m.impl("fwd_sparse_prefill_mla", &boxed_fp8<true>);
    m.impl("fwd_sparse_int8_prefill_mla", &boxed_int8<true>);
    m.impl("fwd_sparse_int8_decode_mla", &boxed_int8<false>);
    m.impl("quantize_int8_ds_mla_rows", &boxed_quantize);
    m.impl("get_mla_metadata", &boxed_get_mla_metadata);
    m.impl("fwd_kvcache_mla", &boxed_fwd_kvcache_mla);
    m.impl("fwd_sparse_decode_mla_planned", &boxed_decode_planned);
    m.impl("write_int8_ds_mla_cache", &boxed_write_int8);
    m.impl("write_fp8_ds_mla_cache", &boxed_write_fp8);
}

// `import flash_mla_cuda` only has to load this library so the static registrars above run.
extern "C" {
__attribute__((visibility("default"))) PyObject *PyInit_flash_mla_cuda(void) {
    static struct PyModuleDef module_def = {PyModuleDef_HEAD_INIT, "flash_mla_cuda", nullptr, -1, nullptr};
    return PyModule_Create(&module_def);
}
}
