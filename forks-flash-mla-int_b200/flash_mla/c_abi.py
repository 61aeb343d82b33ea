"""ctypes view of the C ABI in ``include/sparse_mla_b200.h`` (struct-for-struct).

For hosts that have device pointers but no torch: every argument is a raw pointer or an
integer.  The helpers at the bottom build the structs from torch tensors for the tests.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

from ._loader import CORE_LIB

SMLA_FP8_DS_MLA = 0
SMLA_INT8_DS_MLA = 1
SMLA_STATIC_SCRATCH_BYTES = 64 << 20
SMLA_ETOOBIG = -5

EXPORTS = (
    "smla_version", "smla_error_string", "smla_choose_num_splits", "smla_attn_workspace_bytes",
    "smla_decode_plan", "smla_decode_kernel_launches", "smla_decode_kernel_launches_captured", "smla_sparse_mla_decode", "smla_sparse_mla_decode_static_scratch", "smla_sparse_mla_prefill", "smla_dense_mla_decode",
    "smla_quantize_int8_ds_mla_rows", "smla_write_int8_ds_mla_cache", "smla_write_fp8_ds_mla_cache",
    "smla_read_device_status", "smla_device_status_address",
)


class SmlaStream(C.Structure):
    _fields_ = [
        ("cache", C.c_void_p),
        ("scale", C.c_void_p),
        ("indices", C.c_void_p),
        ("lens", C.c_void_p),
        ("indices_stride", C.c_int64),
        ("topk", C.c_int32),
        ("num_blocks", C.c_int32),
        ("block_size", C.c_int32),
        ("block_stride", C.c_int64),
        ("pos_stride", C.c_int64),
        ("scale_block_stride", C.c_int64),
        ("scale_pos_stride", C.c_int64),
    ]


class SmlaAttnParams(C.Structure):
    _fields_ = [
        ("num_tokens", C.c_int32),
        ("num_heads", C.c_int32),
        ("cache_format", C.c_int32),
        ("softmax_scale", C.c_float),
        ("q", C.c_void_p),
        ("q_token_stride", C.c_int64),
        ("q_head_stride", C.c_int64),
        ("out", C.c_void_p),
        ("out_token_stride", C.c_int64),
        ("out_head_stride", C.c_int64),
        ("attn_sink", C.c_void_p),
        ("swa", SmlaStream),
        ("extra", SmlaStream),
        ("num_splits", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


class SmlaDenseParams(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("seqlen_q", C.c_int32),
        ("num_heads", C.c_int32),
        ("causal", C.c_int32),
        ("head_dim", C.c_int32),
        ("softmax_scale", C.c_float),
        ("q", C.c_void_p),
        ("q_token_stride", C.c_int64),
        ("q_head_stride", C.c_int64),
        ("out", C.c_void_p),
        ("out_token_stride", C.c_int64),
        ("out_head_stride", C.c_int64),
        ("softmax_lse", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("k_block_stride", C.c_int64),
        ("k_row_stride", C.c_int64),
        ("num_blocks", C.c_int32),
        ("page_block_size", C.c_int32),
        ("max_blocks_per_seq", C.c_int32),
        ("block_table", C.c_void_p),
        ("block_table_stride", C.c_int64),
        ("cache_seqlens", C.c_void_p),
        ("num_splits", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
    ]


_lib = None


def load() -> C.CDLL:
    """dlopen the core library and declare the prototypes.  Raises OSError when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(CORE_LIB):
        raise OSError(f"{CORE_LIB} not found; run `python forks-flash-mla-int_b200/build.py`")
    lib = C.CDLL(CORE_LIB)
    lib.smla_version.restype = C.c_char_p
    lib.smla_error_string.restype = C.c_char_p
    lib.smla_error_string.argtypes = [C.c_int]
    lib.smla_choose_num_splits.argtypes = [C.c_int] * 4
    lib.smla_attn_workspace_bytes.restype = C.c_size_t
    lib.smla_attn_workspace_bytes.argtypes = [C.c_int] * 3
    lib.smla_decode_plan.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
    lib.smla_decode_kernel_launches.argtypes = [C.c_int] * 4
    lib.smla_decode_kernel_launches.restype = C.c_int
    lib.smla_decode_kernel_launches_captured.argtypes = [C.c_int] * 4
    lib.smla_decode_kernel_launches_captured.restype = C.c_int
    lib.smla_sparse_mla_decode.argtypes = [C.POINTER(SmlaAttnParams), C.c_void_p]
    lib.smla_sparse_mla_prefill.argtypes = [C.POINTER(SmlaAttnParams), C.c_void_p]
    lib.smla_dense_mla_decode.argtypes = [C.POINTER(SmlaDenseParams), C.c_void_p]
    lib.smla_sparse_mla_decode_static_scratch.argtypes = [C.POINTER(SmlaAttnParams), C.c_void_p]
    lib.smla_quantize_int8_ds_mla_rows.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p,
                                                   C.c_void_p, C.c_void_p]
    lib.smla_write_int8_ds_mla_cache.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int,
                                                 C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_int64, C.c_int,
                                                 C.c_void_p]
    lib.smla_write_fp8_ds_mla_cache.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_void_p, C.c_int,
                                                C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_void_p]
    lib.smla_read_device_status.argtypes = [C.POINTER(C.c_int)]
    lib.smla_device_status_address.argtypes = [C.POINTER(C.c_void_p)]
    lib.smla_device_status_address.restype = C.c_int
    _lib = lib
    return lib


def check(rc: int, what: str = "smla call"):
    if rc != 0:
        raise RuntimeError(f"{what} failed: {load().smla_error_string(rc).decode()} (code {rc})")


def stream_from_tensors(cache, scale, indices, lens) -> SmlaStream:
    """Build one stream descriptor from torch CUDA tensors (cache [nb,bs,*], indices [T,topk])."""
    s = SmlaStream()
    s.cache = cache.data_ptr()
    s.scale = scale.data_ptr() if scale is not None else None
    s.indices = indices.data_ptr()
    s.lens = lens.data_ptr()
    s.indices_stride = indices.stride(0) if indices.shape[0] > 1 else indices.shape[1]
    s.topk = indices.shape[1]
    s.num_blocks = cache.shape[0]
    s.block_size = cache.shape[1]
    s.block_stride = cache.stride(0) * cache.element_size()
    if scale is not None:
        s.pos_stride = cache.stride(1)
        s.scale_block_stride = scale.stride(0)
        s.scale_pos_stride = scale.stride(1)
    else:
        s.pos_stride = 576
    return s


def attn_params(q, out, fmt: int, softmax_scale: float, swa: SmlaStream, extra: Optional[SmlaStream] = None,
                attn_sink=None, num_splits: int = 0, workspace=None) -> SmlaAttnParams:
    p = SmlaAttnParams()
    p.num_tokens, p.num_heads = q.shape[0], q.shape[1]
    p.cache_format = fmt
    p.softmax_scale = softmax_scale
    p.q, p.q_token_stride, p.q_head_stride = q.data_ptr(), q.stride(0), q.stride(1)
    p.out, p.out_token_stride, p.out_head_stride = out.data_ptr(), out.stride(0), out.stride(1)
    p.attn_sink = attn_sink.data_ptr() if attn_sink is not None else None
    p.swa = swa
    if extra is not None:
        p.extra = extra
    p.num_splits = num_splits
    if workspace is not None:
        p.workspace = workspace.data_ptr()
        p.workspace_bytes = workspace.numel() * workspace.element_size()
    return p


def dense_params(q, k_cache, block_table, cache_seqlens, out, lse=None, softmax_scale=None, causal=False,
                 num_splits: int = 0, workspace=None) -> SmlaDenseParams:
    """q [b, s_q, h, 576] contiguous bf16; k_cache [num_blocks, page, 1, 576] bf16; out [b, s_q, h, 512];
    lse fp32 [b, h, s_q] or None."""
    p = SmlaDenseParams()
    p.batch, p.seqlen_q, p.num_heads = q.shape[0], q.shape[1], q.shape[2]
    p.causal = 1 if causal else 0
    p.head_dim = q.shape[3]
    p.softmax_scale = softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5
    p.q, p.q_token_stride, p.q_head_stride = q.data_ptr(), q.stride(1), q.stride(2)
    p.out, p.out_token_stride, p.out_head_stride = out.data_ptr(), out.stride(1), out.stride(2)
    p.softmax_lse = lse.data_ptr() if lse is not None else None
    p.k_cache = k_cache.data_ptr()
    p.k_block_stride, p.k_row_stride = k_cache.stride(0) * 2, k_cache.stride(1) * 2
    p.num_blocks, p.page_block_size = k_cache.shape[0], k_cache.shape[1]
    p.block_table, p.block_table_stride = block_table.data_ptr(), block_table.stride(0)
    p.max_blocks_per_seq = block_table.shape[1]
    p.cache_seqlens = cache_seqlens.data_ptr()
    p.num_splits = num_splits
    if workspace is not None:
        p.workspace = workspace.data_ptr()
        p.workspace_bytes = workspace.numel() * workspace.element_size()
    return p
