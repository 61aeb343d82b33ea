"""Second oracle / GPU baseline (test infrastructure, not product): the REFERENCE's own sparse-MLA
CUDA kernels (Ampere mma.sync code, SASS for sm_100) run on the same GPU through
``oracle/_ref/libref_sparse_mla.so`` (built by ``oracle/ref_gpu/build_ref.py`` from the reference
checkout; absent on machines without it).  The host logic here restates what the reference binding
does around the launch: the split policy ``sparse_mla_num_splits`` (csrc/flash_api.cpp:75-102) and
the scratch tensors it allocates (csrc/flash_api.cpp:388-405, 496-508, 546-550).
"""
from __future__ import annotations

import ctypes as C
import os

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_ref", "libref_sparse_mla.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def _load():
    global _lib
    if _lib is None:
        from flash_mla import c_abi
        lib = C.CDLL(LIB_PATH)
        lib.ref_sparse_mla_decode.argtypes = [C.POINTER(c_abi.SmlaAttnParams), C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p]
        lib.ref_sparse_mla_prefill.argtypes = [C.POINTER(c_abi.SmlaAttnParams), C.c_void_p, C.c_void_p]
        _lib = lib
    return _lib


def ref_num_splits(sm_count: int, T: int, H: int, width: int) -> int:
    """csrc/flash_api.cpp:75-102 for the default (tensor-core) decode: 32 heads per CTA, one CTA per
    SM, 96 rows per split (FLASH_MLA_SLOTS_PER_SPLIT overrides), at most 64 splits."""
    head_blocks = (H + 31) // 32
    splits = sm_count // max(1, T * head_blocks)
    slots = int(os.environ.get("FLASH_MLA_SLOTS_PER_SPLIT", "0")) or 96
    cap = max(1, (width + slots - 1) // slots)
    return max(1, min(splits, min(64, cap)))


def _params(q, out, fmt_int8, scale, swa, extra, sink):
    from flash_mla import c_abi
    st = c_abi.stream_from_tensors
    return c_abi.attn_params(q, out, c_abi.SMLA_INT8_DS_MLA if fmt_int8 else c_abi.SMLA_FP8_DS_MLA, scale,
                             st(*swa), st(*extra) if extra is not None else None, sink)


class RefDecode:
    """Pre-allocates the reference's scratch once (the reference allocates per call) and launches."""

    def __init__(self, q, swa_cache, swa_scale, swa_indices, swa_lens, scale=None, attn_sink=None, extra_cache=None,
                 extra_scale=None, extra_indices=None, extra_lens=None):
        import torch
        self.lib = _load()
        T, H, _ = q.shape
        int8 = swa_scale is not None
        width = swa_indices.shape[1] + (extra_indices.shape[1] if extra_cache is not None else 0)
        sm = torch.cuda.get_device_properties(q.device).multi_processor_count
        self.S = ref_num_splits(sm, T, H, width)
        split = self.S > 1
        dev = q.device
        self.out = torch.empty_like(q)
        self.oaccum = torch.empty((T if split else 1, H, self.S, 512), dtype=torch.float32, device=dev)
        self.mlse = torch.empty((T if split else 1, H, self.S, 2), dtype=torch.float32, device=dev)
        self.counter = torch.zeros((T * ((H + 15) // 16) if split else 1,), dtype=torch.int32, device=dev)
        fused = int8 or split      # fp8 with one split falls to the reference's legacy FMA kernel
        self.sel_kv = torch.empty((T * width if fused else 1, 512), dtype=torch.bfloat16, device=dev)
        self.fused = fused
        self.keep = (q, swa_cache, swa_scale, swa_indices, swa_lens, attn_sink, extra_cache, extra_scale,
                     extra_indices, extra_lens)
        extra = (extra_cache, extra_scale, extra_indices, extra_lens) if extra_cache is not None else None
        self.p = _params(q, self.out, int8, scale if scale is not None else 512 ** -0.5,
                         (swa_cache, swa_scale, swa_indices, swa_lens), extra, attn_sink)

    def __call__(self):
        import torch
        rc = self.lib.ref_sparse_mla_decode(self.p, self.S, self.oaccum.data_ptr(), self.mlse.data_ptr(),
                                            self.counter.data_ptr(), self.sel_kv.data_ptr() if self.fused else None,
                                            torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"reference decode launch failed: cudaError {rc}")
        return self.out


class RefPrefill:
    """The reference's prefill launcher (csrc/flash_sparse_mla_prefill_fused_sm80.cu:468-506): for
    fp8_ds_mla it first dequantises the WHOLE cache into a dense bf16 buffer of swa + extra slots
    (allocated here once, csrc/flash_api.cpp:546-567), for int8_ds_mla the fused kernel gathers raw rows."""

    def __init__(self, q, swa_cache, swa_scale, swa_indices, swa_lens, scale=None, attn_sink=None, extra_cache=None,
                 extra_scale=None, extra_indices=None, extra_lens=None):
        import torch
        self.lib = _load()
        int8 = swa_scale is not None
        self.out = torch.empty_like(q)
        slots = swa_cache.shape[0] * swa_cache.shape[1]
        if extra_cache is not None:
            slots += extra_cache.shape[0] * extra_cache.shape[1]
        self.kv = None if int8 else torch.empty((slots, 512), dtype=torch.bfloat16, device=q.device)
        self.keep = (q, swa_cache, swa_scale, swa_indices, swa_lens, attn_sink, extra_cache, extra_scale,
                     extra_indices, extra_lens)
        extra = (extra_cache, extra_scale, extra_indices, extra_lens) if extra_cache is not None else None
        self.p = _params(q, self.out, int8, scale if scale is not None else 512 ** -0.5,
                         (swa_cache, swa_scale, swa_indices, swa_lens), extra, attn_sink)

    def __call__(self):
        import torch
        rc = self.lib.ref_sparse_mla_prefill(self.p, self.kv.data_ptr() if self.kv is not None else None,
                                             torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"reference prefill launch failed: cudaError {rc}")
        return self.out
