#!/usr/bin/env python3
"""Generate the golden fixtures in this directory FROM THE REFERENCE'S OWN PYTHON CODE.

Run once in a container that has the reference checkout (path in REFERENCE_ROOT, else a
directory named ``reference`` beside this repository); the .npz files it writes are committed and are the only
thing the tests read.  Imported from the reference (nothing is copied):

* ``_ref``                      tests/test_sparse_mla_prefill_adversarial.py:25-53
* ``_fp32_ref``, ``_build_cache`` tests/test_sparse_mla_decode_sm86.py:52-72,110-116
* ``build_cache_fast``          benchmarks/bench_sparse_mla_decode_16k.py:33-58
* ``_build_inline_cache``, ``_build_separate_cache``
                                tests/test_sparse_mla_prefill_int8_adversarial.py:44-74
* ``quantize_int8_ds_mla_rows`` flash_mla/int8_sparse_mla.py:15-26 (loaded by file path,
                                the package __init__ needs the compiled extension)
* ``scaled_dot_product_attention`` tests/test_flash_mla_sm80.py:10-27 (that file imports the compiled
                                package at its top; an empty stand-in module named ``flash_mla`` lets the
                                import go through, the oracle function itself needs nothing from it)

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $REFERENCE_ROOT, else a directory named "reference" beside this repository
REF = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")
sys.path.insert(0, os.path.join(REF, "tests"))
sys.path.insert(0, os.path.join(REF, "benchmarks"))

from test_sparse_mla_prefill_adversarial import _ref  # noqa: E402
from test_sparse_mla_decode_sm86 import _fp32_ref, _build_cache  # noqa: E402
from test_sparse_mla_prefill_int8_adversarial import (  # noqa: E402
    _build_inline_cache, _build_separate_cache)
from bench_sparse_mla_decode_16k import build_cache_fast  # noqa: E402

_spec = importlib.util.spec_from_file_location(
    "ref_int8_sparse_mla", os.path.join(REF, "flash_mla", "int8_sparse_mla.py"))
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
ref_quantize = _mod.quantize_int8_ds_mla_rows


import types  # noqa: E402

if "flash_mla" not in sys.modules:
    _stub = types.ModuleType("flash_mla")
    _stub.get_mla_metadata = _stub.flash_mla_with_kvcache = None
    sys.modules["flash_mla"] = _stub
from test_flash_mla_sm80 import scaled_dot_product_attention as ref_dense_sdpa  # noqa: E402


def bits(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def save(name, **kw):
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **kw)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def quantizer_kat():
    torch.manual_seed(5)
    x = torch.randn(96, 512)
    x[5:10] *= 50.0                       # outlier rows
    x[10] = 0.0                           # all-zero row (amax clamp 1e-12)
    x[11] = 1e-20                         # tiny row
    x[12] = torch.arange(512) % 255 - 127.0   # integers: scale exactly 1
    x[13] = (torch.arange(512) % 254 - 127.0) + 0.5   # exact .5 ties at scale 1 ... 127.5 amax
    x[13, 0] = 127.0
    x[13, 1:] = x[13, 1:].clamp(-126.5, 126.5)
    x[14, :] = 3.0
    x[14, 7] = -381.0                     # negative amax
    xb = x.to(torch.bfloat16)
    q, s = ref_quantize(xb)
    # leading dims are arbitrary in the reference: pin a 3-D call too
    q3, s3 = ref_quantize(xb.view(4, 24, 512))
    assert torch.equal(q3.view(96, 512), q) and torch.equal(s3.view(96), s)
    save("quantizer_kat.npz", x_bf16=bits(xb), q=q.numpy(), scale=s.numpy())


def fp8_decode_single():
    torch.manual_seed(0)
    T, H, topk, bs = 2, 64, 256, 32
    num_slots = topk + 64
    cache, K = _build_cache(num_slots, bs, "cpu")
    q = torch.randn(T, H, 512, dtype=torch.bfloat16)
    lens = torch.tensor([topk, topk - 7], dtype=torch.int32)
    idx = torch.stack([torch.randperm(num_slots)[:topk].to(torch.int32) for _ in range(T)])
    sink = torch.randn(H) * 0.1
    scale = 1.0 / math.sqrt(512)
    out = _fp32_ref(q, K, idx, lens, scale, sink)
    out_nosink = _fp32_ref(q, K, idx, lens, scale, None)
    save("fp8_decode_single.npz", q=bits(q), cache=cache.numpy(), K=bits(K), idx=idx.numpy(),
         lens=lens.numpy(), sink=sink.numpy(), scale=np.float64(scale), out=out.numpy(),
         out_nosink=out_nosink.numpy())


def _two_stream_inputs(seed, T, H, swa_topk, extra_topk, swa_slots, extra_slots):
    torch.manual_seed(seed)
    q = torch.randn(T, H, 512, dtype=torch.bfloat16)
    specials = [0, 1, 15, 16, 17, 31, 32, 33, 63, 64, 65, swa_topk]
    swa_lens = torch.randint(0, swa_topk + 1, (T,), dtype=torch.int32)
    extra_lens = torch.randint(0, extra_topk + 1, (T,), dtype=torch.int32)
    for i, v in enumerate(specials):
        swa_lens[i] = min(v, swa_topk)
        extra_lens[-1 - i] = min(v, extra_topk)
    swa_lens[0] = 0
    extra_lens[0] = 0                      # a token with no rows at all -> zeros
    swa_idx = torch.randint(0, swa_slots, (T, swa_topk), dtype=torch.int32)
    extra_idx = torch.randint(0, extra_slots, (T, extra_topk), dtype=torch.int32)
    swa_idx[3, 2] = -1
    swa_idx[4, 0] = swa_slots + 5
    extra_idx[5, 1] = -1
    swa_idx[-1, 0] = -1                    # invalid ids on a full-length token
    sink = torch.randn(H) * 0.1
    return q, swa_idx, swa_lens, extra_idx, extra_lens, sink


def fp8_two_stream():
    T, H, st, et = 16, 16, 160, 96
    swa_cache, swa_K = _build_cache(st + 40, 32, "cpu")
    extra_cache, extra_K = _build_cache(et + 40, 16, "cpu")
    q, si, sl, ei, el, sink = _two_stream_inputs(7, T, H, st, et, swa_K.shape[0], extra_K.shape[0])
    scale = 1.0 / math.sqrt(512)
    out = _ref(q, swa_K, si, sl, extra_K, ei, el, scale, sink)
    save("fp8_two_stream.npz", q=bits(q), swa_cache=swa_cache.numpy(), swa_K=bits(swa_K),
         extra_cache=extra_cache.numpy(), extra_K=bits(extra_K), swa_idx=si.numpy(),
         swa_lens=sl.numpy(), extra_idx=ei.numpy(), extra_lens=el.numpy(), sink=sink.numpy(),
         scale=np.float64(scale), out=out.numpy())


def int8_two_stream():
    T, H, st, et = 16, 16, 160, 96
    scale = 1.0 / math.sqrt(512)
    for layout, build in (("inline528", _build_inline_cache), ("separate", _build_separate_cache)):
        torch.manual_seed(21)
        swa_cache, swa_scale, swa_K = build(st + 40, 64, "cpu")
        extra_cache, extra_scale, extra_K = build(et + 40, 16, "cpu")
        q, si, sl, ei, el, sink = _two_stream_inputs(23, T, H, st, et, swa_K.shape[0], extra_K.shape[0])
        out = _ref(q, swa_K, si, sl, extra_K, ei, el, scale, sink)
        save(f"int8_two_stream_{layout}.npz", q=bits(q),
             swa_q=swa_cache.contiguous().numpy(), swa_scale=swa_scale.contiguous().numpy(),
             swa_K=bits(swa_K), extra_q=extra_cache.contiguous().numpy(),
             extra_scale=extra_scale.contiguous().numpy(), extra_K=bits(extra_K),
             swa_idx=si.numpy(), swa_lens=sl.numpy(), extra_idx=ei.numpy(), extra_lens=el.numpy(),
             sink=sink.numpy(), scale=np.float64(scale), out=out.numpy())


def config1_cpu_oracle():
    """BASELINE config 1: T=4, H=16, 4096-slot fp8_ds_mla cache, top-k 128, ~2% -1 and ~1%
    out-of-range ids, lens uniform in [1,128], scale=None, no sink, no extra stream, seed 0."""
    torch.manual_seed(0)
    T, H, slots, topk, bs = 4, 16, 4096, 128, 64
    cache, K = build_cache_fast(slots, bs, "cpu", seed=0)
    q = torch.randn(T, H, 512, dtype=torch.bfloat16)
    idx = torch.stack([torch.randperm(slots)[:topk].to(torch.int32) for _ in range(T)])
    r = torch.rand(T, topk)
    idx[r < 0.02] = -1
    big = (r >= 0.02) & (r < 0.03)
    idx[big] = slots + torch.randint(0, 1000, (int(big.sum()),), dtype=torch.int32)
    lens = torch.randint(1, topk + 1, (T,), dtype=torch.int32)
    scale = 512 ** -0.5
    no_sink = torch.full((H,), float("-inf"))
    out = _ref(q, K, idx, lens, None, None, None, scale, no_sink)
    save("config1_cpu_oracle.npz", q=bits(q), cache=cache.numpy(), idx=idx.numpy(),
         lens=lens.numpy(), out=out.numpy())


def dense_mla_small():
    """The dense test's oracle (tests/test_flash_mla_sm80.py:75-93) on a small ragged batch: three sequences,
    two query positions, 16 heads, pages of 32 rows, rows past each length poisoned with NaN as there."""
    torch.manual_seed(11)
    b, s_q, h_q, h_kv, d, dv, block_size = 3, 2, 16, 1, 576, 512, 32
    cache_seqlens = torch.tensor([70, 300, 129], dtype=torch.int32)
    max_seqlen_pad = 512
    q = torch.randn(b, s_q, h_q, d).to(torch.bfloat16)
    # pages in a scrambled order so that the block table matters
    perm = torch.randperm(b * max_seqlen_pad // block_size)
    block_table = perm.to(torch.int32).view(b, max_seqlen_pad // block_size)
    blocked_k = torch.zeros(perm.numel(), block_size, h_kv, d, dtype=torch.bfloat16)
    seq_rows = torch.randn(b, max_seqlen_pad, h_kv, d).to(torch.bfloat16)
    for i in range(b):
        seq_rows[i, cache_seqlens[i].item():] = float("nan")
        blocked_k[block_table[i].long()] = seq_rows[i].view(-1, block_size, h_kv, d)
    res = {}
    for causal in (False, True):
        out = torch.empty(b, s_q, h_q, dv, dtype=torch.float32)
        lse = torch.empty(b, h_q, s_q, dtype=torch.float32)
        for i in range(b):
            n = cache_seqlens[i].item()
            O, LSE = ref_dense_sdpa(q[i].transpose(0, 1), seq_rows[i, :n].transpose(0, 1),
                                    seq_rows[i, :n, :, :dv].transpose(0, 1), h_q=h_q, h_kv=h_kv, is_causal=causal)
            out[i] = O.transpose(0, 1)
            lse[i] = LSE
        res["out_causal" if causal else "out"] = out.numpy()
        res["lse_causal" if causal else "lse"] = lse.numpy()
    save("dense_mla_small.npz", q_bf16=bits(q), k_cache_bf16=bits(blocked_k), block_table=block_table.numpy(),
         cache_seqlens=cache_seqlens.numpy(), **res)


if __name__ == "__main__":
    torch.set_num_threads(8)
    quantizer_kat()
    fp8_decode_single()
    fp8_two_stream()
    int8_two_stream()
    config1_cpu_oracle()
    dense_mla_small()
