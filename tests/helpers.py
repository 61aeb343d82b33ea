"""Shared helpers for the GPU parity tests: cache builders (oracle packers -> device tensors),
the oracle call on device inputs, and the tolerance checks.

Tolerances (stated once).  Outputs are bf16 and P is rounded to bf16 before PV (as in the
reference kernels), so an output of magnitude x carries an error of up to about x * 2^-7 whatever
the implementation: the golden fixtures built with the reference's deterministic packer reach
|x| = 20 and the x50 outlier rows of BASELINE config 3 reach |x| = 160, where a CPU emulation of the
algorithm (bf16 P, fp32 accumulation, bf16 output) is already 1.0 away from the fp32 oracle.  Bounds:
    |out - ref| <= 2e-2 + 2e-2 |ref| + 2^-7 max_d |ref[t, h, :]|   elementwise: the reference's own gate,
                                       assert_close(rtol=2e-2, atol=2e-2), tests/test_sparse_mla_prefill_adversarial.py:92-95,
                                       plus one bf16 quantum of the (token, head) output row: where a few
                                       large rows nearly cancel, the bf16 rounding of their weights is an
                                       error relative to THEIR size, not to the small result
    mean|out - ref| <= 2e-3 + 2^-8 mean|ref|
    cos_diff < 8e-5                    (the reference's gate, same file)
and, for N(0,1)-scale workloads without outlier rows (``strict_abs=True``), the plain north-star
bounds max-abs <= 2e-2 and mean-abs <= 2e-3.
"""
from __future__ import annotations

import numpy as np
import torch

import oracle

MAX_ABS = 2e-2
MEAN_ABS = 2e-3
COS_DIFF = 8e-5


def bf16_from_bits(bits: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)


def to_dev(a, device="cuda"):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)


def fp8_cache_from_latent(latent_f32: np.ndarray, block_size: int, device="cuda"):
    """-> (cache uint8 tensor [nb, bs, 584] on device, K fp32 numpy [nb*bs, 512])."""
    cache, K = oracle.pack_fp8_ds_mla(latent_f32, block_size)
    return to_dev(cache, device), K


def int8_cache_from_latent(latent_f32: np.ndarray, block_size: int, layout: str, device="cuda"):
    """-> (int8 cache view, fp32 scale view, K fp32 numpy, backing buffer or None)."""
    q, s = oracle.quantize_int8_rows(oracle.ds_mla_formats.round_to_bf16(latent_f32))
    n = q.shape[0]
    nb = (n + block_size - 1) // block_size
    K = np.zeros((nb * block_size, 512), np.float32)
    K[:n] = oracle.dequant_int8_ds_mla(q, s)
    if layout == "inline528":
        buf = to_dev(oracle.pack_int8_inline528(q, s, block_size), device)
        data = buf[:, :, :512].view(torch.int8)
        scale = buf[:, :, 512:516].view(torch.float32).squeeze(-1)
        return data, scale, K, buf
    qp = np.zeros((nb * block_size, 512), np.int8)
    sp = np.zeros((nb * block_size,), np.float32)
    qp[:n], sp[:n] = q, s
    return (to_dev(qp.reshape(nb, block_size, 512), device), to_dev(sp.reshape(nb, block_size), device), K, None)


def oracle_out(q, swa_K, swa_idx, swa_lens, extra_K=None, extra_idx=None, extra_lens=None, scale=None, sink=None,
               tokens=None):
    def n(x):
        if x is None:
            return None
        return x.detach().float().cpu().numpy() if x.dtype in (torch.bfloat16, torch.float32) else x.detach().cpu().numpy()
    return oracle.sparse_mla_attention(n(q), swa_K, n(swa_idx), n(swa_lens), extra_K, n(extra_idx), n(extra_lens),
                                       scale=scale, sink=n(sink), tokens=tokens)


def assert_attention_close(out: torch.Tensor, ref: np.ndarray, what="", tokens=None, strict_abs=False):
    got = out.detach().float().cpu().numpy()
    if tokens is not None:
        got, ref = got[tokens], ref[tokens]
    assert not np.isnan(got).any(), f"{what}: NaN in output"
    d = np.abs(got - ref)
    cd = oracle.cos_diff(got, ref) if (np.any(ref) or np.any(got)) else 0.0      # all-zero vs all-zero: equal
    excess = (d - (MAX_ABS + 2e-2 * np.abs(ref) + 2.0 ** -7 * np.abs(ref).max(-1, keepdims=True))).max()
    assert excess <= 0, f"{what}: error exceeds atol 2e-2 + rtol 2e-2 + row quantum by {excess:.3e} (max-abs {d.max():.3e})"
    mean_bound = MEAN_ABS + 2.0 ** -8 * np.abs(ref).mean()
    assert d.mean() <= mean_bound, f"{what}: mean-abs {d.mean():.3e} > {mean_bound:.3e}"
    assert cd < COS_DIFF, f"{what}: cos_diff {cd:.3e} >= {COS_DIFF}"
    if strict_abs:
        assert d.max() <= MAX_ABS, f"{what}: max-abs {d.max():.3e} > {MAX_ABS}"
        assert d.mean() <= MEAN_ABS, f"{what}: mean-abs {d.mean():.3e} > {MEAN_ABS}"


def device_status() -> int:
    import ctypes
    from flash_mla import c_abi
    s = ctypes.c_int(0)
    rc = c_abi.load().smla_read_device_status(ctypes.byref(s))
    assert rc == 0, rc
    return s.value
