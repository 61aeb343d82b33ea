"""fp32 CPU oracle of sparse MLA attention (test infrastructure, not product).

Restates the reference's canonical oracle ``_ref``
(tests/test_sparse_mla_prefill_adversarial.py:25-53) and its single-stream sibling
``_fp32_ref`` (tests/test_sparse_mla_decode_sm86.py:52-72):

* per token the selected rows are ``swa[:swa_len] ++ extra[:extra_len]``;
* a slot id < 0 or >= the stream's slot count is an ALL-ZERO ROW that stays inside the
  softmax (score 0, weight exp(0 - m) in the denominator, nothing in the numerator);
* ``attn_sink`` is one extra logit per head with no value row: it joins the max and adds
  ``exp(sink - m)`` to the denominator once;
* a token with no selected rows outputs zeros;
* everything is fp32 over the dequantised (bf16-representable) rows; V == K.
"""
from __future__ import annotations

import numpy as np
import torch


def cos_diff(x, y) -> float:
    """1 - 2<x,y> / (|x|^2 + |y|^2) in fp64 (tests/test_sparse_mla_decode_sm86.py:47-49)."""
    x = torch.as_tensor(np.asarray(x)).double()
    y = torch.as_tensor(np.asarray(y)).double()
    return 1 - 2 * (x * y).sum().item() / max((x * x + y * y).sum().item(), 1e-12)


def _t(a, dtype=None):
    if a is None:
        return None
    if isinstance(a, torch.Tensor):
        t = a.detach().cpu()
    else:
        t = torch.from_numpy(np.ascontiguousarray(a))
    return t.to(dtype) if dtype is not None else t


def _stream_rows(K, idx_row, n):
    sl = idx_row[:n].long()
    ok = (sl >= 0) & (sl < K.shape[0])
    r = torch.zeros(n, K.shape[1], dtype=torch.float32)
    r[ok] = K[sl[ok]]
    return r


def sparse_mla_attention(q, swa_K, swa_idx, swa_lens, extra_K=None, extra_idx=None,
                         extra_lens=None, scale=None, sink=None, tokens=None) -> np.ndarray:
    """q [T,H,512] (bf16 values); *_K fp32 rows [slots,512]; idx int32 [T,topk]; lens int32 [T].

    ``sink`` fp32 [H] or None.  ``tokens`` optionally restricts the computation to a list of
    token positions (used to time a bounded sample); other tokens' outputs are left zero.
    Returns fp32 [T,H,512].
    """
    q = _t(q, torch.float32)
    swa_K = _t(swa_K, torch.float32)
    extra_K = _t(extra_K, torch.float32)
    swa_idx, swa_lens = _t(swa_idx), _t(swa_lens)
    extra_idx, extra_lens = _t(extra_idx), _t(extra_lens)
    sink = _t(sink, torch.float32)
    T, H, D = q.shape
    if scale is None:
        scale = D ** -0.5
    out = torch.zeros(T, H, D, dtype=torch.float32)
    for t in (range(T) if tokens is None else tokens):
        ns = int(swa_lens[t])
        ne = int(extra_lens[t]) if extra_lens is not None else 0
        rows = []
        if ns:
            rows.append(_stream_rows(swa_K, swa_idx[t], ns))
        if ne:
            rows.append(_stream_rows(extra_K, extra_idx[t], ne))
        if not rows:
            continue
        K = torch.cat(rows)
        sc = (q[t] @ K.t()) * scale
        m = sc.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[:, None])
        ex = torch.exp(sc - m)
        den = ex.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[:, None] - m)
        out[t] = (ex @ K) / den
    return out.numpy()
