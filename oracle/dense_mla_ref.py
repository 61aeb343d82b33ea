"""fp32 CPU oracle of dense paged MLA decode (test infrastructure, not product).

Restates the oracle of the reference's dense test (tests/test_flash_mla_sm80.py:10-27 for the
attention itself, :75-93 for how a sequence's rows are taken out of the paged cache):

* sequence ``b`` attends to rows ``0 .. cache_seqlens[b] - 1`` of its own pages, found through
  ``block_table[b]``; rows past the length are never read (the reference's test poisons them with NaN);
* scores run over all ``d`` = 576 dims, values are the first ``dv`` = 512 dims of the same rows, one kv head;
* the scale defaults to ``d ** -0.5``;
* with ``causal`` query position ``i`` of ``s_q`` sees rows ``0 .. len - s_q + i`` (``tril(diagonal=s_k - s_q)``);
* ``lse`` is the natural-log sum of exponentials of the scaled scores.
"""
from __future__ import annotations

import numpy as np
import torch

from .sparse_mla_ref import _t


def dense_mla_decode(q, k_cache, block_table, cache_seqlens, dv=512, causal=False, softmax_scale=None,
                     sequences=None):
    """q [b, s_q, h, d] (bf16 values); k_cache [num_blocks, page, 1, d]; block_table int32 [b, max_blocks];
    cache_seqlens int32 [b].  ``sequences`` optionally restricts the computation to some batch entries (the
    others' outputs stay zero).  Returns (out fp32 [b, s_q, h, dv], lse fp32 [b, h, s_q])."""
    q = _t(q, torch.float32)
    k_cache = _t(k_cache)
    block_table = _t(block_table).long()
    lens = _t(cache_seqlens).long()
    B, SQ, H, D = q.shape
    page = k_cache.shape[1]
    scale = float(softmax_scale) if softmax_scale is not None else D ** -0.5
    out = torch.zeros(B, SQ, H, dv, dtype=torch.float32)
    lse = torch.zeros(B, H, SQ, dtype=torch.float32)
    rows_of = k_cache.reshape(k_cache.shape[0], page, D)
    for b in (range(B) if sequences is None else sequences):
        n = int(lens[b])
        pages = block_table[b, : (n + page - 1) // page]
        K = rows_of[pages].reshape(-1, D)[:n].float()                     # [n, d]
        s = torch.einsum("ihd,nd->hin", q[b], K) * scale                  # [h, s_q, n]
        if causal and SQ > 1:
            keep = torch.ones(SQ, n, dtype=torch.bool).tril(diagonal=n - SQ)
            s = s.masked_fill(~keep, float("-inf"))
        lse[b] = torch.logsumexp(s, dim=-1)
        p = torch.softmax(s, dim=-1, dtype=torch.float32)
        p = torch.nan_to_num(p, nan=0.0)                                  # a query that sees no row
        out[b] = torch.einsum("hin,nv->ihv", p, K[:, :dv])
    return out.numpy(), lse.numpy()
