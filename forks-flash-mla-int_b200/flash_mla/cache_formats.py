"""Writers for the two paged cache formats the sparse-MLA kernels read (torch ops, any device).

The reference ships no production writer (the vLLM fork owns it); its tests and benchmarks
build caches with ad-hoc packers (tests/test_sparse_mla_decode_sm86.py:23-44,
benchmarks/bench_sparse_mla_decode_16k.py:33-58, tests/test_sparse_mla_prefill_int8_adversarial.py:44-74).
These follow the same byte layouts:

``fp8_ds_mla``  uint8 [num_blocks, block_size, 584]; a block is ``[bs x 576 data][bs x 8 scale]``,
                data = 448 e4m3 + 64 bf16 (RoPE), scale = 7 UE8M0 bytes + 1 pad byte (127).
``int8_ds_mla`` 528-byte tokens: 512 int8 + fp32 scale at +512 + 12 pad, exposed as two strided views.
"""
from __future__ import annotations

import torch

HEAD_DIM = 512
FP8_DIM = 448
ROPE_DIM = 64
SCALE_GROUP = 64
TOKEN_DATA = FP8_DIM + 2 * ROPE_DIM   # 576
TOKEN_BYTES = TOKEN_DATA + 8          # 584
INT8_TOKEN_BYTES = 528


def pack_fp8_ds_mla(latent: torch.Tensor, block_size: int) -> torch.Tensor:
    """latent [N, 512] (any float dtype; RoPE tail stored as bf16) -> uint8 [ceil(N/bs), bs, 584].

    Per 64-dim NoPE group the UE8M0 exponent is the smallest power of two with
    ``amax / 2**e <= 448``; slots past N are zero bytes (they dequantise to zero rows).
    """
    if latent.shape[-1] != HEAD_DIM or latent.dim() != 2:
        raise ValueError(f"expected [N, {HEAD_DIM}], got {tuple(latent.shape)}")
    n, dev = latent.shape[0], latent.device
    nb = (n + block_size - 1) // block_size
    total = nb * block_size
    x = latent.float()
    nope = x[:, :FP8_DIM].view(n, FP8_DIM // SCALE_GROUP, SCALE_GROUP)
    amax = nope.abs().amax(dim=-1)
    exps = torch.where(amax > 0, torch.ceil(torch.log2(amax.clamp_min(1e-30) / 448.0)), torch.zeros_like(amax))
    exps = exps.clamp(-120, 120)
    codes = (nope / torch.exp2(exps).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    data = torch.zeros(total, TOKEN_DATA, dtype=torch.uint8, device=dev)
    data[:n, :FP8_DIM] = codes.view(torch.uint8).view(n, FP8_DIM)
    data[:n, FP8_DIM:] = x[:, FP8_DIM:].to(torch.bfloat16).contiguous().view(torch.uint8).view(n, 2 * ROPE_DIM)
    sc = torch.zeros(total, 8, dtype=torch.uint8, device=dev)
    sc[:n, :7] = (exps + 127).to(torch.uint8)
    sc[:n, 7] = 127
    cache = torch.empty(nb, block_size * TOKEN_BYTES, dtype=torch.uint8, device=dev)
    cache[:, : block_size * TOKEN_DATA] = data.view(nb, block_size * TOKEN_DATA)
    cache[:, block_size * TOKEN_DATA:] = sc.view(nb, block_size * 8)
    return cache.view(nb, block_size, TOKEN_BYTES)


def pack_int8_inline528(q: torch.Tensor, scale: torch.Tensor, block_size: int):
    """int8 rows [N, 512] + fp32 scales [N] -> (buffer uint8 [nb, bs, 528], int8 view [nb, bs, 512]
    with token stride 528, fp32 scale view [nb, bs] with token stride 132)."""
    n, dev = q.shape[0], q.device
    nb = (n + block_size - 1) // block_size
    buf = torch.zeros(nb * block_size, INT8_TOKEN_BYTES, dtype=torch.uint8, device=dev)
    buf[:n, :HEAD_DIM] = q.view(torch.uint8)
    buf[:n, HEAD_DIM:HEAD_DIM + 4] = scale.to(torch.float32).contiguous().view(n, 1).view(torch.uint8)
    buf = buf.view(nb, block_size, INT8_TOKEN_BYTES)
    data_view = buf[:, :, :HEAD_DIM].view(torch.int8)
    scale_view = buf[:, :, HEAD_DIM:HEAD_DIM + 4].view(torch.float32).squeeze(-1)
    return buf, data_view, scale_view
