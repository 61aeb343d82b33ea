"""Writers for the two paged cache formats the sparse-MLA kernels read.

``write_fp8_ds_mla_cache`` / ``write_int8_ds_mla_cache`` are the CUDA writers: one kernel encodes a
batch of new latent rows and scatters them to their slots of a paged cache (the step right before
the attention calls).  ``pack_fp8_ds_mla`` / ``pack_int8_inline528`` are torch composites that build
a whole cache on any device; the synthetic workloads and the CPU tests use them.

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
    # Smallest e with amax <= 448 * 2**e, exactly: amax = m * 2**k, m in [0.5, 1), 448 = 0.875 * 2**9.
    m, k = torch.frexp(amax)
    exps = torch.where(m <= 0.875, k - 9, k - 8)
    exps = torch.where(amax > 0, exps, torch.zeros_like(exps)).clamp(-120, 120).to(torch.float32)
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


def _check_writer_args(latent, slot_mapping, cache, token_bytes):
    if latent.dim() != 2 or latent.shape[1] != HEAD_DIM:
        raise ValueError(f"expected latent [rows, {HEAD_DIM}], got {tuple(latent.shape)}")
    if slot_mapping.dim() != 1 or slot_mapping.shape[0] != latent.shape[0]:
        raise ValueError(f"expected slot_mapping [{latent.shape[0]}], got {tuple(slot_mapping.shape)}")
    if cache.dim() != 3 or cache.shape[2] != token_bytes or cache.element_size() != 1:
        raise ValueError(f"expected a byte cache [num_blocks, block_size, {token_bytes}], got {tuple(cache.shape)}")
    from ._loader import load_torch_extension
    load_torch_extension()


def write_int8_ds_mla_cache(latent: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor,
                            scale_rule: str = "quantizer") -> None:
    """Quantise ``latent`` [rows, 512] (bf16 / fp16 / fp32, CUDA) and write row i to slot
    ``slot_mapping[i]`` (int32 / int64; block ``slot // block_size``, position ``slot % block_size``) of
    ``cache`` uint8 [num_blocks, block_size, 528], in place: 512 int8, the fp32 row scale, 12 zero
    bytes.  Rows with a negative or out-of-range slot are skipped.  ``scale_rule`` "quantizer" gives the
    bytes of ``quantize_int8_ds_mla_rows`` (scale = max(amax, 1e-12) / 127); "writer" uses
    scale = max(amax / 127, 1e-12), the serving engine's writer as the reference's tests restate it
    (tests/test_sparse_mla_prefill_int8_adversarial.py:35-40)."""
    _check_writer_args(latent, slot_mapping, cache, INT8_TOKEN_BYTES)
    rule = {"quantizer": 0, "writer": 1}[scale_rule]
    torch.ops.flash_mla.write_int8_ds_mla_cache(latent, slot_mapping, cache, rule)


def write_fp8_ds_mla_cache(latent: torch.Tensor, slot_mapping: torch.Tensor, cache: torch.Tensor) -> None:
    """Encode ``latent`` [rows, 512] (448 NoPE + 64 RoPE elements; bf16 / fp16 / fp32, CUDA) and write
    row i to slot ``slot_mapping[i]`` of ``cache`` uint8 [num_blocks, block_size, 584], in place, with the
    bytes ``pack_fp8_ds_mla`` produces for that row.  Rows with a negative or out-of-range slot are
    skipped."""
    _check_writer_args(latent, slot_mapping, cache, TOKEN_BYTES)
    torch.ops.flash_mla.write_fp8_ds_mla_cache(latent, slot_mapping, cache)


def int8_ds_mla_cache_views(cache: torch.Tensor):
    """uint8 [nb, bs, 528] -> (int8 rows [nb, bs, 512] with token stride 528, fp32 scales [nb, bs]
    with token stride 132): the two strided views the int8 attention entry points take."""
    return cache[:, :, :HEAD_DIM].view(torch.int8), cache[:, :, HEAD_DIM:HEAD_DIM + 4].view(torch.float32).squeeze(-1)
