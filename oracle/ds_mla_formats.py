"""Byte formats of the sparse-MLA caches, restated in numpy (CPU oracle; test infrastructure).

``fp8_ds_mla`` (reference: docs/sparse_mla_decode_sm86_design.md:23-31,
csrc/flash_sparse_mla_decode_sm80.cu:23-50, tests/test_sparse_mla_decode_sm86.py:14-44):
a paged block of ``bs`` tokens is ``[bs x 576 data bytes][bs x 8 scale bytes]``.
A token's data record is 448 e4m3 bytes (NoPE) + 64 little-endian bf16 (RoPE); its
scale record is 7 UE8M0 bytes (one per 64 NoPE dims) + 1 pad byte.
``K[d] = e4m3(byte[d]) * 2**(scale[d // 64] - 127)`` for d < 448, ``K[448 + j] = rope[j]``.

``int8_ds_mla`` (reference: README.md:166-172, csrc/flash_sparse_mla_decode_sm80.cu:159-175,
tests/test_sparse_mla_prefill_int8_adversarial.py:44-74): 512 int8 per token plus one
fp32 scale; ``K[d] = bf16_rn(float(int8[d]) * scale)``.  The production container is a
528-byte token (512 payload, fp32 scale at +512, 12 pad bytes).

Cache writers (``write_fp8_ds_mla``, ``write_int8_inline528``): the reference has no writer, only
test-side packers that take the fp8 exponents as given, so the exponent rule here
(``ue8m0_exponents``: the smallest power of two that keeps the group within +-448) is this project's
own and is pinned only through the format: rows the reference's packers produced re-encode to caches
that dequantise to the same rows (tests/test_gpu_cache_writers.py), and the int8 tokens are the
reference quantizer's known answers laid out as its tests describe the serving engine's token.

Row quantizer (reference: flash_mla/int8_sparse_mla.py:15-26):
``scale = max(amax|x|, 1e-12) / 127`` and ``q = clamp(rint(x / scale), -127, 127)``, all in
IEEE fp32 with true division and round-half-even.
"""
from __future__ import annotations

import numpy as np

HEAD_DIM = 512
FP8_DIM = 448
ROPE_DIM = 64
SCALE_GROUP = 64
N_GROUPS = FP8_DIM // SCALE_GROUP  # 7
SCALE_BYTES = 8
TOKEN_DATA = FP8_DIM + 2 * ROPE_DIM  # 576
TOKEN_BYTES_FP8 = TOKEN_DATA + SCALE_BYTES  # 584
INT8_TOKEN_BYTES = 528


def _make_e4m3_lut() -> np.ndarray:
    """Value of every e4m3fn byte: 1 sign, 4 exponent (bias 7), 3 mantissa; 0x7f/0xff = NaN."""
    lut = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = float("nan")
        elif e == 0:
            v = (m / 8.0) * 2.0 ** -6
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        lut[b] = s * v
    return lut


E4M3_LUT = _make_e4m3_lut()
_E4M3_POS = E4M3_LUT[:0x7F].astype(np.float64)  # codes 0..126, strictly increasing, max 448


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))
    return (r >> 16).astype(np.uint16)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def encode_e4m3(x: np.ndarray) -> np.ndarray:
    """Nearest e4m3fn code with ties to even, saturating at +-448."""
    a = np.abs(x.astype(np.float64))
    a = np.minimum(a, 448.0)
    hi = np.searchsorted(_E4M3_POS, a, side="left")
    hi = np.clip(hi, 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    dlo = a - _E4M3_POS[lo]
    dhi = _E4M3_POS[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    sign = np.signbit(x).astype(np.uint8) << 7
    return code | sign


def ue8m0_exponents(groups: np.ndarray) -> np.ndarray:
    """fp32 [..., 64] -> int32 [...]: the smallest power-of-two exponent e with
    ``amax|group| <= 448 * 2**e``, clamped to [-120, 120]; 0 for an all-zero group.
    Exact (no logarithm): amax = m * 2**k with m in [0.5, 1) and 448 = 0.875 * 2**9, so
    e = k - 9 when m <= 0.875 and k - 8 otherwise."""
    amax = np.abs(np.asarray(groups, dtype=np.float32)).max(axis=-1)
    m, k = np.frexp(amax)
    e = np.where(m <= np.float32(0.875), k - 9, k - 8)
    e = np.where(amax > 0, e, 0)
    return np.clip(e, -120, 120).astype(np.int32)


def pack_fp8_ds_mla(latent: np.ndarray, block_size: int, exps: np.ndarray | None = None):
    """Pack fp32 rows [N, 512] (bf16-representable RoPE tail) into a paged fp8_ds_mla cache.

    ``exps`` [N, 7] are the per-64-group power-of-two exponents; when None the smallest
    exponent with ``amax / 2**e <= 448`` is used (``ue8m0_exponents``).  The reference ships no production
    writer, so this choice is ours; parity is defined on ``dequant(bytes)``.
    Returns ``(cache uint8 [nb, bs, 584], K fp32 [nb * bs, 512])`` with K the exact
    dequantised rows.  Slots past N are zero bytes (dequantise to zero rows).
    """
    latent = np.asarray(latent, dtype=np.float32)
    n = latent.shape[0]
    nb = (n + block_size - 1) // block_size
    total = nb * block_size
    nope = latent[:, :FP8_DIM].reshape(n, N_GROUPS, SCALE_GROUP)
    if exps is None:
        exps = ue8m0_exponents(nope)
    exps = np.asarray(exps, dtype=np.int32)
    scale = np.exp2(exps.astype(np.float32))[:, :, None]
    codes = encode_e4m3(nope / scale).reshape(n, FP8_DIM)
    rope_bits = f32_to_bf16_bits(latent[:, FP8_DIM:])

    data = np.zeros((total, TOKEN_DATA), dtype=np.uint8)
    data[:n, :FP8_DIM] = codes
    data[:n, FP8_DIM:] = rope_bits.view(np.uint8).reshape(n, 2 * ROPE_DIM)
    sc = np.zeros((total, SCALE_BYTES), dtype=np.uint8)
    sc[:n, :N_GROUPS] = (exps + 127).astype(np.uint8)
    sc[:n, N_GROUPS:] = 127
    cache = np.zeros((nb, block_size * TOKEN_BYTES_FP8), dtype=np.uint8)
    cache[:, : block_size * TOKEN_DATA] = data.reshape(nb, block_size * TOKEN_DATA)
    cache[:, block_size * TOKEN_DATA:] = sc.reshape(nb, block_size * SCALE_BYTES)
    cache = cache.reshape(nb, block_size, TOKEN_BYTES_FP8)
    return cache, dequant_fp8_ds_mla(cache)


def dequant_fp8_ds_mla(cache: np.ndarray) -> np.ndarray:
    """uint8 [nb, bs, 584] -> fp32 [nb * bs, 512] of bf16-representable values."""
    cache = np.ascontiguousarray(cache, dtype=np.uint8)
    nb, bs, tb = cache.shape
    assert tb == TOKEN_BYTES_FP8
    flat = cache.reshape(nb, bs * TOKEN_BYTES_FP8)
    data = flat[:, : bs * TOKEN_DATA].reshape(nb * bs, TOKEN_DATA)
    sc = flat[:, bs * TOKEN_DATA:].reshape(nb * bs, SCALE_BYTES)
    vals = E4M3_LUT[data[:, :FP8_DIM]]
    mult = np.exp2(sc[:, :N_GROUPS].astype(np.float32) - 127.0).astype(np.float32)
    nope = vals * np.repeat(mult, SCALE_GROUP, axis=1)
    rope = bf16_bits_to_f32(np.ascontiguousarray(data[:, FP8_DIM:]).view(np.uint16))
    return round_to_bf16(np.concatenate([nope, rope], axis=1).astype(np.float32))


def quantize_int8_rows(x: np.ndarray):
    """fp32 [..., 512] -> (int8 [..., 512], fp32 scale [...]); bit-exact restatement."""
    x = np.asarray(x, dtype=np.float32)
    if x.shape[-1] != HEAD_DIM:
        raise ValueError(f"expected last dim {HEAD_DIM}, got {x.shape[-1]}")
    amax = np.abs(x).max(axis=-1)
    scale = (np.maximum(amax, np.float32(1e-12)) / np.float32(127.0)).astype(np.float32)
    q = np.rint(x / scale[..., None])
    q = np.clip(q, -127, 127).astype(np.int8)
    return q, scale


def dequant_int8_ds_mla(q: np.ndarray, scale: np.ndarray) -> np.ndarray:
    """int8 [..., 512], fp32 [...] -> fp32 rows [N, 512] of bf16-representable values."""
    q = np.asarray(q).reshape(-1, HEAD_DIM).astype(np.float32)
    s = np.asarray(scale, dtype=np.float32).reshape(-1, 1)
    return round_to_bf16((q * s).astype(np.float32))


def pack_int8_inline528(q: np.ndarray, scale: np.ndarray, block_size: int) -> np.ndarray:
    """Production container: uint8 [nb, bs, 528] = 512 payload + fp32 scale at +512 + 12 pad."""
    q = np.asarray(q, dtype=np.int8).reshape(-1, HEAD_DIM)
    s = np.asarray(scale, dtype=np.float32).reshape(-1)
    n = q.shape[0]
    nb = (n + block_size - 1) // block_size
    buf = np.zeros((nb * block_size, INT8_TOKEN_BYTES), dtype=np.uint8)
    buf[:n, :HEAD_DIM] = q.view(np.uint8)
    buf[:n, HEAD_DIM:HEAD_DIM + 4] = s.view(np.uint8).reshape(n, 4)
    return buf.reshape(nb, block_size, INT8_TOKEN_BYTES)


def quantize_int8_rows_writer(x: np.ndarray):
    """The cache writer's variant of the row quantizer (reference:
    tests/test_sparse_mla_prefill_int8_adversarial.py:35-40, ``_quantize_rows``, stated there to
    mirror the serving engine's writer): ``scale = max(amax|x| / 127, 1e-12)``; the codes are
    computed as in ``quantize_int8_rows``.  Differs from it only for rows with amax < 1.27e-10."""
    x = np.asarray(x, dtype=np.float32)
    amax = np.abs(x).max(axis=-1)
    scale = np.maximum((amax / np.float32(127.0)).astype(np.float32), np.float32(1e-12))
    q = np.clip(np.rint(x / scale[..., None]), -127, 127).astype(np.int8)
    return q, scale


def write_int8_inline528(cache: np.ndarray, latent: np.ndarray, slots: np.ndarray, scale_rule: int = 0) -> None:
    """Quantise rows [N, 512] and scatter them into ``cache`` uint8 [nb, bs, 528] in place:
    row i goes to block ``slots[i] // bs``, position ``slots[i] % bs``; a negative slot or one
    past the cache skips the row.  A written token is 512 int8, the fp32 scale and 12 zero bytes.
    ``scale_rule`` 0 = ``quantize_int8_rows``, 1 = ``quantize_int8_rows_writer``."""
    nb, bs, tb = cache.shape
    assert tb == INT8_TOKEN_BYTES and cache.dtype == np.uint8
    q, s = (quantize_int8_rows if scale_rule == 0 else quantize_int8_rows_writer)(latent)
    flat = cache.reshape(nb * bs, tb)
    for i, slot in enumerate(np.asarray(slots).reshape(-1).tolist()):
        if 0 <= slot < nb * bs:
            flat[slot, :HEAD_DIM] = q[i].view(np.uint8)
            flat[slot, HEAD_DIM:HEAD_DIM + 4] = s[i:i + 1].view(np.uint8)
            flat[slot, HEAD_DIM + 4:] = 0


def write_fp8_ds_mla(cache: np.ndarray, latent: np.ndarray, slots: np.ndarray) -> None:
    """Encode rows [N, 512] and scatter them into ``cache`` uint8 [nb, bs, 584] in place (same
    slot rule as ``write_int8_inline528``).  Bytes per token as ``pack_fp8_ds_mla`` writes them:
    448 e4m3 codes of ``x / 2**e``, 64 bf16 (round-to-nearest-even) and the scale record
    ``[e + 127] * 7 + [127]`` in the block's scale area."""
    nb, bs, tb = cache.shape
    assert tb == TOKEN_BYTES_FP8 and cache.dtype == np.uint8
    latent = np.asarray(latent, dtype=np.float32)
    packed, _ = pack_fp8_ds_mla(latent, 1)                 # [N, 1, 584]: one token per block
    packed = packed.reshape(-1, TOKEN_BYTES_FP8)
    flat = cache.reshape(nb, bs * tb)
    for i, slot in enumerate(np.asarray(slots).reshape(-1).tolist()):
        if 0 <= slot < nb * bs:
            b, p = divmod(slot, bs)
            flat[b, p * TOKEN_DATA:(p + 1) * TOKEN_DATA] = packed[i, :TOKEN_DATA]
            flat[b, bs * TOKEN_DATA + p * SCALE_BYTES: bs * TOKEN_DATA + (p + 1) * SCALE_BYTES] = packed[i, TOKEN_DATA:]
