"""Seeded synthetic sparse-MLA workloads with the shapes, sizes and value distributions of the
benchmark configurations (there is no public dataset for this path; the reference benchmarks
synthetic tensors too, benchmarks/bench_sparse_mla_decode_16k.py:109-143).  Used by ``bench.py`` and
by the tests; not part of the product package.

Every builder returns a dict of keyword arguments for the matching ``flash_mla`` op plus a
``meta`` entry (row counts for roofline arithmetic).  All tensors live on ``device``.  On a CUDA
device the caches are packed with the library's own writers and quantizer (``flash_mla``); on the
CPU -- the reference arm of the benchmark, which must not load the library -- with the numpy oracle
(``oracle.pack_fp8_ds_mla``, ``oracle.quantize_int8_rows``, ``oracle.pack_int8_inline528``), whose
bytes are the same formats.
"""
from __future__ import annotations

from typing import Optional

import torch


def _is_cpu(device) -> bool:
    return torch.device(device).type == "cpu"


def pack_fp8_ds_mla(latent_bf16, block_size):
    if _is_cpu(latent_bf16.device):
        import oracle
        cache, _ = oracle.pack_fp8_ds_mla(latent_bf16.float().numpy(), block_size)
        return torch.from_numpy(cache)
    from flash_mla.cache_formats import pack_fp8_ds_mla as pack
    return pack(latent_bf16, block_size)


def quantize_int8_ds_mla_rows(latent_bf16):
    if _is_cpu(latent_bf16.device):
        import oracle
        q, s = oracle.quantize_int8_rows(latent_bf16.float().numpy())
        return torch.from_numpy(q), torch.from_numpy(s)
    from flash_mla import quantize_int8_ds_mla_rows as quant
    return quant(latent_bf16)


def pack_int8_inline528(q, scale, block_size):
    """-> (backing uint8 buffer [nb, bs, 528], int8 data view [nb, bs, 512], fp32 scale view [nb, bs])."""
    if _is_cpu(q.device):
        import oracle
        buf = torch.from_numpy(oracle.pack_int8_inline528(q.numpy(), scale.numpy(), block_size))
        return buf, buf[:, :, :512].view(torch.int8), buf[:, :, 512:516].view(torch.float32).squeeze(-1)
    from flash_mla.cache_formats import pack_int8_inline528 as pack
    return pack(q, scale, block_size)


def _distinct_indices(gen, T, num_slots, topk, device, mask_frac=0.0):
    """[T, topk] int32, uniform distinct per token; a fraction set to -1."""
    r = torch.rand(T, num_slots, generator=gen, device=device)
    idx = r.argsort(dim=1)[:, :topk].to(torch.int32)
    if mask_frac > 0:
        m = torch.rand(T, topk, generator=gen, device=device) < mask_frac
        idx = torch.where(m, torch.full_like(idx, -1), idx)
    return idx.contiguous()


def _causal_indices(gen, T, num_slots, topk, device, divisor=1):
    """Row p: uniform distinct ids in [0, p // divisor], padded with -1; lens = min(p//divisor + 1, topk)."""
    limit = (torch.arange(T, device=device) // divisor).clamp_max(num_slots - 1)     # inclusive upper id
    r = torch.rand(T, num_slots, generator=gen, device=device)
    cols = torch.arange(num_slots, device=device)
    r = torch.where(cols[None, :] <= limit[:, None], r, torch.full_like(r, 2.0))
    idx = r.argsort(dim=1)[:, :topk].to(torch.int32)
    lens = (limit + 1).clamp_max(topk).to(torch.int32)
    pos = torch.arange(topk, device=device)
    idx = torch.where(pos[None, :] < lens[:, None], idx, torch.full_like(idx, -1))
    return idx.contiguous(), lens.contiguous()


def _latent(gen, n, device, outlier_frac=0.0):
    x = torch.randn(n, 512, generator=gen, device=device)
    if outlier_frac > 0:
        o = torch.rand(n, generator=gen, device=device) < outlier_frac
        x = torch.where(o[:, None], x * 50.0, x)
    return x.to(torch.bfloat16)


def _gen(device, seed):
    return torch.Generator(device=device).manual_seed(seed)


def _count_rows(idx, lens, num_slots):
    """(rows inside lens, rows inside lens with an in-range id)."""
    pos = torch.arange(idx.shape[1], device=idx.device)
    inside = pos[None, :] < lens[:, None]
    valid = inside & (idx >= 0) & (idx < num_slots)
    return int(inside.sum().item()), int(valid.sum().item())


def decode_workload(fmt: str = "fp8", T: int = 128, H: int = 64, swa_slots: int = 65536, swa_block: int = 256,
                    swa_topk: int = 512, extra_slots: int = 16384, extra_block: int = 64, extra_topk: int = 2048,
                    mask_frac: float = 0.02, full_lens: bool = False, sink: bool = True, layout: str = "inline528",
                    outlier_frac: Optional[float] = None, seed: int = 0, device: str = "cuda"):
    """DSV4-Flash absorbed decode shape: q [T, H, 512] ~ N(0,1); swa + extra caches built from bf16
    latents ~ N(0,1); indices uniform distinct per token with ``mask_frac`` set to -1; lens uniform in
    [topk/2, topk] (or == topk with ``full_lens``); attn_sink ~ N(0,1).  ``fmt`` "fp8" or "int8"
    (int8: 5 % of the latent rows scaled x50 unless ``outlier_frac`` says otherwise; ``layout``
    "inline528" or "separate")."""
    g = _gen(device, seed)
    if outlier_frac is None:
        outlier_frac = 0.05 if fmt == "int8" else 0.0
    swa_lat = _latent(g, swa_slots, device, outlier_frac)
    extra_lat = _latent(g, extra_slots, device, outlier_frac) if extra_topk > 0 else None
    q = torch.randn(T, H, 512, generator=g, device=device).to(torch.bfloat16)
    swa_idx = _distinct_indices(g, T, swa_slots, swa_topk, device, mask_frac)
    if full_lens:
        swa_lens = torch.full((T,), swa_topk, dtype=torch.int32, device=device)
    else:
        swa_lens = torch.randint(swa_topk // 2, swa_topk + 1, (T,), generator=g, device=device).to(torch.int32)
    kw = dict(q=q, swa_indices=swa_idx, swa_lens=swa_lens)
    if sink:
        kw["attn_sink"] = torch.randn(H, generator=g, device=device)
    rows_in, rows_valid = _count_rows(swa_idx, swa_lens, swa_slots)
    if extra_topk > 0:
        extra_idx = _distinct_indices(g, T, extra_slots, extra_topk, device, mask_frac)
        if full_lens:
            extra_lens = torch.full((T,), extra_topk, dtype=torch.int32, device=device)
        else:
            extra_lens = torch.randint(extra_topk // 2, extra_topk + 1, (T,), generator=g,
                                       device=device).to(torch.int32)
        kw.update(extra_indices=extra_idx, extra_lens=extra_lens)
        a, b = _count_rows(extra_idx, extra_lens, extra_slots)
        rows_in, rows_valid = rows_in + a, rows_valid + b

    keep = []
    if fmt == "fp8":
        kw["swa_cache"] = pack_fp8_ds_mla(swa_lat, swa_block)
        if extra_topk > 0:
            kw["extra_cache"] = pack_fp8_ds_mla(extra_lat, extra_block)
    else:
        for name, lat, bs in (("swa", swa_lat, swa_block), ("extra", extra_lat, extra_block)):
            if lat is None:
                continue
            qi, sc = quantize_int8_ds_mla_rows(lat)
            if layout == "inline528":
                buf, dv, sv = pack_int8_inline528(qi, sc, bs)
                keep.append(buf)
                kw[f"{name}_cache"], kw[f"{name}_scale"] = dv, sv
            else:
                nb = lat.shape[0] // bs
                kw[f"{name}_cache"] = qi.view(nb, bs, 512)
                kw[f"{name}_scale"] = sc.view(nb, bs)
    row_bytes = 584 if fmt == "fp8" else 516
    meta = dict(fmt=fmt, T=T, H=H, rows_in_lens=rows_in, rows_valid=rows_valid, row_bytes=row_bytes,
                flops=4 * H * 512 * rows_in,
                bytes=rows_valid * row_bytes + 2 * (T * H * 512 * 2) + 4 * rows_in + 8 * T + 4 * H,
                keep=keep)
    return kw, meta


def prefill_int8_workload(T: int = 4096, H: int = 64, swa_slots: int = 16384, swa_block: int = 256,
                          swa_topk: int = 2048, extra_slots: int = 4096, extra_block: int = 64,
                          extra_topk: int = 512, seed: int = 0, device: str = "cuda"):
    """Causal prefill: for query position p the swa ids are uniform distinct in [0, p] padded with -1
    (lens min(p+1, topk)); the compressed extra stream follows the same rule on p // 4."""
    g = _gen(device, seed)
    swa_lat = _latent(g, swa_slots, device, 0.05)
    extra_lat = _latent(g, extra_slots, device, 0.05)
    q = torch.randn(T, H, 512, generator=g, device=device).to(torch.bfloat16)
    swa_idx, swa_lens = _causal_indices(g, T, swa_slots, swa_topk, device, 1)
    extra_idx, extra_lens = _causal_indices(g, T, extra_slots, extra_topk, device, 4)
    sink = torch.randn(H, generator=g, device=device)
    kw = dict(q=q, swa_indices=swa_idx, swa_lens=swa_lens, attn_sink=sink, extra_indices=extra_idx,
              extra_lens=extra_lens)
    keep = []
    for name, lat, bs in (("swa", swa_lat, swa_block), ("extra", extra_lat, extra_block)):
        qi, sc = quantize_int8_ds_mla_rows(lat)
        buf, dv, sv = pack_int8_inline528(qi, sc, bs)
        keep.append(buf)
        kw[f"{name}_cache"], kw[f"{name}_scale"] = dv, sv
    a, b = _count_rows(swa_idx, swa_lens, swa_slots)
    c, d = _count_rows(extra_idx, extra_lens, extra_slots)
    rows_in, rows_valid = a + c, b + d
    meta = dict(fmt="int8", T=T, H=H, rows_in_lens=rows_in, rows_valid=rows_valid, row_bytes=516,
                flops=4 * H * 512 * rows_in,
                bytes=rows_valid * 516 + 2 * (T * H * 512 * 2) + 4 * rows_in + 8 * T + 4 * H, keep=keep)
    return kw, meta


def dense_decode_workload(b: int = 128, s_q: int = 1, mean_sk: int = 4096, h_q: int = 128, varlen: bool = False,
                          block_size: int = 64, seed: int = 0, device="cuda", poison_tail: bool = True, d: int = 576):
    """The reference's dense test case (tests/test_flash_mla_sm80.py:43-63): ``b`` sequences of ``mean_sk`` rows
    (``varlen``: normal around it with sigma mean_sk / 2, at least s_q), q and the bf16 cache N(0, 1), pages in
    a scrambled order, rows past each length NaN so that any read of them shows in the result."""
    gen = _gen(device, seed)
    lens = torch.full((b,), mean_sk, dtype=torch.int32)
    if varlen:
        cpu_gen = torch.Generator().manual_seed(seed + 1)
        lens = (torch.randn(b, generator=cpu_gen) * (mean_sk / 2) + mean_sk).clamp(min=s_q).to(torch.int32)
    max_pad = (int(lens.max()) + 255) // 256 * 256
    pages_per_seq = max_pad // block_size
    perm = torch.randperm(b * pages_per_seq, generator=torch.Generator().manual_seed(seed + 2))
    block_table = perm.to(torch.int32).view(b, pages_per_seq).to(device)
    q = torch.randn(b, s_q, h_q, d, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    k_cache = torch.empty(b * pages_per_seq, block_size, 1, d, device=device, dtype=torch.bfloat16)
    for i in range(b):           # sequence by sequence: a 128 x 8192 batch is 1.2 GB of bf16
        rows = torch.randn(max_pad, 1, d, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        if poison_tail:
            rows[int(lens[i]):] = float("nan")
        k_cache[block_table[i].long()] = rows.view(pages_per_seq, block_size, 1, d)
    lens = lens.to(device)
    rows_total = int(lens.sum()) * s_q        # without the causal trim (at most s_q - 1 rows per query)
    meta = {"flops": 2 * rows_total * h_q * (d + 512),
            "bytes": int(lens.sum()) * 2 * d + b * s_q * h_q * (d + 512) * 2 + b * pages_per_seq * 4,
            "rows_in_lens": rows_total}
    return {"q": q, "k_cache": k_cache, "block_table": block_table, "cache_seqlens": lens}, meta
