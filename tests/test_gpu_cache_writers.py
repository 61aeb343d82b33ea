"""GPU parity tests of the cache writers (encode new latent rows and scatter them into a paged
cache): byte-exact against the oracle's writers on the same seeded inputs, against the golden
vectors generated from the reference's own quantizer and packers, through the Python API and
through the C ABI, plus size-independent properties at a large row count and a writer -> attention
round trip.  The byte formats are the ones the reference's tests build with torch composites
(tests/test_sparse_mla_decode_sm86.py:14-44, tests/test_sparse_mla_prefill_int8_adversarial.py:5-12,35-60).
"""
import math

import numpy as np
import pytest
import torch

from helpers import assert_attention_close, bf16_from_bits, device_status, oracle_out, to_dev
import oracle

pytestmark = pytest.mark.gpu
FILL = 0xA5


@pytest.fixture(scope="module")
def fm():
    import flash_mla
    return flash_mla


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert device_status() == 0


def _rows(n, seed, dtype):
    """Rows with the hard cases mixed in: outlier rows, all-zero rows and groups, tiny rows, exact
    rounding ties, group maxima exactly on and just past a power-of-two boundary of the exponent rule."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 512, generator=g)
    x[1::7] *= 50.0
    x[2::11] *= 1e-3
    if n > 16:
        x[3] = 0.0
        x[4, :64] = 0.0
        x[5] = 1e-11 * torch.randn(512, generator=g)
        x[6] = torch.arange(512) % 9 - 4.0                     # ties after the division
        x[7] = (torch.arange(512) % 255 - 127).float() * 0.5
        x[8, :64] = 0.25
        x[8, 0] = 448.0                                       # amax exactly 448 * 2^0
        x[9, 64:128] = 0.25
        x[9, 64] = 449.0                                      # just past it
        x[10, 128:192] = 3.0e-5
        x[10, 128] = -448.0 * 2.0 ** -20
        x[11] = (6.0e3 if dtype == torch.float16 else 1e30) * torch.randn(512, generator=g).clamp(-3, 3)
        x[12] = 1e-38 * torch.randn(512, generator=g)        # subnormal-range values
        x[13] = torch.arange(512) % 251 - 125.5               # scale 1: every quotient an exact tie
        x[13, 0] = 127.0
        x[14] = x[13] + (torch.arange(512) % 3 - 1.0) * 2.0 ** -17   # ... and just off the tie
        x[14, 0] = 127.0
        x[15] = (torch.arange(512) % 251 - 125.5) * 3.0       # scale 3: ties after an inexact division
        x[15, 0] = 381.0
    return x.to(dtype)


def _slots(n, num_slots, seed, dtype):
    """A random injective slot mapping with a few skipped rows (-1, and one past the cache)."""
    rs = np.random.RandomState(seed)
    s = rs.permutation(num_slots)[:n].astype(np.int64)
    if n > 20:
        s[13] = -1
        s[17] = num_slots
        s[19] = num_slots + 12345
    return torch.from_numpy(s).to(dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("block_size,slot_dtype,rule", [(64, torch.int64, "quantizer"), (16, torch.int32, "writer"),
                                                        (1, torch.int64, "writer"), (3, torch.int32, "quantizer")])
def test_int8_writer_matches_oracle(fm, dtype, block_size, slot_dtype, rule):
    n, nb = 333, (400 + block_size - 1) // block_size
    x = _rows(n, 1, dtype)
    slots = _slots(n, nb * block_size, 2, slot_dtype)
    cache = torch.full((nb, block_size, 528), FILL, dtype=torch.uint8, device="cuda")
    fm.write_int8_ds_mla_cache(x.cuda(), slots, cache, scale_rule=rule)
    ref = np.full((nb, block_size, 528), FILL, np.uint8)
    oracle.write_int8_inline528(ref, x.float().numpy(), slots.cpu().numpy(), 0 if rule == "quantizer" else 1)
    assert np.array_equal(cache.cpu().numpy(), ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("block_size,slot_dtype", [(64, torch.int64), (16, torch.int32), (1, torch.int64),
                                                   (3, torch.int32)])
def test_fp8_writer_matches_oracle(fm, dtype, block_size, slot_dtype):
    n, nb = 333, (400 + block_size - 1) // block_size
    x = _rows(n, 3, dtype)
    slots = _slots(n, nb * block_size, 4, slot_dtype)
    cache = torch.full((nb, block_size, 584), FILL, dtype=torch.uint8, device="cuda")
    fm.write_fp8_ds_mla_cache(x.cuda(), slots, cache)
    ref = np.full((nb, block_size, 584), FILL, np.uint8)
    oracle.write_fp8_ds_mla(ref, x.float().numpy(), slots.cpu().numpy())
    got = cache.cpu().numpy()
    assert np.array_equal(got, ref), f"{np.argwhere(got != ref)[:8]}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_int8_codes_bit_exact_at_scale(fm, dtype):
    """2^16 rows (33 M codes) of mixed magnitude against IEEE division + round-half-even on the CPU:
    the kernels get their codes from a reciprocal multiply and divide only near a rounding tie, so
    this is the check that the short cut never shows.  Rows are scaled so that many quotients land on
    or next to half-integers."""
    n = 1 << 16
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(n, 512, generator=g, device="cuda") * torch.exp2(torch.randint(-20, 21, (n, 1), generator=g, device="cuda").float())
    # every fourth row: multiples of half the scale -> exact ties wherever the multiple is odd
    k = torch.randint(-254, 255, (n // 4, 512), generator=g, device="cuda").float()
    k[:, 0] = 254.0
    step = torch.rand(n // 4, 1, generator=g, device="cuda") + 0.5
    x[::4] = k * step * 0.5
    x = x.to(dtype)
    qo, so = oracle.quantize_int8_rows(x.float().cpu().numpy())
    q, s = fm.quantize_int8_ds_mla_rows(x)
    assert np.array_equal(s.cpu().numpy(), so)
    assert np.array_equal(q.cpu().numpy(), qo)
    cache = torch.zeros(n // 64, 64, 528, dtype=torch.uint8, device="cuda")
    slots = torch.randperm(n, generator=g, device="cuda")
    fm.write_int8_ds_mla_cache(x, slots, cache)
    data, scale = fm.int8_ds_mla_cache_views(cache)
    assert np.array_equal(data.reshape(-1, 512)[slots].cpu().numpy(), qo)
    assert np.array_equal(scale.reshape(-1)[slots].cpu().numpy(), so)


def test_writers_strided_rows_and_alignment_paths(fm):
    """Latent rows as a column slice of a wider tensor: row stride 1152 bytes (32-byte aligned rows:
    256-bit loads), 1040 bytes and a base 16 bytes in (128-bit loads), and an element offset that no
    vector load can take (the binding copies)."""
    n, bs = 200, 16
    nb = (n + bs - 1) // bs
    slots = _slots(n, nb * bs, 5, torch.int64)
    for width, off in ((576, 0), (520, 0), (528, 8), (515, 3)):
        wide = torch.randn(n, width, generator=torch.Generator().manual_seed(width)).to(torch.bfloat16).cuda()
        x = wide[:, off:off + 512]
        ci = torch.zeros(nb, bs, 528, dtype=torch.uint8, device="cuda")
        cf = torch.zeros(nb, bs, 584, dtype=torch.uint8, device="cuda")
        fm.write_int8_ds_mla_cache(x, slots, ci)
        fm.write_fp8_ds_mla_cache(x, slots, cf)
        ri, rf = np.zeros((nb, bs, 528), np.uint8), np.zeros((nb, bs, 584), np.uint8)
        oracle.write_int8_inline528(ri, x.float().cpu().numpy(), slots.cpu().numpy())
        oracle.write_fp8_ds_mla(rf, x.float().cpu().numpy(), slots.cpu().numpy())
        assert np.array_equal(ci.cpu().numpy(), ri), (width, off)
        assert np.array_equal(cf.cpu().numpy(), rf), (width, off)


def test_int8_writer_golden(fm, golden):
    """The reference quantizer's known answers, as tokens of the inline container."""
    g = golden("quantizer_kat.npz")
    x = bf16_from_bits(g["x_bf16"])
    n = x.shape[0]
    cache = torch.zeros(6, 16, 528, dtype=torch.uint8, device="cuda")
    fm.write_int8_ds_mla_cache(x, torch.arange(n, device="cuda"), cache)
    assert np.array_equal(cache.cpu().numpy(), oracle.pack_int8_inline528(g["q"], g["scale"], 16))
    data, scale = fm.int8_ds_mla_cache_views(cache)
    assert np.array_equal(data.cpu().numpy().reshape(-1, 512)[:n], g["q"])
    assert np.array_equal(scale.cpu().numpy().reshape(-1)[:n], g["scale"])


def test_fp8_writer_golden_values(fm, golden):
    """Rows the reference's packer produced (every value representable in the format): writing them
    again must give a cache that dequantises to exactly the same rows, RoPE bytes included."""
    for name, ck, kk in (("fp8_decode_single.npz", "cache", "K"), ("fp8_two_stream.npz", "swa_cache", "swa_K"),
                         ("fp8_two_stream.npz", "extra_cache", "extra_K")):
        g = golden(name)
        K = bf16_from_bits(g[kk])
        nb, bs, _ = g[ck].shape
        assert np.array_equal(oracle.dequant_fp8_ds_mla(g[ck]), K.float().cpu().numpy())
        cache = torch.zeros(nb, bs, 584, dtype=torch.uint8, device="cuda")
        fm.write_fp8_ds_mla_cache(K, torch.arange(K.shape[0], device="cuda", dtype=torch.int32), cache)
        got = cache.cpu().numpy()
        assert np.array_equal(oracle.dequant_fp8_ds_mla(got), K.float().cpu().numpy())
        flat_g, flat_r = got.reshape(nb, -1)[:, :bs * 576].reshape(-1, 576), g[ck].reshape(nb, -1)[:, :bs * 576].reshape(-1, 576)
        assert np.array_equal(flat_g[:, 448:], flat_r[:, 448:])


def test_writers_through_c_abi(fm):
    """Raw pointers through ctypes, and the argument checks of the entry points."""
    from flash_mla import c_abi
    lib = c_abi.load()
    n, bs, nb = 70, 8, 10
    x = _rows(n, 7, torch.bfloat16).cuda()
    slots = _slots(n, nb * bs, 8, torch.int32)
    st = torch.cuda.current_stream().cuda_stream
    ci = torch.zeros(nb, bs, 528, dtype=torch.uint8, device="cuda")
    cf = torch.zeros(nb, bs, 584, dtype=torch.uint8, device="cuda")
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr(), 0, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs,
                                            bs * 528, 528, 1, st) == 0
    assert lib.smla_write_fp8_ds_mla_cache(x.data_ptr(), 0, n, 512, slots.data_ptr(), 0, cf.data_ptr(), nb, bs,
                                           bs * 584, st) == 0
    ri, rf = np.zeros((nb, bs, 528), np.uint8), np.zeros((nb, bs, 584), np.uint8)
    oracle.write_int8_inline528(ri, x.float().cpu().numpy(), slots.cpu().numpy(), 1)
    oracle.write_fp8_ds_mla(rf, x.float().cpu().numpy(), slots.cpu().numpy())
    assert np.array_equal(ci.cpu().numpy(), ri) and np.array_equal(cf.cpu().numpy(), rf)
    # zero rows: nothing to do, nothing touched
    assert lib.smla_write_fp8_ds_mla_cache(None, 0, 0, 512, None, 0, None, 0, 0, 0, st) == 0
    EINVAL, EALIGN = -1, -2
    assert lib.smla_write_int8_ds_mla_cache(None, 0, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs, bs * 528, 528, 0, st) == EINVAL
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr(), 7, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs, bs * 528, 528, 0, st) == EINVAL
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr(), 0, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs, bs * 528, 520, 0, st) == EINVAL
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr(), 0, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs, bs * 528, 528, 2, st) == EINVAL
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr() + 2, 0, n, 512, slots.data_ptr(), 0, ci.data_ptr(), nb, bs, bs * 528, 528, 0, st) == EALIGN
    assert lib.smla_write_fp8_ds_mla_cache(x.data_ptr(), 0, n, 512, slots.data_ptr(), 0, cf.data_ptr(), nb, bs, bs * 584 - 8, st) == EINVAL
    assert lib.smla_write_fp8_ds_mla_cache(x.data_ptr(), 0, n, 515, slots.data_ptr(), 0, cf.data_ptr(), nb, bs, bs * 584, st) == EALIGN
    assert np.array_equal(ci.cpu().numpy(), ri) and np.array_equal(cf.cpu().numpy(), rf)
    with pytest.raises(ValueError):
        fm.write_fp8_ds_mla_cache(x[:, :256], slots, cf)
    with pytest.raises(ValueError):
        fm.write_int8_ds_mla_cache(x, slots[:5], ci)
    with pytest.raises(ValueError):
        fm.write_int8_ds_mla_cache(x, slots, cf)


def test_writers_edge_shapes(fm):
    """No rows, only skipped rows, blocks with padding between them (block stride larger than the
    tokens need), and a slot count no device could hold."""
    from flash_mla import c_abi
    lib = c_abi.load()
    st = torch.cuda.current_stream().cuda_stream
    bs, nb = 8, 6
    for tb, write, owrite in ((528, fm.write_int8_ds_mla_cache, oracle.write_int8_inline528),
                              (584, fm.write_fp8_ds_mla_cache, oracle.write_fp8_ds_mla)):
        cache = torch.full((nb, bs, tb), FILL, dtype=torch.uint8, device="cuda")
        write(torch.empty(0, 512, dtype=torch.bfloat16, device="cuda"), torch.empty(0, dtype=torch.int64, device="cuda"), cache)
        x = _rows(40, 9, torch.bfloat16).cuda()
        write(x, torch.full((40,), -1, dtype=torch.int64, device="cuda"), cache)
        write(x, torch.full((40,), nb * bs, dtype=torch.int32, device="cuda"), cache)
        assert bool((cache == FILL).all())
        # every second block of a larger allocation: block stride = 2 * bs * tb
        big = torch.full((2 * nb, bs, tb), FILL, dtype=torch.uint8, device="cuda")
        view = big[::2]
        slots = _slots(40, nb * bs, 10, torch.int64)
        write(x, slots, view)
        ref = np.full((nb, bs, tb), FILL, np.uint8)
        owrite(ref, x.float().cpu().numpy(), slots.cpu().numpy())
        assert np.array_equal(view.cpu().numpy(), ref)
        assert bool((big[1::2] == FILL).all())
    x = _rows(40, 9, torch.bfloat16).cuda()
    slots = _slots(40, 48, 10, torch.int64)
    ETOOBIG = -5
    assert lib.smla_write_int8_ds_mla_cache(x.data_ptr(), 0, 40, 512, slots.data_ptr(), 1, big.data_ptr(), 1 << 26, 64,
                                            64 * 528, 528, 0, st) == ETOOBIG
    assert lib.smla_write_fp8_ds_mla_cache(x.data_ptr(), 0, 40, 512, slots.data_ptr(), 1, big.data_ptr(), 1 << 26, 64,
                                           64 * 584, st) == ETOOBIG


def _dequant_fp8_torch(cache):
    nb, bs, _ = cache.shape
    flat = cache.view(nb, bs * 584)
    data = flat[:, :bs * 576].reshape(nb * bs, 576)
    sc = flat[:, bs * 576:].reshape(nb * bs, 8)
    nope = data[:, :448].contiguous().view(torch.float8_e4m3fn).float().view(-1, 7, 64)
    nope = (nope * torch.exp2(sc[:, :7].float() - 127.0).unsqueeze(-1)).view(-1, 448)
    rope = data[:, 448:].contiguous().view(torch.bfloat16).float()
    return torch.cat([nope, rope], 1)


def test_writers_properties_at_scale(fm):
    """2^18 rows (256 MiB of bf16 input): error bounds of both formats, untouched slots, and
    idempotence of the fp8 format on its own values."""
    n, bs = 1 << 18, 64
    nb = n // bs + 8
    g = torch.Generator(device="cuda").manual_seed(11)
    x = (torch.randn(n, 512, generator=g, device="cuda") * torch.exp2(torch.randint(-6, 7, (n, 1), generator=g, device="cuda").float())).to(torch.bfloat16)
    slots = torch.randperm(nb * bs, generator=g, device="cuda")[:n]
    used = torch.zeros(nb * bs, dtype=torch.bool, device="cuda")
    used[slots] = True

    ci = torch.full((nb, bs, 528), FILL, dtype=torch.uint8, device="cuda")
    fm.write_int8_ds_mla_cache(x, slots, ci)
    data, scale = fm.int8_ds_mla_cache_views(ci)
    tok = ci.view(nb * bs, 528)
    assert bool((tok[~used] == FILL).all()) and bool((tok[used][:, 516:] == 0).all())
    q, s = data.reshape(-1, 512)[slots].float(), scale.reshape(-1)[slots]
    xf = x.float()
    want_s = np.maximum(xf.abs().amax(-1).cpu().numpy(), np.float32(1e-12)) / np.float32(127.0)   # IEEE division
    assert np.array_equal(s.cpu().numpy(), want_s)
    assert bool(((q * s[:, None] - xf).abs() <= 0.5001 * s[:, None]).all())
    assert int(q.abs().amax(-1).min()) == 127                 # every row uses the full range

    cf = torch.full((nb, bs, 584), FILL, dtype=torch.uint8, device="cuda")
    fm.write_fp8_ds_mla_cache(x, slots, cf)
    blocks = cf.view(nb, bs * 584)
    tokd = blocks[:, :bs * 576].reshape(nb * bs, 576)
    toks = blocks[:, bs * 576:].reshape(nb * bs, 8)
    assert bool((tokd[~used] == FILL).all()) and bool((toks[~used] == FILL).all()) and bool((toks[used][:, 7] == 127).all())
    deq = _dequant_fp8_torch(cf)[slots]
    assert torch.equal(deq[:, 448:], xf[:, 448:])
    grp = xf[:, :448].view(n, 7, 64)
    e = toks[slots][:, :7].float() - 127.0
    amax = grp.abs().amax(-1)
    assert bool((amax <= 448.0 * torch.exp2(e)).all()) and bool((amax > 448.0 * torch.exp2(e - 1)).all())
    # e4m3 has 3 mantissa bits: relative error <= 2^-4 for normal codes, absolute <= 2^-10 * 2^e below
    err = (deq[:, :448].view(n, 7, 64) - grp).abs()
    assert bool((err <= torch.maximum(grp.abs() * 2.0 ** -4, torch.exp2(e - 10).unsqueeze(-1))).all())
    cf2 = torch.zeros_like(cf)
    fm.write_fp8_ds_mla_cache(deq.to(torch.float32), slots, cf2)
    assert torch.equal(_dequant_fp8_torch(cf2)[slots], deq)


@pytest.mark.parametrize("fmt", ["fp8", "int8"])
def test_writer_then_decode(fm, fmt):
    """The writers' caches through the attention kernels: fill a paged cache in three batches of
    scattered slots, run decode on it and compare with the oracle on the oracle-packed rows."""
    T, H, bs, n, topk = 8, 64, 64, 1000, 384
    nb = (n + bs - 1) // bs
    g = torch.Generator().manual_seed(21)
    lat = torch.randn(n, 512, generator=g).to(torch.bfloat16)
    q = torch.randn(T, H, 512, generator=g).to(torch.bfloat16).cuda()
    perm = torch.randperm(nb * bs, generator=g)[:n]             # row i lives in slot perm[i]
    idx = torch.stack([perm[torch.randperm(n, generator=g)[:topk]] for _ in range(T)]).to(torch.int32)
    idx[0, 5] = -1
    lens = torch.tensor([topk, 1, 100, 383, 384, 129, 128, 300], dtype=torch.int32)
    sink = torch.randn(H, generator=g)
    tb = 584 if fmt == "fp8" else 528
    cache = torch.zeros(nb, bs, tb, dtype=torch.uint8, device="cuda")
    write = fm.write_fp8_ds_mla_cache if fmt == "fp8" else fm.write_int8_ds_mla_cache
    for lo, hi in ((0, 1), (1, 400), (400, n)):
        write(lat[lo:hi].cuda(), perm[lo:hi].cuda(), cache)
    K = np.zeros((nb * bs, 512), np.float32)
    if fmt == "fp8":
        _, rows = oracle.pack_fp8_ds_mla(lat.float().numpy(), 1)
        K[perm.numpy()] = rows
        out = fm.sparse_mla_decode_fp8(q, cache, idx.cuda(), lens.cuda(), scale=1 / math.sqrt(512), attn_sink=sink.cuda())
    else:
        qi, sc = oracle.quantize_int8_rows(lat.float().numpy())
        K[perm.numpy()] = oracle.dequant_int8_ds_mla(qi, sc)
        data, scale = fm.int8_ds_mla_cache_views(cache)
        out = fm.sparse_mla_decode_int8(q, data, scale, idx.cuda(), lens.cuda(), scale=1 / math.sqrt(512), attn_sink=sink.cuda())
    ref = oracle_out(q, K, idx, lens, scale=1 / math.sqrt(512), sink=sink)
    assert_attention_close(out, ref, f"writer -> decode {fmt}", strict_abs=True)
