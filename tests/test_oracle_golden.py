"""Pin the CPU oracle against fixtures produced by the reference's own Python code
(tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import pytest

from oracle import (bf16_bits_to_f32, dequant_fp8_ds_mla, dequant_int8_ds_mla, pack_fp8_ds_mla,
                    pack_int8_inline528, quantize_int8_rows, sparse_mla_attention, cos_diff, E4M3_LUT)
from oracle.ds_mla_formats import encode_e4m3, f32_to_bf16_bits


def test_e4m3_lut_matches_torch():
    import torch
    b = torch.arange(256, dtype=torch.uint8)
    ref = b.view(torch.float8_e4m3fn).float().numpy()
    ok = np.isnan(ref) == np.isnan(E4M3_LUT)
    assert ok.all()
    m = ~np.isnan(ref)
    assert np.array_equal(ref[m], E4M3_LUT[m])


def test_e4m3_encode_matches_torch():
    import torch
    g = torch.Generator().manual_seed(1)
    x = torch.randn(20000, generator=g) * 40
    x[:200] = torch.linspace(-448, 448, 200)
    ref = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = encode_e4m3(x.numpy())
    assert np.array_equal(ref, got)


def test_bf16_rounding_matches_torch():
    import torch
    g = torch.Generator().manual_seed(2)
    x = torch.randn(50000, generator=g) * 3
    ref = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ref, f32_to_bf16_bits(x.numpy()))


def test_quantizer_bit_exact(golden):
    g = golden("quantizer_kat.npz")
    x = bf16_bits_to_f32(g["x_bf16"])
    q, s = quantize_int8_rows(x)
    assert np.array_equal(q, g["q"])
    assert np.array_equal(s.view(np.uint32), g["scale"].view(np.uint32))
    q3, s3 = quantize_int8_rows(x.reshape(4, 24, 512))
    assert q3.shape == (4, 24, 512) and s3.shape == (4, 24)
    with pytest.raises(ValueError):
        quantize_int8_rows(np.zeros((3, 256), np.float32))


def test_fp8_dequant_matches_reference_rows(golden):
    for name, ck, kk in (("fp8_decode_single.npz", "cache", "K"),
                         ("fp8_two_stream.npz", "swa_cache", "swa_K"),
                         ("fp8_two_stream.npz", "extra_cache", "extra_K")):
        g = golden(name)
        K = dequant_fp8_ds_mla(g[ck])
        assert np.array_equal(f32_to_bf16_bits(K), g[kk]), (name, ck)


def test_fp8_single_stream(golden):
    g = golden("fp8_decode_single.npz")
    q = bf16_bits_to_f32(g["q"])
    K = dequant_fp8_ds_mla(g["cache"])
    out = sparse_mla_attention(q, K, g["idx"], g["lens"], scale=float(g["scale"]), sink=g["sink"])
    np.testing.assert_allclose(out, g["out"], rtol=2e-5, atol=2e-6)
    out = sparse_mla_attention(q, K, g["idx"], g["lens"], scale=float(g["scale"]))
    np.testing.assert_allclose(out, g["out_nosink"], rtol=2e-5, atol=2e-6)


def test_fp8_two_stream(golden):
    g = golden("fp8_two_stream.npz")
    q = bf16_bits_to_f32(g["q"])
    out = sparse_mla_attention(q, dequant_fp8_ds_mla(g["swa_cache"]), g["swa_idx"], g["swa_lens"],
                               dequant_fp8_ds_mla(g["extra_cache"]), g["extra_idx"], g["extra_lens"],
                               scale=float(g["scale"]), sink=g["sink"])
    np.testing.assert_allclose(out, g["out"], rtol=2e-5, atol=2e-6)
    assert np.all(out[0] == 0)  # token with no selected rows


@pytest.mark.parametrize("layout", ["inline528", "separate"])
def test_int8_two_stream(golden, layout):
    g = golden(f"int8_two_stream_{layout}.npz")
    q = bf16_bits_to_f32(g["q"])
    swa_K = dequant_int8_ds_mla(g["swa_q"], g["swa_scale"])
    extra_K = dequant_int8_ds_mla(g["extra_q"], g["extra_scale"])
    assert np.array_equal(f32_to_bf16_bits(swa_K), g["swa_K"])
    assert np.array_equal(f32_to_bf16_bits(extra_K), g["extra_K"])
    out = sparse_mla_attention(q, swa_K, g["swa_idx"], g["swa_lens"], extra_K, g["extra_idx"],
                               g["extra_lens"], scale=float(g["scale"]), sink=g["sink"])
    np.testing.assert_allclose(out, g["out"], rtol=2e-5, atol=2e-6)
    assert cos_diff(out, g["out"]) < 1e-10


def test_config1_cpu_oracle(golden):
    g = golden("config1_cpu_oracle.npz")
    q = bf16_bits_to_f32(g["q"])
    K = dequant_fp8_ds_mla(g["cache"])
    out = sparse_mla_attention(q, K, g["idx"], g["lens"])  # scale=None -> 512**-0.5, no sink
    np.testing.assert_allclose(out, g["out"], rtol=2e-5, atol=2e-6)


def test_pack_roundtrip():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((70, 512)).astype(np.float32)
    x[3] *= 50
    x[4] = 0
    cache, K = pack_fp8_ds_mla(x, 32)
    assert cache.shape == (3, 32, 584)
    # repacking the dequantised rows reproduces the same bytes for the data records
    cache2, K2 = pack_fp8_ds_mla(K[:70], 32)
    assert np.array_equal(K, K2)
    rel = np.abs(K[:70, :448] - x[:, :448]).max() / np.abs(x).max()
    assert rel < 0.07
    q, s = quantize_int8_rows(x)
    buf = pack_int8_inline528(q, s, 16)
    assert buf.shape == (5, 16, 528)
    assert np.array_equal(buf.reshape(-1, 528)[:70, :512].view(np.int8), q)
    assert np.array_equal(buf.reshape(-1, 528)[:70, 512:516].copy().view(np.float32).ravel(), s)


def test_ue8m0_exponent_rule_is_exact():
    """The writer's exponent is the smallest e with amax <= 448 * 2**e, also right at the boundaries
    (checked in exact rational arithmetic), 0 for a zero group and clamped to [-120, 120]."""
    from fractions import Fraction
    from oracle import ue8m0_exponents
    rng = np.random.default_rng(5)
    amax = np.concatenate([
        np.float32(448.0) * np.exp2(np.arange(-30, 31)).astype(np.float32),                      # on the boundary
        np.nextafter(np.float32(448.0) * np.exp2(np.arange(-30, 31)).astype(np.float32), np.float32(np.inf)),
        np.nextafter(np.float32(448.0) * np.exp2(np.arange(-30, 31)).astype(np.float32), np.float32(0)),
        np.exp(rng.uniform(-60, 60, 400)).astype(np.float32),
        np.array([0.0, 1e-45, 1e-39, 3e38], np.float32)])
    groups = np.zeros((amax.size, 64), np.float32)
    groups[np.arange(amax.size), rng.integers(0, 64, amax.size)] = amax * rng.choice([-1.0, 1.0], amax.size).astype(np.float32)
    e = ue8m0_exponents(groups)
    for a, ei in zip(amax.tolist(), e.tolist()):
        if a == 0.0:
            assert ei == 0
            continue
        fa = Fraction(a)
        want = 0
        while fa > 448 * Fraction(2) ** want:
            want += 1
        while fa <= 448 * Fraction(2) ** (want - 1):
            want -= 1
        assert ei == max(-120, min(120, want)), (a, ei, want)


def test_scatter_writers_match_packers():
    from oracle import quantize_int8_rows_writer, write_fp8_ds_mla, write_int8_inline528
    rng = np.random.default_rng(6)
    x = rng.standard_normal((50, 512)).astype(np.float32)
    x[7] = 0
    x[8] *= 1e-11
    cache, _ = pack_fp8_ds_mla(x, 16)
    mine = np.zeros_like(cache)
    write_fp8_ds_mla(mine, x, np.arange(50))
    assert np.array_equal(mine, cache)
    q, s = quantize_int8_rows(x)
    buf = np.zeros((4, 16, 528), np.uint8)
    write_int8_inline528(buf, x, np.arange(50))
    assert np.array_equal(buf, pack_int8_inline528(q, s, 16))
    # scattered slots, skipped rows, untouched bytes
    slots = rng.permutation(64)[:50]
    slots[3], slots[4] = -1, 64
    buf2 = np.full((4, 16, 528), 0xA5, np.uint8)
    write_int8_inline528(buf2, x, slots, scale_rule=1)
    qw, sw = quantize_int8_rows_writer(x)
    assert sw[8] == np.float32(1e-12) and s[8] != sw[8] and np.array_equal(s[:7], sw[:7])
    flat = buf2.reshape(64, 528)
    for i, sl in enumerate(slots.tolist()):
        if 0 <= sl < 64:
            assert np.array_equal(flat[sl, :512].view(np.int8), qw[i]) and flat[sl, 512:516].view(np.float32)[0] == sw[i]
    untouched = np.setdiff1d(np.arange(64), slots[(slots >= 0) & (slots < 64)])
    assert (flat[untouched] == 0xA5).all()


def test_dense_mla_oracle_matches_reference_oracle(golden):
    """``oracle.dense_mla_decode`` against outputs of the reference's dense oracle
    (tests/test_flash_mla_sm80.py:10-27 on the rows of each sequence), with and without the causal mask;
    rows past a sequence's length are NaN in the fixture and must not reach the result."""
    g = golden("dense_mla_small.npz")
    from oracle import dense_mla_decode
    q = bf16_bits_to_f32(g["q_bf16"])
    kc = bf16_bits_to_f32(g["k_cache_bf16"])
    for causal in (False, True):
        out, lse = dense_mla_decode(q, kc, g["block_table"], g["cache_seqlens"], causal=causal)
        np.testing.assert_allclose(out, g["out_causal" if causal else "out"], rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(lse, g["lse_causal" if causal else "lse"], rtol=2e-5, atol=2e-6)
