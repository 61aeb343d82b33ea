"""GPU parity tests of dense paged MLA decode (``flash_mla_with_kvcache``): the sm_100a kernel through the
reference-shaped Python API and through the C ABI, against the golden fixture made with the reference's own
oracle and against the CPU oracle on seeded inputs.  The cases mirror the reference's dense test,
tests/test_flash_mla_sm80.py:43-121 (batch, query positions, heads, ragged lengths, causal mask, NaN in
every row past a sequence's length), and use its gate: ``cos_diff < 8e-5`` for the output and for the lse.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import bf16_from_bits, device_status
import oracle
from bench_workloads import dense_decode_workload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fm():
    import flash_mla
    return flash_mla


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert device_status() == 0, "a kernel wait ran out (device status word set)"


def check(out, lse, ref_out, ref_lse, what, sequences=None):
    out = out.float().cpu().numpy()
    lse = lse.float().cpu().numpy()
    if sequences is not None:
        out, lse, ref_out, ref_lse = out[sequences], lse[sequences], ref_out[sequences], ref_lse[sequences]
    assert np.isfinite(out).all(), f"{what}: non-finite output (a row past a sequence's length was read?)"
    assert oracle.cos_diff(out, ref_out) < 8e-5, f"{what}: out cos_diff {oracle.cos_diff(out, ref_out):.3e}"
    fin = np.isfinite(ref_lse)
    assert (np.isfinite(lse) == fin).all(), f"{what}: lse finiteness differs"
    assert oracle.cos_diff(lse[fin], ref_lse[fin]) < 8e-5, f"{what}: lse cos_diff"
    # the reference's elementwise bound for the sparse ops holds here too (outputs are O(1))
    assert np.abs(out - ref_out).max() <= 2e-2 + 2e-2 * np.abs(ref_out).max(), f"{what}: max abs {np.abs(out - ref_out).max():.3e}"
    assert np.abs(lse[fin] - ref_lse[fin]).max() <= 2e-3 + 1e-3 * np.abs(ref_lse[fin]).max(), f"{what}: lse max abs"


def run_api(fm, kw, causal):
    meta, splits = fm.get_mla_metadata(kw["cache_seqlens"], kw["q"].shape[1] * kw["q"].shape[2], 1)
    return fm.flash_mla_with_kvcache(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], 512,
                                     meta, splits, causal=causal)


# ----------------------------------------------------------------------------- golden fixture
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("via", ["python", "c_abi"])
def test_dense_golden(fm, golden, causal, via):
    g = golden("dense_mla_small.npz")
    q = bf16_from_bits(g["q_bf16"])
    kc = bf16_from_bits(g["k_cache_bf16"])
    bt = torch.from_numpy(g["block_table"]).cuda()
    lens = torch.from_numpy(g["cache_seqlens"]).cuda()
    if via == "python":
        out, lse = run_api(fm, {"q": q, "k_cache": kc, "block_table": bt, "cache_seqlens": lens}, causal)
    else:
        from flash_mla import c_abi
        lib = c_abi.load()
        out = torch.empty(*q.shape[:3], 512, device="cuda", dtype=torch.bfloat16)
        lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], device="cuda", dtype=torch.float32)
        p = c_abi.dense_params(q, kc, bt, lens, out, lse, causal=causal, num_splits=1)
        c_abi.check(lib.smla_dense_mla_decode(ctypes.byref(p), torch.cuda.current_stream().cuda_stream))
    check(out, lse, g["out_causal" if causal else "out"], g["lse_causal" if causal else "lse"], f"golden {via} causal={causal}")


# ----------------------------------------------------------------------------- the reference test's sweep, reduced
@pytest.mark.parametrize("h_q", [16, 32, 64, 128])
@pytest.mark.parametrize("s_q", [1, 2])
@pytest.mark.parametrize("varlen", [False, True])
def test_dense_sweep(fm, h_q, s_q, varlen):
    kw, _ = dense_decode_workload(b=6, s_q=s_q, mean_sk=1500, h_q=h_q, varlen=varlen, block_size=32, seed=h_q + s_q)
    out, lse = run_api(fm, kw, causal=True)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], causal=True)
    check(out, lse, ref_out, ref_lse, f"h_q={h_q} s_q={s_q} varlen={varlen}")


@pytest.mark.parametrize("b,mean_sk,block_size", [(1, 8192, 64), (2, 4096, 64), (12, 3000, 64), (40, 700, 32), (700, 200, 64)])
def test_dense_every_schedule_and_merge(fm, b, mean_sk, block_size):
    """One sequence spread over the whole GPU (slice merge), a few (combine kernel), dozens (merge in the
    epilogue of the CTA holding a sequence's first rows), many (whole items, nothing to merge)."""
    kw, _ = dense_decode_workload(b=b, s_q=1, mean_sk=mean_sk, h_q=64, varlen=True, block_size=block_size, seed=b)
    out, lse = run_api(fm, kw, causal=False)
    seqs = list(range(min(b, 8))) + ([b - 1] if b > 8 else [])
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], sequences=seqs)
    check(out, lse, ref_out, ref_lse, f"b={b}", sequences=seqs)


@pytest.mark.parametrize("b,mean_sk,h_q", [(1, 20000, 128), (1, 9000, 16), (3, 6000, 8)])
def test_dense_long_sequences_cut_into_many_segments(fm, b, mean_sk, h_q):
    """A sequence cut across 40-70 CTAs leaves every CTA at most one head of the slice merge; the CTA's warps
    then share that head's segments and add their sums in shared memory."""
    kw, _ = dense_decode_workload(b=b, s_q=1, mean_sk=mean_sk, h_q=h_q, varlen=True, seed=7 * b + h_q)
    out, lse = run_api(fm, kw, causal=False)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"])
    check(out, lse, ref_out, ref_lse, f"b={b} s_k~{mean_sk} h_q={h_q}")


@pytest.mark.parametrize("block_size", [16, 32, 64, 128, 256])
def test_dense_page_sizes(fm, block_size):
    """Pages smaller than, equal to and larger than the 128-row tile (the K tile is fetched in boxes of
    min(page, 128) rows), ragged lengths, two query positions with the causal mask."""
    kw, _ = dense_decode_workload(b=5, s_q=2, mean_sk=900, h_q=64, varlen=True, block_size=block_size, seed=block_size)
    out, lse = run_api(fm, kw, causal=True)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], causal=True)
    check(out, lse, ref_out, ref_lse, f"page {block_size}")


@pytest.mark.parametrize("b,seqlen,heads", [(2, 128, 4), (4, 256, 8), (6, 1100, 64)])
def test_dense_head_dim_512(fm, b, seqlen, heads):
    """head_size 512 = head_size_v (the reference's tests/test_flash_mla_dsv4_sm80.py:18-40 shapes and a larger
    one): scores over 512 dims, no RoPE part."""
    kw, _ = dense_decode_workload(b=b, s_q=1, mean_sk=seqlen, h_q=heads, varlen=False, block_size=32, seed=b, d=512)
    out, lse = run_api(fm, kw, causal=True)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"])
    check(out, lse, ref_out, ref_lse, f"d=512 b={b} heads={heads}")


def test_dense_strided_cache_and_q(fm):
    """A cache whose rows are wider than 576 elements (row stride 640) and a q that is a slice of a wider
    tensor: strides are honoured, nothing is copied for the cache."""
    kw, _ = dense_decode_workload(b=4, s_q=1, mean_sk=700, h_q=32, varlen=True, block_size=64, seed=21)
    wide = torch.full((*kw["k_cache"].shape[:3], 640), float("nan"), device="cuda", dtype=torch.bfloat16)
    wide[..., :576] = kw["k_cache"]
    qwide = torch.randn(4, 1, 32, 600, device="cuda").to(torch.bfloat16)
    qwide[..., :576] = kw["q"]
    kw2 = dict(kw, k_cache=wide[..., :576], q=qwide[..., :576])
    out, lse = run_api(fm, kw2, causal=False)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"])
    check(out, lse, ref_out, ref_lse, "strided")


def test_dense_edges(fm):
    """Lengths at the edges: exactly s_q rows (the shortest the reference generates), exact multiples of the
    128-row tile and of the page, one row more, and 12 heads (not a multiple of 8: Q arrives by cp.async)."""
    kw, _ = dense_decode_workload(b=6, s_q=2, mean_sk=512, h_q=12, varlen=False, block_size=64, seed=3)
    kw["cache_seqlens"] = torch.tensor([2, 128, 129, 64, 512, 257], dtype=torch.int32, device="cuda")
    # re-poison the rows past the new lengths
    for i, n in enumerate(kw["cache_seqlens"].tolist()):
        rows = kw["k_cache"][kw["block_table"][i].long()].view(-1, 1, 576)
        rows[n:] = float("nan")
        kw["k_cache"][kw["block_table"][i].long()] = rows.view(-1, 64, 1, 576)
    for causal in (False, True):
        out, lse = run_api(fm, kw, causal)
        ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], causal=causal)
        check(out, lse, ref_out, ref_lse, f"edges causal={causal}")


@pytest.mark.parametrize("h_q,s_q", [(16, 2), (16, 4), (32, 2), (8, 3)])
@pytest.mark.parametrize("causal", [False, True])
def test_dense_folded_query_positions(fm, h_q, s_q, causal):
    """Few heads and several query positions: the positions are folded into the head dimension (one pass over
    the rows).  Lengths shorter than s_q leave early positions without any visible row under the causal mask
    (output zero, lse -inf, as the oracle), lengths around tile and page ends shift the mask across tiles."""
    kw, _ = dense_decode_workload(b=9, s_q=s_q, mean_sk=700, h_q=h_q, varlen=True, block_size=64, seed=h_q * s_q,
                                  poison_tail=False)          # poisoned below, past the lengths set here
    lens = kw["cache_seqlens"].clone()
    lens[:6] = torch.tensor([1, 2, 3, 129, 128, 257], dtype=torch.int32, device="cuda")
    kw["cache_seqlens"] = lens
    for i, n in enumerate(lens.tolist()):
        rows = kw["k_cache"][kw["block_table"][i].long()].view(-1, 1, 576)
        rows[n:] = float("nan")
        kw["k_cache"][kw["block_table"][i].long()] = rows.view(-1, 64, 1, 576)
    out, lse = run_api(fm, kw, causal)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], causal=causal)
    check(out, lse, ref_out, ref_lse, f"folded h={h_q} s_q={s_q} causal={causal}")


def test_dense_length_beyond_block_table_is_clamped(fm):
    """A length larger than the block table row can name must not make the kernel read past the table: it is
    clamped to max_blocks_per_seq * page rows (the sparse ops clamp lens to topk the same way)."""
    kw, _ = dense_decode_workload(b=3, s_q=1, mean_sk=512, h_q=64, varlen=False, block_size=64, seed=2, poison_tail=False)
    cap = kw["block_table"].shape[1] * 64
    kw["cache_seqlens"] = torch.tensor([cap + 1000, 300, 2 ** 30], dtype=torch.int32, device="cuda")
    out, lse = run_api(fm, kw, causal=False)
    clamped = torch.tensor([cap, 300, cap], dtype=torch.int32)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], clamped)
    check(out, lse, ref_out, ref_lse, "clamped lengths")


@pytest.mark.parametrize("b", [2, 40])
def test_dense_replays_from_a_cuda_graph(fm, b):
    """Captured once, replayed with new q, new lengths and a new block table in the same buffers (b = 2: a
    sequence spread over many CTAs; b = 40: merges in the owning CTA's epilogue): every replay must match the
    oracle, i.e. nothing the kernels use to hand partial results between CTAs may depend on the launch."""
    kw, _ = dense_decode_workload(b=b, s_q=1, mean_sk=1800, h_q=64, varlen=True, block_size=64, seed=100 + b, poison_tail=False)
    q, bt, sl, kc = kw["q"], kw["block_table"], kw["cache_seqlens"], kw["k_cache"]
    cap = bt.shape[1] * 64
    md, ns = fm.get_mla_metadata(sl, 64, 1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fm.flash_mla_with_kvcache(q, kc, bt, sl, 512, md, ns)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, lse = fm.flash_mla_with_kvcache(q, kc, bt, sl, 512, md, ns)
    gen = torch.Generator(device="cuda").manual_seed(b)
    for rep in range(3):
        q.copy_(torch.randn(q.shape, device="cuda", generator=gen).to(torch.bfloat16))
        sl.copy_(torch.randint(1, cap + 1, (b,), device="cuda", generator=gen, dtype=torch.int32))
        bt.copy_(bt.flatten()[torch.randperm(bt.numel(), device="cuda", generator=gen)].view_as(bt))
        graph.replay()
        torch.cuda.synchronize()
        seqs = list(range(min(b, 6)))
        ref_out, ref_lse = oracle.dense_mla_decode(q, kc, bt, sl, sequences=seqs)
        check(out, lse, ref_out, ref_lse, f"graph replay {rep}, b={b}", sequences=seqs)


@pytest.mark.parametrize("case", range(16))
def test_dense_random_problems(fm, case):
    """Random small problems: batch, query positions, heads (any count, not only multiples of 8), page size,
    ragged lengths from 1 to several tiles, head_dim 576 or 512, with and without the causal mask."""
    rng = np.random.default_rng(9000 + case)
    b = int(rng.integers(1, 12))
    s_q = int(rng.choice([1, 1, 2, 3, 4]))
    h_q = int(rng.choice([1, 4, 8, 12, 16, 24, 32, 40, 64, 72, 128]))
    page = int(rng.choice([16, 32, 64, 128, 256]))
    d = int(rng.choice([576, 576, 512]))
    causal = bool(rng.integers(0, 2))
    kw, _ = dense_decode_workload(b=b, s_q=s_q, mean_sk=int(rng.integers(64, 1400)), h_q=h_q, varlen=True,
                                  block_size=page, seed=case, poison_tail=False, d=d)
    cap = kw["block_table"].shape[1] * page
    lens = torch.from_numpy(rng.integers(1, cap + 1, b).astype(np.int32)).cuda()
    if case % 4 == 0:
        lens[0] = int(rng.choice([1, 127, 128, 129, 255, 256]))
    kw["cache_seqlens"] = lens
    for i, n in enumerate(lens.tolist()):
        rows = kw["k_cache"][kw["block_table"][i].long()].view(-1, 1, d)
        rows[n:] = float("nan")
        kw["k_cache"][kw["block_table"][i].long()] = rows.view(-1, page, 1, d)
    out, lse = run_api(fm, kw, causal)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], lens, causal=causal)
    check(out, lse, ref_out, ref_lse, f"case {case}: b={b} s_q={s_q} h_q={h_q} page={page} d={d} causal={causal}")


@pytest.mark.parametrize("page,h_q,s_q", [(48, 64, 1), (48, 16, 2), (96, 128, 1), (24, 8, 3)])
def test_dense_page_sizes_the_boxes_cannot_serve(fm, page, h_q, s_q):
    """A 128-row tile is neither a whole number of these pages nor a page a whole number of tiles: the rows are
    copied by the worker threads with cp.async instead of by TMA boxes.  Ragged lengths, NaN behind every sequence."""
    rng = np.random.default_rng(page * 1000 + h_q)
    b = 5
    kw, _ = dense_decode_workload(b=b, s_q=s_q, mean_sk=768, h_q=h_q, varlen=False, block_size=page, seed=page + h_q,
                                  poison_tail=False)
    cap = kw["block_table"].shape[1] * page
    lens = torch.from_numpy(rng.integers(1, cap + 1, b).astype(np.int32)).cuda()
    lens[0] = cap
    lens[1] = 129
    kw["cache_seqlens"] = lens
    for i, n in enumerate(lens.tolist()):
        rows = kw["k_cache"][kw["block_table"][i].long()].view(-1, 1, 576)
        rows[n:] = float("nan")
        kw["k_cache"][kw["block_table"][i].long()] = rows.view(-1, page, 1, 576)
    out, lse = run_api(fm, kw, causal=s_q > 1)
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], lens, causal=s_q > 1)
    check(out, lse, ref_out, ref_lse, f"page {page} h_q={h_q} s_q={s_q}")


def test_dense_full_size_sample(fm):
    """The reference test's own size (b=128, s_k=4096, h_q=128, s_q=2, ragged, causal), checked on a sample
    of the sequences."""
    kw, _ = dense_decode_workload(b=128, s_q=2, mean_sk=4096, h_q=128, varlen=True, block_size=64, seed=1)
    out, lse = run_api(fm, kw, causal=True)
    lens = kw["cache_seqlens"].cpu()
    seqs = sorted({0, 127, int(lens.argmax()), int(lens.argmin()), 17, 63})
    ref_out, ref_lse = oracle.dense_mla_decode(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], causal=True, sequences=seqs)
    check(out, lse, ref_out, ref_lse, "b=128 s_k=4096 h_q=128 s_q=2", sequences=seqs)


def test_dense_split_equals_whole_items(fm):
    """The balanced schedule with in-kernel merges against whole items (num_splits = 1) through the C ABI."""
    from flash_mla import c_abi
    lib = c_abi.load()
    kw, _ = dense_decode_workload(b=24, s_q=1, mean_sk=2500, h_q=64, varlen=True, block_size=64, seed=9)
    q = kw["q"]
    res = []
    for splits in (1, 0):
        out = torch.empty(*q.shape[:3], 512, device="cuda", dtype=torch.bfloat16)
        lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], device="cuda", dtype=torch.float32)
        ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
        p = c_abi.dense_params(q, kw["k_cache"], kw["block_table"], kw["cache_seqlens"], out, lse, num_splits=splits, workspace=ws)
        c_abi.check(lib.smla_dense_mla_decode(ctypes.byref(p), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        res.append((out.float(), lse))
    assert (res[0][0] - res[1][0]).abs().max().item() <= 2 ** -7
    assert (res[0][1] - res[1][1]).abs().max().item() <= 1e-3     # denominators sum bf16-rounded probabilities
