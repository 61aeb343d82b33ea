"""Second pin of parity: this library against the REFERENCE'S OWN CUDA kernels run on the same GPU
(the reference's Ampere mma.sync code compiled for sm_100 from its checkout by
oracle/ref_gpu/build_ref.py into oracle/_ref/, which travels to the GPU box as a built file).
Skipped where that library is absent.  Both outputs are bf16 roundings of the same fp32 quantity
computed with bf16 P, so they must agree to about one bf16 ulp; both are also held to the oracle gate.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,T,H", [("fp8", 2, 64), ("int8", 1, 64), ("int8", 8, 64), ("int8", 96, 32)])
def test_matches_reference_cuda_kernels(fmt, T, H):
    from oracle import ref_gpu, cos_diff
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/libref_sparse_mla.so not built (needs the reference checkout)")
    import flash_mla
    import bench_workloads as synthetic
    kw, meta = synthetic.decode_workload(fmt=fmt, T=T, H=H, swa_slots=4096, extra_slots=4096, swa_topk=256,
                                         extra_topk=768, seed=9, outlier_frac=0.0)
    op = flash_mla.sparse_mla_decode_fp8 if fmt == "fp8" else flash_mla.sparse_mla_decode_int8
    mine = op(**kw).float().cpu().numpy()
    ref = ref_gpu.RefDecode(kw["q"], kw["swa_cache"], kw.get("swa_scale"), kw["swa_indices"], kw["swa_lens"], None,
                            kw.get("attn_sink"), kw.get("extra_cache"), kw.get("extra_scale"), kw.get("extra_indices"),
                            kw.get("extra_lens"))
    theirs = ref().float().cpu().numpy()
    torch.cuda.synchronize()
    d = np.abs(mine - theirs)
    assert d.max() <= 4e-3 and d.mean() <= 2e-4, (d.max(), d.mean())
    assert cos_diff(mine, theirs) < 8e-5


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_match_reference_cuda_kernels(seed):
    """Sixty random decode problems per seed: token counts 1..260 (whole-item and balanced schedules, all
    three merge forms), 16..128 heads, both formats and int8 layouts, with and without the extra stream
    and the sink, ragged lens with empty tokens.  The reference's fp8 kernel returns NaN for a token
    without rows; this library returns zeros there (the Python API's documented result)."""
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/libref_sparse_mla.so not built (needs the reference checkout)")
    import flash_mla
    import bench_workloads as synthetic
    from helpers import device_status
    rng = np.random.default_rng(seed)
    for it in range(60):
        fmt = str(rng.choice(["fp8", "int8"]))
        T = int(rng.choice([1, 2, 3, 5, 8, 13, 21, 40, 75, 100, 150, 260]))
        H = int(rng.choice([16, 32, 64, 128]))
        st = int(rng.choice([64, 128, 256, 512]))
        et = int(rng.choice([0, 128, 640, 1024, 2048]))
        layout = str(rng.choice(["inline528", "separate"]))
        kw, _ = synthetic.decode_workload(fmt=fmt, T=T, H=H, swa_slots=2048, extra_slots=4096, swa_topk=st, extra_topk=et,
                                          seed=int(rng.integers(1 << 30)), outlier_frac=0.0, sink=bool(rng.integers(2)),
                                          layout=layout, mask_frac=float(rng.choice([0.0, 0.05])))
        kw["swa_lens"] = torch.randint(0, st + 1, (T,), device="cuda", dtype=torch.int32)
        if et > 0:
            kw["extra_lens"] = torch.randint(0, et + 1, (T,), device="cuda", dtype=torch.int32)
        if T > 2:
            kw["swa_lens"][0] = 0
            if et > 0:
                kw["extra_lens"][0] = 0
        op = flash_mla.sparse_mla_decode_fp8 if fmt == "fp8" else flash_mla.sparse_mla_decode_int8
        mine = op(**kw).float().cpu().numpy()
        ref = ref_gpu.RefDecode(kw["q"], kw["swa_cache"], kw.get("swa_scale"), kw["swa_indices"], kw["swa_lens"], None,
                                kw.get("attn_sink"), kw.get("extra_cache"), kw.get("extra_scale"), kw.get("extra_indices"),
                                kw.get("extra_lens"))
        theirs = ref().float().cpu().numpy()
        torch.cuda.synchronize()
        what = f"seed {seed} case {it}: {fmt} T={T} H={H} swa {st} extra {et} {layout}"
        assert not np.isnan(mine).any(), what
        rows = (kw["swa_lens"] + (kw["extra_lens"] if et > 0 else 0)).cpu().numpy()
        their_nan = np.isnan(theirs).any(axis=(1, 2))
        assert np.all(rows[their_nan] == 0), what          # the reference only fails on empty tokens ...
        assert np.all(mine[rows == 0] == 0), what          # ... where this library returns zeros
        keep = ~their_nan
        if keep.any():
            d = np.abs(mine[keep] - theirs[keep])
            top = float(np.abs(theirs[keep]).max())
            # two bf16 roundings of (almost) the same fp32 value: at most one ulp of the output apart
            assert d.max() <= max(8e-3, top * 2.0 ** -7), (what, d.max(), top)
            assert d.mean() <= 4e-4 * max(1.0, top), (what, d.mean())
    assert device_status() == 0
