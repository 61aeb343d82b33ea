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
    from flash_mla import synthetic
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
