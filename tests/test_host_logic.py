"""CPU-side tests: the C-ABI library loads and exports every declared symbol, the host-only entry
points (split policy, workspace size, error strings) behave, the Python wrappers validate like the
reference's, and token sharding works across two gloo ranks.  No GPU, no compute calls."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sparse_mla_b200.h")).read()
    return re.findall(r"^SMLA_API\s+[\w\s\*]+?\b(smla_\w+)\s*\(", text, flags=re.M)


def test_library_exports_every_declared_symbol():
    from flash_mla import c_abi
    lib = c_abi.load()
    declared = _declared_symbols()
    assert len(declared) >= 9
    assert set(declared) == set(c_abi.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert b"sm_100a" in lib.smla_version()


def test_struct_layout_matches_header():
    """ctypes mirrors of the three structs: field order as in the header, natural alignment."""
    from flash_mla import c_abi
    text = open(os.path.join(ROOT, "include", "sparse_mla_b200.h")).read()

    def fields(struct):
        body = re.search(r"typedef struct %s \{(.*?)\} %s_t;" % (struct, struct), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                names.append(re.findall(r"(\w+)\s*$", part.strip())[0])
        return names
    assert fields("smla_stream") == [f[0] for f in c_abi.SmlaStream._fields_]
    assert fields("smla_attn_params") == [f[0] for f in c_abi.SmlaAttnParams._fields_]
    assert fields("smla_dense_params") == [f[0] for f in c_abi.SmlaDenseParams._fields_]
    assert ctypes.sizeof(c_abi.SmlaStream) == 88
    assert ctypes.sizeof(c_abi.SmlaAttnParams) == 272


def test_struct_layout_matches_c_compiler(tmp_path):
    """Compile the header as plain C and compare sizeof/offsetof with the ctypes mirrors."""
    import shutil
    from flash_mla import c_abi
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    checks = [("smla_stream_t", c_abi.SmlaStream), ("smla_attn_params_t", c_abi.SmlaAttnParams),
              ("smla_dense_params_t", c_abi.SmlaDenseParams)]
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "sparse_mla_b200.h"', 'int main(void){']
    for cname, cls in checks:
        lines.append(f'printf("%zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'printf("%zu\\n", offsetof({cname}, {fname}));')
    lines.append('return 0;}')
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)],
                   check=True)
    got = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = []
    for _, cls in checks:
        want.append(ctypes.sizeof(cls))
        want += [getattr(cls, f).offset for f, _ in cls._fields_]
    assert got == want


def test_split_policy_and_workspace():
    from flash_mla import c_abi
    lib = c_abi.load()
    os.environ.pop("FLASH_MLA_SLOTS_PER_SPLIT", None)
    f = lib.smla_choose_num_splits
    # >= 4 items (token x block of 64 heads) per SM: whole items per CTA, nothing to merge
    assert f(148, 1024, 64, 2560) == 1
    assert f(148, 296, 128, 2560) == 1
    # otherwise: scratch for (2 * CTAs + 1) slots of 64 heads, expressed per (token, head)
    assert f(148, 128, 64, 2560) == 3            # 148 CTAs: ceil(297 * 64 / (128 * 64))
    assert f(148, 1, 64, 2560) == 41             # 20 tiles -> 20 CTAs -> 41 slots for one token
    assert f(148, 1, 64, 512) == 9
    assert f(148, 8, 64, 2560) == 38
    assert f(148, 8, 128, 2560) == 19            # two head blocks per token
    assert f(148, 1, 64, 100) == 1               # a single tile: one CTA
    assert f(148, 1, 16, 2560) == 41             # slots shrink with the head block (16 heads)
    os.environ["FLASH_MLA_SLOTS_PER_SPLIT"] = "512"
    try:
        assert f(148, 1, 64, 2560) == 11         # at least 512 rows per CTA -> 5 CTAs; read on every call
    finally:
        os.environ.pop("FLASH_MLA_SLOTS_PER_SPLIT")
    # kernels per decode call: the merge is fused unless ~10..70 items are spread over the SMs
    k = lib.smla_decode_kernel_launches
    assert k(148, 128, 64, f(148, 128, 64, 2560)) == 1      # an item cut in two or three: merged in the owner's epilogue
    assert k(148, 1, 64, f(148, 1, 64, 2560)) == 1          # one token on 20 SMs: every CTA merges a slice of the heads
    assert k(148, 8, 64, f(148, 8, 64, 2560)) == 1
    assert k(148, 32, 64, f(148, 32, 64, 2560)) == 2        # in between: attention kernel + combine kernel
    assert k(148, 1024, 64, 1) == 1                         # whole items, nothing to merge
    assert k(148, 128, 64, 2) == 1                          # scratch for 62 CTAs only: still two or three segments per item
    kc = lib.smla_decode_kernel_launches_captured           # on a capturing stream the slice merge gives way to the combine kernel
    assert kc(148, 1, 64, f(148, 1, 64, 2560)) == 2 and kc(148, 8, 64, f(148, 8, 64, 2560)) == 2
    assert kc(148, 128, 64, f(148, 128, 64, 2560)) == 1 and kc(148, 32, 64, f(148, 32, 64, 2560)) == 2
    assert kc(148, 1024, 64, 1) == 1
    w = lib.smla_attn_workspace_bytes
    assert w(4, 64, 1) == 0
    assert w(4, 64, 8) == 4 * 64 * 8 * (512 + 2) * 4
    assert b"alignment" in lib.smla_error_string(-2)
    assert lib.smla_error_string(0) == b"ok"


def test_null_and_bad_arguments_are_rejected_without_a_device_call():
    from flash_mla import c_abi
    lib = c_abi.load()
    assert lib.smla_sparse_mla_decode(None, None) == -1
    assert lib.smla_sparse_mla_prefill(None, None) == -1
    assert lib.smla_quantize_int8_ds_mla_rows(None, 0, 0, 512, None, None, None) == 0   # zero rows: nothing to do
    assert lib.smla_quantize_int8_ds_mla_rows(None, 0, 4, 512, None, None, None) == -1


def test_wrapper_validation_matches_reference():
    """ValueError before any op call (flash_mla/flash_mla_interface.py:8-18,
    flash_mla/int8_sparse_mla.py:22-23,313-324 of the reference)."""
    import flash_mla
    q = torch.zeros(2, 4, 512, dtype=torch.bfloat16)
    idx4 = torch.zeros(2, 1, 1, 8, dtype=torch.int32)
    with pytest.raises(ValueError, match="num_tokens, topk"):
        flash_mla.sparse_mla_decode_fp8(q, torch.zeros(1, 1, 584, dtype=torch.uint8), idx4, torch.zeros(2, dtype=torch.int32))
    with pytest.raises(ValueError, match="head dim"):
        flash_mla.sparse_mla_decode_int8(q[..., :64], None, None, None, None)
    with pytest.raises(ValueError, match="singleton"):
        flash_mla.sparse_mla_prefill_int8(q, None, None, torch.zeros(2, 2, 8, dtype=torch.int32), None)
    with pytest.raises(ValueError, match="last dim"):
        flash_mla.quantize_int8_ds_mla_rows(torch.zeros(3, 100))
    # the ops exist with the reference's schemas
    for name in ("fwd_sparse_decode_mla", "fwd_sparse_prefill_mla", "fwd_sparse_int8_decode_mla",
                 "fwd_sparse_int8_prefill_mla", "quantize_int8_ds_mla_rows"):
        assert hasattr(torch.ops.flash_mla, name)
    s = str(torch.ops.flash_mla.fwd_sparse_int8_decode_mla.default._schema)
    assert "Tensor swa_scale" in s and "Tensor? extra_lens" in s and "float scale" in s


def test_cpu_tensors_fail_loudly():
    """No CPU fallback: the ops are registered for the CUDA dispatch key only."""
    import flash_mla
    q = torch.zeros(1, 4, 512, dtype=torch.bfloat16)
    with pytest.raises((RuntimeError, NotImplementedError)):
        flash_mla.sparse_mla_decode_fp8(q, torch.zeros(1, 2, 584, dtype=torch.uint8),
                                        torch.zeros(1, 2, dtype=torch.int32), torch.ones(1, dtype=torch.int32))
    with pytest.raises((RuntimeError, NotImplementedError)):
        flash_mla.quantize_int8_ds_mla_rows(torch.zeros(3, 512))


def test_token_range():
    from flash_mla.sharding import token_range
    for T in (0, 1, 7, 128, 1024, 1025):
        for w in (1, 2, 3, 4, 8):
            spans = [token_range(T, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == T
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        token_range(4, 2, 2)


def test_cache_writers_match_oracle_packers():
    import oracle
    from flash_mla.cache_formats import pack_fp8_ds_mla, pack_int8_inline528
    torch.manual_seed(3)
    x = torch.randn(75, 512)
    x[3] *= 50
    x[4] = 0
    xb = x.to(torch.bfloat16)
    c = pack_fp8_ds_mla(xb, 32)
    c2, _ = oracle.pack_fp8_ds_mla(xb.float().numpy(), 32)
    assert np.array_equal(c.numpy(), c2)
    q, s = oracle.quantize_int8_rows(xb.float().numpy())
    buf, dv, sv = pack_int8_inline528(torch.from_numpy(q), torch.from_numpy(s), 16)
    assert np.array_equal(buf.numpy(), oracle.pack_int8_inline528(q, s, 16))
    assert dv.stride(1) == 528 and sv.stride(1) == 132


_GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "forks-flash-mla-int_b200"))
import oracle
from flash_mla.sharding import shard_tokens, token_range, gather_outputs
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
rng = np.random.default_rng(0)                      # same inputs on every rank (replicated cache)
T, H, topk, slots = 7, 4, 48, 96
K = oracle.ds_mla_formats.round_to_bf16(rng.standard_normal((slots, 512)).astype(np.float32))
kw = dict(q=torch.from_numpy(oracle.ds_mla_formats.round_to_bf16(rng.standard_normal((T, H, 512)).astype(np.float32))),
          swa_indices=torch.from_numpy(rng.integers(-2, slots + 3, (T, topk)).astype(np.int32)),
          swa_lens=torch.from_numpy(rng.integers(0, topk + 1, (T,)).astype(np.int32)))
full = oracle.sparse_mla_attention(kw["q"], K, kw["swa_indices"], kw["swa_lens"])
mine = shard_tokens(kw, world, rank)
a, b = token_range(T, world, rank)
assert mine["q"].shape[0] == b - a
local = torch.from_numpy(oracle.sparse_mla_attention(mine["q"], K, mine["swa_indices"], mine["swa_lens"]))
allo = gather_outputs(local, T)
assert allo.shape == (T, H, 512)
assert np.array_equal(allo.numpy(), full), "sharded result differs from the unsharded one"
# dense paged MLA: sequences shard the same way (block table and lengths with q, cache replicated)
from flash_mla.sharding import shard_sequences
g = torch.Generator().manual_seed(3)
dkw = dict(q=torch.randn(5, 2, 4, 576, generator=g).to(torch.bfloat16),
           k_cache=torch.randn(20, 16, 1, 576, generator=g).to(torch.bfloat16),
           block_table=torch.randperm(20, generator=g).to(torch.int32).view(5, 4),
           cache_seqlens=torch.tensor([3, 64, 17, 40, 2], dtype=torch.int32))
dfull, dlse = oracle.dense_mla_decode(dkw["q"], dkw["k_cache"], dkw["block_table"], dkw["cache_seqlens"], causal=True)
dm = shard_sequences(dkw, world, rank)
da, db = token_range(5, world, rank)
dloc, _ = oracle.dense_mla_decode(dm["q"], dm["k_cache"], dm["block_table"], dm["cache_seqlens"], causal=True)
dall = gather_outputs(torch.from_numpy(dloc), 5)
assert np.array_equal(dall.numpy(), dfull), "sharded dense result differs from the unsharded one"
dist.barrier(); dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_token_sharding_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29531", WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o}"
        assert f"rank {r} ok" in o
