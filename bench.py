#!/usr/bin/env python3
"""Benchmark of the sparse-MLA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl native|reference]

A step is one pass of the op over one batch of synthetic query tokens.  The headline workload is the
DSV4-Flash absorbed fp8 decode shape (BASELINE config 2: 128 tokens x 64 heads, swa 65536 slots / top-k
512 plus a compressed extra stream of 16384 slots / top-k 2048, attn_sink); every rank of a multi-GPU
run processes its own batch against its own cache replica (token sharding, no collective on the data
path), so the headline scales weakly.  Prints ONE JSON line (rank 0).

Timing: W warm-up steps, then K steps between CUDA events on the launching stream, bracketed by a
barrier + synchronize, max over ranks.  The cache is rotated through replicas whose total size
exceeds the 126 MB L2 so a step never finds its rows cached by the previous one.
`e2e` repeats the measurement through the public API from HOST buffers: the step's inputs (q,
indices, lens, packed in one pinned staging buffer) are copied to the device and the output back to
pinned host memory inside the timed region; the paged KV cache stays resident in HBM, as it does in
serving.  `e2e.pcie_floor_ms` is the time of the same copies alone.  `cpu_baseline` times the fp32 CPU
oracle on a bounded token sample.

With the default workload the line also carries, measured in the same process:
  other_configs  BASELINE config 3 (int8 decode, T in {1, 8, 32, 128, 512} x H in {64, 128}), config 4
                 (int8 prefill, 4096 tokens) and config 5's shapes on one GPU: ms per step, tokens/s,
                 TFLOP/s, roofline, a sampled-token parity check against the CPU oracle and, where the
                 reference's own CUDA kernels were built (oracle/_ref), their time on the same inputs;
  dense_configs  dense bf16 paged MLA decode (flash_mla_with_kvcache) on the reference's dense test shapes
                 (batch 128, 4096 / 8192 rows per sequence, 16 / 64 / 128 heads): ms per step, tokens/s,
                 TFLOP/s, roofline, parity of three sequences against the CPU oracle;
  config5        ONE seeded batch of 1024 tokens (128 heads, 16384-slot caches, top-k 2048 + 512, fp8
                 and int8) cut by token over the N ranks with flash_mla.sharding.shard_tokens, caches
                 replicated: strong scaling against the same batch on one GPU of the same run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "forks-flash-mla-int_b200"))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: (op kind, builder kwargs, description)
    "dsv4_fp8_decode_T128_H64": ("decode_fp8", dict(fmt="fp8", T=128, H=64)),
    **{f"dsv4_int8_decode_T{t}_H{h}": ("decode_int8", dict(fmt="int8", T=t, H=h))
       for t in (1, 8, 32, 128, 512) for h in (64, 128)},
    "ctx16k_fp8_decode_T1024_H128": ("decode_fp8", dict(fmt="fp8", T=1024, H=128, swa_slots=16384, swa_topk=2048,
                                                        extra_slots=16384, extra_topk=512, mask_frac=0.0,
                                                        full_lens=True)),
    "ctx16k_int8_decode_T1024_H128": ("decode_int8", dict(fmt="int8", T=1024, H=128, swa_slots=16384, swa_topk=2048,
                                                          extra_slots=16384, extra_topk=512, mask_frac=0.0,
                                                          full_lens=True)),
    "int8_prefill_T4096_H64": ("prefill_int8", dict(T=4096, H=64)),
    # dense paged MLA decode (flash_mla_with_kvcache): the reference's dense test shapes, bf16 cache, pages of 64
    "dense_bf16_decode_b128_s4096_h128": ("dense", dict(b=128, s_q=1, mean_sk=4096, h_q=128, varlen=False)),
    "dense_bf16_decode_b128_s4096_h16": ("dense", dict(b=128, s_q=1, mean_sk=4096, h_q=16, varlen=False)),
    "dense_bf16_decode_b128_s8192_h64_sq2_varlen": ("dense", dict(b=128, s_q=2, mean_sk=8192, h_q=64, varlen=True)),
    "dense_bf16_decode_b128_s4096_h16_sq2": ("dense", dict(b=128, s_q=2, mean_sk=4096, h_q=16, varlen=False)),
    # latency shapes: few sequences, every sequence cut across many CTAs and merged inside the kernel
    "dense_bf16_decode_b1_s32768_h128": ("dense", dict(b=1, s_q=1, mean_sk=32768, h_q=128, varlen=False)),
    "dense_bf16_decode_b8_s4096_h128": ("dense", dict(b=8, s_q=1, mean_sk=4096, h_q=128, varlen=False)),
    # cache writers (the step before the attention calls): 2^20 new bf16 latent rows scattered into a paged cache
    "write_int8_cache_rows1M": ("write_int8", dict(rows=1 << 20, block_size=64)),
    "write_fp8_cache_rows1M": ("write_fp8", dict(rows=1 << 20, block_size=64)),
    "write_int8_cache_rows256k": ("write_int8", dict(rows=1 << 18, block_size=64)),
    "write_fp8_cache_rows256k": ("write_fp8", dict(rows=1 << 18, block_size=64)),
    # the int8 row quantizer alone (quantize_int8_ds_mla_rows): rows in, int8 rows + fp32 scales out
    "quantize_int8_rows1M": ("write_quantize", dict(rows=1 << 20, block_size=64)),
    "quantize_int8_rows256k": ("write_quantize", dict(rows=1 << 18, block_size=64)),
}
DEFAULT_WORKLOAD = "dsv4_fp8_decode_T128_H64"
# measured next to the headline in the default run (BASELINE configs 3, 4 and 5 on one GPU)
OTHER_CONFIGS = ([f"dsv4_int8_decode_T{t}_H{h}" for h in (64, 128) for t in (1, 8, 32, 128, 512)] +
                 ["int8_prefill_T4096_H64", "ctx16k_fp8_decode_T1024_H128", "ctx16k_int8_decode_T1024_H128"])


# dense paged MLA decode (flash_mla_with_kvcache), measured next to the headline as well
DENSE_CONFIGS = ["dense_bf16_decode_b128_s4096_h128", "dense_bf16_decode_b128_s4096_h16",
                 "dense_bf16_decode_b128_s8192_h64_sq2_varlen", "dense_bf16_decode_b128_s4096_h16_sq2",
                 "dense_bf16_decode_b1_s32768_h128", "dense_bf16_decode_b8_s4096_h128"]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """SM clock and slowdown reasons of one GPU, read through NVML (queries only) by a thread every
    millisecond while the timed region runs; ``sample()`` lets the timing loop add readings of its own
    (taken while the GPU still works through the queued launches)."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, device_index):
        import threading
        self.h = None
        self.samples = []
        self._stop = threading.Event()
        self.thread = None
        try:
            import pynvml
            import torch
            self.nv = pynvml
            pynvml.nvmlInit()
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:
            self.h = None

    def sample(self):
        if self.h is None:
            return
        try:
            sm = float(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            try:
                mask = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:
                mask = int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            self.samples.append((sm, mask))
        except Exception:
            pass

    def _loop(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(0.001)

    def stop(self):
        if self.h is None:
            return None
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if not self.samples:
            return None
        reasons = sorted({name for _, mask in self.samples for bit, name in self.REASONS if mask & bit})
        return {"sm_mhz": statistics.median(x for x, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.samples), "source": "NVML, 1 ms period, during the timed region"}


def build_workload(name, device, seed):
    import bench_workloads as synthetic
    kind, kw = WORKLOADS[name]
    if kind == "prefill_int8":
        args, meta = synthetic.prefill_int8_workload(seed=seed, device=device, **kw)
    else:
        args, meta = synthetic.decode_workload(seed=seed, device=device, **kw)
    return kind, args, meta


def op_for(kind):
    import flash_mla
    return {"decode_fp8": flash_mla.sparse_mla_decode_fp8, "decode_int8": flash_mla.sparse_mla_decode_int8,
            "prefill_int8": flash_mla.sparse_mla_prefill_int8}[kind]


CACHE_KEYS = ("swa_cache", "swa_scale", "extra_cache", "extra_scale")


def cache_replicas(args, meta):
    """Clones of the cache tensors so that the set cycled through is larger than L2."""
    import torch
    per = sum(a.numel() * a.element_size() for a in meta["keep"]) or sum(
        args[k].numel() * args[k].element_size() for k in CACHE_KEYS if k in args)
    n = max(1, min(16, -(-int(1.5 * L2_BYTES) // max(per, 1))))
    reps = [{k: args[k] for k in CACHE_KEYS if k in args}]
    for _ in range(n - 1):
        if meta["keep"]:   # inline-528 views: clone the backing buffers and rebuild the views
            rep = {}
            for name, buf in zip(("swa", "extra"), meta["keep"]):
                b = buf.clone()
                rep[f"{name}_cache"] = b[:, :, :512].view(torch.int8)
                rep[f"{name}_scale"] = b[:, :, 512:516].view(torch.float32).squeeze(-1)
            reps.append(rep)
        else:
            reps.append({k: args[k].clone() for k in CACHE_KEYS if k in args})
    return reps, per * n


def cpu_oracle_inputs(kind, args):
    """Dequantised fp32 rows + CPU copies for the oracle (outside any timed region)."""
    import numpy as np
    import oracle
    cpu = {k: (v.detach().cpu() if hasattr(v, "cpu") else v) for k, v in args.items()}
    if kind == "decode_fp8":
        swa_K = oracle.dequant_fp8_ds_mla(cpu["swa_cache"].numpy())
        extra_K = oracle.dequant_fp8_ds_mla(cpu["extra_cache"].numpy()) if "extra_cache" in cpu else None
    else:
        swa_K = oracle.dequant_int8_ds_mla(cpu["swa_cache"].contiguous().numpy(), cpu["swa_scale"].contiguous().numpy())
        extra_K = (oracle.dequant_int8_ds_mla(cpu["extra_cache"].contiguous().numpy(),
                                              cpu["extra_scale"].contiguous().numpy())
                   if "extra_cache" in cpu else None)
    q = cpu["q"].float().numpy()
    sink = cpu["attn_sink"].numpy() if "attn_sink" in cpu else None
    return dict(q=q, swa_K=swa_K, swa_idx=cpu["swa_indices"].numpy(), swa_lens=cpu["swa_lens"].numpy(),
                extra_K=extra_K, extra_idx=cpu["extra_indices"].numpy() if "extra_indices" in cpu else None,
                extra_lens=cpu["extra_lens"].numpy() if "extra_lens" in cpu else None, sink=sink)


def time_cpu_oracle(oin, T, budget_s=12.0):
    """Times the oracle on the first n tokens, n chosen so the work takes about `budget_s`."""
    import oracle
    import torch
    t0 = time.perf_counter()
    oracle.sparse_mla_attention(**oin, tokens=[0])
    per_tok = max(time.perf_counter() - t0, 1e-4)
    n = int(max(1, min(T, budget_s / per_tok)))
    t0 = time.perf_counter()
    out = oracle.sparse_mla_attention(**oin, tokens=list(range(n)))
    dt = time.perf_counter() - t0
    return n, dt, out, torch.get_num_threads()


# ----------------------------------------------------------------------------- cache-writer workloads
WRITER_TOKEN_BYTES = {"write_int8": 528, "write_fp8": 584, "write_quantize": 516}
WRITER_KERNEL = {"write_int8": "write_ds_mla_cache_kernel<bf16, int8>", "write_fp8": "write_ds_mla_cache_kernel<bf16, fp8>",
                 "write_quantize": "quantize_int8_rows_kernel<bf16>"}


def writer_inputs(kind, kw, device, seed):
    """Seeded latent rows (N(0,1) times a per-row power of two, bf16), a random injective slot mapping
    and an empty paged cache with a few spare blocks."""
    import torch
    n, bs = kw["rows"], kw["block_size"]
    nb = n // bs + 16
    g = torch.Generator(device=device).manual_seed(1234 + seed)
    x = torch.randn(n, 512, generator=g, device=device)
    x *= torch.exp2(torch.randint(-4, 5, (n, 1), generator=g, device=device).float())
    slots = torch.randperm(nb * bs, generator=g, device=device)[:n]
    tb = 528 if kind == "write_quantize" else WRITER_TOKEN_BYTES[kind]     # the quantizer: checked as inline tokens
    cache = torch.zeros(nb, bs, tb, dtype=torch.uint8, device=device)
    return x.to(torch.bfloat16), slots, cache


def writer_oracle(kind, x_np, slots_np, nb, bs):
    import numpy as np
    import oracle
    if kind == "write_quantize":
        t0 = time.perf_counter()
        q, s = oracle.quantize_int8_rows(x_np)
        return (q, s), time.perf_counter() - t0
    ref = np.zeros((nb, bs, WRITER_TOKEN_BYTES[kind]), np.uint8)
    t0 = time.perf_counter()
    (oracle.write_int8_inline528 if kind == "write_int8" else oracle.write_fp8_ds_mla)(ref, x_np, slots_np)
    return ref, time.perf_counter() - t0


def run_writer_reference(a, kind, kw):
    """Reference arm of the writer workloads: the numpy oracle writer on the host, a bounded sample per step."""
    import torch
    x, slots, cache = writer_inputs(kind, dict(kw, rows=1 << 15), "cpu", 0)
    x_np, slots_np = x.float().numpy(), slots.numpy()
    nb, bs = cache.shape[0], cache.shape[1]
    for _ in range(min(a.warmup, 1)):
        writer_oracle(kind, x_np[:2048], slots_np[:2048], nb, bs)
    dt = sum(writer_oracle(kind, x_np, slots_np, nb, bs)[1] for _ in range(a.steps))
    val = x_np.shape[0] * a.steps / dt
    print(json.dumps({
        "impl": "reference", "metric": "rows quantized/s" if kind == "write_quantize" else "cache rows written/s", "value": val, "unit": "rows/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": dt / a.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": a.workload, "rows_per_step_sampled": x_np.shape[0]},
        "cpu_baseline": {"value": val, "unit": "rows/s", "cores": 1, "kind": "port",
                         "sample": f"{x_np.shape[0]} rows per step (numpy oracle writer), {a.steps} steps"},
        "e2e": {"value": val, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_writer(a, kind, kw, world, rank, local, dev, barrier):
    import numpy as np
    import torch
    import torch.distributed as dist
    import flash_mla
    x, slots, cache = writer_inputs(kind, kw, dev, rank)
    n, tb = x.shape[0], WRITER_TOKEN_BYTES[kind]
    if kind == "write_quantize":
        last = {}

        def write(rows, _slots, _cache):
            last["q"], last["s"] = flash_mla.quantize_int8_ds_mla_rows(rows)
        alg_bytes = n * (1024 + tb)          # bf16 row in, int8 row + fp32 scale out
    else:
        write = flash_mla.write_int8_ds_mla_cache if kind == "write_int8" else flash_mla.write_fp8_ds_mla_cache
        alg_bytes = n * (1024 + tb + 8)      # bf16 row in, token out, int64 slot

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(a.warmup):
        write(x, slots, cache)
    sampler = ClockSampler(local) if rank == 0 else None
    ms = timed(lambda: write(x, slots, cache), a.steps)
    clocks = sampler.stop() if sampler else None

    # end to end: the rows and their slots come from pinned host memory every step; the cache is the
    # result and stays in HBM (as in serving), one written token is read back as the step's receipt
    hx, hs = x.cpu().pin_memory(), slots.cpu().pin_memory()
    dx, ds = torch.empty_like(x), torch.empty_like(slots)
    receipt = torch.empty(cache.shape[2], dtype=torch.uint8).pin_memory()
    first = int(slots[0])

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        ds.copy_(hs, non_blocking=True)
        write(dx, ds, cache)
        if kind == "write_quantize":
            receipt[:512].copy_(last["q"][0].view(torch.uint8), non_blocking=True)
        else:
            receipt.copy_(cache.view(-1, cache.shape[2])[first], non_blocking=True)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(a.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps)

    if rank == 0:
        hbm_gbs, _, peak_kind = measured_peaks()
        dur_s = ms / a.steps / 1e3
        roof = {"bound": "hbm", "achieved": alg_bytes / dur_s / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                "traffic": NCU_DRAM_TRAFFIC_BYTES.get(a.workload), "peak_kind": peak_kind,
                "kernel": WRITER_KERNEL[kind],
                "algorithmic_bytes_per_launch": alg_bytes}
        roof["frac"] = roof["achieved"] / roof["peak"]
        line = {
            "metric": "rows quantized/s" if kind == "write_quantize" else "cache rows written/s",
            "value": world * n * a.steps / (ms / 1e3), "unit": "rows/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f8e4m3" if kind == "write_fp8" else "i8", "data": "synthetic",
            "config": {"workload": a.workload, "rows_per_gpu_per_step": n, "block_size": kw["block_size"],
                       "l2": f"{alg_bytes / 2**20:.0f} MiB read + written per step > 126 MiB L2",
                       "sharding": "rows sharded across GPUs, no collective"},
            "roofline": roof,
            "e2e": {"value": world * n * e2e_steps / (ms_e2e / 1e3), "unit": "rows/s",
                    "h2d_bytes_per_step": hx.numel() * 2 + hs.numel() * 8, "d2h_bytes_per_step": tb,
                    "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                    "note": "latent rows and slots from pinned host memory each step; the cache stays in HBM, one token read back"},
            "gpu_launches": a.steps,
        }
        if clocks:
            line["clocks"] = clocks
        if world == 1 and not a.no_cpu_baseline:
            m = 1 << 15                      # bounded sample: the first 32768 rows of the same step
            ref, dt = writer_oracle(kind, x[:m].float().cpu().numpy(), slots[:m].cpu().numpy(), cache.shape[0], cache.shape[1])
            line["cpu_baseline"] = {"value": m / dt, "unit": "rows/s", "cores": 1, "kind": "port",
                                    "sample": f"first {m} of {n} rows of the same step (numpy oracle writer)"}
            # the same rows written by the kernel into an empty cache: the whole cache, byte for byte
            if kind == "write_quantize":
                write(x[:m], None, None)
                exact = bool(np.array_equal(last["q"].cpu().numpy(), ref[0]) and np.array_equal(last["s"].cpu().numpy(), ref[1]))
            else:
                fresh = torch.zeros_like(cache)
                write(x[:m], slots[:m], fresh)
                exact = bool(np.array_equal(fresh.cpu().numpy(), ref))
            line["parity"] = {"rows_checked": m, "bit_exact": exact}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def common_config(name, meta):
    """The part of `config` that both arms (native and reference) print identically."""
    return {"workload": name, "tokens_per_gpu_per_step": meta["T"], "heads": meta["H"], "cache_format": meta["fmt"],
            "sharding": "tokens sharded across GPUs, cache replicated, no collective"}


def run_reference(args_ns):
    """Reference arm: the fp32 CPU oracle (a port of the reference's own torch oracle; the Python
    reference cannot travel to the GPU box) on the host cores, same workload.  Nothing of the product
    is imported: the workload is built on the CPU with the oracle's packers and quantizer."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # all the host threads there are: torchrun sets OMP_NUM_THREADS=1 for its workers
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    name = args_ns.workload
    kind, kw = WORKLOADS[name]
    if kind.startswith("write"):
        run_writer_reference(args_ns, kind, kw)
        return
    kind, wargs, meta = build_workload(name, "cpu", 0)
    oin = cpu_oracle_inputs(kind, wargs)
    T = meta["T"]
    import oracle
    t0 = time.perf_counter()
    oracle.sparse_mla_attention(**oin, tokens=[0])
    per_tok = max(time.perf_counter() - t0, 1e-4)
    # every token of the batch per step when a step then stays under ~3 s, else a bounded sample
    n = T if per_tok * T <= 3.0 else int(max(1, min(T, 2.0 / per_tok)))
    toks = list(range(n))
    for _ in range(args_ns.warmup):
        oracle.sparse_mla_attention(**oin, tokens=toks[: max(1, n // 8)])
    t0 = time.perf_counter()
    for _ in range(args_ns.steps):
        oracle.sparse_mla_attention(**oin, tokens=toks)
    dt = time.perf_counter() - t0
    val = n * args_ns.steps / dt
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": "sparse MLA decode tokens/s" if "decode" in kind else "sparse MLA prefill tokens/s",
        "value": val, "unit": "tokens/s", "n_gpus": args_ns.gpus, "steps": args_ns.steps, "warmup": args_ns.warmup,
        "ms_per_step": dt / args_ns.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": common_config(name, meta),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": (f"all {T} tokens per step" if n == T else f"first {n} of {T} tokens per step") +
                                   f", {args_ns.steps} steps; caches dequantised once outside the timed region"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from ncu captures of this command line
NCU_DRAM_TRAFFIC_BYTES = {"dsv4_fp8_decode_T128_H64": 43.6e6, "dsv4_int8_decode_T128_H64": 39.8e6,
                          "dsv4_int8_decode_T128_H128": 57.3e6, "int8_prefill_T4096_H64": 537.5e6,
                          "dense_bf16_decode_b128_s4096_h16": 618.8e6, "dense_bf16_decode_b128_s4096_h128": 680.1e6,
                          # row kernels: captured on 2^18 rows, scaled by 4
                          "write_int8_cache_rows1M": 1543.6e6, "write_fp8_cache_rows1M": 1567.9e6,
                          "quantize_int8_rows1M": 1495.8e6,
                          "write_int8_cache_rows256k": 385.9e6, "write_fp8_cache_rows256k": 392.0e6,
                          "quantize_int8_rows256k": 374.0e6}


def roofline_record(meta, seconds, workload=None):
    """achieved = algorithmic bytes (or flops) of one launch / its duration, against the measured peaks."""
    hbm_gbs, bf16_tf, peak_kind = measured_peaks()
    t_hbm = meta["bytes"] / (hbm_gbs * 1e9)
    t_mma = meta["flops"] / (bf16_tf * 1e12)
    if t_hbm >= t_mma:
        roof = {"bound": "hbm", "achieved": meta["bytes"] / seconds / 1e9, "peak": hbm_gbs, "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": meta["flops"] / seconds / 1e12, "peak": bf16_tf, "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["traffic"] = NCU_DRAM_TRAFFIC_BYTES.get(workload)
    roof["peak_kind"] = peak_kind
    roof["kernel"] = "sparse_mla_fwd_kernel"
    roof["algorithmic_bytes_per_launch"] = meta["bytes"]
    roof["algorithmic_flops_per_launch"] = meta["flops"]
    roof["rows_in_lens_per_launch"] = meta["rows_in_lens"]
    roof["other_bound_time_us"] = {"hbm": t_hbm * 1e6, "tensor": t_mma * 1e6}
    return roof


def parity_record(got, ref):
    """The tests' gate (tests/helpers.py) on the tokens the CPU oracle computed: the reference's own
    assert_close(rtol=2e-2, atol=2e-2) and cos_diff < 8e-5, plus the north-star absolute bounds."""
    import numpy as np
    err = np.abs(got - ref)
    excess = float((err - (2e-2 + 2e-2 * np.abs(ref))).max())
    excess_q = float((err - (2e-2 + 2e-2 * np.abs(ref) + 2.0 ** -7 * np.abs(ref).max(-1, keepdims=True))).max())
    num = 2.0 * float((got.astype(np.float64) * ref.astype(np.float64)).sum())
    den = float((got.astype(np.float64) ** 2).sum() + (ref.astype(np.float64) ** 2).sum())
    cos_diff = 1.0 - num / max(den, 1e-300)
    return {"tokens_checked": int(got.shape[0]), "max_abs": float(err.max()), "mean_abs": float(err.mean()),
            "max_abs_ref": float(np.abs(ref).max()), "cos_diff": cos_diff,
            "within_gate": bool(excess <= 0 and cos_diff < 8e-5),
            "gate": "|d| <= 2e-2 + 2e-2|ref| (the reference's assert_close) and cos_diff < 8e-5",
            "within_gate_plus_row_quantum": bool(excess_q <= 0 and cos_diff < 8e-5),
            "north_star_abs": {"max_abs": 2e-2, "mean_abs": 2e-3, "met": bool(err.max() <= 2e-2 and err.mean() <= 2e-3)}}


class AttentionRun:
    """One workload on one device: the op, its per-step arguments and cache replicas larger than L2."""

    def __init__(self, name, dev, seed):
        import torch
        self.torch = torch
        self.name, self.dev = name, dev
        self.kind, self.wargs, self.meta = build_workload(name, dev, seed)
        self.op = op_for(self.kind)
        self.reps, self.rep_bytes = cache_replicas(self.wargs, self.meta)
        self.base = {k: v for k, v in self.wargs.items() if k not in CACHE_KEYS}

    def step(self, i, over=None):
        kw = dict(self.base)
        if over:
            kw.update(over)
        kw.update(self.reps[i % len(self.reps)])
        return self.op(**kw)

    def time_ms(self, steps, warmup, barrier=None):
        """ms of `steps` steps between two CUDA events on the launching stream."""
        torch = self.torch
        for i in range(warmup):
            self.step(i)
        (barrier or torch.cuda.synchronize)()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            self.step(i)
        e1.record()
        (barrier or torch.cuda.synchronize)()
        return e0.elapsed_time(e1)

    def launches_per_step(self):
        import ctypes
        from flash_mla import c_abi
        if not self.kind.startswith("decode"):
            return 1, 1
        lib = c_abi.load()
        w = self.wargs
        width = w["swa_indices"].shape[1] + (w["extra_indices"].shape[1] if "extra_indices" in w else 0)
        splits = ctypes.c_int(1)
        lib.smla_decode_plan(self.meta["T"], self.meta["H"], width, ctypes.byref(splits), None)
        sms = self.torch.cuda.get_device_properties(self.dev).multi_processor_count
        return lib.smla_decode_kernel_launches(sms, self.meta["T"], self.meta["H"], splits.value), splits.value

    def sample_parity(self, tokens):
        import oracle
        oin = cpu_oracle_inputs(self.kind, self.wargs)
        ref = oracle.sparse_mla_attention(**oin, tokens=tokens)
        self.oracle_sample = ref[tokens]
        got = self.step(0).float().cpu().numpy()
        return parity_record(got[tokens], ref[tokens])

    def reference_kernel_ms(self, iters=3):
        """The reference's own CUDA kernels (oracle/_ref, built from the reference checkout: its mma.sync
        decode path with the split policy of its binding, or its fused prefill) on the same inputs."""
        torch = self.torch
        try:
            from oracle import ref_gpu
        except Exception:
            return None
        if not ref_gpu.available():
            return None
        w = self.wargs
        cls = ref_gpu.RefPrefill if self.kind.startswith("prefill") else ref_gpu.RefDecode
        run = cls(w["q"], w["swa_cache"], w.get("swa_scale"), w["swa_indices"], w["swa_lens"], None, w.get("attn_sink"),
                  w.get("extra_cache"), w.get("extra_scale"), w.get("extra_indices"), w.get("extra_lens"))
        run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            run()
        e1.record()
        torch.cuda.synchronize()
        if self.kind.startswith("prefill"):
            which = "sparse_prefill_fused_mma_kernel (+ whole-cache dequant for fp8)"
        elif getattr(run, "fused", False):
            which = f"selection dequant + sparse_mla_decode_mma_kernel, {run.S} splits" + (" + combine" if run.S > 1 else "")
        else:
            which = "legacy FMA decode kernel (the reference's fp8 path when its policy picks one split)"
        return {"ms": e0.elapsed_time(e1) / iters, "kernels": which, "warm_l2": True, "out": run.out}


def other_config_record(name, dev, steps=6):
    """One BASELINE configuration next to the headline: timing (cold L2), roofline, sampled parity, the
    reference's CUDA kernels on the same inputs."""
    import torch
    run = AttentionRun(name, dev, seed=0)
    meta = run.meta
    ms = run.time_ms(steps, 3) / steps
    T = meta["T"]
    launches, splits = run.launches_per_step()
    rec = {"workload": name, "tokens": T, "heads": meta["H"], "cache_format": meta["fmt"], "ms_per_step": ms,
           "tokens_per_s": T / (ms / 1e3), "tflops": meta["flops"] / (ms / 1e3) / 1e12,
           "steps": steps, "warmup": 3, "gpu_launches_per_step": launches, "num_splits": splits,
           "roofline": roofline_record(meta, ms / 1e3, name)}
    if name.startswith("int8_prefill"):
        toks = sorted({0, 1, 2047, 2048, T - 1})
    else:
        toks = sorted({0, T // 3, T - 1})
    rec["parity"] = run.sample_parity(toks)
    rec["parity"]["tokens"] = toks
    ref = run.reference_kernel_ms()
    if ref is not None:
        their = ref.pop("out").float().cpu().numpy()
        ref["parity_of_the_reference_kernel"] = parity_record(their[toks], run.oracle_sample)
        rec["ref_gpu_ms"] = ref["ms"]
        rec["ref_gpu"] = ref
        rec["speedup_vs_ref_gpu"] = ref["ms"] / ms
    del run
    torch.cuda.empty_cache()
    return rec


def config5_record(world, rank, dev, barrier, repeats=10, steps=5):
    """BASELINE config 5: one seeded batch of 1024 query tokens (128 heads, 16384-slot caches, top-k
    2048 + 512), identical on every rank, cut by token with flash_mla.sharding.shard_tokens; caches
    replicated; no collective on the data path.  Strong scaling against the whole batch on one GPU,
    timed on every rank of the same run.  Each figure is the median of `repeats` timed loops of `steps`
    steps (max over ranks per loop), with the spread."""
    import torch
    import torch.distributed as dist
    from flash_mla.sharding import shard_tokens

    def timed(fn):
        vals = []
        for _ in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                fn(i)
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1) / steps
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            vals.append(ms)
        vals.sort()
        return {"median_ms": statistics.median(vals), "min_ms": vals[0], "max_ms": vals[-1]}

    out = {"tokens": 1024, "heads": 128, "repeats": repeats, "steps_per_repeat": steps, "n_gpus": world,
           "sharding": "flash_mla.sharding.shard_tokens (contiguous token ranges), caches replicated, no collective"}
    for fmt in ("fp8", "int8"):
        name = f"ctx16k_{fmt}_decode_T1024_H128"
        run = AttentionRun(name, dev, seed=0)            # the same batch on every rank
        full = dict(run.base)
        mine = shard_tokens(full, world, rank)
        mine = {k: (v.contiguous() if hasattr(v, "contiguous") else v) for k, v in mine.items()}
        for i in range(3):
            run.step(i)
            run.step(i, mine)
        whole = timed(lambda i: run.step(i))
        shard = timed(lambda i: run.step(i, mine))
        meta = run.meta
        rec = {"one_gpu_whole_batch": whole, "sharded": shard,
               "tokens_per_s": 1024 / (shard["median_ms"] / 1e3),
               "tokens_per_gpu": int(mine["q"].shape[0]),
               "strong_scaling_efficiency": whole["median_ms"] / (world * shard["median_ms"]),
               "roofline_per_gpu": roofline_record(
                   {k: (v / world if k in ("bytes", "flops", "rows_in_lens") else v) for k, v in meta.items()},
                   shard["median_ms"] / 1e3, name)}
        out[fmt] = rec
        del run
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------- dense paged MLA decode
def dense_oracle_sample(kw, causal, budget_s=12.0):
    """The CPU oracle on as many sequences (from the first) as fit the time budget."""
    import oracle
    import torch
    cpu = {k: v.detach().cpu() for k, v in kw.items()}
    t0 = time.perf_counter()
    oracle.dense_mla_decode(cpu["q"], cpu["k_cache"], cpu["block_table"], cpu["cache_seqlens"], causal=causal, sequences=[0])
    per = max(time.perf_counter() - t0, 1e-4)
    n = int(max(1, min(cpu["q"].shape[0], budget_s / per)))
    t0 = time.perf_counter()
    out, lse = oracle.dense_mla_decode(cpu["q"], cpu["k_cache"], cpu["block_table"], cpu["cache_seqlens"], causal=causal,
                                       sequences=list(range(n)))
    return n, time.perf_counter() - t0, out, lse, torch.get_num_threads()


def dense_config_record(name, dev, steps=6):
    """One dense paged MLA workload next to the headline: timing, roofline, parity on three sequences."""
    import numpy as np
    import torch
    import flash_mla
    import bench_workloads
    import oracle
    kw_build = WORKLOADS[name][1]
    kw, meta = bench_workloads.dense_decode_workload(device=dev, seed=0, **kw_build)
    causal = kw_build["s_q"] > 1
    md, ns = flash_mla.get_mla_metadata(kw["cache_seqlens"], kw_build["s_q"] * kw_build["h_q"], 1)

    def step():
        return flash_mla.flash_mla_with_kvcache(kw["q"], kw["k_cache"], kw["block_table"], kw["cache_seqlens"], 512, md, ns,
                                                causal=causal)
    for _ in range(3):
        out, lse = step()
    torch.cuda.synchronize()
    cache_bytes = kw["k_cache"].numel() * 2
    if cache_bytes > 2 * L2_BYTES:      # every step reads more than L2 holds
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        l2_note = f"{cache_bytes / 2**20:.0f} MiB cache read per step > 126 MiB L2"
    else:                               # a cache that L2 could hold: L2 is overwritten between the timed steps
        flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for e0, e1 in pairs:
            flush.zero_()
            e0.record()
            step()
            e1.record()
        torch.cuda.synchronize()
        ms = sum(e0.elapsed_time(e1) for e0, e1 in pairs) / steps
        l2_note = f"{cache_bytes / 2**20:.0f} MiB cache; {2 * L2_BYTES / 2**20:.0f} MiB written between the timed steps (L2 flush), each step timed by its own events"
        del flush
    tokens = kw_build["b"] * kw_build["s_q"]
    seqs = sorted({0, kw_build["b"] // 2, kw_build["b"] - 1})
    cpu = {k: v.detach().cpu() for k, v in kw.items()}
    ref_out, ref_lse = oracle.dense_mla_decode(cpu["q"], cpu["k_cache"], cpu["block_table"], cpu["cache_seqlens"], causal=causal,
                                               sequences=seqs)
    got, got_lse = out[seqs].float().cpu().numpy(), lse[seqs].cpu().numpy()
    cd_out, cd_lse = oracle.cos_diff(got, ref_out[seqs]), oracle.cos_diff(got_lse, ref_lse[seqs])
    rec = {"workload": name, **kw_build, "tokens": tokens, "ms_per_step": ms, "tokens_per_s": tokens / (ms / 1e3),
           "tflops": meta["flops"] / (ms / 1e3) / 1e12, "steps": steps, "warmup": 3, "gpu_launches_per_step": 1,
           "l2": l2_note,
           "roofline": roofline_record(meta, ms / 1e3, name),
           "parity": {"sequences": seqs, "cos_diff_out": cd_out, "cos_diff_lse": cd_lse,
                      "max_abs_out": float(np.abs(got - ref_out[seqs]).max()),
                      "within_gate": bool(cd_out < 8e-5 and cd_lse < 8e-5),
                      "gate": "cos_diff < 8e-5 for out and lse (the reference's dense test)"}}
    del kw, out, lse
    torch.cuda.empty_cache()
    return rec


def run_dense_reference(a, kw_build):
    """Reference arm of the dense workloads: the reference's dense path is CUDA only (and needs its cutlass
    submodule, absent from the checkout), so the arm times the CPU oracle port on a bounded sample."""
    import bench_workloads
    small = dict(kw_build, b=min(kw_build["b"], 8))
    kw, _ = bench_workloads.dense_decode_workload(device="cpu", seed=0, **small)
    causal = kw_build["s_q"] > 1
    toks = 0
    t_all = 0.0
    for _ in range(a.steps):
        n, dt, _, _, threads = dense_oracle_sample(kw, causal, budget_s=6.0)
        toks += n * kw_build["s_q"]
        t_all += dt
    val = toks / t_all
    print(json.dumps({
        "impl": "reference", "metric": "dense MLA decode tokens/s", "value": val, "unit": "tokens/s", "n_gpus": a.gpus,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": t_all / a.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": a.workload, **kw_build},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{n} sequences of the batch per step, {a.steps} steps"},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def run_dense(a, kw_build, world, rank, local, dev, barrier):
    import numpy as np
    import torch
    import torch.distributed as dist
    import flash_mla
    import bench_workloads
    import oracle
    kw, meta = bench_workloads.dense_decode_workload(device=dev, seed=rank, **kw_build)
    causal = kw_build["s_q"] > 1
    md, ns = flash_mla.get_mla_metadata(kw["cache_seqlens"], kw_build["s_q"] * kw_build["h_q"], 1)
    tokens = kw_build["b"] * kw_build["s_q"]

    def step(q=None):
        return flash_mla.flash_mla_with_kvcache(kw["q"] if q is None else q, kw["k_cache"], kw["block_table"],
                                                kw["cache_seqlens"], 512, md, ns, causal=causal)

    cache_bytes = kw["k_cache"].numel() * 2
    # a cache that L2 could hold: L2 is overwritten between the timed steps and every step has its own events
    flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev) if cache_bytes <= 2 * L2_BYTES else None

    def timed(fn, steps):
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                 for _ in range(steps if flush is not None else 1)]
        barrier()
        if flush is None:
            pairs[0][0].record()
            for _ in range(steps):
                fn()
            pairs[0][1].record()
        else:
            for e0, e1 in pairs:
                flush.zero_()
                e0.record()
                fn()
                e1.record()
        barrier()
        ms = sum(e0.elapsed_time(e1) for e0, e1 in pairs)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(a.warmup):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    ms = timed(step, a.steps)
    clocks = sampler.stop() if sampler else None

    # end to end: q from pinned host memory, out and lse back to pinned host memory, every step (the cache stays in HBM)
    hq = kw["q"].cpu().pin_memory()
    dq = torch.empty_like(kw["q"])
    out0, lse0 = step()
    hout = torch.empty(out0.shape, dtype=out0.dtype).pin_memory()
    hlse = torch.empty(lse0.shape, dtype=lse0.dtype).pin_memory()

    def e2e_step():
        dq.copy_(hq, non_blocking=True)
        o, l = step(dq)
        hout.copy_(o, non_blocking=True)
        hlse.copy_(l, non_blocking=True)

    for _ in range(2):
        e2e_step()
    e2e_steps = max(3, min(a.steps, 10))
    ms_e2e = timed(e2e_step, e2e_steps)

    if rank == 0:
        line = {
            "metric": "dense MLA decode tokens/s", "value": world * tokens * a.steps / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms / a.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": a.workload, **kw_build, "page_block_size": kw["k_cache"].shape[1],
                       "l2": (f"{cache_bytes / 2**20:.0f} MiB cache read per step > 126 MiB L2" if flush is None else
                              f"{cache_bytes / 2**20:.0f} MiB cache; {2 * L2_BYTES / 2**20:.0f} MiB written between the "
                              "timed steps (L2 flush), each step timed by its own events"),
                       "sharding": "sequences sharded across GPUs, no collective"},
            "roofline": roofline_record(meta, ms / a.steps / 1e3, a.workload),
            "tflops": meta["flops"] / (ms / a.steps / 1e3) / 1e12,
            "e2e": {"value": world * tokens * e2e_steps / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": hq.numel() * 2, "d2h_bytes_per_step": hout.numel() * 2 + hlse.numel() * 4,
                    "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                    "note": "q from pinned host memory, out and lse back to pinned host memory, every step; the paged cache stays in HBM"},
            "gpu_launches": a.steps,
            "device_status": int(flash_mla.device_status_tensor().item()),
        }
        if clocks:
            line["clocks"] = clocks
        if world == 1 and not a.no_cpu_baseline:
            n, dt, ref_out, ref_lse, threads = dense_oracle_sample(kw, causal)
            line["cpu_baseline"] = {"value": n * kw_build["s_q"] / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"first {n} of {kw_build['b']} sequences of the same step"}
            got, got_lse = out0[:n].float().cpu().numpy(), lse0[:n].cpu().numpy()
            line["parity"] = {"sequences_checked": n, "cos_diff_out": oracle.cos_diff(got, ref_out[:n]),
                              "cos_diff_lse": oracle.cos_diff(got_lse, ref_lse[:n]),
                              "max_abs_out": float(np.abs(got - ref_out[:n]).max()),
                              "max_abs_lse": float(np.abs(got_lse - ref_lse[:n]).max()),
                              "gate": "cos_diff < 8e-5 for out and lse (the reference's dense test)"}
            line["parity"]["within_gate"] = bool(line["parity"]["cos_diff_out"] < 8e-5 and line["parity"]["cos_diff_lse"] < 8e-5)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip other_configs and config5 (default workload only)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3) if a.impl == "native" else a.warmup

    if a.impl == "reference":
        if WORKLOADS[a.workload][0] == "dense":
            if int(os.environ.get("RANK", "0")) == 0:
                run_dense_reference(a, WORKLOADS[a.workload][1])
            return
        run_reference(a)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if WORKLOADS[a.workload][0].startswith("write"):
        run_writer(a, *WORKLOADS[a.workload], world, rank, local, dev, barrier)
        return
    if WORKLOADS[a.workload][0] == "dense":
        run_dense(a, WORKLOADS[a.workload][1], world, rank, local, dev, barrier)
        return

    run = AttentionRun(a.workload, dev, seed=rank)
    kind, wargs, meta, base, step = run.kind, run.wargs, run.meta, run.base, run.step
    T, H = meta["T"], meta["H"]
    import ctypes
    from flash_mla import c_abi
    lib = c_abi.load()
    # launches per step (claimed): the attention kernel, plus the combine kernel when a few tokens are
    # spread over the whole GPU (otherwise the merge is fused into the attention kernel)
    launches_per_step, num_splits = run.launches_per_step()

    for i in range(a.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        out = step(i)
    e1.record()
    if sampler:
        sampler.sample()      # the GPU is still working through the queued steps
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    ms_per_step = ms / a.steps
    value = world * T * a.steps / (ms / 1e3)

    # ---- end to end through the public API from host buffers: the step's inputs travel as one packed
    # pinned buffer, the output comes back to pinned host memory, every step
    from flash_mla.host_pipeline import HostPipeline, PackedInputs
    host_keys = [k for k in ("q", "swa_indices", "swa_lens", "extra_indices", "extra_lens") if k in base]
    example = {k: base[k] for k in host_keys}
    packed = PackedInputs(example)
    host_buf, host_views = packed.new_host()
    for k in host_keys:
        host_views[k].copy_(base[k])
    dev_buf, dev_views = packed.new_device(dev)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = packed.nbytes
    d2h = host_out.numel() * host_out.element_size()

    def max_over_ranks(*vals):
        if world > 1:
            t = torch.tensor(list(vals), device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return [float(x) for x in t.tolist()]
        return list(vals)

    def timed_loop(fn, steps):
        barrier()
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    def one_stream_step(i):
        dev_buf.copy_(host_buf, non_blocking=True)
        o = step(i, dev_views)
        host_out.copy_(o, non_blocking=True)

    for i in range(3):
        one_stream_step(i)
    ms_serial = timed_loop(one_stream_step, a.steps)

    # the floor: the same copies with no kernel between them, (a) on one stream, (b) each direction on
    # its own stream (what three staggered streams can overlap at best)
    dummy_out = torch.empty_like(out)

    def copies_one_stream(i):
        dev_buf.copy_(host_buf, non_blocking=True)
        host_out.copy_(dummy_out, non_blocking=True)

    for i in range(3):
        copies_one_stream(i)
    ms_copy_serial = timed_loop(copies_one_stream, a.steps)
    s_a, s_b = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def copies_two_streams():
        cur = torch.cuda.current_stream()
        barrier()
        e0.record()
        s_a.wait_event(e0)
        s_b.wait_event(e0)
        for i in range(a.steps):
            with torch.cuda.stream(s_a):
                dev_buf.copy_(host_buf, non_blocking=True)
            with torch.cuda.stream(s_b):
                host_out.copy_(dummy_out, non_blocking=True)
        ea, eb = torch.cuda.Event(), torch.cuda.Event()
        ea.record(s_a)
        eb.record(s_b)
        cur.wait_event(ea)
        cur.wait_event(eb)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    copies_two_streams()
    ms_copy_overlapped = copies_two_streams()

    # consecutive steps staggered over three streams (copy in / kernel / copy out), three buffers deep:
    # every step still moves its inputs from pinned host memory and its output back
    pipe = HostPipeline(lambda d, i: step(i, d), example, out, depth=3)
    for i in range(3):
        pipe.submit(i, host_buf)
    pipe.drain()
    barrier()
    cur = torch.cuda.current_stream()
    e0.record()
    pipe.start_after(e0)
    for i in range(a.steps):
        pipe.submit(i, host_buf)
    pipe.join(cur)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    ms_e2e, ms_serial, ms_copy_serial, ms_copy_overlapped = max_over_ranks(ms_e2e, ms_serial, ms_copy_serial, ms_copy_overlapped)
    e2e_value = world * T * a.steps / (ms_e2e / 1e3)
    e2e_serial = world * T * a.steps / (ms_serial / 1e3)
    # the pipelined result must be the plain call's result
    pipe_ok = bool(torch.equal(pipe.result((a.steps - 1) % 3).to(dev), step(a.steps - 1)))

    status = ctypes.c_int(0)
    lib.smla_read_device_status(ctypes.byref(status))

    extras = (a.workload == DEFAULT_WORKLOAD) and not a.no_extras
    config5 = None
    if extras:
        del pipe
        torch.cuda.empty_cache()
        config5 = config5_record(world, rank, dev, barrier)      # every rank takes part

    if rank == 0:
        roof = roofline_record(meta, ms_per_step / 1e3, a.workload)
        best_ms = min(ms_e2e, ms_serial) / a.steps
        floor_ms = max(ms_copy_overlapped / a.steps, ms_per_step)
        cfg = common_config(a.workload, meta)
        line = {
            "metric": ("sparse MLA decode tokens/s" if kind.startswith("decode") else "sparse MLA prefill tokens/s"),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": cfg,
            "run": {"l2": f"cache rotated over {len(run.reps)} replicas ({run.rep_bytes / 2**20:.0f} MiB) > 126 MiB L2",
                    "num_splits": num_splits, "rows_in_lens_per_step": meta["rows_in_lens"]},
            "roofline": roof,
            # both ways of driving the public API from host buffers were timed; the faster one is the figure
            "e2e": {"value": max(e2e_value, e2e_serial), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": best_ms,
                    "mode": "three_streams" if e2e_value >= e2e_serial else "one_stream",
                    "three_streams": {"value": e2e_value, "ms_per_step": ms_e2e / a.steps},
                    "one_stream": {"value": e2e_serial, "ms_per_step": ms_serial / a.steps},
                    "pcie_floor_ms": ms_copy_overlapped / a.steps,
                    "pcie_floor_one_stream_ms": ms_copy_serial / a.steps,
                    "kernel_ms": ms_per_step,
                    "over_floor": best_ms / floor_ms,
                    "matches_plain_call": pipe_ok,
                    "note": "q/indices/lens packed in ONE pinned staging buffer (one host->device copy per step) and the "
                            "output back to pinned host memory every step; three_streams = steps staggered over copy-in / "
                            "kernel / copy-out streams (flash_mla.host_pipeline.HostPipeline); one_stream = the same on a "
                            "single stream; value = the faster of the two; pcie_floor_ms = the same two copies per step with "
                            "no kernel, one stream per direction; over_floor = e2e ms / max(pcie floor, kernel); KV cache "
                            "resident in HBM; all figures max over ranks"},
            "gpu_launches": a.steps * launches_per_step,
            "device_status": status.value,
        }
        if clocks:
            line["clocks"] = clocks
        if world == 1 and not a.no_cpu_baseline:
            oin = cpu_oracle_inputs(kind, wargs)
            n, dt, ref, cores = time_cpu_oracle(oin, T, budget_s=8.0)
            got = step(0).float().cpu().numpy()[:n]
            line["cpu_baseline"] = {"value": n / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"first {n} of {T} tokens of the same step; caches dequantised once outside the timed region"}
            line["parity"] = parity_record(got, ref[:n])
            del oin
        if config5 is not None:
            line["config5"] = config5
        if extras and world == 1:
            refk = run.reference_kernel_ms()
            if refk is not None:
                refk.pop("out", None)
                line["ref_gpu_ms"] = refk["ms"]
                line["ref_gpu"] = refk
            del run
            torch.cuda.empty_cache()
            others = []
            for name in OTHER_CONFIGS:
                try:
                    others.append(other_config_record(name, dev))
                except Exception as e:      # one broken configuration must not cost the whole line
                    others.append({"workload": name, "error": f"{type(e).__name__}: {e}"[:300]})
            line["other_configs"] = others
            dense = []
            for name in DENSE_CONFIGS:
                try:
                    dense.append(dense_config_record(name, dev))
                except Exception as e:
                    dense.append({"workload": name, "error": f"{type(e).__name__}: {e}"[:300]})
            line["dense_configs"] = dense
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
