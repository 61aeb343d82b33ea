"""Decode without per-call allocation: a plan sized once per (tokens, heads, width) shape.

The reference computes its split count and allocates the partial-result buffers inside every decode
call (csrc/flash_api.cpp:75-102,381-405).  A serving engine that replays CUDA graphs, or that has
handed all device memory to its KV-cache pool, wants that done once: ``get_sparse_mla_decode_plan``
asks the library for the split policy of the current device, allocates the scratch and the output
once, and ``sparse_mla_decode_planned`` runs decode steps into them -- the call itself allocates
nothing, for either cache format, and can be captured in a CUDA graph and replayed.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional

import torch

from . import c_abi
from ._loader import load_torch_extension

HEAD_DIM = 512


@dataclass
class SparseMlaDecodePlan:
    num_tokens: int
    num_heads: int
    max_width: int                 # swa top-k + extra top-k
    num_splits: int                # 1 = whole items per CTA; > 1 = balanced tiles with partial segments in scratch
    workspace_bytes: int
    kernel_launches: int           # kernels one decode call launches on an ordinary stream
    graph_kernel_nodes: int        # kernel nodes of the same call captured in a CUDA graph (the slice-wise merge of a
                                   # few tokens is replaced by the combine kernel under capture: 2 where the above says 1)
    workspace: Optional[torch.Tensor]
    out: torch.Tensor              # bf16 [num_tokens, num_heads, 512], overwritten by every call


def get_sparse_mla_decode_plan(num_tokens: int, num_heads: int, max_width: int,
                               device: Optional[torch.device] = None) -> SparseMlaDecodePlan:
    """Split policy and buffers for decode calls of this shape on ``device`` (default: current)."""
    lib = c_abi.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        splits, nbytes = ctypes.c_int(1), ctypes.c_size_t(0)
        c_abi.check(lib.smla_decode_plan(num_tokens, num_heads, max_width, ctypes.byref(splits), ctypes.byref(nbytes)),
                    "smla_decode_plan")
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        launches = lib.smla_decode_kernel_launches(sms, num_tokens, num_heads, splits.value)
        nodes = lib.smla_decode_kernel_launches_captured(sms, num_tokens, num_heads, splits.value)
        ws = torch.empty((nbytes.value + 3) // 4, dtype=torch.float32, device=dev) if splits.value > 1 else None
        out = torch.empty(num_tokens, num_heads, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    return SparseMlaDecodePlan(num_tokens, num_heads, max_width, splits.value, nbytes.value, launches, nodes, ws, out)


def sparse_mla_decode_planned(plan: SparseMlaDecodePlan, q: torch.Tensor, swa_cache: torch.Tensor,
                              swa_indices: torch.Tensor, swa_lens: torch.Tensor, scale: Optional[float] = None,
                              attn_sink: Optional[torch.Tensor] = None, extra_cache: Optional[torch.Tensor] = None,
                              extra_indices: Optional[torch.Tensor] = None, extra_lens: Optional[torch.Tensor] = None,
                              swa_scale: Optional[torch.Tensor] = None,
                              extra_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One decode step into ``plan.out`` (returned).  Same arguments and results as
    ``sparse_mla_decode_fp8`` (uint8 caches) / ``sparse_mla_decode_int8`` (int8 caches with
    ``swa_scale`` / ``extra_scale``); the shape must be the plan's."""
    load_torch_extension()
    width = swa_indices.shape[-1] + (extra_indices.shape[-1] if extra_indices is not None else 0)
    if tuple(q.shape) != (plan.num_tokens, plan.num_heads, HEAD_DIM) or width > plan.max_width:
        raise ValueError(f"plan is for q {(plan.num_tokens, plan.num_heads, HEAD_DIM)} and width <= {plan.max_width}, "
                         f"got q {tuple(q.shape)} and width {width}")
    if scale is None:
        scale = 1.0 / math.sqrt(HEAD_DIM)
    if swa_indices.dim() == 3:
        swa_indices = swa_indices[:, 0]
    if extra_indices is not None and extra_indices.dim() == 3:
        extra_indices = extra_indices[:, 0]
    torch.ops.flash_mla.fwd_sparse_decode_mla_planned(q, swa_cache, swa_scale, swa_indices, swa_lens, float(scale),
                                                      attn_sink, extra_cache, extra_scale, extra_indices, extra_lens,
                                                      plan.out, plan.workspace)
    return plan.out


class _DeviceWord:
    """Minimal __cuda_array_interface__ view of one int32 in device memory."""

    def __init__(self, address: int):
        self.__cuda_array_interface__ = {"shape": (1,), "typestr": "<i4", "data": (address, False), "version": 2}


def device_status_tensor(device: Optional[torch.device] = None) -> torch.Tensor:
    """The library's per-device status word as a 1-element int32 CUDA tensor (an alias, not a copy).

    The kernels set bits in it when one of their bounded waits runs out (e.g. a CTA waited a second for
    a partial result of another CTA because something else held SMs); the outputs of that launch are
    then not valid although the call returned long before.  A serving loop that must not synchronise
    can copy the word to pinned memory behind each step, ``status.to(pinned, non_blocking=True)`` on
    the decode stream, and look at it when the step's results are consumed; ``status.zero_()`` clears it."""
    lib = c_abi.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        addr = ctypes.c_void_p(0)
        c_abi.check(lib.smla_device_status_address(ctypes.byref(addr)), "smla_device_status_address")
        return torch.as_tensor(_DeviceWord(addr.value), device=dev)
