"""Host-buffer calls with copies overlapped across steps.

A serving loop that holds a step's inputs (q, indices, lens) in pinned host memory and wants the
output back in host memory pays two PCIe transfers around a ~0.1 ms kernel.  Run back to back on one
stream they serialise; the two PCIe directions and the kernel can all work at once when consecutive
steps are staggered over three streams.  ``HostPipeline`` does that with plain CUDA streams and
events: step i's host->device copy runs while step i-1 computes and step i-2's result travels back.
Nothing here synchronises the host except ``result()`` / ``drain()``.
"""
from __future__ import annotations

from typing import Callable, Dict

import torch


class HostPipeline:
    """``run(dev_inputs, i)`` is the device call (e.g. a closure around ``sparse_mla_decode_fp8``) and
    must return the output tensor; ``example`` maps input names to device tensors of the per-step
    shapes.  ``depth`` buffers of inputs and pinned outputs are cycled."""

    def __init__(self, run: Callable[[Dict[str, torch.Tensor], int], torch.Tensor], example: Dict[str, torch.Tensor],
                 out_like: torch.Tensor, depth: int = 3):
        self.run = run
        self.depth = depth
        dev = out_like.device
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.slots = []
        for _ in range(depth):
            self.slots.append({
                "dev_in": {k: torch.empty_like(v) for k, v in example.items()},
                "host_out": torch.empty(out_like.shape, dtype=out_like.dtype).pin_memory(),
                "ev_in": torch.cuda.Event(), "ev_run": torch.cuda.Event(), "ev_out": torch.cuda.Event(),
                "used": False,
            })

    def start_after(self, event: torch.cuda.Event) -> None:
        """Order all three streams after ``event`` (e.g. the start mark of a timed region)."""
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(event)

    def submit(self, i: int, host_in: Dict[str, torch.Tensor]) -> int:
        slot = self.slots[i % self.depth]
        if slot["used"]:
            self.s_in.wait_event(slot["ev_run"])      # the kernel that read these input buffers is done
        with torch.cuda.stream(self.s_in):
            for k, h in host_in.items():
                slot["dev_in"][k].copy_(h, non_blocking=True)
            slot["ev_in"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot["ev_in"])
            out = self.run(slot["dev_in"], i)
            slot["ev_run"].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["ev_run"])
            slot["host_out"].copy_(out, non_blocking=True)
            out.record_stream(self.s_out)
            slot["ev_out"].record(self.s_out)
        slot["used"] = True
        return i % self.depth

    def result(self, ticket: int) -> torch.Tensor:
        """The pinned host tensor of a submitted step, after waiting for its copy (valid until the slot
        is reused ``depth`` submissions later)."""
        slot = self.slots[ticket]
        slot["ev_out"].synchronize()
        return slot["host_out"]

    def join(self, stream: torch.cuda.Stream) -> None:
        """Make ``stream`` wait for everything submitted so far (e.g. before an end mark)."""
        for slot in self.slots:
            if slot["used"]:
                stream.wait_event(slot["ev_out"])

    def drain(self) -> None:
        for s in (self.s_in, self.s_run, self.s_out):
            s.synchronize()
