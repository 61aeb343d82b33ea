"""Host-buffer calls with copies overlapped across steps.

A serving loop that holds a step's inputs (q, indices, lens) in pinned host memory and wants the
output back in host memory pays two PCIe transfers around a ~0.1 ms kernel.  Run back to back on one
stream they serialise; the two PCIe directions and the kernel can all work at once when consecutive
steps are staggered over three streams.  ``HostPipeline`` does that with plain CUDA streams and
events: step i's host->device copy runs while step i-1 computes and step i-2's result travels back.
All inputs of a step live in ONE pinned staging buffer and one device buffer (the per-name tensors
are views at 256-byte aligned offsets), so a step costs one copy each way, not one per tensor.
Nothing here synchronises the host except ``result()`` / ``drain()``.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

import torch


class PackedInputs:
    """Byte layout of a step's inputs inside one buffer: name -> (offset, bytes, dtype, shape)."""

    def __init__(self, example: Dict[str, torch.Tensor]):
        self.layout = {}
        off = 0
        for k, v in example.items():
            n = v.numel() * v.element_size()
            self.layout[k] = (off, n, v.dtype, tuple(v.shape))
            off = (off + n + 255) // 256 * 256
        self.nbytes = max(off, 256)

    def views(self, buf: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {k: buf[off:off + n].view(dt).view(shape) for k, (off, n, dt, shape) in self.layout.items()}

    def new_host(self) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        """A pinned staging buffer and its per-name views (fill the views, submit the buffer)."""
        buf = torch.empty(self.nbytes, dtype=torch.uint8).pin_memory()
        return buf, self.views(buf)

    def new_device(self, device) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        return buf, self.views(buf)


class HostPipeline:
    """``run(dev_inputs, i)`` is the device call (e.g. a closure around ``sparse_mla_decode_fp8``) and
    must return the output tensor; ``example`` maps input names to device tensors of the per-step
    shapes.  ``depth`` device input buffers and pinned outputs are cycled.  If ``run`` returns the same
    output tensor every step (a planned decode does) pass ``reuses_output=True``: the kernel of a step
    then waits for the device->host copy of the step before it instead of overwriting what it reads."""

    def __init__(self, run: Callable[[Dict[str, torch.Tensor], int], torch.Tensor], example: Dict[str, torch.Tensor],
                 out_like: torch.Tensor, depth: int = 3, reuses_output: bool = False):
        self.run = run
        self.depth = depth
        self.reuses_output = reuses_output
        dev = out_like.device
        self.packed = PackedInputs(example)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.slots = []
        for _ in range(depth):
            buf, views = self.packed.new_device(dev)
            self.slots.append({
                "dev_buf": buf, "dev_in": views,
                "host_out": torch.empty(out_like.shape, dtype=out_like.dtype).pin_memory(),
                "ev_in": torch.cuda.Event(), "ev_run": torch.cuda.Event(), "ev_out": torch.cuda.Event(),
                "used": False,
            })
        self.last_out_event = None

    def new_host_inputs(self) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        return self.packed.new_host()

    def start_after(self, event: torch.cuda.Event) -> None:
        """Order all three streams after ``event`` (e.g. the start mark of a timed region)."""
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_event(event)

    def submit(self, i: int, host_buf: torch.Tensor) -> int:
        """``host_buf``: a pinned staging buffer from ``new_host_inputs()`` holding this step's inputs."""
        slot = self.slots[i % self.depth]
        if slot["used"]:
            self.s_in.wait_event(slot["ev_run"])      # the kernel that read these input buffers is done
        with torch.cuda.stream(self.s_in):
            slot["dev_buf"].copy_(host_buf, non_blocking=True)
            slot["ev_in"].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(slot["ev_in"])
            if self.reuses_output and self.last_out_event is not None:
                self.s_run.wait_event(self.last_out_event)   # the previous step's copy still reads the shared output
            out = self.run(slot["dev_in"], i)
            slot["ev_run"].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["ev_run"])
            slot["host_out"].copy_(out, non_blocking=True)
            out.record_stream(self.s_out)
            slot["ev_out"].record(self.s_out)
        self.last_out_event = slot["ev_out"]
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
