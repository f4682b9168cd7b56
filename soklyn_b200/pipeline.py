"""Asynchronous host <-> device staging around a training step.

The reference's `forward_raw` (src/ffn.rs:73-94) uploads the batch, runs the network and
returns a copy of the output, all on one stream with a host sync after every call. Here the
same data movement runs on a copy stream with two device slots: while step s computes, the
inputs of step s+1 are copied from pinned host memory, and the output of step s is copied
back while its backward pass runs. No copy is skipped; they only overlap compute.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .core import TORCH_DTYPE, Tensor
from .function import Precision


class HostFeeder:
    def __init__(self, context, shapes: Sequence[tuple], precision: Precision, slots: int = 2):
        self.ctx = context
        self.copy_stream = torch.cuda.Stream(device=context.device)
        dt = TORCH_DTYPE[precision]
        self.slots = [[Tensor(torch.empty(tuple(s), device=context.device, dtype=dt), precision, take_id=False)
                       for s in shapes] for _ in range(slots)]
        self.ready = [torch.cuda.Event() for _ in range(slots)]
        self.consumed = [torch.cuda.Event() for _ in range(slots)]
        self.out_done = [torch.cuda.Event() for _ in range(slots)]
        self._fetched = [False] * slots
        self.bytes_h2d = 0
        self.bytes_d2h = 0
        for e in self.consumed:
            e.record(context.stream)

    def stage(self, slot: int, host_tensors: Sequence[torch.Tensor]):
        """Start copying pinned host tensors into `slot` (after the step that last used it has finished)."""
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])
            for dst, src in zip(self.slots[slot], host_tensors):
                dst.data.copy_(src, non_blocking=True)
                self.bytes_h2d += src.numel() * src.element_size()
            self.ready[slot].record(self.copy_stream)

    def acquire(self, slot: int):
        """Device tensors of `slot`, valid for work queued on the context's stream from now on."""
        self.ctx.stream.wait_event(self.ready[slot])
        return self.slots[slot]

    def release(self, slot: int):
        self.consumed[slot].record(self.ctx.stream)

    def fetch(self, device_tensor: Tensor, host_out: torch.Tensor, rows: int, slot: int = 0):
        """Copy the first `rows` rows of a device tensor to pinned host memory behind the work
        already queued on the context's stream; `wait_output(slot)` blocks until it has landed. With one
        host buffer per slot the host can wait for step s's output while step s+1 is already queued."""
        produced = torch.cuda.Event()
        produced.record(self.ctx.stream)
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(produced)
            host_out.copy_(device_tensor.data[:rows], non_blocking=True)
            self.out_done[slot].record(self.copy_stream)
        self._fetched[slot] = True
        self.bytes_d2h += host_out.numel() * host_out.element_size()

    def wait_output(self, slot: int = 0):
        if self._fetched[slot]:
            self.out_done[slot].synchronize()
            self._fetched[slot] = False
