"""Running the attention operators on host-resident batches.

A caller whose Q/K/V live in (pinned) host memory pays for the PCIe transfers
on every call.  ``HostPipeline`` overlaps them with the kernels: inputs of step
``i + 1`` are copied host-to-device on one stream while step ``i`` computes on a
second and the output of step ``i - 1`` returns device-to-host on a third, with
two sets of device buffers.  Host-to-device and device-to-host traffic use the
two directions of the link at the same time, so the steady-state step time is
the larger of the two transfers instead of their sum plus the kernel.
"""

from __future__ import annotations

from typing import Callable, List, Sequence

import torch

__all__ = ["HostPipeline"]


class HostPipeline:
    """Double-buffered host -> device -> host pipeline around an operator call.

    ``fn(*device_inputs)`` must return the output tensor (or a tuple whose first
    element is the output).  ``submit(host_inputs, host_output)`` enqueues one
    step and returns immediately; ``flush()`` waits for everything submitted.
    Host tensors should be pinned, or the copies are not asynchronous.
    """

    def __init__(self, fn: Callable, device: torch.device, depth: int = 2) -> None:
        self.fn = fn
        self.device = torch.device(device)
        self.depth = depth
        self.s_in = torch.cuda.Stream(self.device)
        self.s_compute = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._slots: List[dict] = [dict(inputs=None, out=None, free=None) for _ in range(depth)]
        self._step = 0

    def submit(self, host_inputs: Sequence[torch.Tensor], host_output: torch.Tensor) -> None:
        slot = self._slots[self._step % self.depth]
        self._step += 1
        # the slot's device buffers are reusable once its previous output has left
        if slot["free"] is not None:
            self.s_in.wait_event(slot["free"])
        with torch.cuda.stream(self.s_in):
            if slot["inputs"] is None or any(d.shape != h.shape or d.dtype != h.dtype
                                             for d, h in zip(slot["inputs"], host_inputs)):
                slot["inputs"] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in host_inputs]
            for d, h in zip(slot["inputs"], host_inputs):
                d.copy_(h, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(self.s_in)
        self.s_compute.wait_event(copied)
        with torch.cuda.stream(self.s_compute):
            out = self.fn(*slot["inputs"])
            if isinstance(out, tuple):
                out = out[0]
            slot["out"] = out
            computed = torch.cuda.Event()
            computed.record(self.s_compute)
        self.s_out.wait_event(computed)
        with torch.cuda.stream(self.s_out):
            out.record_stream(self.s_out)      # allocated on the compute stream, read here
            host_output.copy_(out, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.s_out)
        slot["free"] = done

    def flush(self) -> None:
        for s in (self.s_in, self.s_compute, self.s_out):
            s.synchronize()
