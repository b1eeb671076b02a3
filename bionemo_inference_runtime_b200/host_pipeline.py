"""Streaming pair tensors that live in host memory through a device function.

A pair tensor of 512 tokens is 64 MiB; over PCIe its copy in and its copy out each take longer than the
triangle-attention nodes themselves.  ``HostPipeline`` overlaps the three: while batch ``i`` is computed,
batch ``i+1`` is copied in and batch ``i-1`` is copied out, on three CUDA streams with ``depth`` device slots.
The copies are plain ``cudaMemcpyAsync`` calls (one per batch) from and to pinned host memory.
"""

from __future__ import annotations

import os
from typing import Callable, Sequence

import torch


def bind_to_gpu_numa_node(device: torch.device | str | int) -> list[int] | None:
    """Restrict this process to the CPU cores of the NUMA node the GPU hangs off, so that pinned buffers allocated
    afterwards are local to the GPU's PCIe root and the copy threads run next to them.  With one process per GPU on
    a two-socket host this keeps host-to-device copies off the socket interconnect.  Returns the core list, or
    ``None`` when the topology cannot be read (nothing is changed then).  Host-side only: no GPU setting is touched.
    """
    try:
        props = torch.cuda.get_device_properties(torch.device(device) if not isinstance(device, int) else device)
        address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{address}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cores: list[int] = []
        for part in spec.split(","):
            lo, _, hi = part.partition("-")
            cores.extend(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cores) & os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


class HostPipeline:
    """Runs ``fn(z_device, slot) -> result_device`` over a sequence of pinned host tensors.

    ``fn`` is called on the compute stream with the device copy of one input and the index of the slot it
    occupies (``0 <= slot < depth``); whatever it returns must stay valid until the same slot is used again
    (e.g. a tensor from a per-slot buffer dict), because the copy-out of batch ``i`` runs while ``fn`` already
    works on batch ``i+1``.  ``fn`` may also work in place and return the slot tensor itself: the next copy into a
    slot waits for the copy-out of the slot's previous result as well as for its compute.  Inputs must all have the
    shape and dtype of ``example``.
    """

    def __init__(self, fn: Callable[[torch.Tensor, int], torch.Tensor], example: torch.Tensor,
                 device: torch.device | str, depth: int = 2):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.fn = fn
        self.device = torch.device(device)
        self.depth = depth
        self.shape, self.dtype = tuple(example.shape), example.dtype
        self.slots = [torch.empty(self.shape, dtype=self.dtype, device=self.device) for _ in range(depth)]
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self.in_done = [torch.cuda.Event() for _ in range(depth)]
        self.cmp_done = [torch.cuda.Event() for _ in range(depth)]
        self.out_done = [torch.cuda.Event() for _ in range(depth)]

    def run(self, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor]) -> None:
        """Processes ``inputs[i] -> outputs[i]`` (pinned host tensors) and returns once every output is written."""
        if len(inputs) != len(outputs):
            raise ValueError("inputs and outputs must have the same length")
        for t in list(inputs) + list(outputs):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostPipeline copies from and to pinned host tensors")
            if tuple(t.shape) != self.shape or t.dtype != self.dtype:
                raise ValueError(f"expected tensors of shape {self.shape} and dtype {self.dtype}")
        start = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(start)
        for i, (src, dst) in enumerate(zip(inputs, outputs)):
            k = i % self.depth
            reused = i >= self.depth
            with torch.cuda.stream(self.s_in):
                if reused:
                    self.s_in.wait_event(self.cmp_done[k])  # the slot's previous batch has been consumed
                    self.s_in.wait_event(self.out_done[k])  # ... and copied out, in case fn returned the slot itself
                self.slots[k].copy_(src, non_blocking=True)
                self.in_done[k].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(self.in_done[k])
                if reused:
                    self.s_cmp.wait_event(self.out_done[k])  # the slot's previous result has been copied out
                result = self.fn(self.slots[k], k)
                self.cmp_done[k].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.cmp_done[k])
                dst.copy_(result, non_blocking=True)
                result.record_stream(self.s_out)  # the copy-out reads it on this stream
                self.out_done[k].record(self.s_out)
        for s in (self.s_in, self.s_cmp, self.s_out):
            start.wait_stream(s)
        start.synchronize()
