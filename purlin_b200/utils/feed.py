"""Host-fed step loop: every step's input comes from pinned host memory and every step's result goes back to the host,
with both transfers overlapped with the neighbouring steps' compute.

The reference is a communication library and has no input pipeline; its benchmarks create data on the device
(csrc/support/purlin/benchmark/data.cuh:79-140).  A serving or training loop around the fused layers needs one, and on a
B200 the PCIe copy of a step's activations (tens of MB) costs as much as a sizeable fraction of the step itself, so it
must not sit on the critical path:

    copy stream     H2D(i+1) ......            H2D(i+2) ......
    compute stream  step(i) ........ D2H r(i)  step(i+1) ........ D2H r(i+1)
    host            wait r(i-1), read it       wait r(i), read it

``depth`` device buffers rotate; a buffer is overwritten only after the step that read it has finished (event), a step
starts only after its input has landed (event), and the host reads the result of step i - (depth - 1) while the later steps
are already queued: with several ranks that wait for one another inside the fused kernels, a host that is late once
(a timer thread, the interpreter lock) would otherwise stall every rank, every time. Every step still performs its own
host->device copy and its own device->host read; nothing is cached or skipped.
"""
from __future__ import annotations

from typing import Callable, Iterable, List, Optional

import torch


class HostFeed:
    def __init__(self, shape, dtype: torch.dtype, device, depth: int = 4):
        if depth < 2:
            raise ValueError("overlap needs at least two device buffers")
        self.device = torch.device(device)
        self.depth = depth
        self.copy_stream = torch.cuda.Stream(self.device)
        self.bufs = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(depth)]
        self.loaded = [torch.cuda.Event() for _ in range(depth)]      # input of the step using this slot is on the device
        self.consumed = [torch.cuda.Event() for _ in range(depth)]    # the step using this slot no longer reads its input
        self.done = [torch.cuda.Event() for _ in range(depth)]        # the step's result is in pinned host memory
        self.results = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(depth)]
        self.h2d_bytes_per_step = 0
        self.d2h_bytes_per_step = self.results[0].numel() * self.results[0].element_size()

    def run(self, host_inputs: Iterable[torch.Tensor], step_fn: Callable[[torch.Tensor], torch.Tensor],
            on_result: Optional[Callable[[int, float], None]] = None) -> List[float]:
        """Calls ``step_fn(device_input)`` once per host input, in order, and returns every step's scalar result.

        ``host_inputs`` yields pinned host tensors of the shape and dtype given to the constructor; ``step_fn`` returns a
        one-element device tensor (the step's loss or metric) and may launch any kernels on the current stream.
        """
        cur = torch.cuda.current_stream(self.device)
        out: List[float] = []
        pending = []     # (slot, step index) of the steps whose results have not been read yet, oldest first
        lag = self.depth - 1   # results are read this many steps late; a result slot is read before it is reused

        def collect():
            slot, idx = pending.pop(0)
            self.done[slot].synchronize()
            v = float(self.results[slot][0])
            out.append(v)
            if on_result is not None:
                on_result(idx, v)

        for i, x_host in enumerate(host_inputs):
            if not x_host.is_pinned():
                raise ValueError("host inputs must live in pinned memory (torch.Tensor.pin_memory)")
            s = i % self.depth
            self.h2d_bytes_per_step = x_host.numel() * x_host.element_size()
            if i >= self.depth:
                self.copy_stream.wait_event(self.consumed[s])          # the step that last read this buffer is finished with it
            with torch.cuda.stream(self.copy_stream):
                self.bufs[s].copy_(x_host, non_blocking=True)
                self.loaded[s].record(self.copy_stream)
            cur.wait_event(self.loaded[s])
            metric = step_fn(self.bufs[s])
            self.consumed[s].record(cur)
            self.results[s].copy_(metric.reshape(1).to(torch.float32), non_blocking=True)
            self.done[s].record(cur)
            pending.append((s, i))
            while len(pending) > lag:
                collect()                                              # step i - lag's result, read while later steps run
        while pending:
            collect()
        return out
