"""Single-GPU emulation of a multi-rank collective.

Kernels of different ranks wait on one another, so they cannot be separate launches on one GPU (nothing
guarantees they run at the same time).  Here ``world`` virtual ranks are rows of ONE cooperative grid: every
row has its own context, plan, buffers and workspace block on the same device, and the "peer" pointers are
ordinary local pointers.  The protocol code is the production code; only the launch differs.  This is how the
reference's fake-provider test (csrc/tests/setup.cu:38-89) is extended to cover the protocol itself.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native, workspace_layout


class EmulatedWorld:
    def __init__(self, world: int, staging_size: int = 1 << 20, device=None, timeout_ms: int = 2000):
        self.lib = _native.cuda()
        self.world = world
        self.device = torch.device(device or "cuda:0")
        self.staging_size = staging_size
        self.layout = workspace_layout(world, staging_size)
        self.blocks = [torch.zeros(self.layout["total_bytes"], dtype=torch.uint8, device=self.device) for _ in range(world)]
        torch.cuda.synchronize(self.device)
        ptrs = (C.c_uint64 * world)(*[b.data_ptr() for b in self.blocks])
        self.stream = torch.cuda.current_stream(self.device).cuda_stream
        self.ctxs = []
        with torch.cuda.device(self.device):
            for r in range(world):
                h = self.lib.purlin_context_create(r, world, ptrs, 0, staging_size, timeout_ms * 1_000_000, self.stream)
                if not h:
                    raise RuntimeError("purlin: " + _native.last_error(self.lib))
                self.ctxs.append(h)

    def run(self, collective: int, srcs: Sequence[torch.Tensor], dsts: Sequence[torch.Tensor], nbytes: int = 0,
            sizes=None, dtype: int = 0, op: int = 0, mode: int = 0, policy=None, absent: int = -1):
        w = self.world
        ctx_arr = (C.c_void_p * w)(*self.ctxs)
        src_arr = (C.c_void_p * w)(*[t.data_ptr() if t.numel() else None for t in srcs])
        dst_arr = (C.c_void_p * w)(*[t.data_ptr() if t.numel() else None for t in dsts])
        flat = None
        if sizes is not None:
            flat = _native.size_array([x for row in sizes for x in row] if isinstance(sizes[0], (list, tuple)) else sizes)
        rc = self.lib.purlin_emu_collective(ctx_arr, w, collective, src_arr, dst_arr, nbytes, flat, dtype, op, mode,
                                            C.byref(policy) if policy is not None else None, absent, self.stream)
        _native.check(self.lib, rc)

    def status(self, rank: int):
        out = (C.c_uint32 * 4)()
        _native.check(self.lib, self.lib.purlin_context_status(self.ctxs[rank], out, self.stream))
        return list(out)

    def clear(self):
        for h in self.ctxs:
            self.lib.purlin_context_clear_status(h, self.stream)
        for b in self.blocks:
            b.zero_()
        torch.cuda.synchronize(self.device)

    def seq(self, rank: int) -> int:
        return int(self.lib.purlin_context_seq(self.ctxs[rank], self.stream))

    def trace(self, rank: int):
        """Device-side timing records of one virtual rank (``PURLIN_TRACE=1`` at construction), or None."""
        from .. import read_trace
        return read_trace(self.lib, self.ctxs[rank], self.stream)

    def close(self):
        for h in self.ctxs:
            self.lib.purlin_context_destroy(h, self.stream)
        self.ctxs = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
