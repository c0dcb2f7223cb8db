"""Expert-parallel MoE token exchange fused with permute and gate-weighted sum (csrc/src/moe.cu).

``ExpertParallelContext`` owns the symmetric receive / expert-output buffers of one process group.
One layer is: ``route`` -> ``dispatch`` -> experts work on ``recv_rows()`` and write ``out_rows()`` -> ``combine``.
``dispatch`` and ``combine`` must alternate on one stream (a call out of order is refused on the device and
``check()`` raises).  A token crosses NVLink once per destination GPU in each direction, however many of that GPU's
experts it was routed to: the receiver fans it out to its expert rows, and the experts' GPU sends back one row per
token, already weighted and summed over its local experts.  The reference offers allToAllV only; a MoE layer needs the exchange fused with the permute and the weighted sum.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from .. import _native
from .symmetric import allocate_symmetric, RawBuffer as _RawBuffer

_declared = False


def _lib():
    global _declared
    lib = _native.cuda()
    if not _declared:
        vp, i, u64, sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
        lib.purlin_moe_workspace_bytes.restype = sz
        lib.purlin_moe_workspace_bytes.argtypes = [i, i, i, i, i]
        lib.purlin_moe_plan.argtypes = [vp, vp, vp, i, vp, vp]
        lib.purlin_moe_create.restype = vp
        lib.purlin_moe_create.argtypes = [i, i, C.POINTER(u64), i, i, i, i, i, u64, vp]
        lib.purlin_moe_destroy.argtypes = [vp, vp]
        lib.purlin_moe_status.argtypes = [vp, C.POINTER(C.c_uint32), vp]
        lib.purlin_moe_clear_status.argtypes = [vp, vp]
        lib.purlin_moe_timing.argtypes = [vp, C.POINTER(u64), vp]
        lib.purlin_moe_recv_buffer.restype = vp
        lib.purlin_moe_recv_buffer.argtypes = [vp]
        lib.purlin_moe_out_buffer.restype = vp
        lib.purlin_moe_out_buffer.argtypes = [vp]
        lib.purlin_moe_route.argtypes = [vp, vp, i, i, vp, vp, vp, vp]
        lib.purlin_moe_dispatch.argtypes = [vp, vp, i, vp, vp, vp, vp, i, vp]
        lib.purlin_moe_combine.argtypes = [vp, vp, i, vp, vp, vp, i, vp]
        _declared = True
    return lib


class ExpertParallelContext:
    def __init__(self, group=None, device=None, max_tokens: int = 4096, hidden: int = 7168, experts: int = 256, topk: int = 8,
                 capacity_factor: float = 2.0, timeout_ms: int = 10000, provider: Optional[str] = None):
        import torch.distributed as dist
        self.lib = _lib()
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.max_tokens, self.hidden, self.experts, self.topk = max_tokens, hidden, experts, topk
        self.experts_per_rank = experts // self.world
        # balanced routing delivers max_tokens * topk rows to each rank; the factor leaves room for imbalance
        self.capacity_rows = int(max_tokens * topk * capacity_factor)
        nbytes = int(self.lib.purlin_moe_workspace_bytes(self.world, max_tokens, self.capacity_rows, hidden, experts))
        if self.world > 1:
            self._owner, self._hdl, peer_ptrs, _ = allocate_symmetric(nbytes, self.device, group, provider)
        else:
            self._owner = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=self.device)
            base = (self._owner.data_ptr() + 1023) // 1024 * 1024
            self._hdl, peer_ptrs = None, [base]
        ptrs = (C.c_uint64 * self.world)(*peer_ptrs)
        self.stream = lambda: torch.cuda.current_stream().cuda_stream
        self.ctx = self.lib.purlin_moe_create(self.rank, self.world, ptrs, max_tokens, hidden, experts, topk, self.capacity_rows,
                                              timeout_ms * 1_000_000, self.stream())
        if not self.ctx:
            raise RuntimeError("purlin: " + _native.last_error(self.lib))
        dev = self.device
        self.topk_idx = torch.empty(max_tokens, topk, dtype=torch.int32, device=dev)
        self.topk_weight = torch.empty(max_tokens, topk, dtype=torch.float32, device=dev)
        self.slot = torch.empty(max_tokens, topk, dtype=torch.int32, device=dev)
        self.sent_row = torch.empty(max_tokens, topk, dtype=torch.int32, device=dev)
        self.recv_counts = torch.zeros(self.experts_per_rank + 1, dtype=torch.int32, device=dev)
        shape = (self.capacity_rows, hidden)
        self._recv = torch.as_tensor(_RawBuffer(self.lib.purlin_moe_recv_buffer(self.ctx), shape, "<u2"), device=dev).view(torch.bfloat16)
        self._out = torch.as_tensor(_RawBuffer(self.lib.purlin_moe_out_buffer(self.ctx), shape, "<u2"), device=dev).view(torch.bfloat16)

    # -- the four steps of a layer ----------------------------------------------------------------------------
    def route(self, logits: torch.Tensor, normalize: bool = True):
        """softmax + top-k of fp32 ``logits [tokens, experts]``; returns (expert ids, gate weights)."""
        t = logits.shape[0]
        if logits.dtype != torch.float32 or not logits.is_contiguous() or logits.shape[1] != self.experts:
            raise ValueError("logits must be contiguous fp32 [tokens, experts]")
        rc = self.lib.purlin_moe_route(self.ctx, logits.data_ptr(), t, int(normalize), self.topk_idx.data_ptr(),
                                       self.topk_weight.data_ptr(), self.slot.data_ptr(), self.stream())
        _native.check(self.lib, rc)
        return self.topk_idx[:t], self.topk_weight[:t]

    def plan(self, topk_idx: torch.Tensor, topk_weight: torch.Tensor):
        """Adopts routing the caller computed: int32 ``topk_idx`` and fp32 ``topk_weight`` of shape [tokens, topk]."""
        t = topk_idx.shape[0]
        if topk_idx.dtype != torch.int32 or topk_weight.dtype != torch.float32 or topk_idx.shape != (t, self.topk) or topk_weight.shape != (t, self.topk):
            raise ValueError("routing must be int32 ids and fp32 weights of shape [tokens, topk]")
        self.topk_idx[:t].copy_(topk_idx)
        self.topk_weight[:t].copy_(topk_weight)
        rc = self.lib.purlin_moe_plan(self.ctx, self.topk_idx.data_ptr(), self.topk_weight.data_ptr(), t, self.slot.data_ptr(), self.stream())
        _native.check(self.lib, rc)
        return self.topk_idx[:t], self.topk_weight[:t]

    def dispatch(self, x: torch.Tensor, blocks: int = 0):
        """Sends every token to its experts' GPUs; returns (rows in expert-major order, rows per local expert).
        ``blocks`` > 0 sets the number of sending CTAs (the rest of the grid copies rows to their expert rows);
        ``PURLIN_MOE_SENDERS`` in the environment sets the default."""
        blocks = blocks or int(os.environ.get("PURLIN_MOE_SENDERS", 0))
        t = x.shape[0]
        if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] != self.hidden:
            raise ValueError("x must be contiguous bf16 [tokens, hidden]")
        rc = self.lib.purlin_moe_dispatch(self.ctx, x.data_ptr(), t, self.topk_idx.data_ptr(), self.slot.data_ptr(),
                                          self.sent_row.data_ptr(), self.recv_counts.data_ptr(), blocks, self.stream())
        _native.check(self.lib, rc)
        return self._recv, self.recv_counts

    def recv_rows(self) -> torch.Tensor:
        return self._recv

    def out_rows(self) -> torch.Tensor:
        """Where the experts write their outputs, row for row with ``recv_rows()``."""
        return self._out

    def combine(self, tokens: int, out: Optional[torch.Tensor] = None, blocks: int = 0) -> torch.Tensor:
        """``blocks`` > 0 sets the number of CTAs that form and push the per-GPU partial sums (the rest add the rows that
        arrive); ``PURLIN_MOE_PUSHERS`` in the environment sets the default."""
        blocks = blocks or int(os.environ.get("PURLIN_MOE_PUSHERS", 0))
        if out is None:
            out = torch.empty(tokens, self.hidden, dtype=torch.bfloat16, device=self.device)
        rc = self.lib.purlin_moe_combine(self.ctx, out.data_ptr(), tokens, self.topk_idx.data_ptr(), self.topk_weight.data_ptr(),
                                         self.sent_row.data_ptr(), blocks, self.stream())
        _native.check(self.lib, rc)
        return out

    def check(self):
        out = (C.c_uint32 * 4)()
        self.lib.purlin_moe_status(self.ctx, out, self.stream())
        if out[0]:
            self.lib.purlin_moe_clear_status(self.ctx, self.stream())
            what = {2: "receive buffer capacity exceeded", 3: "more rows for one destination than the staging area holds",
                    7: "an expert id outside [0, experts)", 9: "dispatch called twice without a combine in between",
                    10: "combine called without a matching dispatch"}.get(out[1], "bad plan") if out[0] == 6 else "a wait timed out"
            raise RuntimeError(f"purlin: MoE exchange failed: {what} (where {out[1]}, peer {out[2]})")

    def timing(self):
        """Device-side phase times in microseconds since the previous call of this method (contexts created with
        ``PURLIN_MOE_TIMING=1``): from the first CTA's start to the last sender / last receiver / first sender leaving the
        dispatch, and the same for the pushers and finishers of the combine. Synchronises the stream."""
        out = (C.c_uint64 * 8)()
        _native.check(self.lib, self.lib.purlin_moe_timing(self.ctx, out, self.stream()))
        us = [v / 1e3 for v in out]
        return {"dispatch": {"last_sender": us[0], "last_receiver": us[1], "first_sender": us[2]},
                "combine": {"last_pusher": us[4], "last_finisher": us[5], "first_pusher": us[6]}}

    def close(self):
        if self.ctx:
            self._recv = self._out = None
            self.lib.purlin_moe_destroy(self.ctx, self.stream())
            self.ctx = None
        self._owner = self._hdl = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
