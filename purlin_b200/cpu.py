"""CPU executor: the same Plan the GPU kernels run, executed over a gloo process group.

The reference has no CPU path.  This one exists so that the layout engine and
the Python binding surface can be exercised with real processes and no GPU: each
rank asks the native layout engine for its plan, performs its stage steps into a
byte buffer that plays the role of its symmetric staging half, lets gloo play
the role of NVLink (an all-gather of the staged bytes makes every peer's staging
readable), then performs its consume / reduce / gather / packet steps against
the peers' bytes at the offsets the plan names.  Reductions accumulate in fp32
in ascending rank order, as the deterministic device path does.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _native

_TORCH_DTYPE = {0: torch.bfloat16, 1: torch.float16, 2: torch.float8_e4m3fn, 3: torch.float8_e5m2, 4: torch.float32}


def _bytes_view(t: torch.Tensor) -> torch.Tensor:
    return t.view(-1).view(torch.uint8)


class CpuContext:
    def __init__(self, group, rank: int, world: int, staging_size: int):
        self.group, self.rank, self.world, self.staging_size = group, rank, world, staging_size
        self.seq = 0

    # -- plan ---------------------------------------------------------------------------------------------
    def _plan(self, collective, nbytes, sizes, out_sizes, dtype, op, mode, in_place, policy):
        lib = _native.host()
        plan = _native.Plan()
        s_arr = _native.size_array(sizes) if sizes is not None else None
        o_arr = _native.size_array(out_sizes) if out_sizes is not None else None
        rc = lib.purlin_plan_build(collective, self.world, self.rank, nbytes, s_arr, o_arr, dtype, op, mode, 0, int(in_place),
                                   self.staging_size, C.byref(policy) if policy is not None else None, C.byref(plan), None)
        _native.check(lib, rc)
        return plan

    # -- transport ----------------------------------------------------------------------------------------
    def _exchange(self, mine: torch.Tensor, extent: int):
        """All ranks publish the first ``extent`` bytes of a staging image; returns every rank's image."""
        ext = torch.tensor([extent], dtype=torch.int64)
        dist.all_reduce(ext, op=dist.ReduceOp.MAX, group=self.group)
        n = int(ext.item())
        send = torch.zeros(max(n, 1), dtype=torch.uint8)
        send[: min(n, mine.numel())] = mine[:n]
        recv = [torch.empty_like(send) for _ in range(self.world)]
        dist.all_gather(recv, send, group=self.group)
        return recv

    @staticmethod
    def _reduce(parts, dtype, op):
        td = _TORCH_DTYPE[dtype]
        acc = None
        for p in parts:   # ascending rank order, fp32 accumulation
            x = p.view(td).to(torch.float32)
            if acc is None:
                acc = x.clone()
            elif op == 0:
                acc += x
            elif op == 1:
                acc *= x
            else:
                acc = torch.maximum(acc, x)
        return _bytes_view(acc.to(td))

    # -- one collective -----------------------------------------------------------------------------------
    def run(self, collective, src, dst, nbytes, sizes, out_sizes, dtype, op, mode, policy=None):
        if self.world == 1:
            n = sizes[0] if sizes is not None else nbytes
            _bytes_view(dst)[:n] = _bytes_view(src)[:n]
            return
        in_place = src.data_ptr() == dst.data_ptr()
        plan = self._plan(collective, nbytes, sizes, out_sizes, dtype, op, mode, in_place, policy)
        steps = plan.active_steps()
        if any(s.flags & _native.FLAG_CYCLIC for s in steps):
            raise NotImplementedError("the gloo executor keeps streams resident; use a staging size that holds the payload")
        s8 = _bytes_view(src).clone()   # in-place calls read the original input
        d8 = _bytes_view(dst)
        W, r = self.world, self.rank

        # throughput staging image and packet image (payload bytes only; a flag is implied by the exchange)
        tr_extent = max([s.dstOff + s.bytes for s in steps if s.role == _native.ROLE_STAGE], default=0)
        tr = torch.zeros(tr_extent, dtype=torch.uint8)
        # packet image: slot for destination d at [d * stride, ...): what I send to d
        put = [s for s in steps if s.role == _native.ROLE_PACKET_PUT]
        stride = max([s.dstOff + s.bytes for s in put], default=0)
        lr = torch.zeros(stride * W, dtype=torch.uint8)
        for s in steps:
            if s.role == _native.ROLE_STAGE:
                tr[s.dstOff:s.dstOff + s.bytes] = s8[s.srcOff:s.srcOff + s.bytes]
            elif s.role == _native.ROLE_PACKET_PUT:
                for d in (range(W) if s.peer < 0 else [s.peer]):
                    at = s.srcOff + (d * s.bytes if s.flags & _native.FLAG_SCATTER else 0)     # scatter: peer d gets slice d
                    lr[d * stride + s.dstOff: d * stride + s.dstOff + s.bytes] = s8[at:at + s.bytes]
            elif s.role == _native.ROLE_LOCAL:
                d8[s.dstOff:s.dstOff + s.bytes] = s8[s.srcOff:s.srcOff + s.bytes]
        # every rank performs every exchange, whatever its own plan holds, so the group calls always match
        peers_tr = self._exchange(tr, tr_extent)
        strides = [torch.zeros(1, dtype=torch.int64) for _ in range(W)]
        dist.all_gather(strides, torch.tensor([stride], dtype=torch.int64), group=self.group)
        peers_lr = self._exchange(lr, lr.numel())

        def packet_from(q, off, n):   # what rank q sent to me
            st = int(strides[q].item())
            return peers_lr[q][r * st + off: r * st + off + n]

        seam = torch.zeros(0, dtype=torch.uint8)
        seam_extent = 0
        result_pub = {}   # packet reduce results published to peers: offset -> bytes
        for s in steps:
            if s.role == _native.ROLE_CONSUME:
                d8[s.dstOff:s.dstOff + s.bytes] = peers_tr[s.peer][s.srcOff:s.srcOff + s.bytes]
            elif s.role == _native.ROLE_REDUCE:
                out = self._reduce([peers_tr[q][s.srcOff:s.srcOff + s.bytes] for q in range(W)], dtype, op)
                if s.flags & _native.FLAG_TO_DST:
                    d8[s.dstOff:s.dstOff + s.bytes] = out
                if s.flags & _native.FLAG_TO_SEAM:
                    seam_extent = s.seamOff + s.bytes
                    seam = torch.zeros(seam_extent, dtype=torch.uint8)
                    seam[s.seamOff:seam_extent] = out
            elif s.role == _native.ROLE_PACKET_GET and not (s.flags & _native.FLAG_RESULT_HALF):
                # peer -1: the packets of every peer in one step, slice q at dstOff + q * bytes
                for q in ([s.peer] if s.peer >= 0 else [q for q in range(W) if q != r]):
                    at = s.dstOff + (q * s.bytes if s.peer < 0 else 0)
                    d8[at:at + s.bytes] = packet_from(q, s.srcOff, s.bytes)
            elif s.role == _native.ROLE_PACKET_REDUCE:
                parts = [s8[s.seamOff:s.seamOff + s.bytes] if q == r else packet_from(q, s.srcOff, s.bytes) for q in range(W)]
                out = self._reduce(parts, dtype, op)
                d8[s.dstOff:s.dstOff + s.bytes] = out
                if s.flags & _native.FLAG_PUBLISH:
                    result_pub[0] = out
        # composition tail: reduced shards travel back (throughput: through the seam; latency: result packets)
        peers_seam = self._exchange(seam, seam_extent)
        for s in steps:
            if s.role == _native.ROLE_GATHER:
                d8[s.dstOff:s.dstOff + s.bytes] = peers_seam[s.peer][s.srcOff:s.srcOff + s.bytes]
        mine = result_pub.get(0, torch.zeros(0, dtype=torch.uint8))
        peers_res = self._exchange(mine, mine.numel())
        for s in steps:
            if s.role == _native.ROLE_PACKET_GET and (s.flags & _native.FLAG_RESULT_HALF):
                for q in ([s.peer] if s.peer >= 0 else [q for q in range(W) if q != r]):
                    at = s.dstOff + (q * s.bytes if s.peer < 0 else 0)
                    d8[at:at + s.bytes] = peers_res[q][s.srcOff:s.srcOff + s.bytes]
        self.seq += 1
