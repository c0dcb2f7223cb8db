"""Data-parallel and sharded-data-parallel helpers on zero-copy symmetric tensors.

The reference implements no parallelism strategy; it offers the collectives a strategy is built from (allReduce for
gradient averaging, allGather / reduceScatter for sharded parameters: csrc/include/purlin/host/allReduce.cuh:310-327,
allGather.cuh, reduceScatter.cuh).  These helpers put the buffers a strategy owns anyway (gradient buckets, flat
parameter shards) into symmetric memory once, so that every step's collective runs in place on them with no staging
pass: ``all_reduce_symm`` for gradient buckets, ``all_gather_symm`` / ``reduce_scatter_symm`` for sharded parameters.

``GradientBuckets``       DDP-style: parameters' ``.grad`` tensors are views into a few large symmetric buckets;
                          ``reduce()`` all-reduces every bucket in place and (optionally) averages.
``ShardedFlatParameter``  ZeRO-3 / FSDP-style: one flat parameter of ``world`` slices in symmetric memory; a rank owns
                          slice ``rank``; ``gather()`` materialises the full parameter in place on every rank,
                          ``reduce_scatter_grad()`` leaves each rank with the reduced gradient of its own slice.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from .. import ReduceOp, ReductionMode, all_gather_symm, all_reduce_symm, reduce_scatter_symm, symm_empty


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class GradientBuckets:
    """Gradients of ``params`` live in symmetric buckets of about ``bucket_bytes``; ``reduce()`` sums them over the group."""

    def __init__(self, params: Iterable[torch.nn.Parameter], handle, bucket_bytes: int = 64 << 20, dtype: Optional[torch.dtype] = None):
        self.handle = handle
        self.world = handle.world
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no parameter requires a gradient")
        self.dtype = dtype or self.params[0].dtype
        esz = torch.empty(0, dtype=self.dtype).element_size()
        align = 32 // esz                                   # every gradient view starts on a 32-byte boundary
        self.buckets = []                                   # SymmetricTensor per bucket
        self.views: List[torch.Tensor] = []
        plan, cur, cur_elems = [], [], 0
        for p in self.params:
            n = _round_up(p.numel(), align)
            if cur and (cur_elems + n) * esz > bucket_bytes:
                plan.append((cur, cur_elems))
                cur, cur_elems = [], 0
            cur.append((p, cur_elems))
            cur_elems += n
        plan.append((cur, cur_elems))
        for members, elems in plan:
            st = symm_empty((_round_up(elems, align * self.world),), self.dtype, handle)
            st.tensor.zero_()
            self.buckets.append(st)
            for p, off in members:
                view = st.tensor[off:off + p.numel()].view_as(p)
                p.grad = view                               # autograd accumulates straight into the bucket
                self.views.append(view)

    def zero(self):
        for st in self.buckets:
            st.tensor.zero_()

    def reduce(self, average: bool = True, reduction_mode=ReductionMode.NON_DETERMINISTIC):
        """In-place all-reduce of every bucket on the current stream; gradients become the sum (or mean) over ranks."""
        for st in self.buckets:
            all_reduce_symm(st, ReduceOp.ADD, reduction_mode)
            if average:
                st.tensor.mul_(1.0 / self.world)

    def status(self) -> int:
        return max(st.status() for st in self.buckets)


class ShardedFlatParameter:
    """A flat parameter of ``world`` equal slices in symmetric memory; this rank owns (and updates) slice ``rank``."""

    def __init__(self, numel: int, dtype: torch.dtype, handle):
        self.handle = handle
        self.world, self.rank = handle.world, handle.rank
        esz = torch.empty(0, dtype=dtype).element_size()
        self.numel = numel
        self.slice_elems = _round_up(_round_up(numel, self.world) // self.world, 32 // esz)
        self.full = symm_empty((self.slice_elems * self.world,), dtype, handle)         # gathered parameter
        self.full.tensor.zero_()
        self.grad_full = symm_empty((self.slice_elems * self.world,), dtype, handle)    # full local gradient, input of the reduce-scatter
        self.grad_full.tensor.zero_()
        self.grad_shard = torch.zeros(self.slice_elems, dtype=dtype, device=handle.device)

    @property
    def shard(self) -> torch.Tensor:
        """The slice this rank owns (a view into the gathered tensor: updating it updates the next gather's source)."""
        return self.full.tensor[self.rank * self.slice_elems:(self.rank + 1) * self.slice_elems]

    def gather(self) -> torch.Tensor:
        """Every rank's slice lands in every rank's tensor, in place; returns the full flat parameter."""
        all_gather_symm(self.full)
        return self.full.tensor[:self.numel]

    def reduce_scatter_grad(self, average: bool = True, reduction_mode=ReductionMode.NON_DETERMINISTIC) -> torch.Tensor:
        """Sums ``grad_full`` over ranks and returns the slice of the result that belongs to this rank's shard."""
        reduce_scatter_symm(self.grad_full, self.grad_shard, ReduceOp.ADD, reduction_mode)
        if average:
            self.grad_shard.mul_(1.0 / self.world)
        return self.grad_shard

    def status(self) -> int:
        return max(self.full.status(), self.grad_full.status())
