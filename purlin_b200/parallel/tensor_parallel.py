"""Tensor-parallel linear layers whose collective is fused into the GEMM kernel.

``TensorParallelContext`` owns the symmetric buffers of the fused kernels (csrc/src/gemm_sm100.cu):
  * ``ag_gemm``  : all-gather of sequence-sharded activations fused into the GEMM that consumes them
  * ``gemm_rs``  : GEMM whose output tiles are reduce-scattered by sequence from the epilogue
The reference offers only the separate collectives (allGather, reduceScatter; csrc/include/purlin/host/allGather.cuh,
reduceScatter.cuh of the reference); a tensor-parallel layer wants the transfer hidden under the math.  With a world of one the same tcgen05 kernel runs without its communication warps.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native
from ..ops import gemm as _gemm
from .symmetric import allocate_symmetric

_declared = False


def _lib():
    global _declared
    lib = _native.cuda()
    if not _declared:
        vp, i, u64, sz = C.c_void_p, C.c_int, C.c_uint64, C.c_size_t
        lib.purlin_tp_workspace_bytes.restype = sz
        lib.purlin_tp_workspace_bytes.argtypes = [i, i, i, i]
        lib.purlin_tp_create.restype = vp
        lib.purlin_tp_create.argtypes = [i, i, C.POINTER(u64), i, i, i, u64, vp]
        lib.purlin_tp_destroy.argtypes = [vp, vp]
        lib.purlin_tp_status.argtypes = [vp, C.POINTER(C.c_uint32), vp]
        lib.purlin_tp_clear_status.argtypes = [vp, vp]
        lib.purlin_tp_ag_gemm.argtypes = [vp, vp, vp, vp, i, i, i, i, vp]
        lib.purlin_tp_gemm_rs.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        _gemm._lib()
        _declared = True
    return lib


class TensorParallelContext:
    """Symmetric workspace + native context for fused TP kernels over ``group`` (collective constructor)."""

    def __init__(self, group=None, device=None, max_tokens: int = 8192, k_ag: int = 8192, n_rs: int = 8192,
                 timeout_ms: int = 10000, provider: Optional[str] = None):
        import torch.distributed as dist
        self.lib = _lib()
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.group = group
        self.max_tokens, self.k_ag, self.n_rs = max_tokens, k_ag, n_rs
        self.ctx = None
        self._owner = self._hdl = None
        if self.world > 1:
            nbytes = int(self.lib.purlin_tp_workspace_bytes(self.world, max_tokens, k_ag, n_rs))
            self._owner, self._hdl, peer_ptrs, _ = allocate_symmetric(nbytes, self.device, group, provider)
            ptrs = (C.c_uint64 * self.world)(*peer_ptrs)
            self.ctx = self.lib.purlin_tp_create(self.rank, self.world, ptrs, max_tokens, k_ag, n_rs,
                                                 timeout_ms * 1_000_000, torch.cuda.current_stream().cuda_stream)
            if not self.ctx:
                raise RuntimeError("purlin: " + _native.last_error(self.lib))

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, swiglu: bool = False):
        """``epilogue(all_gather(x_local) @ w.T)``; x_local is this rank's [tokens / world, K] slice of the sequence."""
        if self.world == 1:
            return _gemm.gemm_swiglu(x_local, w, out) if swiglu else _gemm.gemm(x_local, w, out)
        _gemm._check(x_local, w)
        m, k, n = x_local.shape[0] * self.world, x_local.shape[1], w.shape[0]
        if out is None:
            out = torch.empty(m, n // 2 if swiglu else n, dtype=torch.bfloat16, device=x_local.device)
        rc = self.lib.purlin_tp_ag_gemm(self.ctx, x_local.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                        _gemm.EPI_SWIGLU if swiglu else _gemm.EPI_STORE, torch.cuda.current_stream().cuda_stream)
        _native.check(self.lib, rc)
        return out

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None):
        """This rank's [tokens / world, N] rows of ``sum over ranks (a @ w.T)``; a is [tokens, K / world]."""
        if self.world == 1:
            return _gemm.gemm(a, w, out)
        _gemm._check(a, w)
        m, k, n = a.shape[0], a.shape[1], w.shape[0]
        if out is None:
            out = torch.empty(m // self.world, n, dtype=torch.bfloat16, device=a.device)
        rc = self.lib.purlin_tp_gemm_rs(self.ctx, a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                        torch.cuda.current_stream().cuda_stream)
        _native.check(self.lib, rc)
        return out

    def check(self):
        """Synchronises and raises if a bounded wait inside a fused kernel gave up."""
        if self.ctx is None:
            torch.cuda.synchronize(self.device)
            return
        out = (C.c_uint32 * 4)()
        self.lib.purlin_tp_status(self.ctx, out, torch.cuda.current_stream().cuda_stream)
        if out[0]:
            self.lib.purlin_tp_clear_status(self.ctx, torch.cuda.current_stream().cuda_stream)
            raise TimeoutError(f"purlin: fused kernel wait timed out (where {out[1]}, {out[2]}, {out[3]})")

    def close(self):
        if self.ctx is not None:
            self.lib.purlin_tp_destroy(self.ctx, torch.cuda.current_stream().cuda_stream)
            self.ctx = None
        self._owner = self._hdl = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
