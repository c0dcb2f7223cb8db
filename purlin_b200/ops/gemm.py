"""Python face of the tcgen05 GEMM (csrc/src/gemm_sm100.cu).

``gemm(a, w)`` computes ``a @ w.T`` for bf16 ``a [M, K]`` and ``w [N, K]`` (the nn.Linear weight layout) with
fp32 accumulation in tensor memory.  ``gemm_swiglu(a, w_interleaved)`` fuses ``silu(gate) * up`` into the
epilogue; ``interleave_gate_up`` prepares the weight for it once at load time.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native

EPI_STORE, EPI_SWIGLU = 0, 1
_declared = False


def _lib():
    global _declared
    lib = _native.cuda()
    if not _declared:
        vp, i = C.c_void_p, C.c_int
        lib.purlin_gemm_bf16.argtypes = [vp, vp, vp, i, i, i, i, i, vp, vp]
        _declared = True
    return lib


def _check(a: torch.Tensor, w: torch.Tensor):
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError("the tcgen05 GEMM takes bf16 operands")
    if not (a.is_cuda and w.is_cuda and a.is_contiguous() and w.is_contiguous()):
        raise ValueError("operands must be contiguous CUDA tensors")
    if a.shape[1] != w.shape[1]:
        raise ValueError("a is [M, K] and w is [N, K]")


def gemm(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    _check(a, w)
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=a.device)
    lib = _lib()
    rc = lib.purlin_gemm_bf16(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, EPI_STORE, bn, None,
                              torch.cuda.current_stream().cuda_stream)
    _native.check(lib, rc)
    return out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up weights -> [2I, K] with rows alternating 16 of gate and 16 of up, so that one 32-column
    slice of an accumulator tile holds both factors of 16 output columns."""
    i, k = w_gate.shape
    if i % 16:
        raise ValueError("the intermediate size must be a multiple of 16")
    g = w_gate.reshape(i // 16, 16, k)
    u = w_up.reshape(i // 16, 16, k)
    return torch.stack([g, u], dim=1).reshape(2 * i, k).contiguous()


def gemm_swiglu(a: torch.Tensor, w_gu: torch.Tensor, out: Optional[torch.Tensor] = None, bn: int = 0) -> torch.Tensor:
    """out[M, I] = silu(a @ w_gate.T) * (a @ w_up.T) with ``w_gu = interleave_gate_up(w_gate, w_up)``."""
    _check(a, w_gu)
    m, k = a.shape
    n = w_gu.shape[0]
    if out is None:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=a.device)
    lib = _lib()
    rc = lib.purlin_gemm_bf16(a.data_ptr(), w_gu.data_ptr(), out.data_ptr(), m, n, k, EPI_SWIGLU, bn, None,
                              torch.cuda.current_stream().cuda_stream)
    _native.check(lib, rc)
    return out
