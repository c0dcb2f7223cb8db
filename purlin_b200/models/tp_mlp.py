"""Llama-style MLP block under tensor + sequence parallelism, every collective fused into a GEMM.

    x_local [T / W, H]  --all-gather->GEMM (gate|up, SwiGLU epilogue)-->  h [T, I / W]
                        --GEMM->reduce-scatter (down)-->                  y_local [T / W, H]

Shapes of the Llama-3-70B MLP at TP = 8: H = 8192, I = 28672 (3584 per rank), T = 8192 tokens.  Weights are
random N(0, 0.02) from a seed, activations N(0, 1); there is no checkpoint loading here.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.gemm import interleave_gate_up
from ..parallel.tensor_parallel import TensorParallelContext


class TensorParallelMLP:
    def __init__(self, hidden: int = 8192, intermediate: int = 28672, tokens: int = 8192, group=None, device=None,
                 seed: int = 3, tp: Optional[TensorParallelContext] = None):
        self.hidden, self.intermediate, self.tokens = hidden, intermediate, tokens
        self.tp = tp or TensorParallelContext(group, device, max_tokens=tokens, k_ag=hidden, n_rs=hidden)
        w, r = self.tp.world, self.tp.rank
        if intermediate % (w * 16):
            raise ValueError("the intermediate size per rank must be a multiple of 16")
        self.i_local = intermediate // w
        dev = self.tp.device
        g = torch.Generator(device=dev).manual_seed(seed * 1000 + r)
        def init(rows, cols):
            return (torch.randn(rows, cols, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        self.w_gate = init(self.i_local, hidden)      # this rank's columns of the gate projection, [I / W, H]
        self.w_up = init(self.i_local, hidden)
        self.w_down = init(hidden, self.i_local)      # this rank's rows of the down projection, [H, I / W]
        self.w_gu = interleave_gate_up(self.w_gate, self.w_up)
        self.h = torch.empty(tokens, self.i_local, dtype=torch.bfloat16, device=dev)
        self._feed = None
        self._y = None

    def forward(self, x_local: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        t = x_local.shape[0] * self.tp.world
        h = self.h[:t]
        self.tp.ag_gemm(x_local, self.w_gu, h, swiglu=True)
        return self.tp.gemm_rs(h, self.w_down, out)

    __call__ = forward

    def run_host_batches(self, host_batches, out: Optional[torch.Tensor] = None, on_result=None):
        """Serving loop over activations that live in pinned host memory: one forward per batch, its input copied to the
        device and its metric (the L2 norm of this rank's output rows) read back to the host every step, with both
        transfers overlapped with the neighbouring steps (``purlin_b200.utils.feed.HostFeed``). Returns the metrics."""
        from ..utils.feed import HostFeed
        rows = self.tokens // self.tp.world
        if self._feed is None:
            self._feed = HostFeed((rows, self.hidden), torch.bfloat16, self.tp.device)
        y = out if out is not None else self._y_rows(rows)

        def step(x_dev):
            self.forward(x_dev, y)
            return torch.linalg.vector_norm(y, dtype=torch.float32)

        return self._feed.run(host_batches, step, on_result)

    def _y_rows(self, rows: int) -> torch.Tensor:
        if self._y is None or self._y.shape[0] != rows:
            self._y = torch.empty(rows, self.hidden, dtype=torch.bfloat16, device=self.tp.device)
        return self._y

    def flops(self, tokens: int) -> float:
        """Floating-point operations of one forward over ``tokens`` tokens, whole job (all ranks)."""
        return 2.0 * tokens * self.hidden * self.intermediate * 3

    def reference(self, x_full: torch.Tensor) -> torch.Tensor:
        """fp32 PyTorch result of this rank's partial contribution (before the reduction over ranks)."""
        xf = x_full.float()
        h = torch.nn.functional.silu(xf @ self.w_gate.float().t()) * (xf @ self.w_up.float().t())
        return h.to(torch.bfloat16).float() @ self.w_down.float().t()


def smoke_mlp():
    """Tiny forward on one GPU, checked against the fp32 reference."""
    mlp = TensorParallelMLP(hidden=512, intermediate=1024, tokens=256, device="cuda:0")
    g = torch.Generator(device="cuda:0").manual_seed(3)
    x = torch.randn(256, 512, generator=g, device="cuda:0").to(torch.bfloat16)
    y = mlp(x)
    torch.cuda.synchronize()
    ref = mlp.reference(x)
    err = (y.float() - ref).abs().max().item()
    assert err <= 3e-2 * ref.abs().max().item() + 1e-3, f"MLP smoke mismatch: {err}"
