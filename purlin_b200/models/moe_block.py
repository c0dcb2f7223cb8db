"""Mixture-of-experts feed-forward block under expert parallelism.

    logits = x @ w_router.T                                  (tcgen05 GEMM)
    route: softmax + top-k                                   (one kernel)
    dispatch: tokens -> their experts' GPUs, expert-major    (one kernel over peer memory)
    experts: SwiGLU MLP per local expert on its rows         (tcgen05 GEMMs on contiguous row ranges)
    combine: gate-weighted sum of the top-k outputs          (one kernel over peer memory)

DeepSeek-V3-like shapes are the defaults of the benchmark: hidden 7168, 256 experts (32 per GPU at 8 GPUs), top-8.
Weights are random N(0, 0.02) from a seed; there is no checkpoint loading here.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.gemm import gemm, gemm_swiglu, interleave_gate_up
from ..parallel.expert_parallel import ExpertParallelContext


class ExpertParallelMoE:
    def __init__(self, hidden: int = 7168, intermediate: int = 2048, experts: int = 256, topk: int = 8, max_tokens: int = 4096,
                 group=None, device=None, seed: int = 11, ep: Optional[ExpertParallelContext] = None, capacity_factor: float = 2.0):
        self.ep = ep or ExpertParallelContext(group, device, max_tokens=max_tokens, hidden=hidden, experts=experts, topk=topk,
                                              capacity_factor=capacity_factor)
        self.hidden, self.intermediate, self.experts, self.topk = hidden, intermediate, experts, topk
        dev = self.ep.device
        g = torch.Generator(device=dev).manual_seed(seed)                      # the router is replicated: same seed everywhere
        self.w_router = (torch.randn(experts, hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        ge = torch.Generator(device=dev).manual_seed(seed * 1000 + 1 + self.ep.rank)
        n = self.ep.experts_per_rank
        def init(*shape):
            return (torch.randn(*shape, generator=ge, device=dev) * 0.02).to(torch.bfloat16)
        self.w_gate, self.w_up = init(n, intermediate, hidden), init(n, intermediate, hidden)
        self.w_down = init(n, hidden, intermediate)
        self.w_gu = torch.stack([interleave_gate_up(self.w_gate[e], self.w_up[e]) for e in range(n)])
        self._h = torch.empty(self.ep.capacity_rows, intermediate, dtype=torch.bfloat16, device=dev)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        t = x.shape[0]
        logits = gemm(x, self.w_router).float()
        self.ep.route(logits)
        recv, counts = self.ep.dispatch(x)
        offs = [0] + torch.cumsum(counts[: self.ep.experts_per_rank], 0).tolist()   # one host read per layer: row ranges of the experts
        outb = self.ep.out_rows()
        for e in range(self.ep.experts_per_rank):
            a, b = offs[e], offs[e + 1]
            if b > a:
                h = gemm_swiglu(recv[a:b], self.w_gu[e], self._h[a:b])
                gemm(h, self.w_down[e], outb[a:b])
        return self.ep.combine(t, out)

    __call__ = forward

    def reference(self, x: torch.Tensor, all_gate=None, all_up=None, all_down=None) -> torch.Tensor:
        """fp32 PyTorch result for a world of one (all experts local)."""
        xf = x.float()
        probs = torch.softmax((x.float() @ self.w_router.float().t()).to(torch.bfloat16).float(), dim=-1)
        w, idx = torch.topk(probs, self.topk, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        y = torch.zeros_like(xf)
        for e in range(self.experts):
            tok, k = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            xe = xf[tok]
            h = torch.nn.functional.silu(xe @ self.w_gate[e].float().t()) * (xe @ self.w_up[e].float().t())
            o = (h.to(torch.bfloat16).float() @ self.w_down[e].float().t()).to(torch.bfloat16).float()
            y.index_add_(0, tok, o * w[tok, k].unsqueeze(-1))
        return y
