"""One MoE dispatch + combine on ONE GPU (a world of one: every expert is local); used for profiler captures:
python examples/moe_single.py [tokens hidden experts topk]"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from purlin_b200.parallel.expert_parallel import ExpertParallelContext  # noqa: E402

t, h, e, k = (int(v) for v in sys.argv[1:5]) if len(sys.argv) >= 5 else (4096, 7168, 256, 8)
ep = ExpertParallelContext(None, "cuda:0", max_tokens=t, hidden=h, experts=e, topk=k, capacity_factor=1.0)
g = torch.Generator(device="cuda:0").manual_seed(11)
logits = torch.randn(t, e, generator=g, device="cuda:0")
x = torch.randn(t, h, generator=g, device="cuda:0").to(torch.bfloat16)
y = torch.empty_like(x)
ep.route(logits)
for _ in range(3):
    ep.dispatch(x)
    ep.combine(t, y)
ep.check()
print("ok", float(y.float().abs().mean()))
ep.close()
