"""One tcgen05 GEMM launch at a small shape (used for profiler captures): python examples/gemm_single.py [M N K [swiglu]]"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from purlin_b200.ops.gemm import gemm, gemm_swiglu  # noqa: E402

m, n, k = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (4096, 4096, 4096)
a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
fused = len(sys.argv) >= 5 and sys.argv[4] == "swiglu"     # w then holds gate and up rows interleaved; the output has N / 2 columns
out = torch.empty(m, n // 2 if fused else n, device="cuda", dtype=torch.bfloat16)
for _ in range(4):
    gemm_swiglu(a, w, out) if fused else gemm(a, w, out)
torch.cuda.synchronize()
print("ok", float(out.float().abs().mean()))
