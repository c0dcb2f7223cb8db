"""One rank of the fused tensor-parallel correctness run (launched by test_gpu_tp.py)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from purlin_b200.models.tp_mlp import TensorParallelMLP  # noqa: E402
from purlin_b200.parallel.tensor_parallel import TensorParallelContext  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    T, H, I = int(os.environ.get("TP_TOKENS", 1024 * world // 2)), 1024, 512 * world
    T = max(T // (128 * world), 1) * 128 * world
    tp = TensorParallelContext(dist.group.WORLD, dev, max_tokens=T, k_ag=H, n_rs=H, timeout_ms=5000)
    fails = []
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    for it in range(3):   # three calls: both buffer parities and flag growth
        # ---- all-gather -> GEMM ----
        x_local = torch.randn(T // world, H, generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn(768, H, generator=g, device=dev) * 0.05).to(torch.bfloat16)
        out = tp.ag_gemm(x_local, w)
        tp.check()
        xs = [torch.empty_like(x_local) for _ in range(world)]
        dist.all_gather(xs, x_local)
        ref = torch.cat(xs).float() @ w.float().t()
        err = (out.float() - ref).abs().max().item()
        if err > 2e-2 * ref.abs().max().item() + 1e-3:
            fails.append(f"ag_gemm it{it} err {err}")
        # ---- GEMM -> reduce-scatter ----
        a = torch.randn(T, 256, generator=g, device=dev).to(torch.bfloat16)
        w2 = (torch.randn(H, 256, generator=g, device=dev) * 0.05).to(torch.bfloat16)
        y = tp.gemm_rs(a, w2)
        tp.check()
        part = (a.float() @ w2.float().t())
        full = part.clone()
        dist.all_reduce(full)
        ref2 = full[rank * (T // world):(rank + 1) * (T // world)]
        err2 = (y.float() - ref2).abs().max().item()
        if err2 > 3e-2 * ref2.abs().max().item() + 1e-3:
            fails.append(f"gemm_rs it{it} err {err2}")
    # ---- the MLP block ----
    mlp = TensorParallelMLP(hidden=H, intermediate=I, tokens=T, tp=tp)
    x_local = torch.randn(T // world, H, generator=g, device=dev).to(torch.bfloat16)
    for it in range(2):
        y = mlp(x_local)
        tp.check()
    xs = [torch.empty_like(x_local) for _ in range(world)]
    dist.all_gather(xs, x_local)
    part = mlp.reference(torch.cat(xs))
    dist.all_reduce(part)
    ref = part[rank * (T // world):(rank + 1) * (T // world)]
    err = (y.float() - ref).abs().max().item()
    if err > 3e-2 * ref.abs().max().item() + 1e-3:
        fails.append(f"mlp err {err} vs max {ref.abs().max().item()}")
    ok = torch.tensor([0 if fails else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in fails:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print(f"tp worker world {world} tokens {T}: all ranks ok: {bool(ok.item())}", flush=True)
    tp.close()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
