"""One rank of the multi-GPU run of the strategy helpers (data parallel, sharded parameters, sequence parallel)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import purlin_b200 as purlin  # noqa: E402
from purlin_b200.parallel import data_parallel as dp  # noqa: E402
from purlin_b200.parallel import sequence_parallel as sp  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    h = purlin.initialize(dist.group.WORLD, dev, 100, None, staging_size=8 << 20, timeout_ms=5000)
    failures = []

    # ---- gradient buckets: two steps of a tiny model, gradients averaged in place, compared with NCCL ----
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.GELU(), torch.nn.Linear(96, 40)).to(dev)
    buckets = dp.GradientBuckets(model.parameters(), h, bucket_bytes=16 << 10)     # small buckets: several of them
    if len(buckets.buckets) < 2:
        failures.append("expected more than one gradient bucket")
    for step in range(2):
        buckets.zero()
        g = torch.Generator(device=dev).manual_seed(100 * step + rank)
        x = torch.randn(32, 64, generator=g, device=dev)
        model(x).square().mean().backward()
        want = []
        for p in model.parameters():
            t = p.grad.detach().clone()
            dist.all_reduce(t)
            want.append(t / world)
        buckets.reduce(average=True, reduction_mode=purlin.ReductionMode.DETERMINISTIC)
        if buckets.status() != 0:
            failures.append("gradient buckets: device wait timed out")
        for p, t in zip(model.parameters(), want):
            if not torch.allclose(p.grad, t, rtol=1e-5, atol=1e-6):
                failures.append(f"gradient buckets step {step}: max diff {(p.grad - t).abs().max().item():.3e}")
                break

    # ---- sharded flat parameter: gather, then reduce-scatter of a gradient ----
    sh = dp.ShardedFlatParameter(1000 * world + 3, torch.float32, h)
    sh.shard.fill_(float(rank + 1))
    full = sh.gather()
    for q in range(world):
        part = sh.full.tensor[q * sh.slice_elems:(q + 1) * sh.slice_elems]
        if not torch.all(part == float(q + 1)).item():
            failures.append(f"sharded parameter: slice {q} after gather")
    if full.numel() != 1000 * world + 3:
        failures.append("sharded parameter: wrong gathered length")
    sh.grad_full.tensor.copy_(torch.arange(sh.slice_elems * world, device=dev, dtype=torch.float32) % 7 + rank)
    got = sh.reduce_scatter_grad(average=False)
    base = torch.arange(sh.slice_elems * world, device=dev, dtype=torch.float32)[rank * sh.slice_elems:(rank + 1) * sh.slice_elems] % 7
    if sh.status() != 0 or not torch.equal(got, base * world + sum(range(world))):
        failures.append("sharded parameter: reduce-scatter of the gradient")

    # ---- Ulysses exchange and its inverse, sequence gather, ring rotation ----
    s_local, heads, d = 24, 4 * world, 16
    g = torch.Generator().manual_seed(7)
    whole = torch.randn(s_local * world, heads, d, generator=g).to(torch.bfloat16)     # the same on every rank
    mine = whole[rank * s_local:(rank + 1) * s_local].to(dev)
    by_heads = sp.seq_to_heads(mine, h)
    hg = heads // world
    if not torch.equal(by_heads.cpu(), whole[:, rank * hg:(rank + 1) * hg]):
        failures.append("seq_to_heads")
    back = sp.heads_to_seq(by_heads, h)
    if not torch.equal(back.cpu(), whole[rank * s_local:(rank + 1) * s_local]):
        failures.append("heads_to_seq")
    if not torch.equal(sp.gather_sequence(mine, h).cpu(), whole):
        failures.append("gather_sequence")
    for step in (1, 2, world):
        shifted = sp.ring_shift(mine, h, step=step)
        src = (rank - step) % world
        if not torch.equal(shifted.cpu(), whole[src * s_local:(src + 1) * s_local]):
            failures.append(f"ring_shift step {step}")
    try:
        purlin.check(h)
    except TimeoutError as e:
        failures.append(str(e))
    del buckets, sh
    purlin.finalize(h)
    ok = torch.tensor([0 if failures else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in failures:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print(f"strategy helpers: all ranks ok: {bool(ok.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
