"""Data-parallel, sharded-parameter and sequence-parallel helpers in one small script.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node <gpus> --master-addr 127.0.0.1 examples/strategies.py
  python examples/strategies.py --cpu        # two gloo processes on the CPU (gloo stand-ins for the symmetric tensors)

The reference ships the collectives these strategies are built from and no strategy code; here gradient buckets and
parameter shards live in symmetric memory, so their collectives run in place (purlin_b200/parallel/data_parallel.py),
and the Ulysses / gather / ring exchanges are thin wrappers over all_to_all(_v) and all_gather (sequence_parallel.py).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import purlin_b200 as purlin  # noqa: E402
from purlin_b200.parallel import data_parallel as dp  # noqa: E402
from purlin_b200.parallel import sequence_parallel as sp  # noqa: E402


def run(rank: int, world: int, cpu: bool):
    if cpu:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        device, stream = torch.device("cpu"), 0
    else:
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=device)
        stream = torch.cuda.current_stream().cuda_stream
    h = purlin.initialize(dist.group.WORLD, device, 100, stream, staging_size=16 << 20)

    # 1. DDP-style: gradients are views into symmetric buckets; one in-place all-reduce per bucket
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).to(device)
    buckets = dp.GradientBuckets(model.parameters(), h, bucket_bytes=32 << 10)
    g = torch.Generator(device=device).manual_seed(rank)
    model(torch.randn(16, 64, generator=g, device=device)).square().mean().backward()
    buckets.reduce(average=True)
    norm = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in model.parameters()))

    # 2. ZeRO-3-style: a flat parameter of `world` slices; gather in place, reduce-scatter the gradient
    shard = dp.ShardedFlatParameter(10_000, torch.float32, h)
    shard.shard.fill_(float(rank))
    full = shard.gather()
    shard.grad_full.tensor.fill_(1.0)
    grad = shard.reduce_scatter_grad(average=False)

    # 3. Ulysses: [S / W, H, D] <-> [S, H / W, D], and one ring step
    x = torch.randn(8, 4 * world, 16, device=device).to(torch.bfloat16 if not cpu else torch.float32)
    by_heads = sp.seq_to_heads(x, h)
    back = sp.heads_to_seq(by_heads, h)
    neighbour = sp.ring_shift(x, h)
    if not cpu:
        purlin.check(h)
    if rank == 0:
        print(f"{world} ranks: {len(buckets.buckets)} gradient buckets, averaged gradient norm {float(norm):.4f}")
        print(f"gathered parameter: {full.numel()} elements, slice means {[float(full[i * shard.slice_elems]) for i in range(world)]}")
        print(f"reduce-scattered gradient: {grad.numel()} elements, every entry {float(grad[0])} (= world)")
        print(f"Ulysses {tuple(x.shape)} -> {tuple(by_heads.shape)} -> {tuple(back.shape)}, round trip exact: {bool(torch.equal(back, x))}; "
              f"ring step received {tuple(neighbour.shape)}")
    del buckets, shard
    purlin.finalize(h, stream)
    dist.destroy_process_group()


def _cpu_child(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    run(rank, world, cpu=True)


if __name__ == "__main__":
    if "--cpu" in sys.argv:
        import socket
        import torch.multiprocessing as mp
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        mp.spawn(_cpu_child, args=(2, port), nprocs=2, join=True)
    else:
        run(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), cpu=False)
