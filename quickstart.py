"""Smallest end-to-end use of the package: initialize, one all-reduce, print, finalize.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node <gpus> --master-addr 127.0.0.1 quickstart.py
  python quickstart.py --cpu       # two gloo processes on the CPU, no GPU needed

Counterpart of quickstart.py in the reference (an fp16 2x4 tensor all-reduced over the process group).
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import purlin_b200 as purlin  # noqa: E402


def run(rank: int, world: int, cpu: bool):
    if cpu:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        device = torch.device("cpu")
        stream = 0
    else:
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=device)
        stream = torch.cuda.current_stream().cuda_stream
    handle = purlin.initialize(dist.group.WORLD, device, 100, stream)
    x = torch.full((2, 16), float(rank + 1), dtype=torch.float16, device=device)
    out = torch.empty_like(x)
    purlin.all_reduce(x, out, handle, stream)
    purlin.check(handle)
    if rank == 0:
        print(f"all_reduce over {world} ranks -> {out[0, :4].tolist()} (expected {world * (world + 1) / 2})")
    purlin.finalize(handle, stream)
    dist.destroy_process_group()


def _cpu_child(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    run(rank, world, cpu=True)


if __name__ == "__main__":
    if "--cpu" in sys.argv:
        import socket
        import torch.multiprocessing as mp
        s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
        mp.spawn(_cpu_child, args=(2, port), nprocs=2, join=True)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        run(int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), cpu=False)
