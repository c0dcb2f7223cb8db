"""Point-to-point copy through the Atom over a peer pointer: push (remote stores) and pull (remote loads), with the
copy-engine baseline (cudaMemcpyAsync to the same peer pointer).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node=2 --master-addr 127.0.0.1 examples/p2p_push_pull.py

Counterpart of the reference's csrc/examples/p2p/{push,pull}.cu and csrc/examples/p2p/ce_p2p.cu: the device-side
`superCopy` is given a pointer into another GPU's symmetric memory; the direction decides whether NVLink carries
stores or load requests and responses. Rank 0 measures, rank 1 only lends its memory.
"""
import ctypes as C
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from purlin_b200 import _native  # noqa: E402
from purlin_b200.parallel.expert_parallel import _RawBuffer  # noqa: E402
from purlin_b200.parallel.symmetric import allocate_symmetric  # noqa: E402


def timed(fn, runs=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(runs):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / runs * 1e3   # us


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    lib = _native.cuda()
    nbytes = int(os.environ.get("P2P_BYTES", 256 << 20))
    owner, hdl, ptrs, _ = allocate_symmetric(nbytes, dev, dist.group.WORLD)
    peer = ptrs[(rank + 1) % world]
    local_buf = torch.ones(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    if rank == 0:
        print("direction,blocks,threads,bytes,us,GB/s")
        for blocks in (8, 16, 32, 64, 128):
            for name, dst, src in (("push", peer, local_buf.data_ptr()), ("pull", local_buf.data_ptr(), peer)):
                us = timed(lambda: _native.check(lib, lib.purlin_p2p_copy(dst, src, nbytes, blocks, 256, stream)))
                print(f"{name},{blocks},256,{nbytes},{us:.1f},{nbytes / us / 1e3:.1f}", flush=True)
        remote = torch.as_tensor(_RawBuffer(peer, (nbytes,), "|u1"), device=dev)
        us = timed(lambda: remote.copy_(local_buf, non_blocking=True))
        print(f"copy-engine-push,-,-,{nbytes},{us:.1f},{nbytes / us / 1e3:.1f}", flush=True)
        us = timed(lambda: local_buf.copy_(remote, non_blocking=True))
        print(f"copy-engine-pull,-,-,{nbytes},{us:.1f},{nbytes / us / 1e3:.1f}", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
