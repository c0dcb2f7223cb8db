"""Multi-GPU correctness: spawns one process per GPU and runs tests/distributed_worker.py on all of them.

Counterpart of tests/test_python_collectives_distributed.py in the reference (all 7 collectives, element types,
both reduction modes, exact equality), widened to every protocol band, CUDA-graph replay and empty partitions.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("provider", ["torch", "vmm", "ipc"])
def test_all_collectives_all_gpus(provider):
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ)
    env["PURLIN_PROVIDER"] = provider
    if provider != "torch":
        env["PURLIN_TEST_SUBSET"] = "1"   # the protocol bands were covered by the first pass; this one is about the memory
    env.setdefault("NCCL_NVLS_ENABLE", "0")   # NCCL only bootstraps here; keep its multicast objects out of the picture
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29581", os.path.join(here, "distributed_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    sys.stdout.write(res.stdout[-4000:])
    sys.stderr.write(res.stderr[-4000:])
    assert res.returncode == 0


def test_strategy_helpers_all_gpus():
    """Gradient buckets and sharded parameters on zero-copy symmetric tensors, Ulysses / gather / ring exchanges."""
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29583", os.path.join(here, "parallel_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(res.stdout[-4000:])
    sys.stderr.write(res.stderr[-4000:])
    assert res.returncode == 0
