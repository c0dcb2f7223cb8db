"""The host-fed step loop: inputs from pinned host memory, results back to the host, transfers overlapped with compute."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_feed_order_and_values():
    from purlin_b200.utils.feed import HostFeed
    n = 1 << 20
    feed = HostFeed((n,), torch.float32, "cuda:0", depth=2)
    batches = [torch.full((n,), float(i + 1)).pin_memory() for i in range(7)]
    seen = []

    def step(x):
        # enough work that the next copy really overlaps this step; the result depends on every element of the input
        y = x
        for _ in range(4):
            y = y * 1.0
        return y.sum(dtype=torch.float64).to(torch.float32) / n

    out = feed.run(iter(batches), step, on_result=lambda i, v: seen.append(i))
    assert out == [float(i + 1) for i in range(7)]          # every step saw its own input, results in step order
    assert seen == list(range(7))
    assert feed.h2d_bytes_per_step == n * 4 and feed.d2h_bytes_per_step == 4
    # a second run on the same feed (buffers and events are reused)
    out = feed.run(iter(batches[:3]), step)
    assert out == [1.0, 2.0, 3.0]


def test_host_feed_rejects_pageable_memory():
    from purlin_b200.utils.feed import HostFeed
    feed = HostFeed((16,), torch.float32, "cuda:0")
    with pytest.raises(ValueError):
        feed.run(iter([torch.zeros(16)]), lambda x: x.sum())


def test_mlp_run_host_batches_matches_forward():
    from purlin_b200.models.tp_mlp import TensorParallelMLP
    mlp = TensorParallelMLP(hidden=512, intermediate=1024, tokens=256, device="cuda:0")
    g = torch.Generator().manual_seed(5)
    hosts = [torch.randn(256, 512, generator=g).to(torch.bfloat16).pin_memory() for _ in range(4)]
    got = mlp.run_host_batches(iter(hosts))
    want = []
    for h in hosts:
        y = mlp.forward(h.cuda())
        want.append(float(torch.linalg.vector_norm(y, dtype=torch.float32)))
    assert got == pytest.approx(want, rel=1e-6)
