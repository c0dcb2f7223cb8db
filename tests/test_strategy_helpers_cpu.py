"""Bucket and shard book-keeping of the data-parallel helpers, on the CPU with recording stand-ins for the symmetric
tensors and their collectives (the GPU run of the same helpers is tests/parallel_worker.py)."""
import types

import pytest
import torch

from purlin_b200.parallel import data_parallel as dp


class FakeSymm:
    def __init__(self, shape, dtype):
        self.tensor = torch.zeros(shape, dtype=dtype)

    def status(self):
        return 0


@pytest.fixture
def fakes(monkeypatch):
    calls = []
    monkeypatch.setattr(dp, "symm_empty", lambda shape, dtype, handle: FakeSymm(shape, dtype))
    monkeypatch.setattr(dp, "all_reduce_symm", lambda st, op, mode: calls.append(("ar", st)) or st.tensor.mul_(2.0))   # "sum over two equal ranks"
    monkeypatch.setattr(dp, "all_gather_symm", lambda st: calls.append(("ag", st)))

    def rs(st, out, op, mode):
        calls.append(("rs", st))
        n = out.numel()
        out.copy_(st.tensor[n:2 * n] * 2.0)     # rank 1's slice, two equal ranks
    monkeypatch.setattr(dp, "reduce_scatter_symm", rs)
    return calls


def handle(world=2, rank=1):
    return types.SimpleNamespace(world=world, rank=rank, device=torch.device("cpu"), group=None)


def test_gradient_buckets_layout_and_reduce(fakes):
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(30, 50), torch.nn.Linear(50, 7))     # 1500 + 50 + 350 + 7 parameters
    b = dp.GradientBuckets(model.parameters(), handle(), bucket_bytes=4096)
    assert len(b.buckets) >= 2                                   # 6 KB of weights cannot share one 4 KB bucket
    for st in b.buckets:
        assert (st.tensor.numel() * 4) % (32 * 2) == 0           # a whole number of 32-byte slices per rank
    for p in model.parameters():
        owner = [st for st in b.buckets if st.tensor.data_ptr() <= p.grad.data_ptr() < st.tensor.data_ptr() + st.tensor.numel() * 4]
        assert len(owner) == 1 and (p.grad.data_ptr() - owner[0].tensor.data_ptr()) % 32 == 0
        assert p.grad.shape == p.shape
    model(torch.randn(4, 30)).sum().backward()
    local = [p.grad.clone() for p in model.parameters()]
    assert any(st.tensor.abs().sum() > 0 for st in b.buckets)    # autograd wrote straight into the buckets
    b.reduce(average=True)
    assert [c[0] for c in fakes] == ["ar"] * len(b.buckets)
    for p, g in zip(model.parameters(), local):
        assert torch.allclose(p.grad, g)                         # (g + g) / 2
    b.zero()
    assert all(float(p.grad.abs().sum()) == 0.0 for p in model.parameters())
    assert b.status() == 0


def test_gradient_buckets_need_a_trainable_parameter(fakes):
    p = torch.nn.Parameter(torch.zeros(3), requires_grad=False)
    with pytest.raises(ValueError):
        dp.GradientBuckets([p], handle())


def test_sharded_flat_parameter(fakes):
    sh = dp.ShardedFlatParameter(1003, torch.float32, handle(world=2, rank=1))
    assert sh.slice_elems % 8 == 0 and sh.slice_elems * 2 >= 1003
    assert sh.shard.data_ptr() == sh.full.tensor.data_ptr() + sh.slice_elems * 4
    sh.shard.fill_(3.0)
    full = sh.gather()
    assert full.numel() == 1003 and [c[0] for c in fakes] == ["ag"]
    assert float(sh.full.tensor[sh.slice_elems]) == 3.0
    sh.grad_full.tensor.copy_(torch.arange(sh.slice_elems * 2, dtype=torch.float32))
    g = sh.reduce_scatter_grad(average=True)
    assert torch.equal(g, torch.arange(sh.slice_elems, 2 * sh.slice_elems, dtype=torch.float32))   # (x + x) / 2
    assert fakes[-1][0] == "rs" and sh.status() == 0
