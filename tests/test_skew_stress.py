"""Skewed, sparse and hot-ring variable-length traffic through the CPU interpreter (and, on a GPU, the emulated ranks).

Counterpart of csrc/tests/{agvskew,rsvskew,a2avskew}.cu in the reference: integer-only seeded inputs, skew of
0/25/50 % of the payload moved onto one heavy rank, sparse mode (k ranks exchange 64 KiB, the rest nothing),
hot-ring mode (90 % of every rank's bytes go to the next rank), Zipf splits for every supported exponent.
The plans are the ones the GPU kernel executes; the interpreter walks them step by step on the CPU.
"""
import pytest
import torch

from helpers import AGV, RSV, A2AV, ELEM, TORCH_DT, expected, in_out_bytes, ints, policy, sim
from purlin_b200.utils import split_policy as sp


def _check(coll, world, sizes, pol=None, staging=1 << 20, dtype=4):
    status, outs, exp = sim(coll, world, sizes=sizes, dtype=dtype, staging=staging, policy=pol)
    assert status[0] == 0, f"status {status}"
    for r in range(world):
        assert torch.equal(outs[r].view(torch.uint8), exp[r].view(torch.uint8)), f"coll {coll} world {world} rank {r} sizes {sizes}"


def _matrix_from_rows(world, row_of):
    return [row_of(r) for r in range(world)]


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("percent", [0, 25, 50])
@pytest.mark.parametrize("coll", [AGV, RSV])
def test_skewed_lists(coll, world, percent):
    sizes = sp.skew_splits(world * (48 << 10), world, percent, seed=11 + percent)
    assert sum(sizes) == world * (48 << 10)
    for pol in (None, policy(weighted=1, chunkBytes=16384), policy(weighted=0)):
        _check(coll, world, sizes, pol)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("percent", [0, 25, 50])
def test_skewed_all_to_all_v(world, percent):
    # every sender skews its own row with its own seed: columns (what a rank receives) are skewed too
    mat = _matrix_from_rows(world, lambda r: sp.skew_splits(world * (16 << 10), world, percent, seed=100 * percent + r))
    _check(A2AV, world, mat)
    _check(A2AV, world, mat, policy(perStreamThreshold=8192, chunkBytes=16384, putBlocks=max(4, world), consumeBlocks=2 * world))


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("active", [1, 2, 3])
def test_sparse_all_to_all_v(world, active):
    mat = sp.sparse_matrix(world, active, 64 << 10, seed=5)
    assert sum(map(sum, mat)) > 0
    _check(A2AV, world, mat)
    _check(A2AV, world, mat, policy(perStreamThreshold=4096, chunkBytes=32768, putBlocks=max(4, world), consumeBlocks=2 * world))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_hot_ring_all_to_all_v(world):
    mat = sp.hot_ring_matrix(world, 128 << 10, 90)
    for r in range(world):
        assert mat[r][(r + 1) % world] >= 0.85 * sum(mat[r])
    _check(A2AV, world, mat)
    # a staging window smaller than the hot stream: the hot stream runs cyclic while the cold ones stay packets
    _check(A2AV, world, mat, policy(perStreamThreshold=2048, chunkBytes=16384, putBlocks=max(4, world), consumeBlocks=2 * world), staging=256 << 10)


@pytest.mark.parametrize("eighths", [0, 1, 2, 4, 8])
def test_zipf_lists_every_exponent(eighths):
    world = 8
    sizes = sp.zipf_splits(world * (32 << 10), world, eighths)
    _check(AGV, world, sizes)
    _check(RSV, world, sizes, dtype=0)


def test_self_only_and_single_sender():
    world = 4
    diag = [[(8 << 10) if r == q else 0 for q in range(world)] for r in range(world)]
    _check(A2AV, world, diag)                       # every rank talks only to itself
    one = [[(4 << 10) * (q + 1) if r == 2 else 0 for q in range(world)] for r in range(world)]
    _check(A2AV, world, one)                        # one sender, everyone else idle
    _check(AGV, world, [0, 0, 96 << 10, 0])         # one contributor
    _check(RSV, world, [0, 64 << 10, 0, 32])        # two owners, one of them tiny


# ---- the same traffic on a GPU: virtual ranks as rows of one cooperative grid ----
@pytest.fixture(scope="module")
def emulated():
    from purlin_b200.utils.emulation import EmulatedWorld
    cache = {}

    def get(world):
        if world not in cache:
            cache[world] = EmulatedWorld(world, 1 << 20)
        return cache[world]
    yield get
    for w in cache.values():
        w.close()


def _run_gpu(ew, coll, sizes, pol=None, dtype=0):
    world, e = ew.world, ELEM[dtype]
    for rep in range(2):
        ins, outs = [], []
        for r in range(world):
            ib, ob = in_out_bytes(coll, world, r, 0, sizes)
            ins.append(ints(ib // e, dtype, 7000 + rep * 100 + r).cuda())
            outs.append(torch.full((ob // e,), 7.0, device="cuda").to(TORCH_DT[dtype]))
        ew.run(coll, ins, outs, nbytes=0, sizes=sizes, dtype=dtype, op=0, mode=0, policy=pol)
        torch.cuda.synchronize()
        cpu_in = [t.cpu() for t in ins]
        for r in range(world):
            assert ew.status(r)[0] == 0, f"rank {r} status {ew.status(r)}"
            exp = expected(coll, world, r, cpu_in, 0, sizes, dtype, 0)
            assert torch.equal(outs[r].cpu().view(torch.uint8), exp.view(torch.uint8)), f"coll {coll} world {world} rank {r} rep {rep}"


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_gpu_skew_sparse_hot_ring(emulated, world):
    ew = emulated(world)
    for percent in (0, 25, 50):
        sizes = sp.skew_splits(world * (48 << 10), world, percent, seed=3 + percent)
        _run_gpu(ew, AGV, sizes)
        _run_gpu(ew, RSV, sizes)
    _run_gpu(ew, A2AV, sp.hot_ring_matrix(world, 128 << 10, 90))
    _run_gpu(ew, A2AV, sp.sparse_matrix(world, 1, 64 << 10, seed=5))
    _run_gpu(ew, A2AV, [[(8 << 10) if r == q else 0 for q in range(world)] for r in range(world)])
