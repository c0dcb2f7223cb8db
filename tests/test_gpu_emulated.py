"""Every collective and protocol variant on ONE GPU: virtual ranks are rows of a cooperative grid.

Mirrors the reference's multi-GPU correctness binaries (csrc/tests/{ar,ag,agv,rs,rsv,a2a,a2av}.cu: seeded
inputs, exact comparison; integers in [-2, 2] so every summation order is exact) and its robustness cases
(csrc/tests/varlen_empty.cu: empty partitions, idle ranks, back-to-back calls reusing one context).
"""
import pytest
import torch

from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, ELEM, TORCH_DT, expected, in_out_bytes, ints, policy

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def worlds():
    from purlin_b200.utils.emulation import EmulatedWorld
    cache = {}

    def get(world, staging=1 << 20):
        key = (world, staging)
        if key not in cache:
            cache[key] = EmulatedWorld(world, staging)
        return cache[key]
    yield get
    for w in cache.values():
        w.close()


def run_case(ew, coll, nbytes=0, sizes=None, dtype=0, op=0, mode=0, pol=None, seed=0, reps=2):
    world = ew.world
    e = ELEM[dtype]
    if pol is not None and world >= 8:
        # eight virtual ranks share one GPU's 148 SMs, one CTA per SM: keep each rank's grid within 18 CTAs
        pol.consumeBlocks = min(pol.consumeBlocks, 2) if coll in (AR, RS, RSV) else min(pol.consumeBlocks, 8)
        pol.gatherBlocks = min(pol.gatherBlocks, 7)
        pol.localBlocks = 1
        pol.lrBlocks = min(pol.lrBlocks, 16)
    for rep in range(reps):   # consecutive calls alternate staging halves and grow the flag values
        ins, outs = [], []
        for r in range(world):
            ib, ob = in_out_bytes(coll, world, r, nbytes, sizes)
            lo, hi = (1, 2) if op == 1 else (-2, 2)
            ins.append(ints(ib // e, dtype, seed * 1000 + rep * 100 + r, lo, hi).cuda())
            outs.append(torch.full((ob // e,), 7.0, device="cuda").to(TORCH_DT[dtype]))
        ew.run(coll, ins, outs, nbytes=nbytes, sizes=sizes, dtype=dtype, op=op, mode=mode, policy=pol)
        torch.cuda.synchronize()
        for r in range(world):
            assert ew.status(r)[0] == 0, f"rank {r} status {ew.status(r)}"
        cpu_in = [t.cpu() for t in ins]
        for r in range(world):
            exp = expected(coll, world, r, cpu_in, nbytes, sizes, dtype, op)
            got = outs[r].cpu()
            assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8)), f"coll {coll} world {world} rank {r} rep {rep}"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kw", [dict(), dict(chunkBytes=32768), dict(regime=0)])
@pytest.mark.parametrize("coll", [AG, RS, A2A])
def test_fixed_collectives(worlds, coll, world, kw):
    for dtype in (0, 4):
        run_case(worlds(world), coll, nbytes=98304 + 64, dtype=dtype, pol=policy(**kw))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kw", [dict(arPath=0), dict(arPath=1), dict(arPath=1, chunkBytes=65536), dict(regime=0, arPath=0), dict(regime=0, arPath=1)])
def test_all_reduce_variants(worlds, world, kw):
    for dtype, op in ((0, 0), (4, 0), (1, 0), (0, 2), (4, 1)):
        run_case(worlds(world), AR, nbytes=world * 32 * 257, dtype=dtype, op=op, pol=policy(**kw))


@pytest.mark.parametrize("dtype", [2, 3])
def test_all_reduce_fp8(worlds, dtype):
    for kw in (dict(arPath=1), dict(regime=0, arPath=0)):
        run_case(worlds(4), AR, nbytes=4 * 32 * 64, dtype=dtype, pol=policy(**kw))


@pytest.mark.parametrize("world", [2, 4])
def test_cyclic_staging(worlds, world):
    st = 256 << 10
    for coll, n in ((AG, 1 << 20), (RS, 1 << 19), (A2A, 1 << 19), (AR, 1 << 20)):
        run_case(worlds(world, st), coll, nbytes=n, dtype=4, pol=policy(chunkBytes=32768, arPath=0))


def _sizes(world, seed, scale=65536, zero_every=0):
    g = torch.Generator().manual_seed(seed)
    v = (torch.randint(0, scale // 32, (world,), generator=g) * 32).tolist()
    return [0 if zero_every and i % zero_every == 0 else x for i, x in enumerate(v)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_variable_length(worlds, world):
    for seed, kw in enumerate((dict(), dict(chunkBytes=8192), dict(regime=0))):
        sizes = _sizes(world, seed, scale=16384 if kw.get("regime") == 0 else 65536, zero_every=3 if seed == 1 else 0)
        for coll in (AGV, RSV):
            run_case(worlds(world), coll, sizes=sizes, dtype=0, pol=policy(**kw), seed=seed)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("threshold", [0, 4096, 1 << 20])
def test_all_to_all_v(worlds, world, threshold):
    for seed in range(2):
        mat = [_sizes(world, seed * 17 + r, scale=32768, zero_every=4 if seed else 0) for r in range(world)]
        run_case(worlds(world), A2AV, sizes=mat, dtype=0, pol=policy(perStreamThreshold=threshold, chunkBytes=8192), seed=seed)


def test_idle_ranks_and_context_reuse(worlds):
    ew = worlds(4)
    mat = [[0] * 4 for _ in range(4)]
    for r in range(4):
        mat[r][r] = 256
    run_case(ew, A2AV, sizes=mat, pol=policy(perStreamThreshold=128))
    run_case(ew, AGV, sizes=[0, 0, 64, 0], pol=policy())
    # one context serves different collectives and grid sizes back to back
    for coll, kw in ((AR, dict(arPath=1)), (AG, dict(regime=0)), (RS, dict(consumeBlocks=3)), (A2A, dict(putBlocks=6)), (AR, dict(regime=0, arPath=1))):
        run_case(ew, coll, nbytes=4 * 32 * 33, dtype=4, pol=policy(**kw), reps=3)
    assert ew.seq(0) == ew.seq(3) and ew.seq(0) > 10


def test_default_policies(worlds):
    # no forced policy: the built-in codesign table picks the band for each size
    ew = worlds(4)
    for n in (4096, 262144):
        for coll in (AR, AG, RS, A2A):
            run_case(ew, coll, nbytes=n, dtype=0, pol=None, reps=1)


def test_absent_rank_times_out_and_context_recovers():
    # A rank that never launches: the others' bounded waits give up, the host reads a status, and after
    # clearing it the same contexts run a correct collective. Nothing traps, faults or spins forever.
    from purlin_b200.utils.emulation import EmulatedWorld
    ew = EmulatedWorld(4, 1 << 20, timeout_ms=100)
    ins = [ints(4096, 4, r).cuda() for r in range(4)]
    outs = [torch.zeros(4096, device="cuda") for r in range(4)]
    ew.run(AR, ins, outs, nbytes=16384, dtype=4, policy=policy(arPath=1), absent=2)
    torch.cuda.synchronize()
    st = [ew.status(r) for r in range(4)]
    assert all(st[r][0] in (1, 2, 3) for r in (0, 1, 3))
    assert st[2][0] == 0
    ew.close()
    ew = EmulatedWorld(4, 1 << 20, timeout_ms=2000)
    run_case(ew, AR, nbytes=16384, dtype=4, pol=policy(arPath=1))
    ew.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("depth", [2, 5, 13])
def test_bulk_async_engine(worlds, world, depth):
    # the copy roles stream through the cp.async.bulk ring: uneven tails, chunk boundaries inside and across tiles,
    # CTAs with no bytes in a chunk, cyclic slots, composed all-reduce (stage and gather on the ring, reduce in registers)
    for coll, n, kw in ((AG, 98304 + 64, dict()), (AG, 200000 // 32 * 32, dict(chunkBytes=32768)), (A2A, 65536 + 32, dict(chunkBytes=16384)),
                        (RS, 65536, dict(chunkBytes=8192)), (AR, world * 32 * 771, dict(arPath=1)),
                        (AR, world * 32 * 771, dict(arPath=1, chunkBytes=world * 4096)), (AR, 1 << 17, dict(arPath=0, chunkBytes=16384))):
        run_case(worlds(world), coll, nbytes=n, dtype=4, pol=policy(stageDepth=depth, **kw))
    sizes = _sizes(world, 5, scale=131072, zero_every=3)
    for coll in (AGV, RSV):
        run_case(worlds(world), coll, sizes=sizes, dtype=0, pol=policy(stageDepth=depth, chunkBytes=16384), seed=5)
    mat = [_sizes(world, 40 + r, scale=65536, zero_every=4) for r in range(world)]
    run_case(worlds(world), A2AV, sizes=mat, dtype=0, pol=policy(stageDepth=depth, perStreamThreshold=4096, chunkBytes=16384), seed=6)


@pytest.mark.parametrize("world", [2, 4])
def test_bulk_async_engine_cyclic(worlds, world):
    st = 256 << 10
    for coll, n in ((AG, 1 << 20), (RS, 1 << 19), (A2A, 1 << 19), (AR, 1 << 20)):
        run_case(worlds(world, st), coll, nbytes=n, dtype=4, pol=policy(chunkBytes=32768, arPath=0, stageDepth=6))


def test_device_side_trace(monkeypatch):
    """PURLIN_TRACE=1: every call leaves its device timestamps, logical bytes and kind in the context's ring."""
    from purlin_b200.utils.emulation import EmulatedWorld
    quiet = EmulatedWorld(2, 1 << 20)
    assert quiet.trace(0) is None                       # off unless asked for
    quiet.close()
    monkeypatch.setenv("PURLIN_TRACE", "1")
    ew = EmulatedWorld(2, 1 << 20)
    try:
        sizes = [4096, 65536, 4096 * 3]
        for n in sizes:
            run_case(ew, AG, nbytes=n, dtype=0, reps=1)
        run_case(ew, AR, nbytes=2 * 32 * 100, dtype=4, reps=1)
        for r in range(2):
            rec = ew.trace(r)
            assert [x["call"] for x in rec] == [0, 1, 2, 3]
            assert [x["collective"] for x in rec] == ["all_gather"] * 3 + ["all_reduce"]
            assert [x["bytes"] for x in rec[:3]] == sizes            # all-gather: bytes per rank
            assert all(x["end_ns"] >= x["start_ns"] > 0 and x["us"] < 1e6 for x in rec)
            assert all(b["start_ns"] >= a["start_ns"] for a, b in zip(rec, rec[1:]))
    finally:
        ew.close()
