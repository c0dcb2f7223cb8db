"""The static bounds check every plan passes before it can be launched or interpreted.

Stands in for the sanitizer runs the reference does not have either (its correctness rests on static_asserts inside
the templates, e.g. csrc/include/purlin/snac.cuh:55-56): worlds 2-16, every collective, sizes around the boundaries
where the policy changes protocol (packets / resident / chunked / cyclic / segmented), forced policies, and plans
corrupted on purpose.
"""
import copy

import pytest

import purlin_b200 as P
from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, in_out_bytes, policy

STAGING = 1 << 20


def _sizes_for(coll, world, unit):
    if coll in (AGV, RSV):
        return [unit * ((q * 7) % 5) for q in range(world)], None
    if coll == A2AV:
        mat = [[unit * ((r * 3 + q * 5) % 4) for q in range(world)] for r in range(world)]
        return mat, None
    return None, None


@pytest.mark.parametrize("world", [2, 3, 4, 5, 8, 12, 16])
@pytest.mark.parametrize("coll", [AR, AG, RS, A2A])
def test_fixed_size_plans_pass_around_every_boundary(world, coll):
    unit = 32 * world
    # band boundaries of the built-in policy are powers of two between 1 KiB and the staging size; probe one unit either side
    probes = set()
    for shift in range(10, 23):
        for d in (-unit, 0, unit):
            n = ((1 << shift) + d) // unit * unit
            if n >= unit:
                probes.add(n)
    probes.update({unit, 2 * unit, STAGING // world // unit * unit, STAGING, STAGING + unit, 3 * STAGING})
    checked = 0
    for n in sorted(probes):
        for rank in {0, world - 1}:
            try:
                plan, _ = P.build_plan(coll, world, rank, n, dtype=P.DataType.BF16, staging_size=STAGING)
            except RuntimeError as e:
                assert "plan check" not in str(e), f"coll {coll} world {world} bytes {n}: {e}"
                continue   # a size the engine refuses outright (e.g. beyond what the staging buffer can stream)
            ib, ob = in_out_bytes(coll, world, rank, n, None)
            assert P.check_plan(plan, world, ib, ob, STAGING) == ""
            checked += 1
    assert checked > 20


@pytest.mark.parametrize("world", [2, 4, 7, 16])
@pytest.mark.parametrize("coll", [AGV, RSV, A2AV])
def test_variable_length_plans_pass(world, coll):
    for unit in (32, 4096, 96 << 10):
        sizes, _ = _sizes_for(coll, world, unit)
        for rank in range(world):
            if coll == A2AV:
                ins, outs = sizes[rank], [sizes[q][rank] for q in range(world)]
                plan, _ = P.build_plan(coll, world, rank, 0, sizes=ins, out_sizes=outs, staging_size=STAGING)
            else:
                plan, _ = P.build_plan(coll, world, rank, 0, sizes=sizes, staging_size=STAGING)
            ib, ob = in_out_bytes(coll, world, rank, 0, sizes)
            assert P.check_plan(plan, world, ib, ob, STAGING) == ""


@pytest.mark.parametrize("kw", [dict(), dict(chunkBytes=32768), dict(regime=0), dict(arPath=0), dict(regime=0, arPath=0),
                                dict(chunkBytes=65536, arPath=1)])
def test_forced_policies_pass(kw):
    for world in (2, 4, 8):
        for coll in (AR, AG, RS, A2A):
            n = 32 * world * 96
            plan, _ = P.build_plan(coll, world, 1, n, staging_size=STAGING, policy=policy(**kw))
            ib, ob = in_out_bytes(coll, world, 1, n, None)
            assert P.check_plan(plan, world, ib, ob, STAGING) == ""


def test_corrupted_plans_are_caught():
    world, n = 4, 32 * 4 * 512
    plan, _ = P.build_plan(AG, world, 0, n, staging_size=STAGING, policy=policy(chunkBytes=16384))
    ib, ob = in_out_bytes(AG, world, 0, n, None)
    assert P.check_plan(plan, world, ib, ob, STAGING) == ""
    assert "source" in P.check_plan(plan, world, ib - 32, ob, STAGING)            # the caller's buffer is shorter than claimed
    assert "destination" in P.check_plan(plan, world, ib, ob - 32, STAGING)

    def mutated(fn):
        p = copy.deepcopy(plan)
        fn(p)
        return P.check_plan(p, world, ib, ob, STAGING)

    stage = next(i for i in range(plan.nSteps) if plan.steps[i].role == 0)
    consume = next(i for i in range(plan.nSteps) if plan.steps[i].role == 2)
    assert "staging window" in mutated(lambda p: setattr(p.steps[stage], "dstOff", STAGING - 64))
    assert "staging window" in mutated(lambda p: setattr(p.steps[consume], "srcOff", STAGING))
    assert "CTA range" in mutated(lambda p: setattr(p.steps[consume], "blockBegin", p.blocks))
    assert "chunks" in mutated(lambda p: setattr(p.steps[stage], "chunks", p.steps[stage].chunks + 1))
    assert "aligned" in mutated(lambda p: setattr(p.steps[consume], "dstOff", p.steps[consume].dstOff + 8))
    assert "peer" in mutated(lambda p: setattr(p.steps[consume], "peer", world))
    assert "grid size" in mutated(lambda p: setattr(p, "blocks", 0))
    # packets: an all-reduce small enough for the latency regime
    small, _ = P.build_plan(AR, world, 0, 32 * world * 4, staging_size=STAGING, policy=policy(regime=0, arPath=1, lrBlocks=2))
    nb = 32 * world * 4
    assert P.check_plan(small, world, nb, nb, STAGING) == ""
    put = next(i for i in range(small.nSteps) if small.steps[i].role >= 5)
    bad = copy.deepcopy(small)
    bad.steps[put].dstOff = 8 << 20
    assert "packet slot" in P.check_plan(bad, world, nb, nb, STAGING)


def test_output_coverage_gaps_and_overlaps_are_caught():
    world, n = 4, 32 * 4 * 512
    plan, _ = P.build_plan(AG, world, 1, n, staging_size=STAGING, policy=policy())
    ib, ob = in_out_bytes(AG, world, 1, n, None)
    assert P.check_plan(plan, world, ib, ob, STAGING) == ""
    consumers = [i for i in range(plan.nSteps) if plan.steps[i].role == 2]
    assert len(consumers) == world - 1

    def mutated(fn):
        p = copy.deepcopy(plan)
        fn(p)
        return P.check_plan(p, world, ib, ob, STAGING)

    # two consumers write the same slice: an overlap, and the slice the second one left is a gap
    msg = mutated(lambda p: setattr(p.steps[consumers[1]], "dstOff", p.steps[consumers[0]].dstOff))
    assert "both write the output" in msg or "no step writes" in msg
    # a consumer that copies less than its slice leaves stale bytes behind
    def shorten(p):
        s = p.steps[consumers[0]]
        s.bytes -= 32
        s.chunkBytes = s.bytes
    assert "no step writes the output bytes" in mutated(shorten)
    # dropping the self copy leaves the rank's own slice unwritten
    local = next(i for i in range(plan.nSteps) if plan.steps[i].role == 1)
    assert "no step writes the output bytes" in mutated(lambda p: setattr(p.steps[local], "bytes", 0))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_table_driven_nvls_and_in_place_plans_pass(world):
    """What a GPU run sees and the interpreter does not: the measured table installed, a multicast alias on offer,
    in-place calls, both reduction modes, sizes up to 1 GiB. None may be refused by the plan check."""
    from purlin_b200 import tuning
    built = 0
    try:
        for use_table in (False, True):
            tuning.clear()
            if use_table:
                assert tuning.load_for("NVIDIA B200", world) is not None
            for coll in (AR, AG, RS, A2A):
                for size in (32 * world, 8 << 10, 512 << 10, 4 << 20, 32 << 20, 256 << 20, 1 << 30):
                    size = size // (32 * world) * (32 * world)
                    for mc in (False, True):
                        for in_place in (False, True):
                            for mode in (P.ReductionMode.NON_DETERMINISTIC, P.ReductionMode.DETERMINISTIC):
                                try:
                                    P.build_plan(coll, world, world - 1, size, multicast=mc, in_place=in_place, mode=mode)
                                    built += 1
                                except RuntimeError as e:
                                    assert "plan check" not in str(e), f"coll {coll} world {world} bytes {size} mc {mc} in-place {in_place}: {e}"
            for kw in (dict(arPath=1, memType=1), dict(arPath=1, memType=1, chunkBytes=1 << 20), dict(regime=0, arPath=0, lrMulticast=1),
                       dict(regime=0, arPath=1, lrMulticast=1)):
                for size in (32 * world * 8, 1 << 20, 16 << 20):
                    try:
                        P.build_plan(AR, world, 0, size, multicast=True, policy=policy(**kw))
                        built += 1
                    except RuntimeError as e:
                        assert "plan check" not in str(e), f"forced {kw} world {world} bytes {size}: {e}"
    finally:
        tuning.clear()
    assert built > 250   # in-place reduce-scatter and all-to-all are refused by design


def test_forced_tiny_chunks_are_raised_to_fit_the_arrival_counters():
    """A resident stream may not have more chunks than last-arrival counters (1024): a forced 4 KiB chunk over 16 MiB
    would give 4096, so the engine raises the chunk size instead."""
    from purlin_b200 import _native
    for coll in (P.Collective.ALL_GATHER, P.Collective.ALL_TO_ALL, P.Collective.REDUCE_SCATTER):
        _, chosen = P.build_plan(coll, 4, 1, 16 << 20)
        chosen.regime = 1
        chosen.chunkBytes = 4096
        plan, _ = P.build_plan(coll, 4, 1, 16 << 20, policy=chosen)
        for s in plan.active_steps():
            assert s.chunks <= 1024 or (s.flags & _native.FLAG_CYCLIC and s.slots <= 1024), (int(coll), s.role, s.chunks)


@pytest.mark.parametrize("coll", [P.Collective.REDUCE_SCATTER, P.Collective.REDUCE_SCATTER_V, P.Collective.ALL_TO_ALL, P.Collective.ALL_TO_ALL_V])
def test_in_place_reduce_scatter_and_all_to_all_are_refused(coll):
    sizes = [1024] * 4 if coll in (P.Collective.REDUCE_SCATTER_V, P.Collective.ALL_TO_ALL_V) else None
    outs = [1024] * 4 if coll == P.Collective.ALL_TO_ALL_V else None
    with pytest.raises(RuntimeError, match="in place"):
        P.build_plan(coll, 4, 2, 0 if sizes else 4096, sizes=sizes, out_sizes=outs, in_place=True)
    P.build_plan(coll, 4, 2, 0 if sizes else 4096, sizes=sizes, out_sizes=outs, in_place=False)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_cta_budget_is_honoured_by_every_collective(world):
    """With a budget of 64 CTAs (the reference's cap) every plan fits it, and the interpreter still gets exact results."""
    import torch
    from helpers import sim
    old = P.set_max_ctas(64)
    try:
        for coll in (AR, AG, RS, A2A):
            for size in (8 << 10, 512 << 10, 4 << 20, 64 << 20, 256 << 20):
                size = size // (32 * world) * (32 * world)
                for mc in (False, True):
                    plan, _ = P.build_plan(coll, world, 1, size, multicast=mc)
                    assert plan.blocks <= 64, (int(coll), world, size, mc, plan.blocks)
        for coll in (AR, AG, RS, A2A):
            status, outs, exp = sim(coll, world, 32 * world * 40, None, dtype=4)
            assert status[0] == 0
            for r in range(world):
                assert torch.equal(outs[r], exp[r])
    finally:
        P.set_max_ctas(old)
    plan, _ = P.build_plan(AR, world, 0, 64 << 20)
    assert P.set_max_ctas(0) == 0
