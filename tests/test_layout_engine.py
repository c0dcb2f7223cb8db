"""Layout engine and SNAC plan: properties checked on the CPU, plus the CPU interpreter on every collective.

Models the reference's host-only and fake-provider tests (csrc/tests/variable_counts.cpp, csrc/tests/setup.cu)
and adds what it lacks: an execution of the protocol itself without a GPU.
"""
import ctypes as C

import pytest
import torch

import purlin_b200 as P
from purlin_b200 import _native
from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, sim, policy, in_out_bytes


def test_workspace_layout_matches_reference_format():
    for world in (2, 4, 8, 16):
        w = P.workspace_layout(world, 256 << 20)
        assert w["lr_offset"] == 2 * (256 << 20)
        assert w["signal_offset"] == 2 * ((256 << 20) + (8 << 20))
        assert w["gather_offset"] == w["signal_offset"] + 8 * world
        assert w["consumed_offset"] == w["signal_offset"] + 16 * world
        assert w["varlen_offset"] % 32 == 0 and w["varlen_offset"] >= w["signal_offset"] + 24 * world
        assert w["total_bytes"] == w["varlen_offset"] + 2 * world * 16
        assert w["packet_stride"] == ((8 << 20) // world) // 32 * 32


def test_topology_table():
    lib = _native.host()
    out = (C.c_int * 8)()
    # (in, out, op) -> perDest, perStream, variable, arrival, selfDirect, reduceWhole
    cases = {
        (0, 2, 0): (0, 0, 0, 0, 1, 0),   # all-gather
        (1, 3, 0): (0, 0, 1, 1, 1, 0),   # all-gather-v
        (2, 4, 0): (1, 0, 0, 0, 1, 0),   # all-to-all
        (3, 5, 0): (1, 1, 1, 1, 1, 0),   # all-to-all-v
        (2, 0, 1): (1, 0, 0, 0, 0, 0),   # reduce-scatter
        (3, 1, 1): (1, 0, 1, 1, 0, 0),   # reduce-scatter-v
        (0, 0, 1): (0, 0, 0, 0, 0, 1),   # all-reduce direct
    }
    for (i, o, op), want in cases.items():
        assert lib.purlin_topology(i, o, op, 0, out) == 0
        assert tuple(out[:6]) == want
    assert lib.purlin_topology(0, 4, 0, 0, out) != 0      # packed -> transposed is not a collective
    assert lib.purlin_topology(1, 2, 0, 0, out) != 0      # V and fixed layouts do not mix
    assert lib.purlin_topology(2, 4, 0, 1, out) == 0 and out[7] == 2   # cyclic per-destination: single drain
    assert lib.purlin_topology(0, 2, 0, 1, out) == 0 and out[7] == 1   # cyclic packed: all ranks drain


@pytest.mark.parametrize("world", [2, 3, 4, 8, 16])
@pytest.mark.parametrize("coll", [AR, AG, RS, A2A])
def test_plan_ctas_are_disjoint_and_cover_streams(world, coll):
    for nbytes in (32, 4096, 1 << 20, 48 << 20):
        plan, pol = P.build_plan(coll, world, world - 1, nbytes, staging_size=256 << 20)
        steps = plan.active_steps()
        assert plan.blocks <= 148
        if plan.regime == 1:
            spans = sorted((s.blockBegin, s.blockBegin + s.blockCount) for s in steps if s.role < 5)
            for a, b in zip(spans, spans[1:]):
                assert a[1] <= b[0], "throughput roles must own disjoint CTA ranges"
        for s in steps:
            assert s.bytes % 32 == 0 and s.chunkBytes % 32 == 0
            assert s.chunks == -(-s.bytes // s.chunkBytes)
            assert 1 <= s.slots <= max(s.chunks, 1)


def test_rejects_bad_arguments():
    with pytest.raises(RuntimeError):
        P.build_plan(AR, 2, 0, 33)                       # not a multiple of 32 bytes
    with pytest.raises(RuntimeError):
        P.build_plan(AR, 17, 0, 64)
    with pytest.raises(RuntimeError):
        P.build_plan(AGV, 2, 0, sizes=[64, 48])          # 48 is not a multiple of 32
    with pytest.raises(RuntimeError):
        P.build_plan(AR, 4, 1, 8 << 20, policy=policy(regime=0, arPath=0))   # too large for a packet slot


def test_compose_requires_matching_layouts():
    # the composed all-reduce is reduce-scatter followed by all-gather through the seam: the plan has one reduce
    # step that writes the seam and notifies, and one gather step per remote shard
    plan, _ = P.build_plan(AR, 4, 2, 1 << 20, policy=policy(arPath=1, consumeBlocks=4))
    roles = [s.role for s in plan.active_steps()]
    assert roles.count(_native.ROLE_STAGE) == 4 and roles.count(_native.ROLE_REDUCE) == 1 and roles.count(_native.ROLE_GATHER) == 3
    red = [s for s in plan.active_steps() if s.role == _native.ROLE_REDUCE][0]
    assert red.flags & _native.FLAG_TO_SEAM and red.flags & _native.FLAG_NOTIFY_GATHER and red.flags & _native.FLAG_TO_DST
    plan, _ = P.build_plan(AR, 4, 2, 1 << 20, policy=policy(arPath=0, consumeBlocks=4))
    roles = [s.role for s in plan.active_steps()]
    assert roles.count(_native.ROLE_GATHER) == 0 and roles.count(_native.ROLE_STAGE) == 1


def test_multimem_only_when_allowed():
    pol = policy(memType=1, arPath=1)
    plan, _ = P.build_plan(AR, 8, 0, 1 << 20, multicast=True, policy=pol)
    red = [s for s in plan.active_steps() if s.role == _native.ROLE_REDUCE][0]
    assert red.flags & _native.FLAG_MULTIMEM_LOAD and red.flags & _native.FLAG_MULTICAST_OUT
    assert all(s.flags & _native.FLAG_LOCAL_SOURCE for s in plan.active_steps() if s.role == _native.ROLE_GATHER)
    for kw in (dict(multicast=False), dict(multicast=True, mode=P.ReductionMode.DETERMINISTIC)):
        plan, _ = P.build_plan(AR, 8, 0, 1 << 20, policy=pol, **kw)
        red = [s for s in plan.active_steps() if s.role == _native.ROLE_REDUCE][0]
        assert not red.flags & _native.FLAG_MULTIMEM_LOAD


def test_weighted_apportionment_follows_stream_sizes():
    sizes = [32, 32, 1 << 20, 32]
    plan, _ = P.build_plan(AGV, 4, 0, sizes=sizes, policy=policy(consumeBlocks=12))
    cons = {s.peer: s.blockCount for s in plan.active_steps() if s.role == _native.ROLE_CONSUME}
    assert cons[2] > cons[1] and cons[2] > cons[3] and sum(cons.values()) == 12
    empty = [0, 64, 0, 64]
    plan, _ = P.build_plan(AGV, 4, 1, sizes=empty, policy=policy(consumeBlocks=6))
    assert {s.peer for s in plan.active_steps() if s.role == _native.ROLE_CONSUME} == {3}


LR = dict(regime=0)
CASES = [
    ("tr", dict()),
    ("tr_chunked", dict(chunkBytes=4096)),
    ("lr", LR),
]


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("name,kw", CASES)
@pytest.mark.parametrize("coll", [AG, RS, A2A])
def test_interpreter_fixed_collectives(coll, world, name, kw):
    for dtype in (4, 0):
        status, outs, exp = sim(coll, world, nbytes=16384 + 64, dtype=dtype, policy=policy(**kw))
        assert status[0] == 0
        for o, e in zip(outs, exp):
            assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("kw", [dict(arPath=0), dict(arPath=1), dict(arPath=1, chunkBytes=8192), dict(arPath=0, chunkBytes=4096),
                                dict(regime=0, arPath=0), dict(regime=0, arPath=1)])
def test_interpreter_all_reduce_variants(world, kw):
    for dtype, op in ((4, 0), (0, 0), (1, 2), (4, 1)):
        status, outs, exp = sim(AR, world, nbytes=world * 1024 * 3, dtype=dtype, op=op, policy=policy(**kw))
        assert status[0] == 0
        for o, e in zip(outs, exp):
            assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_interpreter_cyclic_streams(world):
    # staging of 256 KiB per half and payloads several times larger: slots are reused under back-pressure
    st = 256 << 10
    for coll, n in ((AG, 1 << 20), (RS, 1 << 18), (A2A, 1 << 18), (AR, 1 << 20)):
        kw = dict(chunkBytes=16384, arPath=0)
        status, outs, exp = sim(coll, world, nbytes=n, dtype=4, staging=st, policy=policy(**kw))
        assert status[0] == 0, (coll, status)
        plan, _ = P.build_plan(coll, world, 0, n, staging_size=st, policy=policy(**kw))
        assert any(s.flags & _native.FLAG_CYCLIC for s in plan.active_steps())
        for o, e in zip(outs, exp):
            assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))


def _rand_sizes(world, seed, scale=4096, zero_every=0):
    g = torch.Generator().manual_seed(seed)
    v = (torch.randint(0, scale // 32, (world,), generator=g) * 32).tolist()
    if zero_every:
        v = [0 if i % zero_every == 0 else x for i, x in enumerate(v)]
    return v


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("kw", [dict(), dict(chunkBytes=1024), dict(regime=0)])
def test_interpreter_variable_length(world, kw):
    for seed in range(3):
        sizes = _rand_sizes(world, seed, zero_every=3 if seed == 2 else 0)
        for coll in (AGV, RSV):
            status, outs, exp = sim(coll, world, sizes=sizes, dtype=4, policy=policy(**kw), seed=seed)
            assert status[0] == 0
            for o, e in zip(outs, exp):
                assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("threshold", [0, 1024, 1 << 20])
def test_interpreter_all_to_all_v_per_stream(world, threshold):
    # streams at most `threshold` long travel as packets, the rest through staging windows; some are empty
    for seed in range(3):
        mat = [_rand_sizes(world, seed * 31 + r, scale=8192, zero_every=4 if seed else 0) for r in range(world)]
        status, outs, exp = sim(A2AV, world, sizes=mat, dtype=4, policy=policy(perStreamThreshold=threshold, chunkBytes=2048), seed=seed)
        assert status[0] == 0
        for o, e in zip(outs, exp):
            assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))


def test_interpreter_idle_and_self_only_ranks():
    world = 4
    # fully idle ranks and self-only traffic (the cases of csrc/tests/varlen_empty.cu in the reference)
    mat = [[0] * world for _ in range(world)]
    for r in range(world):
        mat[r][r] = 256
    status, outs, exp = sim(A2AV, world, sizes=mat, policy=policy(perStreamThreshold=128))
    assert status[0] == 0
    for o, e in zip(outs, exp):
        assert torch.equal(o, e)
    status, outs, exp = sim(AGV, world, sizes=[0, 0, 0, 0], policy=policy())
    assert status[0] == 0


@pytest.mark.parametrize("coll", [AR, AG, RS, A2A, AGV])
def test_absent_rank_is_reported_not_hung(coll):
    # a rank that never joins: every wait that depends on it ends with a status instead of spinning forever
    kw = dict(sizes=[64, 64, 64, 64]) if coll == AGV else dict(nbytes=4096)
    status, _, _ = sim(coll, 4, policy=policy(), drop=2, **kw)
    assert status[0] in (1, 2, 3)
    status, _, _ = sim(coll, 4, policy=policy(regime=0), drop=1, **kw)
    assert status[0] in (1, 2, 3)


@pytest.mark.parametrize("world", [3, 5, 6, 7, 12, 16])
def test_borrowed_tuning_tables_give_sound_plans(world):
    """A world size without its own measured table borrows the nearest one; every plan built from it must still pass
    the interpreter bit for bit (policies that do not fit fall back to the built-in bands)."""
    from purlin_b200 import tuning
    tuning.clear()
    try:
        used = tuning.load_for("NVIDIA B200", world)
        assert used is not None and f"_w{world}." not in used.name
        for coll in (AR, AG, RS, A2A):
            for n in (32 * world, 32 * world * 40, 32 * world * 1031, (1 << 20) // (32 * world) * (32 * world)):
                status, outs, exp = sim(coll, world, nbytes=n, dtype=0, staging=4 << 20)
                assert status[0] == 0, f"coll {coll} world {world} bytes {n}: status {status}"
                for r in range(world):
                    assert torch.equal(outs[r].view(torch.uint8), exp[r].view(torch.uint8)), f"coll {coll} world {world} bytes {n} rank {r}"
    finally:
        tuning.clear()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_variable_length_forms_borrow_measured_bands(world):
    """With a measured table installed, AGV / RSV / A2AV take the CTA counts and chunk size of their fixed-size sibling's band
    (never its switch variant) and still run bit for bit through the interpreter, whole range of stream sizes."""
    from purlin_b200 import tuning
    tuning.clear()
    try:
        assert tuning.load_for("NVIDIA B200", world) is not None
        big = 3 << 20
        sizes = [big // 32 * 32 if q % 2 == 0 else (big // 3) // 32 * 32 for q in range(world)]
        _, fixed = P.build_plan(AG, world, 0, max(sizes), staging_size=64 << 20)
        _, borrowed = P.build_plan(AGV, world, 0, 0, sizes=sizes, staging_size=64 << 20)
        assert (borrowed.putBlocks, borrowed.consumeBlocks, borrowed.chunkBytes) == (fixed.putBlocks, fixed.consumeBlocks, fixed.chunkBytes)
        _, rs = P.build_plan(RSV, world, 0, 0, sizes=sizes, staging_size=64 << 20, multicast=True)
        assert rs.memType == 0                                    # the switch variant is not borrowed
        for scale in (1, 40, 3000):
            lst = [32 * scale * ((q * 5) % 4) for q in range(world)]
            mat = [[32 * scale * ((r + 2 * q) % 3) for q in range(world)] for r in range(world)]
            for coll, sz in ((AGV, lst), (RSV, lst), (A2AV, mat)):
                status, outs, exp = sim(coll, world, sizes=sz, dtype=0, staging=4 << 20)
                assert status[0] == 0, f"coll {coll} world {world} scale {scale}: {status}"
                for r in range(world):
                    assert torch.equal(outs[r].view(torch.uint8), exp[r].view(torch.uint8)), f"coll {coll} world {world} scale {scale} rank {r}"
    finally:
        tuning.clear()


@pytest.mark.parametrize("world", [2, 4, 8, 16])
def test_latency_plans_fetch_all_peers_in_one_step(world):
    # fixed-size forms: ONE get step for the packets of every peer (slices of equal size at q * bytes), so a rank polls its
    # peers at the same time; the variable-length forms keep one step per peer (their slices differ)
    for coll, nbytes in ((AG, 4096), (A2A, 4096), (AR, 4096 * world)):
        plan, _ = P.build_plan(coll, world, 1, nbytes, policy=policy(regime=0, arPath=1))
        gets = [s for s in plan.active_steps() if s.role == _native.ROLE_PACKET_GET]
        assert len(gets) == 1 and gets[0].peer == -1 and gets[0].seamOff == 1
        assert gets[0].bytes == 4096 and gets[0].dstOff == 0
    # ... and ONE put step where every peer gets its own slice (all-to-all, reduce-scatter, the scatter half of a two-shot all-reduce)
    for coll, nbytes in ((A2A, 4096), (RS, 4096), (AR, 4096 * world)):
        plan, _ = P.build_plan(coll, world, 1, nbytes, policy=policy(regime=0, arPath=1))
        puts = [s for s in plan.active_steps() if s.role == _native.ROLE_PACKET_PUT]
        assert len(puts) == 1 and puts[0].peer == -1 and puts[0].flags & _native.FLAG_SCATTER and puts[0].seamOff == 1
        assert puts[0].bytes == 4096 and puts[0].srcOff == 0
    puts = [s for s in P.build_plan(AG, world, 1, 4096, policy=policy(regime=0))[0].active_steps() if s.role == _native.ROLE_PACKET_PUT]
    assert len(puts) == 1 and not puts[0].flags & _native.FLAG_SCATTER          # the same words to everyone
    sizes = [64 * (q + 1) for q in range(world)]
    plan, _ = P.build_plan(AGV, world, 1, 0, sizes=sizes, policy=policy(regime=0))
    gets = [s for s in plan.active_steps() if s.role == _native.ROLE_PACKET_GET]
    assert len(gets) == world - 1 and all(s.peer >= 0 for s in gets)
    # the interpreter runs the fused step on every rank
    for coll in (AG, A2A, RS, AR):
        status, outs, exp = sim(coll, world, nbytes=2048 * world if coll == AR else 2048, dtype=4, policy=policy(regime=0, arPath=1))
        assert status[0] == 0
        for o, e in zip(outs, exp):
            assert torch.equal(o.view(torch.uint8), e.view(torch.uint8))
