"""Back-to-back calls with no barrier between them, under seeded random schedules, through the CPU interpreter.

The ordering invariant of the protocol (a rank can start call k+2, which reuses the staging half of call k, only after
every peer finished call k; variable-length forms add an arrival handshake because a rank with nothing to receive waits on
nothing) cannot be shown by running one call at a time. Here every rank moves on to its next call as soon as its own steps
are done and a random scheduler interleaves all ranks' agents one chunk at a time, so fast ranks really run ahead; every
output of every call must still be exact, and no schedule may end with nobody able to move. Counterpart of the
reference's back-to-back robustness runs (csrc/tests/varlen_empty.cu:199-223: 32 unsynchronised calls, data changing per
iteration, one context across collective kinds), which need GPUs; this needs none.
"""
import random

import pytest
import torch

from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, policy, sim_sequence


def _check(calls, world, **kw):
    status, outs, exp = sim_sequence(calls, world, **kw)
    assert status[0] == 0, f"status {status} for {calls}"
    for c in range(len(calls)):
        for r in range(world):
            assert torch.equal(outs[c][r].view(torch.uint8), exp[c][r].view(torch.uint8)), f"call {c} ({calls[c][0]}) rank {r} world {world} {kw}"


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
def test_same_collective_many_times(world, seed):
    n = 32 * world * 24
    for coll in (AR, AG, RS, A2A):
        _check([(coll, n, None)] * 6, world, seed=seed, dtype=0)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("seed", range(8))
def test_mixed_kinds_and_sizes(world, seed):
    rng = random.Random(1000 * world + seed)
    calls = []
    for _ in range(7):
        coll = rng.choice([AR, AG, RS, A2A, AGV, RSV, A2AV])
        if coll in (AGV, RSV):
            calls.append((coll, 0, [32 * rng.choice([0, 1, 9, 300]) for _ in range(world)]))
        elif coll == A2AV:
            calls.append((coll, 0, [[32 * rng.choice([0, 0, 2, 40, 500]) for _ in range(world)] for _ in range(world)]))
        else:
            calls.append((coll, 32 * world * rng.choice([1, 5, 64, 700]), None))
    _check(calls, world, seed=seed, dtype=4)


@pytest.mark.parametrize("kw", [dict(chunkBytes=4096), dict(regime=0), dict(regime=0, arPath=0), dict(arPath=0, chunkBytes=8192),
                                dict(chunkBytes=4096, perStreamThreshold=2048)])
@pytest.mark.parametrize("seed", [11, 12, 13])
def test_forced_protocols_back_to_back(kw, seed):
    world = 4
    n = 32 * world * 96
    calls = [(AR, n, None), (AG, n // world, None), (AR, n, None), (RS, n // world, None), (A2A, n // world, None), (AR, n, None)]
    _check(calls, world, seed=seed, dtype=0, policy=policy(**kw))


@pytest.mark.parametrize("seed", [21, 22, 23, 24])
def test_cyclic_windows_back_to_back(seed):
    # payloads larger than their staging windows: slots are reused inside a call as well as across calls
    world, staging = 2, 256 << 10
    calls = [(AG, staging // 2 + 4096, None), (A2A, staging // 2, None), (AG, staging // 2 + 4096, None), (RS, staging // 4, None)]
    _check(calls, world, seed=seed, dtype=4, staging=staging, policy=policy(chunkBytes=32768, putBlocks=4, consumeBlocks=4))


@pytest.mark.parametrize("seed", [31, 32, 33, 34, 35, 36])
def test_idle_ranks_cannot_race_ahead(seed):
    # ranks with nothing to send or receive finish their own steps at once; only the arrival handshake holds them back
    world = 4
    lone = [[(1 << 14) if (r, q) == (0, 3) else 0 for q in range(world)] for r in range(world)]
    calls = [(A2AV, 0, lone), (AGV, 0, [0, 0, 1 << 13, 0]), (A2AV, 0, lone), (RSV, 0, [1 << 12, 0, 0, 0]), (A2AV, 0, lone), (AGV, 0, [0, 32, 0, 0])]
    _check(calls, world, seed=seed, dtype=4)


def test_coarse_and_fine_schedules_agree():
    world = 4
    calls = [(AR, 32 * world * 300, None), (AG, 32 * 300, None), (RS, 32 * 300, None)] * 2
    for quantum in (1, 3, 0):
        _check(calls, world, seed=5, dtype=0, quantum=quantum, policy=policy(chunkBytes=8192))


@pytest.mark.parametrize("kw", [dict(arPath=1, memType=1), dict(arPath=1, memType=1, chunkBytes=8192), dict(regime=0, arPath=0, lrMulticast=1),
                                dict(regime=0, arPath=1, lrMulticast=1)])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_switch_variants_back_to_back(kw, world):
    """The NVLS plans (in-switch reduction, results broadcast into every rank's staging or packet slots, gathered from the
    rank's own memory) under the same overlapped schedules: the interpreter models multimem.ld_reduce as a read of every
    rank's staging and multimem.st as a write to every rank's."""
    n = 32 * world * 48
    calls = [(AR, n, None), (AR, n, None), (AG, n // world, None), (AR, n, None), (RS, n // world, None), (AR, n, None)]
    for seed in (41, 42, 43):
        _check(calls, world, seed=seed, dtype=0, policy=policy(**kw), multicast=True)


@pytest.mark.parametrize("kw", [dict(), dict(arPath=0), dict(regime=0, arPath=0), dict(regime=0, arPath=1), dict(chunkBytes=4096)])
@pytest.mark.parametrize("world", [2, 4])
def test_in_place_all_reduce_back_to_back(kw, world):
    # source and destination are one buffer: a rank's result must not reach the buffer before every peer has taken its input
    n = 32 * world * 40
    calls = [(AR, n, None), (AG, n // world, None), (AR, n, None), (AR, n, None)]
    for seed in (51, 52, 53):
        _check(calls, world, seed=seed, dtype=4, policy=policy(**kw) if kw else None, in_place_ar=True)


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("kw", [dict(), dict(chunkBytes=16384), dict(chunkBytes=4096, putBlocks=8, consumeBlocks=8, gatherBlocks=8),
                                dict(arPath=1, memType=1, chunkBytes=8192)])
def test_all_reduce_larger_than_staging_runs_as_one_plan(kw, world):
    """Payloads beyond the staging half stream through per-rank windows under back-pressure: producers are released by the
    reducers' gather signals, the seam slots by the gatherers. Back to back with other calls, under random schedules."""
    staging = 256 << 10
    n = (staging * 3 + 32 * world * 17) // (32 * world) * (32 * world)
    small = 32 * world * 24
    calls = [(AR, n, None), (AR, small, None), (AR, n, None), (AG, small // world, None), (AR, n + 32 * world, None), (RS, small // world, None)]
    for seed in (61, 62, 63):
        _check(calls, world, seed=seed, dtype=0, staging=staging, policy=policy(**kw) if kw else None, multicast=bool(kw.get("memType")))
