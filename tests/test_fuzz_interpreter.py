"""Seeded random sweep of (collective, world, sizes, element type, staging size, forced policy) through the CPU
interpreter: every accepted combination must complete and match the reference bit for bit; a refusal must come from
the argument checks, never from the plan bounds check. (Thousands of such cases were run while the engine was
written; this keeps a few hundred as a regression net.)"""
import random

import pytest
import torch

from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, policy, sim


def _case(rng, n):
    world = rng.choice([2, 3, 4, 5, 6, 7, 8, 12, 16])
    coll = rng.choice([AR, AG, AGV, RS, RSV, A2A, A2AV])
    dtype = rng.choice([0, 4, 1])
    staging = rng.choice([256 << 10, 512 << 10, 1 << 20])
    kw = {}
    if rng.random() < 0.7:
        kw = dict(regime=rng.choice([0, 1]), arPath=rng.choice([0, 1]), putBlocks=rng.choice([1, 2, 4, 8, 13]),
                  consumeBlocks=rng.choice([1, 3, 8, 16, 31]), gatherBlocks=rng.choice([1, 4, 8]), localBlocks=rng.choice([1, 2]),
                  lrBlocks=rng.choice([1, 2, 7]), chunkBytes=rng.choice([0, 0, 4096, 32768, 65536, 3200]),
                  perStreamThreshold=rng.choice([0, 2048, 16384]), weighted=rng.choice([0, 1]))
    sizes, nbytes = None, 0
    if coll in (AGV, RSV):
        sizes = [32 * rng.choice([0, 0, 1, 3, 17, 100, 1000, 5000]) for _ in range(world)]
    elif coll == A2AV:
        sizes = [[32 * rng.choice([0, 0, 0, 1, 5, 64, 700, 3000]) for _ in range(world)] for _ in range(world)]
    else:
        nbytes = 32 * rng.choice([1, 2, 3, 9, 64, 257, 1024, 4099, 20000]) * (world if coll == AR else 1)
    return dict(coll=coll, world=world, nbytes=nbytes, sizes=sizes, dtype=dtype, staging=staging, policy=policy(**kw) if kw else None, seed=n), kw


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_cases_match_the_reference(seed):
    rng = random.Random(seed)
    ran = 0
    for n in range(60):
        args, kw = _case(rng, n)
        try:
            status, outs, exp = sim(**args)
        except RuntimeError as e:
            assert "plan check" not in str(e), f"{args} {kw}: {e}"
            continue
        assert status[0] == 0, f"{args} {kw}: status {status}"
        for r, (o, x) in enumerate(zip(outs, exp)):
            assert torch.equal(o.view(torch.uint8), x.view(torch.uint8)), f"{args} {kw}: rank {r}"
        ran += 1
    assert ran >= 40
