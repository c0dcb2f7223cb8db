"""One emulated multi-rank collective on ONE GPU (virtual ranks are rows of a cooperative grid); used for profiler
captures of the SNAC kernel:  python examples/emulated_collective.py [collective world MiB_per_rank]
collective: 0 all-reduce, 1 all-gather, 3 reduce-scatter, 5 all-to-all."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from purlin_b200 import _native  # noqa: E402
from purlin_b200.utils.emulation import EmulatedWorld  # noqa: E402

coll, world, mib = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (1, 4, 32)
n = mib << 20
ew = EmulatedWorld(world, staging_size=64 << 20)
in_b = n if coll in (0, 1) else n * world
out_b = n * world if coll in (1, 5) else n
srcs = [torch.full((in_b // 2,), float(r + 1), dtype=torch.bfloat16, device="cuda") for r in range(world)]
dsts = [torch.zeros(out_b // 2, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
per_rank = 148 // world
pol = _native.Policy.from_dict(dict(regime=1, threads=256, putBlocks=max(per_rank // 4, world), localBlocks=2, consumeBlocks=per_rank // 2,
                                    gatherBlocks=max(per_rank // 5, world - 1), lrBlocks=8, memType=0, mmDepth=4, unroll=8, stageDepth=0, arPath=1,
                                    lrMulticast=0, weighted=1, chunkBytes=4 << 20, perStreamThreshold=0))
for _ in range(3):
    ew.run(coll, srcs, dsts, nbytes=n, dtype=0, policy=pol)
torch.cuda.synchronize()
assert all(ew.status(r)[0] == 0 for r in range(world))
print("ok", float(dsts[0][:8].float().sum()))
ew.close()
