"""Launcher of the collective sweep / tuner (see purlin_b200/utils/sweep.py for the options).

  python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 bench_collectives.py --min-bytes 8K --max-bytes 1G
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from purlin_b200.utils.sweep import main  # noqa: E402

if __name__ == "__main__":
    main()
