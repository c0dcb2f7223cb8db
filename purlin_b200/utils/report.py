"""Turns the CSV rows of ``bench_collectives.py`` (or ``multi_gpu_bench``) into a comparison table.

    python -m purlin_b200.utils.report sweep.csv [--markdown]

The reference's harness prints one CSV row per size (csrc/support/purlin/benchmark/purlin_report.cuh:21-41) and leaves the
comparison to the reader; this reads those rows (lines that are not CSV data, such as launcher chatter and ``#`` comments,
are skipped), pairs every implementation with the NCCL row of the same collective and size, and prints time, bandwidth
and speed-up side by side.
"""
from __future__ import annotations

import csv
import sys
from collections import OrderedDict
from typing import Dict, Iterable, List, Tuple

LONG = {"ar": "AllReduce", "ag": "AllGather", "rs": "ReduceScatter", "a2a": "AllToAll", "agv": "AllGatherV", "rsv": "ReduceScatterV",
        "a2av": "AllToAllV"}


def _size(n: int) -> str:
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= (1 << shift) and n % (1 << shift) == 0:
            return f"{n >> shift} {unit}"
    return f"{n} B"


def parse(lines: Iterable[str]) -> "OrderedDict[Tuple[str, int], Dict[str, Tuple[float, float, float]]]":
    """(collective, bytes) -> {implementation: (microseconds, bus GB/s, error %)}; unknown lines are ignored."""
    table: "OrderedDict[Tuple[str, int], Dict[str, Tuple[float, float, float]]]" = OrderedDict()
    for row in csv.reader(lines):
        if len(row) < 9 or row[0].startswith("#") or row[0] == "collective":
            continue
        try:
            coll, impl, nbytes = row[0].strip(), row[1].strip(), int(row[3])
            us, bus, err = float(row[5]), float(row[7]), float(row[8])
        except ValueError:
            continue
        table.setdefault((coll, nbytes), {})[impl] = (us, bus, err)
    return table


def render(table, markdown: bool = False, baseline: str = "nccl") -> List[str]:
    impls: List[str] = []
    for per in table.values():
        for impl in per:
            if impl != baseline and impl not in impls:
                impls.append(impl)
    out: List[str] = []
    head = ["collective", "logical bytes"] + [f"{i} us (bus GB/s)" for i in impls] + [f"{baseline} us (bus GB/s)"] + [f"{i} speed-up" for i in impls]
    if markdown:
        out.append("| " + " | ".join(head) + " |")
        out.append("|" + "---|" * len(head))
    else:
        out.append("  ".join(head))
    for (coll, nbytes), per in table.items():
        base = per.get(baseline)
        cells = [LONG.get(coll, coll), _size(nbytes)]
        for i in impls:
            v = per.get(i)
            cells.append("-" if v is None else f"{v[0]:.1f} ({v[1]:.1f})" + ("" if v[2] == 0 else f" ERROR {v[2]:.0f}%"))
        cells.append("-" if base is None else f"{base[0]:.1f} ({base[1]:.1f})")
        for i in impls:
            v = per.get(i)
            cells.append("-" if v is None or base is None or v[0] <= 0 else f"{base[0] / v[0]:.2f}x")
        out.append(("| " + " | ".join(cells) + " |") if markdown else "  ".join(cells))
    return out


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    markdown = "--markdown" in argv
    paths = [a for a in argv if not a.startswith("--")]
    if not paths:
        print(__doc__)
        return 2
    for p in paths:
        with open(p, newline="") as f:
            for line in render(parse(f), markdown):
                print(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
