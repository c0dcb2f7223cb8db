"""Prints the plan the layout engine builds for a call: roles, CTA ranges, regions, flags, chunking.

    python -m purlin_b200.utils.explain all_reduce --world 8 --bytes 64M
    python -m purlin_b200.utils.explain all_to_all_v --world 4 --sizes 0,65536,1048576,32 --rank 1
    python -m purlin_b200.utils.explain reduce_scatter --world 8 --bytes 4M --multicast --staging 256M

In the reference the orchestration of a collective is the result of nested template instantiation
(csrc/include/purlin/snac.cuh:36-78, 572-807) and cannot be looked at; here it is a small table the kernel interprets,
so it can be printed. No GPU is needed. The policy comes from the measured table of ``--gpu`` when one is installed for
that world size (or the nearest one), else from the built-in bands, exactly as at run time.
"""
from __future__ import annotations

import argparse
import sys
from typing import List

import purlin_b200 as purlin
from purlin_b200.utils.bench import parse_size

ROLES = ["stage", "local", "consume", "reduce", "gather", "packet-put", "packet-get", "packet-reduce"]
FLAGS = ["to-seam", "to-dst", "multimem-load", "multicast-out", "local-source", "cyclic", "publish", "result-half", "notify-gather",
         "drain-self", "drain-gather", "scatter"]
KINDS = {"all_reduce": 0, "all_gather": 1, "all_gather_v": 2, "reduce_scatter": 3, "reduce_scatter_v": 4, "all_to_all": 5, "all_to_all_v": 6}


def _fmt(n: int) -> str:
    for unit, shift in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= (1 << shift) and n % (1 << (shift - 2)) == 0:
            return f"{n / (1 << shift):g} {unit}"
    return f"{n} B"


def describe(plan, chosen) -> List[str]:
    """Human-readable lines for one rank's plan."""
    regime = "latency (packets)" if plan.regime == 0 else "throughput (staged)"
    out = [f"{list(KINDS)[plan.collective]}: {regime}, grid {plan.blocks} x {plan.threads} threads, payload {_fmt(plan.payloadBytes)}"
           + (", arrival handshake" if plan.varLenArrival else "") + (", deterministic" if plan.deterministic else "")]
    out.append("policy: " + ", ".join(f"{k}={v}" for k, v in chosen.as_dict().items() if v))
    out.append(f"{'#':>2} {'role':<13} {'CTAs':<9} {'peer':>4} {'bytes':>10} {'chunks x size':>16} {'slots':>5}  {'src off':>10} {'dst off':>10} {'seam off':>10}  flags")
    for i, s in enumerate(plan.active_steps()):
        flags = [name for bit, name in enumerate(FLAGS) if s.flags & (1 << bit)]
        ctas = f"{s.blockBegin}-{s.blockBegin + s.blockCount - 1}"
        chunks = f"{s.chunks} x {_fmt(s.chunkBytes)}" if s.role < 5 and s.role != 1 else "-"
        out.append(f"{i:>2} {ROLES[s.role] if 0 <= s.role < len(ROLES) else s.role:<13} {ctas:<9} {s.peer if s.peer >= 0 else 'all':>4} "
                   f"{_fmt(s.bytes):>10} {chunks:>16} {s.slots if s.role < 5 and s.role != 1 else '-':>5}  {s.srcOff:>10} {s.dstOff:>10} {s.seamOff:>10}  "
                   + " ".join(flags))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("collective", choices=list(KINDS))
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--bytes", default="1M", help="fixed-size forms: the size the host API takes (all-reduce: whole buffer; "
                                                 "all-gather: per rank in; reduce-scatter: per rank out; all-to-all: per peer)")
    ap.add_argument("--sizes", default="", help="variable-length forms: comma-separated bytes, one per rank (all-to-all-v: this rank's "
                                               "row; the column is taken equal to it)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--multicast", action="store_true", help="an NVLS alias is available")
    ap.add_argument("--staging", default="256M")
    ap.add_argument("--gpu", default="NVIDIA B200", help="whose measured table to install (empty: built-in bands only)")
    args = ap.parse_args(argv)
    kind = KINDS[args.collective]
    if args.gpu:
        from purlin_b200 import tuning
        used = tuning.load_for(args.gpu, args.world)
        print(f"# policy table: {used.name if used else 'none (built-in bands)'}")
    dtype = {"bf16": purlin.DataType.BF16, "fp16": purlin.DataType.FP16, "fp32": purlin.DataType.FP32}[args.dtype]
    mode = purlin.ReductionMode.DETERMINISTIC if args.deterministic else purlin.ReductionMode.NON_DETERMINISTIC
    sizes = out_sizes = None
    nbytes = 0
    if kind in (2, 4, 6):
        if not args.sizes:
            print("variable-length forms need --sizes", file=sys.stderr)
            return 2
        sizes = [parse_size(x) for x in args.sizes.split(",")]
        if len(sizes) != args.world:
            print(f"--sizes needs {args.world} entries", file=sys.stderr)
            return 2
        out_sizes = list(sizes) if kind == 6 else None
    else:
        nbytes = parse_size(args.bytes)
    plan, chosen = purlin.build_plan(kind, args.world, args.rank, nbytes, sizes=sizes, out_sizes=out_sizes, dtype=dtype, mode=mode,
                                     multicast=args.multicast, staging_size=parse_size(args.staging))
    for line in describe(plan, chosen):
        print(line)
    return 0


if __name__ == "__main__":
    sys.exit(main())
