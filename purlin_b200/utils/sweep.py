"""Message-size sweep of every collective against NCCL, and the tuner that fills the codesign table.

Run with one process per GPU:
  python -m torch.distributed.run --nnodes=1 --nproc-per-node=8 --master-addr 127.0.0.1 \
      -m purlin_b200.utils.sweep --collectives ar,ag,rs,a2a --min-bytes 8K --max-bytes 1G [--tune] [--csv out.csv]

Counterpart of the reference's benchmark binaries (csrc/tests/{ar,ag,rs,a2a}.cu: power-of-two sweep, an
exact-correctness run before timing, CSV on stdout).  ``--tune`` measures a set of candidate policies
(one-shot / two-shot packets, staged unicast, NVLS; several chunk sizes and grid sizes) for each size and
writes the winners as the measured codesign table that ``purlin_b200.tuning`` loads at ``initialize``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

import purlin_b200 as purlin
from purlin_b200 import _native
from purlin_b200.utils import bench

NAMES = {"ar": purlin.Collective.ALL_REDUCE, "ag": purlin.Collective.ALL_GATHER, "rs": purlin.Collective.REDUCE_SCATTER,
         "a2a": purlin.Collective.ALL_TO_ALL}


def _policy(**kw):
    base = dict(regime=1, threads=256, putBlocks=32, localBlocks=8, consumeBlocks=48, gatherBlocks=32, lrBlocks=32, memType=0,
                mmDepth=4, unroll=8, stageDepth=0, arPath=1, lrMulticast=0, weighted=1, chunkBytes=0, perStreamThreshold=128 << 10)
    base.update(kw)
    return _native.Policy.from_dict(base)


def candidates(coll: str, world: int, nbytes: int, layout: dict, multicast: bool):
    """Policies worth measuring for one (collective, size). `nbytes` is the dispatch size."""
    slot = layout["packet_stride"] // 2
    out = []
    lr_blocks = sorted({min(max(-(-nbytes // 4096), 1), 64), min(max(-(-nbytes // 2048), 1), 128), 16, 32})
    if coll == "ar":
        if nbytes <= slot:
            for b in lr_blocks:
                out.append(("lr1", _policy(regime=0, arPath=0, lrBlocks=b)))
                if multicast:
                    out.append(("lr1-mc", _policy(regime=0, arPath=0, lrBlocks=b, lrMulticast=1)))
        if world > 2 and nbytes <= (slot // 2) * world and nbytes % (world * 32) == 0:
            for b in (28, 56, 112):
                out.append(("lr2", _policy(regime=0, arPath=1, lrBlocks=b)))
                if multicast:
                    out.append(("lr2-mc", _policy(regime=0, arPath=1, lrBlocks=b, lrMulticast=1)))
        if nbytes >= 64 << 10:
            chunks = [0] if nbytes <= 2 << 20 else [c for c in (1 << 20, 2 << 20, 8 << 20, 32 << 20) if c < nbytes and nbytes // c <= 64] + ([0] if nbytes <= 16 << 20 else [])
            for c in chunks:
                for ring in (0,):
                    for put, con, gat in ((16, 32, 16), (32, 64, 32), (24, 96, 24), (32, 80, 32)):
                        if world == 2:
                            out.append((f"tr-direct-r{ring}", _policy(arPath=0, putBlocks=put, consumeBlocks=con + gat, chunkBytes=c, stageDepth=ring)))
                        out.append((f"tr-2shot-r{ring}", _policy(arPath=1, putBlocks=put, consumeBlocks=con, gatherBlocks=gat, chunkBytes=c, stageDepth=ring)))
                    if multicast:
                        for put, con, gat, depth in ((16, 32, 16, 4), (32, 64, 32, 8), (24, 96, 24, 8), (32, 32, 32, 8), (48, 48, 48, 8), (40, 64, 40, 4)):
                            out.append((f"nvls-r{ring}", _policy(arPath=1, memType=1, putBlocks=put, consumeBlocks=con, gatherBlocks=gat, mmDepth=depth, chunkBytes=c, stageDepth=ring)))
    else:
        per_rank_total = nbytes * world
        if nbytes <= slot:
            for b in lr_blocks:
                out.append(("lr", _policy(regime=0, lrBlocks=b)))
        if per_rank_total >= 64 << 10:
            chunks = [0] if nbytes <= 1 << 20 else [c for c in (256 << 10, 1 << 20, 4 << 20, 16 << 20) if c < nbytes and nbytes // c <= 64] + ([0] if nbytes <= 8 << 20 else [])
            for c in chunks:
                for ring in (0,):
                    for put, con in ((16, 32), (32, 64), (32, 96), (24, 112)):
                        out.append((f"tr-r{ring}", _policy(putBlocks=max(put, world), consumeBlocks=con, chunkBytes=c, stageDepth=ring)))
                    if coll == "rs" and multicast:
                        out.append((f"nvls-r{ring}", _policy(memType=1, putBlocks=32, consumeBlocks=64, mmDepth=8, chunkBytes=c, stageDepth=ring)))
    return out


def variable_length_section(args, h, rank, world, dev, td, esz, table=None):
    """AllGatherV, ReduceScatterV and AllToAllV at per-rank element counts uniform in [0.5, 1.5] x ``args.variable`` (seed 7,
    multiples of 16 elements), against NCCL on buffers padded to the largest count (the usual way to run uneven sizes on a
    library that wants equal ones). Inputs are integers in [-2, 2] generated on the device (seed 42 + rank), so the untimed
    comparison with NCCL's result is exact in any summation order. With ``--tune`` the candidate policies of the fixed-size
    sibling are measured for each form and the fastest exact one is appended to ``table`` under the form's own collective id,
    keyed by the largest stream of the call (the size ``selectPolicy`` dispatches on)."""
    from .split_policy import uniform_counts
    unit = max(32 // esz, 1)
    counts = uniform_counts(world, base_elems=args.variable, seed=7, multiple=unit)
    sizes = [c * esz for c in counts]
    total, biggest = sum(sizes), max(counts)
    gen = torch.Generator(device=dev).manual_seed(42 + rank)

    def ints(n):
        return torch.randint(-2, 3, (n,), generator=gen, device=dev).to(td)

    def row(coll, impl, t, ok=True, logical=None):
        if rank == 0:
            print(bench.csv_row(coll, impl, world, total if logical is None else logical, args.dtype, t, 0.0 if ok else 100.0), flush=True)

    def agree(ok):
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item())

    def best_of(coll, sibling, kind, dispatch, call, correct, scrub):
        """Default-policy row, and with --tune the fastest exact candidate (recorded in the table)."""
        t = bench.measure(lambda: call(None), args.warmup, args.runs, args.graph)
        if not (args.tune and table is not None):
            return t
        best = None
        for label, pol in candidates(sibling, world, dispatch, h.layout, False):
            if kind == purlin.Collective.ALL_TO_ALL_V and pol.regime != 1:
                continue                                   # packets are chosen per stream inside an all-to-all-v plan
            try:
                scrub()                                    # a candidate that writes nothing must not pass on old results
                call(pol)
                purlin.check(h)
                if not agree(correct()):
                    continue
                tc = bench.measure(lambda: call(pol), args.warmup, args.runs, args.graph)
            except (RuntimeError, TimeoutError) as e:
                if rank == 0:
                    print(f"# skipped {coll} {label}: {e}", flush=True)
                purlin.clear_status(h)
                continue
            if rank == 0:
                print("# " + bench.csv_row(coll, f"cand:{label}:{pol.putBlocks}/{pol.consumeBlocks}/c{pol.chunkBytes >> 10}K", world, total, args.dtype, tc), flush=True)
            if best is None or tc.us < best[0].us:
                best = (tc, label, pol)
        if best is not None and best[0].us < t.us:
            table.append({"collective": int(kind), "world": world, "bytes": dispatch, "label": best[1], "us": best[0].us, "policy": best[2].as_dict()})
            return best[0]
        return t

    # all-gather-v: rank r contributes counts[r] elements
    x, out = ints(counts[rank]), torch.empty(sum(counts), dtype=td, device=dev)
    xp = torch.zeros(biggest, dtype=td, device=dev)
    xp[:counts[rank]] = x
    outp = torch.empty(world * biggest, dtype=td, device=dev)
    dist.all_gather_into_tensor(outp, xp)
    purlin.all_gather_v(x, out, sizes, h, None)
    purlin.check(h)
    ok, off = True, 0
    for q in range(world):
        ok = ok and torch.equal(out[off:off + counts[q]], outp[q * biggest:q * biggest + counts[q]])
        off += counts[q]
    def agv_ok():
        good, at = True, 0
        for q in range(world):
            good = good and torch.equal(out[at:at + counts[q]], outp[q * biggest:q * biggest + counts[q]])
            at += counts[q]
        return good

    row("agv", "purlin_b200", best_of("agv", "ag", purlin.Collective.ALL_GATHER_V, max(sizes),
                                      lambda pol: purlin.all_gather_v(x, out, sizes, h, None, policy=pol), agv_ok, lambda: out.fill_(7)), agree(ok))
    if not args.no_nccl:
        row("agv", "nccl:padded", bench.measure(lambda: dist.all_gather_into_tensor(outp, xp), args.warmup, args.runs, args.graph))
    del xp, outp

    # reduce-scatter-v: every rank holds sum(counts) elements, rank r receives counts[r] of the sum
    x, out = ints(sum(counts)), torch.empty(counts[rank], dtype=td, device=dev)
    ref = x.clone()
    dist.all_reduce(ref)
    purlin.reduce_scatter_v(x, out, sizes, h, None)
    purlin.check(h)
    off = sum(counts[:rank])
    want = ref[off:off + counts[rank]].clone()
    ok = torch.equal(out, want)
    del ref
    row("rsv", "purlin_b200", best_of("rsv", "rs", purlin.Collective.REDUCE_SCATTER_V, max(sizes),
                                      lambda pol: purlin.reduce_scatter_v(x, out, sizes, h, None, policy=pol), lambda: torch.equal(out, want),
                                      lambda: out.fill_(7)), agree(ok))
    if not args.no_nccl:
        xp = torch.zeros(world * biggest, dtype=td, device=dev)
        outp = torch.empty(biggest, dtype=td, device=dev)
        row("rsv", "nccl:padded", bench.measure(lambda: dist.reduce_scatter_tensor(outp, xp), args.warmup, args.runs, args.graph))
        del xp, outp

    # all-to-all-v: rank r sends counts[(r + q) % world] / world elements to rank q (rows are rotations of one list)
    def cell(r, q):
        return (counts[(r + q) % world] // world) // unit * unit

    send = [cell(rank, q) for q in range(world)]
    recv = [cell(q, rank) for q in range(world)]
    x, out = ints(sum(send)), torch.empty(sum(recv), dtype=td, device=dev)
    ref = torch.empty_like(out)
    dist.all_to_all_single(ref, x, output_split_sizes=recv, input_split_sizes=send)
    splits = [c * esz for c in send] + [c * esz for c in recv]
    purlin.all_to_all_v(x, out, splits, h, None)
    purlin.check(h)
    ok = torch.equal(out, ref)
    moved = sum(cell(0, q) for q in range(world)) * esz * world     # what rank 0 sends, times the ranks: the reference's convention
    row("a2av", "purlin_b200", best_of("a2av", "a2a", purlin.Collective.ALL_TO_ALL_V, max(max(send), max(recv)) * esz,
                                       lambda pol: purlin.all_to_all_v(x, out, splits, h, None, policy=pol), lambda: torch.equal(out, ref),
                                       lambda: out.fill_(7)), agree(ok), moved)
    if not args.no_nccl:
        row("a2av", "nccl", bench.measure(lambda: dist.all_to_all_single(ref, x, output_split_sizes=recv, input_split_sizes=send),
                                          args.warmup, args.runs, args.graph), True, moved)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--collectives", default="ar,ag,rs,a2a")
    ap.add_argument("--min-bytes", default="8K")
    ap.add_argument("--max-bytes", default="256M")
    ap.add_argument("--factor", type=int, default=8)
    ap.add_argument("--dtype", default="bf16")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--runs", type=int, default=20)
    ap.add_argument("--graph", type=int, default=0)
    ap.add_argument("--tune", action="store_true")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--symm", action="store_true", help="also time the zero-copy all-reduce on symmetric tensors")
    ap.add_argument("--variable", type=int, default=0, metavar="ELEMS",
                    help="also run the variable-length collectives: per-rank counts uniform in [0.5, 1.5] x ELEMS from seed 7")
    ap.add_argument("--reference", default="", metavar="DIR",
                    help="also time the reference's own collectives: DIR holds its installed package (purlin/) and, beside it, "
                         "DIR_cache with its prebuilt binding module (see baseline/build_reference_module.py)")
    ap.add_argument("--csv", default="")
    ap.add_argument("--table-out", default="")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    if args.tune:
        os.environ["PURLIN_NO_TUNING_TABLE"] = "1"   # candidates are forced; the built-in policy is the fallback
    h = purlin.initialize(dist.group.WORLD, dev, 100, None)
    ref_mod = ref_h = None
    if args.reference:
        # the reference's Python API, unmodified; its JIT finds the prebuilt module through its own cache directory
        os.environ["PURLIN_CACHE_DIR"] = args.reference.rstrip("/") + "_cache"
        sys.path.insert(0, args.reference)
        import purlin as ref_mod   # noqa: E402  (the reference's package is called purlin; this one is purlin_b200)
        ref_h = ref_mod.initialize(dist.group.WORLD, dev, 100, torch.cuda.current_stream().cuda_stream)
    td = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[args.dtype]
    esz = torch.empty(0, dtype=td).element_size()
    lo, hi = bench.parse_size(args.min_bytes), bench.parse_size(args.max_bytes)
    rows, table = [], []
    if rank == 0:
        print(bench.CSV_HEADER, flush=True)
    for coll in args.collectives.split(","):
        n = lo
        while n <= hi:
            # n = per-rank payload in bytes (all-reduce: whole payload; all-gather: input; others: per-rank total in/out)
            if coll == "ar":
                in_b, out_b, disp = n, n, n
            elif coll == "ag":
                in_b, out_b, disp = n // world, n, n // world
            elif coll == "rs":
                in_b, out_b, disp = n, n // world, n // world
            else:
                in_b, out_b, disp = n, n, n // world
            disp = disp // 32 * 32
            if coll == "ag":
                in_b, out_b = disp, disp * world
            elif coll == "rs":
                in_b, out_b = disp * world, disp
            elif coll == "a2a":
                in_b = out_b = disp * world
            g = torch.Generator().manual_seed(42 + rank)
            x = torch.randint(-2, 3, (in_b // esz,), generator=g).to(td).to(dev)
            out = torch.empty(out_b // esz, dtype=td, device=dev)
            ref = torch.empty_like(out)
            total = bench.logical_bytes(coll, n if coll == "ar" else disp, world)
            runs = args.runs if n <= (64 << 20) else max(args.runs // 4, 3)

            def nccl_call():
                if coll == "ar":
                    ref.copy_(x); dist.all_reduce(ref)
                elif coll == "ag":
                    dist.all_gather_into_tensor(ref, x)
                elif coll == "rs":
                    dist.reduce_scatter_tensor(ref, x)
                else:
                    dist.all_to_all_single(ref, x)

            def nccl_timed():
                if coll == "ar":
                    dist.all_reduce(ref)   # in place, as NCCL users call it
                else:
                    nccl_call()

            def ours(pol=None):
                if coll == "ar":
                    purlin.all_reduce(x, out, h, None, policy=pol)
                elif coll == "ag":
                    purlin.all_gather(x, out, h, None, policy=pol)
                elif coll == "rs":
                    purlin.reduce_scatter(x, out, h, None, policy=pol)
                else:
                    purlin.all_to_all(x, out, h, None, policy=pol)

            nccl_call()
            torch.cuda.synchronize()
            expect = ref.clone()

            def verify(pol, label):
                out.fill_(7)
                ours(pol)
                purlin.check(h)
                ok = torch.equal(out, expect)
                flag = torch.tensor([1 if ok else 0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if not flag.item() and rank == 0:
                    print(f"# MISMATCH {coll} {n} {label}", flush=True)
                return bool(flag.item())

            best = None
            if args.tune:
                for label, pol in candidates(coll, world, disp if coll != "ar" else n, h.layout, h.has_multicast):
                    try:
                        if not verify(pol, label):
                            continue
                        t = bench.measure(lambda: ours(pol), args.warmup, runs, args.graph)
                    except RuntimeError as e:
                        if rank == 0:
                            print(f"# skipped {coll} {n} {label}: {e}", flush=True)
                        continue
                    if rank == 0:
                        print("# " + bench.csv_row(coll, f"cand:{label}:{pol.putBlocks}/{pol.consumeBlocks}/{pol.gatherBlocks}/{pol.lrBlocks}/c{pol.chunkBytes >> 10}K/d{pol.mmDepth}", world, total, args.dtype, t), flush=True)
                    if best is None or t.us < best[0].us:
                        best = (t, label, pol)
                if best is not None:
                    table.append({"collective": int(NAMES[coll]), "world": world, "bytes": disp if coll != "ar" else n, "label": best[1], "us": best[0].us, "policy": best[2].as_dict()})
                    if rank == 0:
                        print(bench.csv_row(coll, "purlin_b200:" + best[1], world, total, args.dtype, best[0]), flush=True)
            else:
                ok = verify(None, "default")
                t = bench.measure(lambda: ours(None), args.warmup, runs, args.graph)
                if rank == 0:
                    print(bench.csv_row(coll, "purlin_b200", world, total, args.dtype, t, 0.0 if ok else 100.0), flush=True)
                    rows.append((coll, "purlin_b200", n, t.us))
            if coll == "ar" and args.symm and not args.tune:
                # zero-copy variant: the tensor lives in symmetric memory, no staging passes
                stt = purlin.symm_empty((in_b // esz,), td, h)
                stt.tensor.copy_(x)
                purlin.all_reduce_symm(stt)
                oks = torch.equal(stt.tensor, expect) and stt.status() == 0
                t = bench.measure(lambda: purlin.all_reduce_symm(stt), args.warmup, runs, args.graph)
                if rank == 0:
                    print(bench.csv_row(coll, "purlin_b200:symm-zero-copy", world, total, args.dtype, t, 0.0 if oks else 100.0), flush=True)
                del stt
            if coll == "rs" and args.symm and not args.tune:
                # inputs in symmetric memory: peers (or the switch) read them in place, no staging pass
                stt = purlin.symm_empty((in_b // esz,), td, h)
                stt.tensor.copy_(x)
                out.fill_(7)
                purlin.reduce_scatter_symm(stt, out)
                oks = stt.status() == 0 and torch.equal(out, expect)
                t = bench.measure(lambda: purlin.reduce_scatter_symm(stt, out), args.warmup, runs, args.graph)
                if rank == 0:
                    print(bench.csv_row(coll, "purlin_b200:symm-zero-copy", world, total, args.dtype, t, 0.0 if oks else 100.0), flush=True)
                del stt
            if coll == "ag" and args.symm and not args.tune:
                # the gathered tensor lives in symmetric memory: every rank pushes its slice into all of them in place
                stt = purlin.symm_empty((out.numel(),), td, h)
                per = x.numel()
                for via, tag in ((None, "symm-zero-copy"), (False, "symm-zero-copy:stores"), (True, "symm-zero-copy:switch")):
                    stt.tensor.fill_(7)
                    stt.tensor[rank * per:(rank + 1) * per].copy_(x.reshape(-1))
                    purlin.all_gather_symm(stt, via_switch=via)
                    oks = stt.status() == 0 and torch.equal(stt.tensor, expect.reshape(-1))
                    t = bench.measure(lambda: purlin.all_gather_symm(stt, via_switch=via), args.warmup, runs, args.graph)
                    if rank == 0:
                        print(bench.csv_row(coll, "purlin_b200:" + tag, world, total, args.dtype, t, 0.0 if oks else 100.0), flush=True)
                del stt
            if ref_mod is not None and not args.tune:
                rout = torch.empty_like(out)

                def ref_call():
                    rstream = torch.cuda.current_stream().cuda_stream     # at call time: under graph capture this is the capturing stream
                    if coll == "ar":
                        ref_mod.all_reduce(x, rout, ref_h, rstream)
                    elif coll == "ag":
                        ref_mod.all_gather(x, rout, ref_h, rstream)
                    elif coll == "rs":
                        ref_mod.reduce_scatter(x, rout, ref_h, rstream)
                    else:
                        ref_mod.all_to_all(x, rout, ref_h, rstream)

                ref_call()
                torch.cuda.synchronize()
                okr = torch.equal(rout, expect)
                t = bench.measure(ref_call, args.warmup, runs, args.graph)
                if rank == 0:
                    print(bench.csv_row(coll, "reference", world, total, args.dtype, t, 0.0 if okr else 100.0), flush=True)
                del rout
            if not args.no_nccl:
                t = bench.measure(nccl_timed, args.warmup, runs, args.graph)
                if rank == 0:
                    print(bench.csv_row(coll, "nccl", world, total, args.dtype, t), flush=True)
            n *= args.factor
    if args.variable:
        variable_length_section(args, h, rank, world, dev, td, esz, table)
    if args.tune and rank == 0:
        from purlin_b200 import tuning
        path = args.table_out or os.path.join("tuning_out", str(tuning.table_path(torch.cuda.get_device_name(), world).name))
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump({"gpu": torch.cuda.get_device_name(), "world": world, "dtype": args.dtype, "entries": table}, f, indent=1, sort_keys=True)
        print(f"# wrote {path}", flush=True)
    if ref_mod is not None:
        ref_mod.finalize(ref_h, torch.cuda.current_stream().cuda_stream)
    purlin.finalize(h)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
