"""One rank of the multi-GPU correctness run (launched by test_gpu_distributed.py through torch.distributed.run).

Every rank regenerates every peer's seeded input locally, so expected outputs need no communication
(the approach of csrc/support/purlin/benchmark/data.cuh:46-61 in the reference). Inputs are integers in
[-2, 2]: exact in every element type and in any summation order, so NVLS results compare bit-exactly too.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import purlin_b200 as purlin  # noqa: E402
from helpers import AR, AG, AGV, RS, RSV, A2A, A2AV, ELEM, TORCH_DT, expected, in_out_bytes, ints, policy  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    staging = int(os.environ.get("PURLIN_TEST_STAGING", 8 << 20))
    h = purlin.initialize(dist.group.WORLD, dev, 100, None, staging_size=staging, timeout_ms=5000)
    failures = []
    count = 0

    def case(name, coll, nbytes=0, sizes=None, dtype=0, op=0, mode=0, pol=None, seed=0, reps=2, graph=False):
        nonlocal count
        e = ELEM[dtype]
        for rep in range(reps):
            ins = []
            for r in range(world):
                ib, _ = in_out_bytes(coll, world, r, nbytes, sizes)
                lo, hi = (1, 2) if op == 1 else (-2, 2)
                ins.append(ints(ib // e, dtype, seed * 1000 + rep * 100 + r, lo, hi))
            _, ob = in_out_bytes(coll, world, rank, nbytes, sizes)
            x = ins[rank].to(dev)
            out = torch.full((ob // e,), 7.0, device=dev).to(TORCH_DT[dtype])
            kw = dict(policy=pol)

            def call():
                if coll == AR:
                    purlin.all_reduce(x, out, h, None, mode, purlin.ReduceOp(op), **kw)
                elif coll == AG:
                    purlin.all_gather(x, out, h, None, **kw)
                elif coll == AGV:
                    purlin.all_gather_v(x, out, sizes, h, None, **kw)
                elif coll == RS:
                    purlin.reduce_scatter(x, out, h, None, mode, purlin.ReduceOp(op), **kw)
                elif coll == RSV:
                    purlin.reduce_scatter_v(x, out, sizes, h, None, mode, purlin.ReduceOp(op), **kw)
                elif coll == A2A:
                    purlin.all_to_all(x, out, h, None, **kw)
                else:
                    purlin.all_to_all_v(x, out, list(sizes[rank]) + [sizes[q][rank] for q in range(world)], h, None, **kw)

            if graph:
                g = torch.cuda.CUDAGraph()
                s = torch.cuda.Stream()
                with torch.cuda.stream(s):
                    with torch.cuda.graph(g, stream=s):
                        call()
                for _ in range(3):
                    g.replay()
            else:
                call()
            try:
                purlin.check(h)
            except TimeoutError as err:
                failures.append(f"{name}: {err}")
                purlin.clear_status(h)
                return
            exp = expected(coll, world, rank, ins, nbytes, sizes, dtype, op)
            if not torch.equal(out.cpu().view(torch.uint8), exp.view(torch.uint8)):
                bad = (out.cpu().view(torch.uint8) != exp.view(torch.uint8)).nonzero()
                failures.append(f"{name} rep {rep}: {bad.numel()} bytes differ, first at {int(bad[0]) if bad.numel() else -1}")
                return
        count += 1

    mc = h.has_multicast
    if rank == 0:
        print(f"world {world} multicast {mc} staging {staging} provider {os.environ.get('PURLIN_PROVIDER', 'torch')}", flush=True)
    W = world
    subset = bool(os.environ.get("PURLIN_TEST_SUBSET"))   # second pass with another provider: defaults, NVLS and V cases only
    # all-reduce: every band, forced
    ar_cases = [("one-shot packets", dict(regime=0, arPath=0, lrBlocks=8), 32 * W * 8),
                ("two-shot packets", dict(regime=0, arPath=1, lrBlocks=8), 32 * W * 64),
                ("staged direct", dict(arPath=0, consumeBlocks=16, putBlocks=8), 1 << 20),
                ("staged composed", dict(arPath=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8), 1 << 20),
                ("staged composed chunked", dict(arPath=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8, chunkBytes=256 << 10), 3 << 20),
                ("segmented", dict(arPath=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8, chunkBytes=1 << 20), staging * 2 + W * 32 * 8)]
    for name, kw, n in ([] if subset else ar_cases):
        os.environ["PURLIN_AR_SEGMENTS"] = "1" if name == "segmented" else "0"     # the default depends on the world size
        for dtype in (0, 4, 1):
            case(f"AR {name} dt{dtype}", AR, nbytes=n, dtype=dtype, pol=policy(**kw))
        case(f"AR {name} max", AR, nbytes=n, dtype=0, op=2, pol=policy(**kw))
        case(f"AR {name} deterministic", AR, nbytes=n, dtype=0, mode=1, pol=policy(**kw))
    if mc:
        for name, kw, n in (("nvls two-shot", dict(arPath=1, memType=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8), 1 << 20),
                            ("nvls chunked", dict(arPath=1, memType=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8, chunkBytes=256 << 10), 4 << 20),
                            ("nvls packets one-shot", dict(regime=0, arPath=0, lrMulticast=1, lrBlocks=8), 32 * W * 8),
                            ("nvls packets two-shot", dict(regime=0, arPath=1, lrMulticast=1, lrBlocks=8), 32 * W * 64)):
            for dtype in (0, 4, 1):
                case(f"AR {name} dt{dtype}", AR, nbytes=n, dtype=dtype, pol=policy(**kw))
            case(f"AR {name} max", AR, nbytes=n, dtype=0, op=2, pol=policy(**kw))
        case("RS nvls", RS, nbytes=1 << 18, dtype=0, pol=policy(memType=1, consumeBlocks=16, putBlocks=8))
    for coll, cname in (() if subset else ((AG, "AG"), (RS, "RS"), (A2A, "A2A"))):
        for name, kw, n in (("packets", dict(regime=0, lrBlocks=8), 32 * 40), ("staged", dict(), 1 << 19),
                            ("chunked", dict(chunkBytes=128 << 10), (1 << 20) + 64), ("cyclic", dict(chunkBytes=256 << 10), staging // 2)):
            case(f"{cname} {name}", coll, nbytes=n, dtype=0, pol=policy(putBlocks=max(8, W), consumeBlocks=max(16, 2 * W), **kw))
    # default policies over sizes (the built-in table chooses)
    for n in (32 * W, 8 << 10, 64 << 10, 512 << 10, 4 << 20):
        for coll, cname in ((AR, "AR"), (AG, "AG"), (RS, "RS"), (A2A, "A2A")):
            case(f"{cname} default {n}", coll, nbytes=n, dtype=0, reps=1)
    # a CTA budget of 64 (the reference's cap on a collective): the same calls must stay exact with the smaller grids
    old_budget = purlin.set_max_ctas(64)
    for n in (64 << 10, 4 << 20):
        for coll, cname in ((AR, "AR"), (AG, "AG"), (RS, "RS"), (A2A, "A2A")):
            case(f"{cname} budget 64 CTAs {n}", coll, nbytes=n, dtype=0, reps=1)
    purlin.set_max_ctas(old_budget)
    # an all-reduce beyond the staging size is one kernel; here with the reduction done by the switch
    os.environ["PURLIN_AR_SEGMENTS"] = "0"
    if mc and not subset:
        case("AR cyclic nvls", AR, nbytes=staging * 2 + W * 32 * 8, dtype=0,
             pol=policy(arPath=1, memType=1, consumeBlocks=16, putBlocks=8, gatherBlocks=8, chunkBytes=1 << 20))
    os.environ.pop("PURLIN_AR_SEGMENTS", None)
    case("AR default graph", AR, nbytes=64 << 10, dtype=0, reps=1, graph=True)
    case("AR default graph large", AR, nbytes=2 << 20, dtype=0, reps=1, graph=True)
    # variable-length
    g = torch.Generator().manual_seed(7)
    base = 1 << 16
    sizes = [int(base * (0.5 + float(torch.rand(1, generator=g)))) // 32 * 32 for _ in range(W)]
    for coll, cname in ((AGV, "AGV"), (RSV, "RSV")):
        case(f"{cname} random", coll, sizes=sizes, dtype=0)
        case(f"{cname} with empty", coll, sizes=[0 if q % 2 else s for q, s in enumerate(sizes)], dtype=0)
        case(f"{cname} small", coll, sizes=[32 * (q + 1) for q in range(W)], dtype=0)
    mat = [[int(base * float(torch.rand(1, generator=g))) // 32 * 32 if (r + q) % 3 else 0 for q in range(W)] for r in range(W)]
    case("A2AV mixed", A2AV, sizes=mat, dtype=0, pol=policy(putBlocks=max(8, W), consumeBlocks=max(16, 2 * W), perStreamThreshold=16384, chunkBytes=32768))
    case("A2AV default", A2AV, sizes=mat, dtype=0)
    idle = [[0] * W for _ in range(W)]
    case("A2AV idle", A2AV, sizes=idle, dtype=0)
    # back-to-back unsynchronised calls on one context
    x = torch.ones(1 << 16, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(x)
    for i in range(32):
        purlin.all_reduce(x, out, h, None)
    purlin.check(h)
    if not torch.all(out == W).item():
        failures.append("back-to-back all-reduce")
    # a delayed rank: the last rank's stream is busy for a while before it joins; the others wait inside their bound
    if rank == W - 1:
        torch.cuda._sleep(200_000_000)      # about 0.1 s of device time, far below the 5 s limit of the waits
    case("AR after a delayed rank", AR, nbytes=1 << 20, dtype=0, reps=1)
    case("A2AV after a delayed rank", A2AV, sizes=mat, dtype=0, reps=1)
    # skewed and hot-ring traffic (the split policies of the benchmark harness)
    from purlin_b200.utils import split_policy as sp
    for percent in (25, 50):
        sk = sp.skew_splits(W * (96 << 10), W, percent, seed=percent)
        case(f"AGV skew {percent}", AGV, sizes=sk, dtype=0, reps=1)
        case(f"RSV skew {percent}", RSV, sizes=sk, dtype=0, reps=1)
    case("A2AV hot ring", A2AV, sizes=sp.hot_ring_matrix(W, 256 << 10, 90), dtype=0, reps=1)
    case("A2AV sparse", A2AV, sizes=sp.sparse_matrix(W, 1, 64 << 10, seed=5), dtype=0, reps=1)
    case("A2AV self only", A2AV, sizes=[[(8 << 10) if r == q else 0 for q in range(W)] for r in range(W)], dtype=0, reps=1)
    # one context, mixed collective kinds and grid sizes, 32 calls back to back without synchronisation, inputs changed
    # on the device between calls (a stale read of an earlier call's staging would show), in a stream and from a graph
    n = 32 * W * 16
    src = torch.zeros(n, device=dev, dtype=torch.float32)
    ar_out = torch.empty(n, device=dev, dtype=torch.float32)
    ag_out = torch.empty(n * W, device=dev, dtype=torch.float32)
    rs_out = torch.empty(n // W, device=dev, dtype=torch.float32)
    aa_out = torch.empty(n, device=dev, dtype=torch.float32)

    def mixed_round():
        src.add_(1.0)                                     # the "device counter": data differ in every round
        purlin.all_reduce(src, ar_out, h, None)
        purlin.all_gather(src, ag_out, h, None)
        purlin.reduce_scatter(src, rs_out, h, None)
        purlin.all_to_all(src, aa_out, h, None)

    for _ in range(8):
        mixed_round()
    purlin.check(h)
    rounds = 8
    gr = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(gr, stream=side):
            for _ in range(8):
                mixed_round()
    for _ in range(4):
        gr.replay()
        rounds += 8
    try:
        purlin.check(h)
        good = (torch.all(ar_out == rounds * W).item() and torch.all(ag_out == rounds).item()
                and torch.all(rs_out == rounds * W).item() and torch.all(aa_out == rounds).item())
        if not good:
            failures.append(f"mixed back-to-back calls: expected round {rounds}, all-reduce saw {float(ar_out[0])}, all-gather {float(ag_out[0])}")
        else:
            count += 1
    except TimeoutError as err:
        failures.append(f"mixed back-to-back calls: {err}")
        purlin.clear_status(h)
    # zero-copy all-reduce on a tensor allocated in symmetric memory (NVLS when offered, peer loads otherwise)
    for dtype, n in ((torch.bfloat16, 1 << 20), (torch.float32, 32 * W * 9)):
        st = purlin.symm_empty((n,), dtype, h)
        for mode in (purlin.ReductionMode.NON_DETERMINISTIC, purlin.ReductionMode.DETERMINISTIC):
            for rep in range(2):
                parts = [ints(n, 0 if dtype == torch.bfloat16 else 4, 900 + rep * 10 + r) for r in range(W)]
                st.tensor.copy_(parts[rank].to(dev))
                purlin.all_reduce_symm(st, reduction_mode=mode)
                if st.status() != 0:
                    failures.append(f"symm all-reduce {dtype} mode {int(mode)}: status {st.status()}")
                    break
                exp = expected(AR, W, rank, parts, n * parts[0].element_size(), None, 0 if dtype == torch.bfloat16 else 4)
                if not torch.equal(st.tensor.cpu().view(torch.uint8), exp.view(torch.uint8)):
                    failures.append(f"symm all-reduce {dtype} mode {int(mode)} rep {rep}")
        count += 1
        del st
    # zero-copy reduce-scatter (symmetric inputs -> ordinary output) and in-place all-gather of a symmetric tensor
    for dtype, code, n_slice in ((torch.bfloat16, 0, 1 << 18), (torch.float32, 4, 8 * 11)):
        st = purlin.symm_empty((W * n_slice,), dtype, h)
        out_rs = torch.empty(n_slice, dtype=dtype, device=dev)
        for mode in (purlin.ReductionMode.NON_DETERMINISTIC, purlin.ReductionMode.DETERMINISTIC):
            for rep in range(2):
                parts = [ints(W * n_slice, code, 1300 + rep * 10 + r) for r in range(W)]
                st.tensor.copy_(parts[rank].to(dev))
                out_rs.fill_(7.0)
                purlin.reduce_scatter_symm(st, out_rs, reduction_mode=mode)
                st.tensor.fill_(9.0)     # the inputs may be overwritten as soon as the call is done in stream order
                exp = expected(RS, W, rank, parts, n_slice * parts[0].element_size(), None, code)
                if st.status() != 0 or not torch.equal(out_rs.cpu().view(torch.uint8), exp.view(torch.uint8)):
                    failures.append(f"symm reduce-scatter {dtype} mode {int(mode)} rep {rep} status {st.status()}")
        for via in (None, False, True):
            for rep in range(2):
                parts = [ints(n_slice, code, 1500 + rep * 10 + r) for r in range(W)]
                st.tensor.fill_(5.0)
                st.tensor[rank * n_slice:(rank + 1) * n_slice].copy_(parts[rank].to(dev))
                purlin.all_gather_symm(st, via_switch=via)
                exp = torch.cat(parts)
                if st.status() != 0 or not torch.equal(st.tensor.cpu().view(torch.uint8), exp.view(torch.uint8)):
                    failures.append(f"symm all-gather {dtype} via_switch {via} rep {rep} status {st.status()}")
        count += 1
        del st
    purlin.finalize(h)
    purlin.finalize(h)
    ok = torch.tensor([0 if failures else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in failures:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print(f"cases passed on rank 0: {count}; all ranks ok: {bool(ok.item())}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
