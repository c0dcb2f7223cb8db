"""CPU plumbing over gloo, world size 2: the Python surface drives the native layout engine in real processes.

Shapes and seeds of the CPU configuration: all-reduce (sum) of 1,048,576 fp32 per rank, N(0,1) from seed
1234 + rank, elementwise against the torch sum (atol 1e-5); all-gather of 262,144 fp32 per rank.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, what, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import purlin_b200 as purlin
    try:
        h = purlin.initialize(dist.group.WORLD, torch.device("cpu"), 100, 0, staging_size=16 << 20)
        ok = True
        if what == "all_reduce":
            g = torch.Generator().manual_seed(1234 + rank)
            x = torch.randn(1_048_576, generator=g)
            out = torch.empty_like(x)
            purlin.all_reduce(x, out, h, 0)
            ref = x.clone()
            dist.all_reduce(ref)
            ok = torch.allclose(out, ref, atol=1e-5, rtol=0)
            # deterministic mode and in-place
            purlin.all_reduce(x, x, h, 0, purlin.ReductionMode.DETERMINISTIC)
            ok = ok and torch.allclose(x, ref, atol=1e-5, rtol=0)
        elif what == "all_gather":
            g = torch.Generator().manual_seed(1234 + rank)
            x = torch.randn(262_144, generator=g)
            out = torch.empty(262_144 * world)
            purlin.all_gather(x, out, h, 0)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            ok = torch.equal(out, torch.cat(parts))
        elif what == "others":
            n = 4096
            x = torch.arange(n * world, dtype=torch.float32) + 1000 * rank
            out = torch.empty(n)
            purlin.reduce_scatter(x, out, h, 0)
            ref = sum((torch.arange(n * world, dtype=torch.float32) + 1000 * q)[rank * n:(rank + 1) * n] for q in range(world))
            ok = torch.equal(out, ref)
            out2 = torch.empty(n * world)
            purlin.all_to_all(x, out2, h, 0)
            ref2 = torch.cat([(torch.arange(n * world, dtype=torch.float32) + 1000 * q)[rank * n:(rank + 1) * n] for q in range(world)])
            ok = ok and torch.equal(out2, ref2)
            # variable-length variants, bf16, with an empty partition
            sizes = [0, 256] if world == 2 else [64 * (q % 3) for q in range(world)]
            xb = (torch.arange(sizes[rank] // 2) % 5).to(torch.bfloat16)
            outb = torch.empty(sum(sizes) // 2, dtype=torch.bfloat16)
            purlin.all_gather_v(xb, outb, sizes, h, 0)
            refb = torch.cat([(torch.arange(sizes[q] // 2) % 5).to(torch.bfloat16) for q in range(world)])
            ok = ok and torch.equal(outb, refb)
            xin = torch.ones(sum(sizes) // 2, dtype=torch.bfloat16) * (rank + 1)
            outr = torch.empty(sizes[rank] // 2, dtype=torch.bfloat16)
            purlin.reduce_scatter_v(xin, outr, sizes, h, 0)
            ok = ok and torch.equal(outr, torch.full_like(outr, sum(range(1, world + 1))))
            splits_in = [32 * ((rank + d) % 3) for d in range(world)]
            splits_out = [32 * ((q + rank) % 3) for q in range(world)]
            xa = torch.full((sum(splits_in),), rank, dtype=torch.uint8)
            outa = torch.empty(sum(splits_out), dtype=torch.uint8)
            purlin.all_to_all_v(xa, outa, splits_in + splits_out, h, 0)
            refa = torch.cat([torch.full((splits_out[q],), q, dtype=torch.uint8) for q in range(world)])
            ok = ok and torch.equal(outa, refa)
        elif what == "sequence_parallel":
            from purlin_b200.parallel import sequence_parallel as sp
            s_local, heads, d = 8, 2 * world, 4
            g = torch.Generator().manual_seed(7)
            whole = torch.randn(s_local * world, heads, d, generator=g)      # the same on every rank
            mine = whole[rank * s_local:(rank + 1) * s_local].clone()
            hg = heads // world
            by_heads = sp.seq_to_heads(mine, h)
            ok = torch.equal(by_heads, whole[:, rank * hg:(rank + 1) * hg])
            ok = ok and torch.equal(sp.heads_to_seq(by_heads, h), mine)
            ok = ok and torch.equal(sp.gather_sequence(mine, h), whole)
            for step in (1, world - 1, world):
                src = (rank - step) % world
                ok = ok and torch.equal(sp.ring_shift(mine, h, step=step), whole[src * s_local:(src + 1) * s_local])
        elif what == "strategies":
            from purlin_b200.parallel import data_parallel as dp
            torch.manual_seed(0)
            model = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Tanh(), torch.nn.Linear(40, 8))
            buckets = dp.GradientBuckets(model.parameters(), h, bucket_bytes=2048)
            ok = len(buckets.buckets) >= 2
            for step in range(2):
                buckets.zero()
                g = torch.Generator().manual_seed(10 * step + rank)
                model(torch.randn(16, 24, generator=g)).square().mean().backward()
                want = []
                for p in model.parameters():
                    t = p.grad.detach().clone()
                    dist.all_reduce(t)
                    want.append(t / world)
                buckets.reduce(average=True)
                ok = ok and all(torch.allclose(p.grad, t, rtol=1e-5, atol=1e-7) for p, t in zip(model.parameters(), want))
            sh = dp.ShardedFlatParameter(100 * world + 3, torch.float32, h)
            sh.shard.fill_(float(rank + 1))
            full = sh.gather()
            ok = ok and full.numel() == 100 * world + 3
            for peer in range(world):
                ok = ok and bool(torch.all(sh.full.tensor[peer * sh.slice_elems:(peer + 1) * sh.slice_elems] == float(peer + 1)))
            sh.grad_full.tensor.copy_(torch.arange(sh.slice_elems * world, dtype=torch.float32) % 5 + rank)
            got = sh.reduce_scatter_grad(average=False)
            base = torch.arange(sh.slice_elems * world, dtype=torch.float32)[rank * sh.slice_elems:(rank + 1) * sh.slice_elems] % 5
            ok = ok and torch.equal(got, base * world + sum(range(world)))
            # the same surface on 16-bit elements
            st = purlin.symm_empty((64 * world,), torch.bfloat16, h)
            st.tensor.fill_(float(rank + 1))
            purlin.all_reduce_symm(st)
            ok = ok and bool(torch.all(st.tensor == float(sum(range(1, world + 1)))))
            st.tensor.zero_()
            st.tensor[rank * 64:(rank + 1) * 64] = float(rank + 7)
            purlin.all_gather_symm(st)
            ok = ok and all(bool(torch.all(st.tensor[peer * 64:(peer + 1) * 64] == float(peer + 7))) for peer in range(world))
        purlin.finalize(h, 0)
        purlin.finalize(h, 0)   # idempotent
        q.put((rank, bool(ok), ""))
    except Exception as e:   # surface the failure in the parent
        import traceback
        q.put((rank, False, traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("what,world", [("all_reduce", 2), ("all_gather", 2), ("others", 2), ("sequence_parallel", 2),
                                        ("sequence_parallel", 3), ("others", 3), ("strategies", 2), ("strategies", 3)])
def test_gloo_world2(what, world):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, what, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(60)
    for rank, ok, err in results:
        assert ok, f"rank {rank}: {err}"
