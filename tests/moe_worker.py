"""One rank of the MoE dispatch/combine correctness run (also runs alone as a world of one)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from purlin_b200.parallel.expert_parallel import ExpertParallelContext  # noqa: E402


def run(rank, world, dev, tokens=512, hidden=1024, experts=64, topk=8, iters=3):
    group = dist.group.WORLD if world > 1 else None
    ep = ExpertParallelContext(group, dev, max_tokens=tokens, hidden=hidden, experts=experts, topk=topk, timeout_ms=5000)
    fails = []
    epr = experts // world
    for it in range(iters):
        g = torch.Generator(device=dev).manual_seed(11 + 100 * it + rank)
        logits = torch.randn(tokens, experts, generator=g, device=dev)
        x = torch.randn(tokens, hidden, generator=g, device=dev).to(torch.bfloat16)
        idx, w = ep.route(logits)
        # routing against torch
        probs = torch.softmax(logits, dim=-1)
        tw, ti = torch.topk(probs, topk, dim=-1)
        tw = tw / tw.sum(-1, keepdim=True)
        if not torch.equal(torch.sort(idx.long(), dim=-1).values, torch.sort(ti, dim=-1).values):
            fails.append(f"it{it}: top-k ids differ")
        if not torch.allclose(torch.sort(w, dim=-1).values, torch.sort(tw, dim=-1).values, atol=1e-5, rtol=1e-4):
            fails.append(f"it{it}: gate weights differ")
        recv, counts = ep.dispatch(x)
        ep.check()
        counts_h = counts.cpu()
        total = int(counts_h[epr])
        # every rank knows who sent what: gather (expert id) histograms to check the counts
        hist = torch.bincount(idx.flatten().long(), minlength=experts)
        hists = [torch.zeros_like(hist) for _ in range(world)]
        if world > 1:
            dist.all_gather(hists, hist)
        else:
            hists = [hist]
        want = sum(hists)[rank * epr:(rank + 1) * epr].cpu()
        if not torch.equal(counts_h[:epr].long(), want):
            fails.append(f"it{it}: receive counts differ")
        # the experts: expert e scales its rows by (e + 1) / 16, so the combined result has a closed form
        offs = torch.cumsum(torch.cat([torch.zeros(1, dtype=torch.long), counts_h[:epr].long()]), 0)
        out = ep.out_rows()
        for e in range(epr):
            a, b = int(offs[e]), int(offs[e + 1])
            out[a:b] = (recv[a:b].float() * ((rank * epr + e + 1) / 16.0)).to(torch.bfloat16)
        # rows of one expert: the multiset of rows received must equal the rows routed there by all ranks
        if it == 0:
            xs = [torch.empty_like(x) for _ in range(world)]
            ids = [torch.empty_like(idx) for _ in range(world)]
            if world > 1:
                dist.all_gather(xs, x); dist.all_gather(ids, idx.contiguous())
            else:
                xs, ids = [x], [idx]
            e = 0
            a, b = int(offs[e]), int(offs[e + 1])
            sent = torch.cat([xs[s][(ids[s] == rank * epr + e).any(-1)] for s in range(world)])
            got = recv[a:b]
            if sent.shape != got.shape or not torch.equal(torch.sort(sent.float().sum(-1)).values, torch.sort(got.float().sum(-1)).values):
                fails.append(f"it{it}: rows of expert {rank * epr} differ")
        y = ep.combine(tokens)
        ep.check()
        scale = ((idx.float() + 1) / 16.0 * w).unsqueeze(-1)                       # [T, k, 1]
        xe = (x.float().unsqueeze(1) * ((idx.float() + 1) / 16.0).unsqueeze(-1)).to(torch.bfloat16).float()   # expert output rounding
        ref = (xe * w.unsqueeze(-1)).sum(1)
        err = (y.float() - ref).abs().max().item()
        if err > 2e-2 * ref.abs().max().item() + 1e-3:
            fails.append(f"it{it}: combine error {err}")
        if total != tokens * topk * world // world and world == 1:
            fails.append(f"it{it}: total rows {total}")
    ep.close()
    return fails


def main():
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    fails = run(rank, world, dev)
    ok = torch.tensor([0 if fails else 1], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    for f in fails:
        print(f"[rank {rank}] FAIL {f}", flush=True)
    if rank == 0:
        print(f"moe worker world {world}: all ranks ok: {bool(ok.item())}", flush=True)
    if world > 1:
        dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
