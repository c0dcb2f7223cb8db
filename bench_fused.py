"""Fused paths against their rooflines and against the unfused NCCL + cuBLAS composition.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench_fused.py [--what tp,moe]

Tensor parallel (Llama-3-70B MLP at TP = world): all-gather->GEMM over activations [8192, 8192] sharded by sequence with
W_gate|W_up per rank [2 * 28672 / world, 8192]; GEMM->reduce-scatter with W_down per rank [8192, 28672 / world].
MoE (DeepSeek-V3-like): 4096 tokens per rank, hidden 7168, 256 experts, top-8; dispatch fused with the permute, combine
fused with the gate-weighted sum. Seeds follow the benchmark configurations (3 for TP, 11 for the gating logits).

Roofline of a fused path = the slower of (FLOPs / measured cuBLAS bf16 peak) and (bytes that must cross NVLink per
GPU / 770 GB/s, the measured peer-copy rate). Times are CUDA-event device times, max over ranks. One JSON line per
measurement on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from purlin_b200.models.tp_mlp import TensorParallelMLP  # noqa: E402
from purlin_b200.parallel.expert_parallel import ExpertParallelContext  # noqa: E402
from purlin_b200.utils.bench import measure  # noqa: E402

LINK_GBPS = 770.0


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


ROWS = []      # every row emitted by this process (bench.py reads them back instead of parsing stdout)
QUIET = False


def emit(rank, **kw):
    ROWS.append(kw)
    if rank == 0 and not QUIET:
        print(json.dumps(kw), flush=True)


def bench_tp(rank, world, dev, args):
    T, H, I = 8192, 8192, 28672
    burst, sustained, how = peaks()
    mlp = TensorParallelMLP(H, I, T, group=dist.group.WORLD if world > 1 else None, device=dev, seed=3)
    tp = mlp.tp
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x_local = torch.randn(T // world, H, generator=g, device=dev).to(torch.bfloat16)
    h = mlp.h
    y = torch.empty(T // world, H, dtype=torch.bfloat16, device=dev)
    il = I // world
    # ---- all-gather -> GEMM (+ SwiGLU) ----
    t = measure(lambda: tp.ag_gemm(x_local, mlp.w_gu, h, swiglu=True), args.warmup, args.runs)
    tp.check()
    flops = 2.0 * T * H * 2 * il
    link_bytes = (world - 1) / world * T * H * 2
    roof_us = max(flops / (burst * 1e12), link_bytes / (LINK_GBPS * 1e9)) * 1e6
    emit(rank, path="all_gather->GEMM(gate|up)+SwiGLU", world=world, shape=[T, 2 * il, H], us=round(t.us, 1), tflops_per_gpu=round(flops / t.us / 1e6, 1),
         roofline_us=round(roof_us, 1), roofline_frac=round(roof_us / t.us, 3), peak=f"{how} cuBLAS burst {burst} TFLOPS; link {LINK_GBPS} GB/s")
    # unfused: NCCL all-gather, then cuBLAS GEMMs and an eager SwiGLU
    xs = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    wg, wu = mlp.w_gate, mlp.w_up

    def unfused_ag():
        if world > 1:
            dist.all_gather_into_tensor(xs, x_local)
        else:
            xs.copy_(x_local)
        return torch.nn.functional.silu(xs @ wg.t()) * (xs @ wu.t())
    tu = measure(unfused_ag, args.warmup, args.runs)
    emit(rank, path="unfused: nccl all_gather + cuBLAS x2 + silu*mul", world=world, us=round(tu.us, 1), speedup_of_fused=round(tu.us / t.us, 2))
    # ---- GEMM -> reduce-scatter ----
    t2 = measure(lambda: tp.gemm_rs(h, mlp.w_down, y), args.warmup, args.runs)
    tp.check()
    flops2 = 2.0 * T * il * H
    roof2 = max(flops2 / (burst * 1e12), link_bytes / (LINK_GBPS * 1e9)) * 1e6
    emit(rank, path="GEMM(down)->reduce_scatter", world=world, shape=[T, H, il], us=round(t2.us, 1), tflops_per_gpu=round(flops2 / t2.us / 1e6, 1),
         roofline_us=round(roof2, 1), roofline_frac=round(roof2 / t2.us, 3))
    full = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def unfused_rs():
        torch.matmul(h, mlp.w_down.t(), out=full)
        if world > 1:
            dist.reduce_scatter_tensor(y, full)
    tu2 = measure(unfused_rs, args.warmup, args.runs)
    emit(rank, path="unfused: cuBLAS + nccl reduce_scatter", world=world, us=round(tu2.us, 1), speedup_of_fused=round(tu2.us / t2.us, 2))
    # ---- the whole block ----
    t3 = measure(lambda: mlp.forward(x_local, y), args.warmup, args.runs)
    tp.check()
    flops3 = mlp.flops(T) / world
    roof3 = max(flops3 / (sustained * 1e12), 2 * link_bytes / (LINK_GBPS * 1e9)) * 1e6
    emit(rank, path="MLP block (both fused kernels)", world=world, us=round(t3.us, 1), tflops_per_gpu=round(flops3 / t3.us / 1e6, 1),
         roofline_us=round(roof3, 1), roofline_frac=round(roof3 / t3.us, 3), peak=f"{how} cuBLAS sustained {sustained} TFLOPS")
    tp.close()


def bench_moe(rank, world, dev, args, unfused=True):
    T, H, E, K = 4096, 7168, 256, 8
    ep = ExpertParallelContext(dist.group.WORLD if world > 1 else None, dev, max_tokens=T, hidden=H, experts=E, topk=K, capacity_factor=1.5)
    g = torch.Generator(device=dev).manual_seed(11 + rank)
    logits = torch.randn(T, E, generator=g, device=dev)
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    idx, w = ep.route(logits)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    # Bytes that must cross NVLink: one row per (token, destination GPU) with the destination != this rank (a token
    # routed to several experts of one GPU travels once). The count per (token, expert) pair is reported beside it.
    epr = E // world
    dest = idx // epr                                                       # [T, K]
    onehot = torch.zeros(T, world, dtype=torch.bool, device=dev)
    onehot.scatter_(1, dest.long(), True)
    onehot[:, rank] = False
    remote = int(onehot.sum().item())
    remote_pairs = int((dest != rank).sum().item())
    rt = torch.tensor([remote, remote_pairs], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(rt, op=dist.ReduceOp.MAX)
    link_bytes = float(rt[0].item()) * H * 2
    pair_bytes = float(rt[1].item()) * H * 2
    hbm_bytes = 2.0 * T * K * H * 2            # every expert row is written once on dispatch and read once on combine
    roof_us = max(link_bytes / (LINK_GBPS * 1e9), hbm_bytes / 6.5e12) * 1e6
    pair_roof_us = max(pair_bytes / (LINK_GBPS * 1e9), hbm_bytes / 6.5e12) * 1e6

    def both():
        ep.dispatch(x)
        ep.combine(T, y)
    ep.dispatch(x)
    ep.out_rows().copy_(ep.recv_rows())    # identity experts: the combine reads real rows
    ep.combine(T, y)
    ep.check()
    # dispatch and combine alternate by contract, so each is timed inside the pair and the pair is split by two extra runs
    t_pair = measure(both, args.warmup, args.runs)
    ep.check()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    d_us, c_us = 0.0, 0.0
    for _ in range(args.runs):
        ev[0].record(); ep.dispatch(x); ev[1].record(); ep.combine(T, y); ev[2].record()
        ev[2].synchronize()
        d_us += ev[0].elapsed_time(ev[1]) * 1e3
        c_us += ev[1].elapsed_time(ev[2]) * 1e3
    tt = torch.tensor([d_us / args.runs, c_us / args.runs], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    d_us, c_us = float(tt[0]), float(tt[1])
    # optional: the same split for other CTA counts of the pushing roles ("senders:pushers,...")
    for pair in [c for c in getattr(args, "moe_sweep", "").split(",") if c]:
        os.environ["PURLIN_MOE_SENDERS"], os.environ["PURLIN_MOE_PUSHERS"] = pair.split(":")
        for _ in range(3):
            both()
        sd, sc = 0.0, 0.0
        for _ in range(args.runs):
            ev[0].record(); ep.dispatch(x); ev[1].record(); ep.combine(T, y); ev[2].record()
            ev[2].synchronize()
            sd += ev[0].elapsed_time(ev[1]) * 1e3
            sc += ev[1].elapsed_time(ev[2]) * 1e3
        st = torch.tensor([sd / args.runs, sc / args.runs], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        emit(rank, path="MoE CTA sweep", world=world, senders=int(os.environ["PURLIN_MOE_SENDERS"]), pushers=int(os.environ["PURLIN_MOE_PUSHERS"]),
             dispatch_us=round(float(st[0]), 1), combine_us=round(float(st[1]), 1))
    if getattr(args, "moe_sweep", ""):
        os.environ.pop("PURLIN_MOE_SENDERS", None)
        os.environ.pop("PURLIN_MOE_PUSHERS", None)
    emit(rank, path="MoE dispatch (+permute)", world=world, tokens_per_rank=T, hidden=H, experts=E, topk=K, us=round(d_us, 1),
         roofline_us=round(roof_us, 1), roofline_frac=round(roof_us / d_us, 3), link_GB=round(link_bytes / 1e9, 3),
         achieved_link_GBps=round(link_bytes / d_us / 1e3, 1), per_pair_link_GB=round(pair_bytes / 1e9, 3),
         frac_of_per_pair_roofline=round(pair_roof_us / d_us, 3))
    emit(rank, path="MoE combine (+gate-weighted sum)", world=world, us=round(c_us, 1), roofline_us=round(roof_us, 1),
         roofline_frac=round(roof_us / c_us, 3), achieved_link_GBps=round(link_bytes / c_us / 1e3, 1),
         frac_of_per_pair_roofline=round(pair_roof_us / c_us, 3))
    emit(rank, path="MoE dispatch+combine pair", world=world, us=round(t_pair.us, 1), roofline_frac=round(2 * roof_us / t_pair.us, 3))
    if os.environ.get("PURLIN_MOE_TIMING"):
        # device-side phase times of one pair (max over ranks): where the senders / pushers and the receivers / finishers end
        ep.timing()
        if world > 1:
            dist.barrier()
        both()
        ph = ep.timing()
        flat = [ph["dispatch"]["first_sender"], ph["dispatch"]["last_sender"], ph["dispatch"]["last_receiver"],
                ph["combine"]["first_pusher"], ph["combine"]["last_pusher"], ph["combine"]["last_finisher"]]
        pt = torch.tensor(flat, device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
        names = ("dispatch_first_sender_us", "dispatch_last_sender_us", "dispatch_last_receiver_us",
                 "combine_first_pusher_us", "combine_last_pusher_us", "combine_last_finisher_us")
        emit(rank, path="MoE phases (device clock, from each kernel's first CTA)", world=world,
             **{n: round(float(v), 1) for n, v in zip(names, pt.tolist())})
    # unfused baseline: sort rows by destination, NCCL all-to-all of the counts and of the rows, and back, then a weighted sum
    if world > 1 and unfused:
        flat = idx.flatten().long()
        order = torch.argsort(flat // epr * E + flat, stable=True)
        rows = x.repeat_interleave(K, dim=0)
        send_counts = torch.bincount(flat // epr, minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv = torch.empty(sum(rc), H, dtype=torch.bfloat16, device=dev)
        back = torch.empty(sum(sc), H, dtype=torch.bfloat16, device=dev)

        def unfused():
            permuted = rows[order]
            dist.all_to_all_single(recv, permuted, rc, sc)
            dist.all_to_all_single(back, recv, sc, rc)
            un = torch.empty_like(back)
            un[order] = back
            return (un.view(T, K, H).float() * w.unsqueeze(-1)).sum(1).to(torch.bfloat16)
        tu = measure(unfused, 2, max(args.runs // 2, 3))
        emit(rank, path="unfused: permute + nccl all_to_all x2 + unpermute + weighted sum", world=world, us=round(tu.us, 1),
             speedup_of_fused=round(tu.us / t_pair.us, 2))
    ep.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="tp,moe")
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--moe-sweep", default="", help='extra MoE rows for other CTA counts: "senders:pushers,senders:pushers"')
    ap.add_argument("--no-unfused", action="store_true", help="skip the NCCL + torch compositions")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    if "tp" in args.what:
        bench_tp(rank, world, dev, args)
    if "moe" in args.what:
        bench_moe(rank, world, dev, args, unfused=not args.no_unfused)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
