"""Headline benchmark: one Llama-3-70B MLP block under tensor + sequence parallelism, collectives fused into the GEMMs.

  python bench.py --gpus 1 --steps 20 --warmup 5
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Step = all-gather->GEMM (gate|up, SwiGLU epilogue) + GEMM->reduce-scatter (down) over 8192 tokens, hidden 8192,
intermediate 28672 split over the N ranks (strong scaling: the whole job's work is fixed).  Rank 0 prints one JSON
line: tokens/s of the whole job (device-timed, max over ranks), the fraction of the measured bf16 GEMM roofline,
an end-to-end figure through the public API including the host->device copy of each step's activations and the
device->host read of a result scalar, the clocks sampled during the timed region, and, for N >= 2, bus GB/s of
the stand-alone collectives against NCCL at a few message sizes.

`--impl reference` runs the unmodified reference package from baseline/_ref through its own entry point.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TOKENS, HIDDEN, INTERMEDIATE = 8192, 8192, 28672
METRIC = "llama3_70b_mlp_fused_tp_tokens_per_s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops_sustained"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 1400.0, 1590.0, "fallback"


class ClockSampler:
    """Reads SM clocks and throttle reasons through NVML (read-only) on a thread while a timed region runs.

    It lives in this file so that the reference arm imports nothing of this repository's package. One sampler can
    bracket several regions (``with sampler: ...`` more than once); the samples accumulate.
    """

    def __init__(self, index=0, period_s=0.001):
        import threading
        self.samples, self.reasons, self.max_mhz = [], set(), 0
        self.period = period_s
        self._stop, self._thread, self._threading = threading.Event(), None, threading
        self._nvml = self._handle = None
        self._names = {}
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                self._handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except Exception:
                self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self._names = {
                pynvml.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
                pynvml.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                pynvml.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            }
            self._sample()          # warms the NVML calls; dropped
            self.samples.clear()
            self.reasons.clear()
        except Exception as e:
            self._nvml = None
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def _sample(self):
        self.samples.append(self._nvml.nvmlDeviceGetClockInfo(self._handle, self._nvml.NVML_CLOCK_SM))
        r = self._nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        for bit, n in self._names.items():
            if r & bit:
                self.reasons.add(n)

    def _run(self):
        try:
            while not self._stop.is_set():
                self._sample()
                self._stop.wait(self.period)
        except Exception as e:
            self.reasons.add(f"nvml_error:{type(e).__name__}")

    def __enter__(self):
        if self._nvml is not None:
            self._stop.clear()
            self._thread = self._threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(2.0)
            self._thread = None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else 0, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def run_reference(args):
    """The same metric on the unmodified reference: its Python API (purlin.initialize / all_gather / reduce_scatter from
    baseline/_ref) around cuBLAS GEMMs, which is how a user of the reference runs this block, since the reference has no
    GEMM of its own. Its binding module cannot be built by its own CMake project without a network; it is built once,
    offline, by baseline/build_reference_module.py from the reference's own sources and found through the reference's own
    JIT cache. Prints one JSON line with "impl": "reference", or the reason the arm is unavailable."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)

    ref = os.path.join(ROOT, "baseline", "_ref")
    cache = os.path.join(ROOT, "baseline", "_ref_cache")
    if not os.path.isdir(os.path.join(ref, "purlin")):
        return unavailable("baseline/_ref is absent (reference not installed)")
    try:
        sys.path.insert(0, ref)
        import purlin as reference                     # the reference's package, unmodified
        from purlin import jit
        from purlin.bindings import purlin_bindings
        key = jit._cache_key(100, purlin_bindings.substitute(mod_name="purlin_1000"), "purlin_1000")
    except Exception as e:   # never fail the arm
        return unavailable(f"the reference package could not be imported: {type(e).__name__}: {e}")
    if not os.path.exists(os.path.join(cache, key, "purlin_1000.so")):
        return unavailable("the reference builds its binding at first use through CMake + CPM downloads (CPM itself, CCCL, NVTX, "
                           "pybind11), which needs a network; the offline build (baseline/build_reference_module.py) has not been run")
    if world == 1:
        return unavailable("at one GPU the block has no collective, so nothing of the reference would run (it has no GEMM)")
    try:
        os.environ["PURLIN_CACHE_DIR"] = cache
        _reference_arm(args, reference, rank, world)
    except Exception as e:
        unavailable(f"the reference arm failed: {type(e).__name__}: {str(e)[:300]}")


def _reference_arm(args, reference, rank, world):
    """All-gather (reference) -> gate/up GEMMs + SwiGLU (torch) -> down GEMM (torch) -> reduce-scatter (reference)."""
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)
    stream = torch.cuda.current_stream().cuda_stream
    h = reference.initialize(dist.group.WORLD, dev, 100, stream)
    T, rows, inter = args.tokens, args.tokens // world, INTERMEDIATE // world
    g = torch.Generator(device=dev).manual_seed(3 * 1000 + rank)

    def init(r, c):
        return (torch.randn(r, c, generator=g, device=dev) * 0.02).to(torch.bfloat16)

    w_gate, w_up, w_down = init(inter, HIDDEN), init(inter, HIDDEN), init(HIDDEN, inter)
    gc = torch.Generator(device="cpu").manual_seed(3 + rank)
    x_host = torch.randn(rows, HIDDEN, generator=gc).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev, non_blocking=True)
    x_full = torch.empty(T, HIDDEN, dtype=torch.bfloat16, device=dev)
    y = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=dev)
    result_host = torch.zeros(1, dtype=torch.float32).pin_memory()

    def step():
        reference.all_gather(x_dev, x_full, h, stream)
        mid = torch.nn.functional.silu(x_full @ w_gate.t()) * (x_full @ w_up.t())
        part = mid @ w_down.t()
        reference.reduce_scatter(part, y, h, stream)

    def barrier():
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        step()
    clocks = ClockSampler(local)
    barrier()
    with clocks:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        b.synchronize()
        barrier()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        step()
        result_host.copy_(torch.linalg.vector_norm(y, dtype=torch.float32).reshape(1), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    with clocks:
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        for _ in range(args.steps):
            e2e_step()
        eb.record()
        eb.synchronize()
        barrier()
    te = torch.tensor([ea.elapsed_time(eb)], dtype=torch.float64, device=dev)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te.item()) / args.steps
    reference.finalize(h, stream)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": round(T / (ms_per_step * 1e-3), 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (activations N(0,1) seed 3+rank, weights N(0,0.02) seed 3; random-init)",
            "config": {"model": "Llama-3-70B MLP block (hidden 8192, intermediate 28672): reference all_gather -> cuBLAS GEMMs + SwiGLU "
                                "-> reference reduce_scatter", "global_batch": T, "seq_len": T, "parallelism": f"tp{world}+sp",
                       "l2": "weights read every step exceed the 126 MB L2 (no flush needed)"},
            "clocks": clocks.summary(),
            "e2e": {"value": round(T / (e2e_ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": x_host.numel() * x_host.element_size(), "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "impl": "reference",
        }), flush=True)
    dist.destroy_process_group()


def collective_samples(purlin, dist, dev, world, steps):
    """Bus GB/s of the stand-alone collectives vs NCCL at a few sizes (device-timed, max over ranks), each compared
    exactly with the NCCL result on integer-valued inputs before it is timed."""
    import torch
    from purlin_b200.utils import bench
    h = purlin.initialize(dist.group.WORLD, dev, 100, None)
    rank = dist.get_rank()
    rows = []

    def sample(name, key, n, ours, nccl, out, ref):
        runs = max(steps // 2, 5) if n <= (32 << 20) else 5
        out.fill_(-7)
        ours()
        nccl()
        purlin.check(h)
        ok = torch.tensor([1 if torch.equal(out, ref) else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        t = bench.measure(ours, 5, runs)
        tn = bench.measure(nccl, 5, runs)
        f = bench.bus_factor(key, world)
        total = bench.logical_bytes(key, n, world) if key != "ar" else n
        rows.append({"collective": name, "bytes": total, "us": round(t.us, 2), "busbw_GBps": round(total / t.us / 1e3 * f, 2),
                     "nccl_us": round(tn.us, 2), "nccl_busbw_GBps": round(total / tn.us / 1e3 * f, 2), "correct": bool(ok.item())})

    for n in (8 << 10, 512 << 10, 32 << 20, 256 << 20):
        x = ((torch.arange(n // 2, device=dev) + rank) % 5).to(torch.bfloat16)
        out, ref = torch.empty_like(x), torch.empty_like(x)
        sample("all_reduce", "ar", n, lambda: purlin.all_reduce(x, out, h, None), lambda: (ref.copy_(x), dist.all_reduce(ref)), out, ref)
    for n in (512 << 10, 32 << 20):      # bytes per rank
        per = n // world // 32 * 32
        x = ((torch.arange(per // 2, device=dev) + 3 * rank) % 7).to(torch.bfloat16)
        out, ref = torch.empty(per // 2 * world, dtype=torch.bfloat16, device=dev), torch.empty(per // 2 * world, dtype=torch.bfloat16, device=dev)
        sample("all_gather", "ag", per, lambda: purlin.all_gather(x, out, h, None), lambda: dist.all_gather_into_tensor(ref, x), out, ref)
        xin = ((torch.arange(per // 2 * world, device=dev) + rank) % 5).to(torch.bfloat16)
        o2, r2 = torch.empty(per // 2, dtype=torch.bfloat16, device=dev), torch.empty(per // 2, dtype=torch.bfloat16, device=dev)
        sample("reduce_scatter", "rs", per, lambda: purlin.reduce_scatter(xin, o2, h, None), lambda: dist.reduce_scatter_tensor(r2, xin), o2, r2)
        o3, r3 = torch.empty_like(xin), torch.empty_like(xin)
        sample("all_to_all", "a2a", per, lambda: purlin.all_to_all(xin, o3, h, None), lambda: dist.all_to_all_single(r3, xin), o3, r3)
    purlin.finalize(h)
    return rows


def moe_samples(dist, dev, rank, world):
    """MoE dispatch / combine at the DeepSeek-V3-like shape (4096 tokens per rank, hidden 7168, 256 experts, top-8):
    microseconds and fractions of the roofline over de-duplicated NVLink bytes (device-timed, max over ranks)."""
    import bench_fused

    class A:
        warmup, runs = 3, 10
    bench_fused.QUIET = True
    del bench_fused.ROWS[:]
    had = os.environ.get("PURLIN_MOE_TIMING")
    os.environ["PURLIN_MOE_TIMING"] = "1"          # the kernels stamp where their CTA roles end (one extra row, device clock)
    try:
        bench_fused.bench_moe(rank, world, dev, A, unfused=False)
    finally:
        if had is None:
            os.environ.pop("PURLIN_MOE_TIMING", None)
        else:
            os.environ["PURLIN_MOE_TIMING"] = had
    keep = ("path", "us", "roofline_us", "roofline_frac", "link_GB", "achieved_link_GBps", "per_pair_link_GB", "frac_of_per_pair_roofline")
    return [{k: v for k, v in r.items() if k in keep or k.endswith("_us")} for r in bench_fused.ROWS]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=TOKENS)
    ap.add_argument("--no-collectives", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    import purlin_b200 as purlin
    from purlin_b200.models.tp_mlp import TensorParallelMLP

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} processes (found WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world, device_id=dev)

    T = args.tokens
    mlp = TensorParallelMLP(HIDDEN, INTERMEDIATE, T, group=dist.group.WORLD if world > 1 else None, device=dev, seed=3)
    rows_local = T // world
    g = torch.Generator(device="cpu").manual_seed(3 + rank)
    x_host = torch.randn(rows_local, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev, non_blocking=True)
    y = torch.empty(rows_local, HIDDEN, dtype=torch.bfloat16, device=dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def step():
        mlp.forward(x_dev, y)

    for _ in range(args.warmup):
        step()
    mlp.tp.check()

    # ---- device-timed region: exactly `steps` steps, one event pair per rank, max over ranks ----
    clocks = ClockSampler(local)   # NVML is brought up here, outside the timed region
    barrier()
    with clocks:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        b.synchronize()
        barrier()
    ms = a.elapsed_time(b)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    mlp.tp.check()

    # ---- end to end through the public API (TensorParallelMLP.run_host_batches): every step copies its activations
    # from pinned host memory to the device and returns its metric to the host; the copies overlap the neighbouring steps
    x_host2 = torch.randn(rows_local, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()

    def host_batches(n):
        for i in range(n):
            yield x_host if i % 2 == 0 else x_host2

    mlp.run_host_batches(host_batches(3), out=y)
    barrier()
    with clocks:   # same sampler: the clock record covers both timed regions
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        metrics = mlp.run_host_batches(host_batches(args.steps), out=y)
        eb.record()
        eb.synchronize()
        barrier()
    assert len(metrics) == args.steps and all(m == m and m > 0.0 for m in metrics), "every step must return a finite metric"
    e2e_ms = ea.elapsed_time(eb)   # device time from before the first copy to after the last read, host gaps included
    te = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(te.item()) / args.steps

    sustained, burst, how = _peaks()
    flops = mlp.flops(T)
    tflops_per_gpu = flops / world / (ms_per_step * 1e-3) / 1e12
    # Roofline of the fused step per GPU: the slower of compute at the measured GEMM peak and NVLink bytes at 770 GB/s.
    # The burst peak applies when the timed region ran without the power cap (short regions at full clock), the
    # sustained one when the cap was active; both fractions are printed, `roofline_frac` is the one that applies.
    nvlink_bytes = (world - 1) / world * T * HIDDEN * 2 * 2 if world > 1 else 0.0   # gathered rows in + partial rows out
    t_link = nvlink_bytes / 770e9
    capped = "sw_power_cap" in clocks.summary()["reasons"]
    frac_burst = max(flops / world / (burst * 1e12), t_link) / (ms_per_step * 1e-3)
    frac_sustained = max(flops / world / (sustained * 1e12), t_link) / (ms_per_step * 1e-3)
    peak_used = sustained if capped else burst
    t_compute = flops / world / (peak_used * 1e12)

    # ---- correctness of what was timed, outside the timed regions: one fused MLP output against the fp32 PyTorch
    # reference of the same block (partial products all-reduced over the ranks)
    fused_correct, fused_err = None, None
    try:
        y_chk = mlp.forward(x_dev, y).float()
        mlp.tp.check()
        if world > 1:
            xs = [torch.empty_like(x_dev) for _ in range(world)]
            dist.all_gather(xs, x_dev)
            part = mlp.reference(torch.cat(xs))
            dist.all_reduce(part)
            ref = part[rank * rows_local:(rank + 1) * rows_local]
            del part, xs
        else:
            ref = mlp.reference(x_dev)
        err = (y_chk - ref).abs().max()
        ok_t = (err <= 3e-2 * ref.abs().max() + 1e-3).to(torch.int32)
        if world > 1:
            dist.all_reduce(ok_t, op=dist.ReduceOp.MIN)
        fused_correct, fused_err = bool(ok_t.item()), float(err.item())
        del ref, y_chk
    except Exception as e:
        fused_correct, fused_err = False, f"{type(e).__name__}: {e}"

    collectives = None
    if world > 1 and not args.no_collectives:
        try:
            collectives = collective_samples(purlin, dist, dev, world, args.steps)
        except Exception as e:   # the headline number must survive a failure here
            collectives = {"error": f"{type(e).__name__}: {e}"}
    moe = None
    if world > 1 and not args.no_collectives:
        try:
            moe = moe_samples(dist, dev, rank, world)
        except Exception as e:
            moe = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        line = {
            "metric": METRIC,
            "value": round(T / (ms_per_step * 1e-3), 1),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic (activations N(0,1) seed 3+rank, weights N(0,0.02) seed 3; random-init)",
            "config": {"model": "Llama-3-70B MLP block (hidden 8192, intermediate 28672), all-gather->GEMM + SwiGLU + GEMM->reduce-scatter",
                       "global_batch": T, "seq_len": T, "parallelism": f"tp{world}+sp",
                       "l2": "weights read every step exceed the 126 MB L2 (no flush needed)"},
            "tflops_per_gpu": round(tflops_per_gpu, 1),
            "roofline_frac": round(frac_sustained if capped else frac_burst, 4),
            "roofline": {"peak_tflops": peak_used, "peak_source": how + (" cuBLAS bf16 sustained (power cap active)" if capped else " cuBLAS bf16 burst (no power cap in the timed region)"),
                         "frac_of_burst_peak": round(frac_burst, 4), "frac_of_sustained_peak": round(frac_sustained, 4), "nvlink_GBps": 770,
                         "compute_ms": round(t_compute * 1e3, 4), "link_ms": round(t_link * 1e3, 4)},
            "fused_correct": fused_correct, "fused_max_abs_err": fused_err,
            "clocks": clocks.summary(),
            "e2e": {"value": round(T / (e2e_ms_per_step * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms_per_step, 4),
                    "h2d_bytes_per_step": mlp._feed.h2d_bytes_per_step, "d2h_bytes_per_step": mlp._feed.d2h_bytes_per_step,
                    "api": "TensorParallelMLP.run_host_batches (HostFeed: the copy of step i+1 and the read of step i-1 overlap step i)"},
            "gpu_launches": 2 * args.steps,
            "impl": "ours",
        }
        if collectives is not None:
            line["collectives"] = collectives
        if moe is not None:
            line["moe"] = moe
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
