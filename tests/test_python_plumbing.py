"""Python binding surface on the CPU with a recording stand-in for the native library.

Counterpart of tests/test_python_plumbing.py in the reference: wrappers forward exact pointers, byte counts,
element types, context, stream and reduction mode; initialize asks the provider for the reference's workspace size
and forwards the multicast pointer; finalize is idempotent; non-contiguous tensors and bad modes are rejected.
"""
import ctypes as C
import os

import pytest
import torch

import purlin_b200 as purlin
from purlin_b200 import _native


class RecordingLib:
    """Looks like the ctypes library to the wrappers; records every native call."""

    def __init__(self):
        self.calls = []
        self.destroyed = 0

    def purlin_collective(self, ctx, coll, src, dst, nbytes, sizes, out_sizes, dtype, op, mode, policy, stream):
        self.calls.append(dict(ctx=ctx, coll=int(coll), src=src, dst=dst, nbytes=nbytes,
                               sizes=None if sizes is None else list(sizes), out_sizes=None if out_sizes is None else list(out_sizes),
                               dtype=int(dtype), op=int(op), mode=int(mode), policy=policy, stream=stream))
        return 0

    def purlin_call_fixed(self, ctx, coll, src, dst, nbytes, traits, stream):
        # the short signature of the fixed-size collectives: traits = dtype | op << 8 | mode << 16
        return self.purlin_collective(ctx, coll, src, dst, nbytes, None, None, traits & 0xff, (traits >> 8) & 0xff, traits >> 16, None, stream)

    def purlin_context_create(self, rank, world, ptrs, mc, staging, timeout, stream):
        self.calls.append(dict(create=True, rank=rank, world=world, ptrs=list(ptrs), mc=mc, staging=staging, stream=stream))
        return 0xC0FFEE

    def purlin_context_destroy(self, ctx, stream):
        self.destroyed += 1
        return 0

    def purlin_context_has_multicast(self, ctx):
        return 1

    def purlin_last_error(self):
        return b"recorded"

    def purlin_tuning_add(self, *a):
        return 0


def make_handle(world=4, rank=1):
    lib = RecordingLib()
    h = purlin.ContextHandle(lib, 0xC0FFEE, object(), object(), rank, world, torch.device("cuda", 0), None, 1 << 20, {})
    return lib, h


def test_wrappers_forward_pointers_bytes_types_and_mode():
    lib, h = make_handle(world=4)
    x = torch.zeros(4 * 64, dtype=torch.bfloat16)
    y = torch.zeros(4 * 64, dtype=torch.bfloat16)
    purlin.all_reduce(x, y, h, 77, purlin.ReductionMode.DETERMINISTIC)
    c = lib.calls[-1]
    assert (c["coll"], c["src"], c["dst"], c["nbytes"], c["dtype"], c["mode"], c["stream"], c["ctx"]) == \
           (0, x.data_ptr(), y.data_ptr(), 512, int(purlin.DataType.BF16), 1, 77, 0xC0FFEE)
    purlin.all_gather(x, y, h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["nbytes"]) == (1, 512)
    purlin.all_gather_v(x, y, [32, 64, 96, 128], h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["sizes"]) == (2, [32, 64, 96, 128])
    purlin.reduce_scatter(x, y, h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["nbytes"]) == (3, 128)          # total bytes / world
    purlin.reduce_scatter_v(x.float(), y.float(), [32, 32, 32, 32], h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["dtype"]) == (4, int(purlin.DataType.FP32))
    purlin.all_to_all(x, y, h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["nbytes"]) == (5, 128)
    purlin.all_to_all_v(x, y, [32, 0, 64, 32, 0, 32, 32, 64], h, 5)
    assert (lib.calls[-1]["coll"], lib.calls[-1]["sizes"], lib.calls[-1]["out_sizes"]) == (6, [32, 0, 64, 32], [0, 32, 32, 64])


def test_element_type_map_and_arch():
    assert purlin.buffer_type(torch.float16) == purlin.DataType.FP16
    assert purlin.buffer_type(torch.float8_e4m3fn) == purlin.DataType.FP8_E4M3
    assert purlin.buffer_type(torch.float8_e5m2) == purlin.DataType.FP8_E5M2
    with pytest.raises(TypeError):
        purlin.buffer_type(torch.int32)
    assert [purlin.normalize_arch(a) for a in (70, 80, 90, 100, 103)] == [700, 800, 900, 1000, 1000]


def test_rejections():
    lib, h = make_handle()
    x = torch.zeros(8, 8)
    with pytest.raises(ValueError):
        purlin.all_reduce(x.t(), x, h, 0)                      # non-contiguous
    with pytest.raises(ValueError):
        purlin.all_reduce(x, x, h, 0, reduction_mode=7)         # not a ReductionMode
    with pytest.raises(ValueError):
        purlin.all_gather_v(x, x, [32], h, 0)                   # one entry per rank
    with pytest.raises(ValueError):
        purlin.all_to_all_v(x, x, [32] * 4, h, 0)
    assert not lib.calls


def test_finalize_is_idempotent_and_blocks_later_calls():
    lib, h = make_handle()
    purlin.finalize(h, 3)
    purlin.finalize(h, 3)
    assert lib.destroyed == 1 and h.ctx is None and h.buf is None and h.hdl is None
    with pytest.raises(RuntimeError):
        purlin.all_reduce(torch.zeros(8), torch.zeros(8), h, 0)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_initialize_asks_for_the_reference_workspace_and_forwards_multicast(monkeypatch, world):
    import torch.distributed as dist
    from purlin_b200 import tuning
    from purlin_b200.parallel import symmetric
    lib = RecordingLib()
    asked = {}

    def fake_alloc(nbytes, device, group, provider=None):
        asked["nbytes"] = nbytes
        return "buf", "hdl", [0x1000 * (q + 1) for q in range(world)], 0xABC000

    monkeypatch.setattr(dist, "get_rank", lambda g=None: 1)
    monkeypatch.setattr(dist, "get_world_size", lambda g=None: world)
    monkeypatch.setattr(symmetric, "allocate_symmetric", fake_alloc)
    monkeypatch.setattr(_native, "cuda", lambda: lib)
    monkeypatch.setattr(tuning, "load_for", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "get_device_name", lambda d=None: "NVIDIA B200")
    h = purlin.initialize("group", torch.device("cuda", 0), 100, 1234)
    staging = 2 * (purlin.STAGING_BUFFER_SIZE + purlin.PACKET_EPOCH_BYTES)
    assert staging == 528 << 20                                           # the reference's 528 MiB of staging
    assert asked["nbytes"] >= staging + 3 * world * 8 + 2 * world * 16 and asked["nbytes"] < staging + 4096
    c = lib.calls[0]
    assert c["create"] and c["rank"] == 1 and c["world"] == world and c["mc"] == 0xABC000 and c["stream"] == 1234
    assert c["ptrs"] == [0x1000 * (q + 1) for q in range(world)] and c["staging"] == purlin.STAGING_BUFFER_SIZE
    assert h.ctx == 0xC0FFEE and h.buf == "buf" and h.has_multicast


def test_vmm_provider_fails_cleanly_without_a_driver():
    """On a machine without a CUDA driver the native virtual-memory provider reports an error instead of crashing."""
    import ctypes as C
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is about machines without a GPU")
    from purlin_b200 import _native
    lib = _native.cuda()
    lib.purlin_vmm_create.restype = C.c_void_p
    lib.purlin_vmm_create.argtypes = [C.c_int, C.c_size_t, C.c_int, C.c_int]
    assert not lib.purlin_vmm_create(0, 1 << 20, 0, 2)
    assert "vmm provider" in _native.last_error(lib)
    assert lib.purlin_vmm_multicast_supported(0) == -1


def test_report_pairs_rows_with_the_baseline():
    from purlin_b200.utils import report
    lines = [
        "NCCL version 2.28.9+cuda12.9",
        "collective,impl,world,totalBytes,datatype,lat(us),algbw(GB/s),busbw(GB/s),error(%),GPUName,warmup,runs,graph_launches",
        "# cand rows are comments",
        "ar,purlin_b200,8,1048576,bf16,20.00,52.4,91.7,0.000,NVIDIA B200,-,20,0",
        "ar,purlin_b200:symm-zero-copy,8,1048576,bf16,16.00,65.5,114.7,0.000,NVIDIA B200,-,20,0",
        "ar,nccl,8,1048576,bf16,40.00,26.2,45.9,0.000,NVIDIA B200,-,20,0",
        "ag,purlin_b200,8,8192,bf16,10.00,0.8,0.7,100.000,NVIDIA B200,-,20,0",
    ]
    table = report.parse(lines)
    assert list(table) == [("ar", 1048576), ("ag", 8192)]
    assert table[("ar", 1048576)]["nccl"] == (40.0, 45.9, 0.0)
    text = "\n".join(report.render(table, markdown=True))
    assert "| AllReduce | 1 MiB | 20.0 (91.7) | 16.0 (114.7) | 40.0 (45.9) | 2.00x | 2.50x |" in text
    assert "ERROR 100%" in text and "| AllGather | 8 KiB |" in text


def test_unswept_world_size_borrows_the_nearest_table(tmp_path, monkeypatch):
    import json
    from purlin_b200 import tuning
    monkeypatch.setattr(tuning, "TABLE_DIR", tmp_path)
    monkeypatch.delenv("PURLIN_TUNING_TABLE", raising=False)
    monkeypatch.delenv("PURLIN_NO_TUNING_TABLE", raising=False)
    tuning.clear()
    try:
        def table(world, chunk):
            pol = _native.Policy()
            pol.regime, pol.threads, pol.putBlocks, pol.localBlocks, pol.consumeBlocks, pol.gatherBlocks = 1, 256, 8, 1, 16, 8
            pol.lrBlocks, pol.mmDepth, pol.unroll, pol.arPath, pol.weighted, pol.chunkBytes = 2, 4, 4, 1, 1, chunk
            return {"gpu": "Test GPU", "world": world, "entries": [{"collective": 0, "world": world, "bytes": 1 << 20, "policy": pol.as_dict()}]}
        for world, chunk in ((4, 65536), (8, 131072)):
            with open(tuning.table_path("Test GPU", world), "w") as f:
                json.dump(table(world, chunk), f)
        assert tuning.nearest_table("Test GPU", 6).name.endswith("_w8.json")      # tie between 4 and 8: the larger
        assert tuning.nearest_table("Test GPU", 3).name.endswith("_w4.json")
        assert tuning.nearest_table("Other GPU", 3) is None
        used = tuning.load_for("Test GPU", 6)
        assert used is not None and used.name.endswith("_w8.json")
        _, chosen = purlin.build_plan(purlin.Collective.ALL_REDUCE, 6, 0, 6 * 32 * 4096, staging_size=8 << 20)
        assert chosen.chunkBytes == 131072                                        # the borrowed band is in force at world 6
        _, other = purlin.build_plan(purlin.Collective.ALL_REDUCE, 5, 0, 5 * 32 * 4096, staging_size=8 << 20)
        assert other.chunkBytes != 131072                                         # nothing was installed for world 5
    finally:
        tuning.clear()


def test_reference_arm_always_prints_one_json_line():
    """`bench.py --impl reference` must exit 0 with one JSON line, whatever the state of the reference install."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for env_extra in ({}, {"WORLD_SIZE": "2", "RANK": "0"}):
        env = dict(os.environ, **env_extra)
        env.pop("PURLIN_REFERENCE_ARM", None)
        res = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", env_extra.get("WORLD_SIZE", "1")],
                             capture_output=True, text=True, timeout=300, env=env)
        assert res.returncode == 0, res.stderr[-2000:]
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        assert len(lines) == 1
        rec = json.loads(lines[0])
        assert rec["impl"] == "reference" and ("unavailable" in rec or "value" in rec)


def test_strategies_example_runs_on_cpu():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "examples", "strategies.py"), "--cpu"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-2000:]
    assert "round trip exact: True" in res.stdout and "every entry 2.0" in res.stdout


def test_plan_explainer_prints_roles_and_regions(capsys):
    from purlin_b200 import tuning
    from purlin_b200.utils import explain
    tuning.clear()
    try:
        assert explain.main(["all_reduce", "--world", "4", "--bytes", "8K", "--gpu", ""]) == 0
        text = capsys.readouterr().out
        assert "latency (packets)" in text and "packet-put" in text and "packet-reduce" in text
        assert explain.main(["all_gather", "--world", "8", "--bytes", "4M", "--gpu", ""]) == 0
        text = capsys.readouterr().out
        assert "throughput (staged)" in text and text.count("consume") >= 7 and "stage" in text
        assert explain.main(["all_to_all_v", "--world", "4", "--sizes", "0,64K,1M,32", "--rank", "1", "--gpu", ""]) == 0
        text = capsys.readouterr().out
        assert "arrival handshake" in text and "local" in text
        assert explain.main(["all_gather_v", "--world", "4", "--gpu", ""]) == 2      # sizes are required
    finally:
        tuning.clear()


def test_fastcall_extension_passes_the_seven_scalars_unchanged():
    """The CPython extension of the launch-bound path: arguments arrive as given (pointers beyond 2^63 included), the
    status comes back, and the loader binds it to the real library (whose answer to a null context is an error, no GPU needed)."""
    import ctypes as C
    import importlib.util
    from purlin_b200 import _build
    path = _build.build_fastcall()
    spec = importlib.util.spec_from_file_location("_purlin_fastcall", str(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with pytest.raises(RuntimeError):
        mod.call_fixed(1, 2, 3, 4, 5, 6, 7)                                   # nothing bound yet
    seen = []
    proto = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_uint, C.c_void_p)

    def target(ctx, collective, src, dst, nbytes, traits, stream):
        seen.append((ctx, collective, src, dst, nbytes, traits, stream))
        return 7 if collective == 5 else 0
    cb = proto(target)
    mod.bind(C.cast(cb, C.c_void_p).value)
    big = (1 << 64) - 32
    assert mod.call_fixed(0xC0FFEE, 3, big, 0x7F0000001000, 1 << 40, (1 << 16) | (2 << 8) | 4, 0xABCDEF) == 0
    assert seen[-1] == (0xC0FFEE, 3, big, 0x7F0000001000, 1 << 40, (1 << 16) | (2 << 8) | 4, 0xABCDEF)
    assert mod.call_fixed(1, 5, 0, 0, 0, 0, 0) == 7
    assert seen[-1][2] is None and seen[-1][6] is None                        # null pointers stay null
    with pytest.raises(TypeError):
        mod.call_fixed(1, 2, 3)
    with pytest.raises((TypeError, OverflowError)):
        mod.call_fixed(1, 2, 3, 4, -1, 6, 7)                                  # a negative byte count is refused, not wrapped
    # the loader: bound to the library itself
    from purlin_b200 import _native
    lib = _native.cuda()
    fast = _native.fast_call_fixed(lib)
    assert fast is not lib.purlin_call_fixed or os.environ.get("PURLIN_NO_FASTCALL")
    assert fast(0, 0, 0, 0, 64, 4, 0) == 1
    assert "null context" in _native.last_error(lib)
