"""purlin_b200: single-kernel NVLink collectives for B200, with the Python surface of purlin.

Public functions (same names, argument order and byte conventions as the
reference package, purlin/__init__.py:62-145): ``initialize``, ``finalize``,
``all_reduce``, ``all_gather``, ``all_gather_v``, ``reduce_scatter``,
``reduce_scatter_v``, ``all_to_all``, ``all_to_all_v``, plus ``ReductionMode``,
``DataType``, ``normalize_arch`` and ``buffer_type``.

Differences a user sees:
  * the native library is prebuilt in-tree (no CMake, no download at first call);
  * ``stream_ptr`` may be omitted (the current torch stream is used);
  * a CPU device selects a gloo-backed executor of the same schedule, so the API
    can be exercised without a GPU;
  * device waits are bounded: ``check(handle)`` raises if a peer never showed up.
"""
from __future__ import annotations

import ctypes as C
import os
from enum import IntEnum
from typing import Optional, Sequence

import torch

from . import _native

__version__ = "1.0.0"

STAGING_BUFFER_SIZE = 256 * 1024 * 1024
PACKET_EPOCH_BYTES = 8 * 1024 * 1024
ACCESS_ALIGNMENT = 32


class ReductionMode(IntEnum):
    """DETERMINISTIC reduces in ascending rank order on the SMs and never uses the NVSwitch reduction."""
    NON_DETERMINISTIC = 0
    DETERMINISTIC = 1


class DataType(IntEnum):
    BF16 = 0
    FP16 = 1
    FP8_E4M3 = 2
    FP8_E5M2 = 3
    FP32 = 4


class ReduceOp(IntEnum):
    ADD = 0
    MUL = 1
    MAX = 2


class Collective(IntEnum):
    ALL_REDUCE = 0
    ALL_GATHER = 1
    ALL_GATHER_V = 2
    REDUCE_SCATTER = 3
    REDUCE_SCATTER_V = 4
    ALL_TO_ALL = 5
    ALL_TO_ALL_V = 6


def normalize_arch(arch: int) -> int:
    """Only Blackwell is built; older values are accepted for source compatibility and map to themselves."""
    if arch >= 100:
        return 1000
    if arch >= 90:
        return 900
    if arch >= 80:
        return 800
    return 700


_DTYPES = {
    torch.float16: DataType.FP16,
    torch.bfloat16: DataType.BF16,
    torch.float32: DataType.FP32,
    torch.float8_e5m2: DataType.FP8_E5M2,
    torch.float8_e4m3fn: DataType.FP8_E4M3,
}


def buffer_type(t: torch.dtype) -> DataType:
    try:
        return _DTYPES[t]
    except KeyError:
        raise TypeError(f"unsupported element type {t}") from None


class ContextHandle:
    """Everything one process group needs: the native context, the symmetric block and its rendezvous handle."""
    __slots__ = ("mod", "ctx", "buf", "hdl", "sig_buf", "sig_hdl", "v_sig_buf", "v_sig_hdl",
                 "rank", "world", "device", "group", "staging_size", "cpu", "layout", "call_fixed")

    def __init__(self, mod, ctx, buf, hdl, rank, world, device, group, staging_size, layout, cpu=None):
        self.mod, self.ctx, self.buf, self.hdl = mod, ctx, buf, hdl
        # the entry point of the launch-bound path: the C extension when it loads, else the ctypes function
        self.call_fixed = _native.fast_call_fixed(mod) if cpu is None and hasattr(mod, "purlin_call_fixed") else None
        # the reference keeps three symmetric tensors; here all regions live in one block, these are views of it
        self.sig_buf = self.sig_hdl = self.v_sig_buf = self.v_sig_hdl = None
        self.rank, self.world, self.device, self.group = rank, world, device, group
        self.staging_size, self.layout, self.cpu = staging_size, layout, cpu

    @property
    def has_multicast(self) -> bool:
        return bool(self.ctx) and self.cpu is None and bool(self.mod.purlin_context_has_multicast(self.ctx))


def workspace_layout(world: int, staging_size: int = STAGING_BUFFER_SIZE) -> dict:
    lib = _native.host()
    out = (C.c_size_t * 8)()
    _native.check(lib, lib.purlin_workspace_layout(world, staging_size, out))
    names = ["staging_tr_size", "lr_offset", "signal_offset", "gather_offset", "consumed_offset", "varlen_offset", "total_bytes", "packet_stride"]
    return dict(zip(names, [int(v) for v in out]))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(stream_ptr: Optional[int]) -> int:
    """The caller's stream handle, or the current stream of the current device (about a tenth of the cost of building a
    ``torch.cuda.Stream`` object per call, which matters for the launch-bound small collectives)."""
    if stream_ptr is None:
        if _raw_stream is not None:
            return _raw_stream(torch.cuda.current_device())
        return torch.cuda.current_stream().cuda_stream
    return int(stream_ptr)


def initialize(group=None, device: Optional[torch.device] = None, arch: int = 100, stream_ptr: Optional[int] = None,
               staging_size: Optional[int] = None, timeout_ms: Optional[int] = None) -> ContextHandle:
    """Collective over ``group``: allocates the symmetric workspace, exchanges peer mappings, builds the context."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    if staging_size is None:
        staging_size = int(os.environ.get("PURLIN_STAGING_TR_SIZE", STAGING_BUFFER_SIZE))
    if device.type == "cpu":
        from .cpu import CpuContext
        layout = workspace_layout(world, staging_size)
        cpu = CpuContext(group, rank, world, staging_size)
        return ContextHandle(_native.host(), cpu, None, None, rank, world, device, group, staging_size, layout, cpu=cpu)
    normalize_arch(arch)
    mod = _native.cuda()
    layout = workspace_layout(world, staging_size)
    from .parallel.symmetric import allocate_symmetric
    buf, hdl, peer_ptrs, mc_ptr = allocate_symmetric(layout["total_bytes"], device, group)
    stream = _stream(stream_ptr)
    ptrs = (C.c_uint64 * world)(*peer_ptrs)
    timeout_ns = int(timeout_ms) * 1_000_000 if timeout_ms else 0
    ctx = mod.purlin_context_create(rank, world, ptrs, int(mc_ptr or 0), staging_size, timeout_ns, stream)
    if not ctx:
        raise RuntimeError("purlin: " + _native.last_error(mod))
    from . import tuning
    tuning.load_for(torch.cuda.get_device_name(device), world, lib=mod)   # measured codesign table, if one exists
    return ContextHandle(mod, ctx, buf, hdl, rank, world, device, group, staging_size, layout)


def finalize(handle: ContextHandle, stream_ptr: Optional[int] = None) -> None:
    """Idempotent. Waits for collectives in flight on the stream, then frees the native context."""
    if handle.ctx is None:
        return
    if handle.cpu is None:
        handle.mod.purlin_context_destroy(handle.ctx, _stream(stream_ptr))
    if hasattr(handle.buf, "close"):
        handle.buf.close()   # native providers release their mappings here (the vmm provider does so collectively)
    handle.ctx = None
    handle.cpu = None
    handle.hdl = None
    handle.sig_hdl = None
    handle.v_sig_hdl = None
    handle.buf = None
    handle.sig_buf = None
    handle.v_sig_buf = None


def check(handle: ContextHandle, stream_ptr: Optional[int] = None) -> None:
    """Synchronises the stream and raises if a bounded device wait gave up since the last check."""
    if handle.cpu is not None or handle.ctx is None:
        return
    out = (C.c_uint32 * 4)()
    _native.check(handle.mod, handle.mod.purlin_context_status(handle.ctx, out, _stream(stream_ptr)))
    if out[0]:
        names = {1: "signal", 2: "packet", 3: "arrival", 4: "tile", 5: "barrier", 6: "plan"}
        raise TimeoutError(f"purlin: device wait timed out ({names.get(out[0], out[0])}; step {out[1]}, peer {out[2]}, chunk {out[3]})")


_COLLECTIVE_NAMES = ["all_reduce", "all_gather", "all_gather_v", "reduce_scatter", "reduce_scatter_v", "all_to_all", "all_to_all_v"]


def read_trace(lib, ctx, stream: int, max_records: int = 256):
    """Decodes the device-side timing ring of a native context (see ``trace``)."""
    lib.purlin_context_trace.argtypes = [C.c_void_p, C.POINTER(C.c_uint64), C.c_int, C.c_void_p]
    buf = (C.c_uint64 * (4 * max_records))()
    n = lib.purlin_context_trace(ctx, buf, max_records, stream)
    if n < 0:
        return None
    out = []
    for i in range(n):
        call, start, end, packed = (int(buf[4 * i + k]) for k in range(4))
        kind = packed >> 56
        out.append({"call": call, "collective": _COLLECTIVE_NAMES[kind] if kind < len(_COLLECTIVE_NAMES) else str(kind),
                    "bytes": packed & ((1 << 56) - 1), "start_ns": start, "end_ns": end, "us": (end - start) / 1000.0})
    return out


def trace(handle: ContextHandle, stream_ptr: Optional[int] = None, max_records: int = 256):
    """Device-side timing of the most recent collectives on this context, oldest first: one dict per call with the call
    number, collective, payload bytes of the plan (all-reduce: the buffer; all-gather: bytes per rank; reduce-scatter and
    all-to-all: this rank's whole input) and the device timestamps taken by the first CTA in and the last CTA out.
    Needs ``PURLIN_TRACE=1`` in the environment when the context is created; returns ``None`` otherwise.
    Synchronises the stream."""
    if handle.cpu is not None or handle.ctx is None:
        return None
    return read_trace(handle.mod, handle.ctx, _stream(stream_ptr), max_records)


def clear_status(handle: ContextHandle, stream_ptr: Optional[int] = None) -> None:
    if handle.cpu is None and handle.ctx is not None:
        _native.check(handle.mod, handle.mod.purlin_context_clear_status(handle.ctx, _stream(stream_ptr)))


def _contig(*tensors):
    for t in tensors:
        if not t.is_contiguous():
            raise ValueError("purlin collectives need contiguous tensors")


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _mode(m) -> int:
    return m if (m == 0 or m == 1) and type(m) is int else int(ReductionMode(m))


def _call(handle, collective, src, dst, nbytes, sizes, out_sizes, dtype, op, mode, stream_ptr, policy=None):
    if handle.ctx is None:
        raise RuntimeError("purlin: the context was finalized")
    if handle.cpu is not None:
        return handle.cpu.run(int(collective), src, dst, nbytes, sizes, out_sizes, int(dtype), int(op), int(mode), policy)
    s_arr = _native.size_array(sizes) if sizes is not None else None
    o_arr = _native.size_array(out_sizes) if out_sizes is not None else None
    pol = C.byref(policy) if policy is not None else None
    rc = handle.mod.purlin_collective(handle.ctx, int(collective), src.data_ptr(), dst.data_ptr(), nbytes, s_arr, o_arr,
                                      int(dtype), int(op), int(mode), pol, _stream(stream_ptr))
    _native.check(handle.mod, rc)


def _call_fixed(handle, collective: int, src, dst, nbytes: int, traits: int, stream_ptr, policy):
    """The launch-bound path of the fixed-size collectives: the fewest Python operations and the shortest native
    signature that do the job (a small collective costs about as much on the host as on the device)."""
    if policy is not None or handle.cpu is not None or handle.ctx is None:
        return _call(handle, collective, src, dst, nbytes, None, None, traits & 0xff, (traits >> 8) & 0xff, traits >> 16, stream_ptr, policy)
    if not (src.is_contiguous() and dst.is_contiguous()):
        raise ValueError("purlin collectives need contiguous tensors")
    if handle.call_fixed(handle.ctx, collective, src.data_ptr(), dst.data_ptr(), nbytes, traits,
                         stream_ptr if stream_ptr is not None else _stream(None)):
        _native.check(handle.mod, 1)


_AR, _AG, _RS, _A2A = int(Collective.ALL_REDUCE), int(Collective.ALL_GATHER), int(Collective.REDUCE_SCATTER), int(Collective.ALL_TO_ALL)


def all_gather(in_tensor, out_tensor, handle, stream_ptr=None, policy=None):
    _call_fixed(handle, _AG, in_tensor, out_tensor, in_tensor.numel() * in_tensor.element_size(), 0, stream_ptr, policy)


def all_gather_v(in_tensor, out_tensor, bytes_list: Sequence[int], handle, stream_ptr=None, policy=None):
    _contig(in_tensor, out_tensor)
    if len(bytes_list) != handle.world:
        raise ValueError("bytes_list needs one entry per rank")
    _call(handle, Collective.ALL_GATHER_V, in_tensor, out_tensor, 0, list(bytes_list), None, 0, 0, 0, stream_ptr, policy)


_TRAITS = {}       # (torch dtype, op, reduction mode) -> dtype | op << 8 | mode << 16, computed once per combination


def _traits(dtype, op, reduction_mode) -> int:
    key = (dtype, op, reduction_mode)
    t = _TRAITS.get(key)
    if t is None:
        t = _TRAITS[key] = int(buffer_type(dtype)) | (int(op) << 8) | (_mode(reduction_mode) << 16)
    return t


def all_reduce(in_tensor, out_tensor, handle, stream_ptr=None, reduction_mode=ReductionMode.NON_DETERMINISTIC,
               op: ReduceOp = ReduceOp.ADD, policy=None):
    _call_fixed(handle, _AR, in_tensor, out_tensor, in_tensor.numel() * in_tensor.element_size(),
                _traits(in_tensor.dtype, op, reduction_mode), stream_ptr, policy)


def all_to_all(in_tensor, out_tensor, handle, stream_ptr=None, policy=None):
    """``in_tensor`` holds one equal slice per peer; the native call takes bytes per slice (total // world)."""
    _call_fixed(handle, _A2A, in_tensor, out_tensor, in_tensor.numel() * in_tensor.element_size() // handle.world, 0, stream_ptr, policy)


def all_to_all_v(in_tensor, out_tensor, splits: Sequence[int], handle, stream_ptr=None, policy=None):
    """``splits`` = input splits followed by output splits, in bytes (2 x world entries)."""
    _contig(in_tensor, out_tensor)
    w = handle.world
    if len(splits) != 2 * w:
        raise ValueError("splits needs world input sizes followed by world output sizes")
    _call(handle, Collective.ALL_TO_ALL_V, in_tensor, out_tensor, 0, list(splits[:w]), list(splits[w:]), 0, 0, 0, stream_ptr, policy)


def reduce_scatter(in_tensor, out_tensor, handle, stream_ptr=None, reduction_mode=ReductionMode.NON_DETERMINISTIC,
                   op: ReduceOp = ReduceOp.ADD, policy=None):
    _call_fixed(handle, _RS, in_tensor, out_tensor, in_tensor.numel() * in_tensor.element_size() // handle.world,
                _traits(in_tensor.dtype, op, reduction_mode), stream_ptr, policy)


def reduce_scatter_v(in_tensor, out_tensor, bytes_list: Sequence[int], handle, stream_ptr=None,
                     reduction_mode=ReductionMode.NON_DETERMINISTIC, op: ReduceOp = ReduceOp.ADD, policy=None):
    _contig(in_tensor, out_tensor)
    if len(bytes_list) != handle.world:
        raise ValueError("bytes_list needs one entry per rank")
    _call(handle, Collective.REDUCE_SCATTER_V, in_tensor, out_tensor, 0, list(bytes_list), None,
          buffer_type(in_tensor.dtype), op, _mode(reduction_mode), stream_ptr, policy)


def set_max_ctas(max_ctas: int) -> int:
    """CTA budget of every collective planned from now on in this process (0 = the whole GPU, the default; the reference
    caps its collectives at 64 so that they can run beside compute kernels). Returns the previous value. The environment
    variable ``PURLIN_MAX_CTAS`` sets the initial value."""
    old = 0
    for lib in (_native.host(), _native.cuda() if torch.cuda.is_available() else None):
        if lib is not None:
            old = int(lib.purlin_set_max_ctas(int(max_ctas)))
    return old


def build_plan(collective, world, rank, nbytes=0, sizes=None, out_sizes=None, dtype=DataType.BF16, op=ReduceOp.ADD,
               mode=ReductionMode.NON_DETERMINISTIC, multicast=False, in_place=False, staging_size=STAGING_BUFFER_SIZE,
               policy=None):
    """Runs the layout engine for one rank and returns ``(Plan, Policy)`` (CPU only; useful for inspection and tests)."""
    lib = _native.host()
    plan, chosen = _native.Plan(), _native.Policy()
    s_arr = _native.size_array(sizes) if sizes is not None else None
    o_arr = _native.size_array(out_sizes) if out_sizes is not None else None
    rc = lib.purlin_plan_build(int(collective), world, rank, nbytes, s_arr, o_arr, int(dtype), int(op), int(mode),
                               int(multicast), int(in_place), staging_size,
                               C.byref(policy) if policy is not None else None, C.byref(plan), C.byref(chosen))
    _native.check(lib, rc)
    return plan, chosen


def reduce_scatter_symm(symm_tensor, out, op: ReduceOp = ReduceOp.ADD, reduction_mode=ReductionMode.NON_DETERMINISTIC, blocks: int = 0):
    """Reduce-scatter straight out of ``symm_empty`` input tensors (no staging pass): ``out`` receives the reduction over
    ranks of this rank's slice. The inputs may be reused as soon as the call completes in stream order."""
    return symm_tensor.reduce_scatter(out, int(op), _mode(reduction_mode), blocks)


def all_gather_symm(symm_tensor, via_switch=None, blocks: int = 0):
    """In-place all-gather of a ``symm_empty`` tensor of ``world`` slices: every rank's own slice is pushed into the same
    slice of every peer's tensor (one switch-replicated store, or one store per peer)."""
    return symm_tensor.all_gather_(via_switch, blocks)


def check_plan(plan, world, src_bytes, dst_bytes, staging_size=STAGING_BUFFER_SIZE) -> str:
    """Static bounds check of a plan against one rank's buffer extents. Returns "" when sound, else the first violation
    (every plan ``build_plan`` or a collective call produces has already passed this check)."""
    lib = _native.host()
    lib.purlin_plan_check.argtypes = [C.c_void_p, C.c_int, C.c_size_t, C.c_size_t, C.c_size_t]
    rc = lib.purlin_plan_check(C.byref(plan), world, staging_size, src_bytes, dst_bytes)
    return "" if rc == 0 else _native.last_error(lib)


Policy = _native.Policy


def symm_empty(shape, dtype, handle_or_group=None, device=None):
    """Allocates a tensor in symmetric memory (collective over the group). See ``all_reduce_symm``.
    With a CPU handle the result is a gloo-backed stand-in with the same methods."""
    from .parallel.symmetric import HostSymmetricTensor, SymmetricTensor
    group = getattr(handle_or_group, "group", handle_or_group)
    dev = device or getattr(handle_or_group, "device", None) or torch.device("cuda", torch.cuda.current_device())
    if torch.device(dev).type == "cpu":
        return HostSymmetricTensor(shape, dtype, group)
    return SymmetricTensor(shape, dtype, dev, group)


def all_reduce_symm(symm_tensor, op: ReduceOp = ReduceOp.ADD, reduction_mode=ReductionMode.NON_DETERMINISTIC, blocks: int = 0):
    """In-place all-reduce of a ``symm_empty`` tensor with no staging copies: the NVSwitch reduces every rank's shard
    straight out of the tensors and broadcasts it straight back (plain peer loads/stores when there is no multicast
    alias or the mode is deterministic)."""
    return symm_tensor.all_reduce_(int(op), _mode(reduction_mode), blocks)
