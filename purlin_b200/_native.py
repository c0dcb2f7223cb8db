"""ctypes view of the native libraries: structs mirrored from the C++ headers and typed entry points.

``host()`` returns the CPU-only library (layout engine, tuning, CPU interpreter);
``cuda()`` returns the full library and fails loudly when it is missing, so a GPU
run can never fall back silently to Python code.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import _build

K_MAX_RANKS = 16
K_MAX_STEPS = 56

ROLE_NAMES = ["stage", "local", "consume", "reduce", "gather", "packet_put", "packet_get", "packet_reduce"]
FLAG_TO_SEAM, FLAG_TO_DST, FLAG_MULTIMEM_LOAD, FLAG_MULTICAST_OUT = 1, 2, 4, 8
FLAG_LOCAL_SOURCE, FLAG_CYCLIC, FLAG_PUBLISH, FLAG_RESULT_HALF = 16, 32, 64, 128
FLAG_NOTIFY_GATHER, FLAG_DRAIN_SELF, FLAG_DRAIN_GATHER, FLAG_SCATTER = 256, 512, 1024, 2048
(ROLE_STAGE, ROLE_LOCAL, ROLE_CONSUME, ROLE_REDUCE, ROLE_GATHER,
 ROLE_PACKET_PUT, ROLE_PACKET_GET, ROLE_PACKET_REDUCE) = range(8)


class Step(C.Structure):
    _fields_ = [
        ("role", C.c_int32), ("peer", C.c_int32), ("blockBegin", C.c_int32), ("blockCount", C.c_int32),
        ("srcOff", C.c_uint64), ("dstOff", C.c_uint64), ("bytes", C.c_uint64), ("chunkBytes", C.c_uint64),
        ("seamOff", C.c_uint64),
        ("chunks", C.c_uint32), ("slots", C.c_uint32), ("flags", C.c_uint32), ("counterBase", C.c_uint32),
    ]


class Plan(C.Structure):
    _fields_ = [
        ("collective", C.c_int32), ("regime", C.c_int32), ("consumeOp", C.c_int32), ("reduceOp", C.c_int32),
        ("dtype", C.c_int32), ("deterministic", C.c_int32), ("blocks", C.c_int32), ("threads", C.c_int32),
        ("nSteps", C.c_int32), ("varLenArrival", C.c_int32), ("mmDepth", C.c_int32), ("unroll", C.c_int32),
        ("stageDepth", C.c_int32), ("reserved", C.c_int32),
        ("smemBytes", C.c_uint64), ("payloadBytes", C.c_uint64),
        ("steps", Step * K_MAX_STEPS),
    ]

    def active_steps(self):
        return [self.steps[i] for i in range(self.nSteps)]


class Policy(C.Structure):
    _fields_ = [
        ("regime", C.c_int32), ("threads", C.c_int32), ("putBlocks", C.c_int32), ("localBlocks", C.c_int32),
        ("consumeBlocks", C.c_int32), ("gatherBlocks", C.c_int32), ("lrBlocks", C.c_int32), ("memType", C.c_int32),
        ("mmDepth", C.c_int32), ("unroll", C.c_int32), ("stageDepth", C.c_int32), ("arPath", C.c_int32),
        ("lrMulticast", C.c_int32), ("weighted", C.c_int32),
        ("chunkBytes", C.c_uint64), ("perStreamThreshold", C.c_uint64),
        ("maxCtas", C.c_int32), ("reserved", C.c_int32),
    ]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}

    @classmethod
    def from_dict(cls, d):
        """A policy from a stored table entry. Fields that are newer than the entry keep the engine's defaults
        (no CTA budget); fields the engine no longer has are ignored."""
        p = cls()
        names = {n for n, _ in cls._fields_}
        for k, v in d.items():
            if k in names:
                setattr(p, k, int(v))
        return p


_host = None
_cuda = None


def _resolve(name: str, builder):
    """The in-tree library, rebuilt first when its sources changed (content key); a tree without a compiler
    uses the library it was shipped with."""
    path = _build.LIB_DIR / name
    try:
        return builder(force=bool(os.environ.get("PURLIN_REBUILD")))
    except Exception:
        if path.exists():
            return path
        raise


def _declare_common(lib):
    lib.purlin_last_error.restype = C.c_char_p
    lib.purlin_plan_sizeof.restype = C.c_size_t
    lib.purlin_policy_sizeof.restype = C.c_size_t
    lib.purlin_tuning_size.restype = C.c_size_t
    lib.purlin_workspace_layout.argtypes = [C.c_int, C.c_size_t, C.POINTER(C.c_size_t)]
    lib.purlin_plan_build.argtypes = [C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                      C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.purlin_default_policy.argtypes = [C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p]
    lib.purlin_topology.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]
    lib.purlin_tuning_add.argtypes = [C.c_int, C.c_int, C.c_uint64, C.c_void_p]
    lib.purlin_sim_run.argtypes = [C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_size_t, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_uint32)]
    assert lib.purlin_plan_sizeof() == C.sizeof(Plan), "Plan struct mirror is out of date"
    assert lib.purlin_policy_sizeof() == C.sizeof(Policy), "Policy struct mirror is out of date"


def host():
    """The CPU-only library; built on first use."""
    global _host
    if _host is None:
        path = _resolve("libpurlin_host.so", _build.build_host)
        _host = C.CDLL(str(path))
        _declare_common(_host)
    return _host


def cuda():
    """The full library (CUDA kernels + host half). Raises if it cannot be loaded."""
    global _cuda
    if _cuda is None:
        path = _resolve("libpurlin_cuda.so", _build.build_cuda)
        lib = C.CDLL(str(path))
        _declare_common(lib)
        vp, sz, i, u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint64
        lib.purlin_context_create.restype = vp
        lib.purlin_context_create.argtypes = [i, i, C.POINTER(u64), u64, sz, u64, vp]
        lib.purlin_context_destroy.argtypes = [vp, vp]
        lib.purlin_context_status.argtypes = [vp, C.POINTER(C.c_uint32), vp]
        lib.purlin_context_clear_status.argtypes = [vp, vp]
        lib.purlin_context_set_timeout.argtypes = [vp, u64]
        lib.purlin_context_seq.restype = u64
        lib.purlin_context_seq.argtypes = [vp, vp]
        lib.purlin_context_has_multicast.argtypes = [vp]
        lib.purlin_context_sizeof.restype = sz
        lib.purlin_collective.argtypes = [vp, i, vp, vp, sz, vp, vp, i, i, i, vp, vp]
        lib.purlin_call_fixed.argtypes = [vp, i, vp, vp, sz, C.c_uint, vp]
        lib.purlin_all_reduce.argtypes = [vp, vp, vp, sz, i, i, i, vp]
        lib.purlin_all_gather.argtypes = [vp, vp, vp, sz, vp]
        lib.purlin_all_gather_v.argtypes = [vp, vp, vp, vp, vp]
        lib.purlin_reduce_scatter.argtypes = [vp, vp, vp, sz, i, i, i, vp]
        lib.purlin_reduce_scatter_v.argtypes = [vp, vp, vp, vp, i, i, i, vp]
        lib.purlin_all_to_all.argtypes = [vp, vp, vp, sz, vp]
        lib.purlin_all_to_all_v.argtypes = [vp, vp, vp, vp, vp, vp]
        lib.purlin_emu_collective.argtypes = [vp, i, i, vp, vp, sz, vp, i, i, i, vp, i, vp]
        lib.purlin_p2p_copy.argtypes = [vp, vp, sz, i, i, vp]
        _cuda = lib
    return _cuda


_fastcall = None


def fast_call_fixed(lib):
    """``purlin_call_fixed`` of ``lib`` behind a CPython extension that takes the seven scalars as they are (a third of
    the per-call cost of the ctypes foreign call); the ctypes function itself when the extension cannot be built or loaded
    (``PURLIN_NO_FASTCALL=1`` forces that). One library per process is bound; a second one gets the ctypes function."""
    global _fastcall
    if os.environ.get("PURLIN_NO_FASTCALL") or not isinstance(lib, C.CDLL):
        return lib.purlin_call_fixed
    if _fastcall is None:
        try:
            import importlib.util
            path = _resolve(_build.fastcall_name(), _build.build_fastcall)
            spec = importlib.util.spec_from_file_location("_purlin_fastcall", str(path))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.bind(C.cast(lib.purlin_call_fixed, C.c_void_p).value)
            _fastcall = (lib, mod)
        except Exception:
            _fastcall = (None, None)
    return _fastcall[1].call_fixed if _fastcall[0] is lib else lib.purlin_call_fixed


def last_error(lib) -> str:
    return (lib.purlin_last_error() or b"").decode()


def check(lib, rc: int):
    if rc != 0:
        raise RuntimeError("purlin: " + last_error(lib))


def size_array(values):
    arr = (C.c_size_t * len(values))(*[int(v) for v in values])
    return arr
