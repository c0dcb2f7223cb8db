"""Split policies for variable-length collectives (Python face of csrc/src/split_policy.cpp).

``zipf_splits`` / ``skew_splits`` divide a total among ranks; ``sparse_matrix`` / ``hot_ring_matrix`` build
all-to-all-v traffic matrices; ``uniform_counts`` is the generator of the variable-length benchmark configuration
(per-rank element counts uniform in [0.5x, 1.5x] of a base, rounded to 16-element multiples, from a seed).
Every function is deterministic in its arguments, so all ranks derive the same lists without communicating.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List

from .. import _native

_ZIPF = {"0": 0, "0.125": 1, "0.25": 2, "0.5": 4, "1": 8}
_declared = False


def _lib():
    global _declared
    lib = _native.host()
    if not _declared:
        sz, i, u64 = C.c_size_t, C.c_int, C.c_uint64
        lib.purlin_split_unit.restype = sz
        lib.purlin_split_unit.argtypes = [sz, i]
        lib.purlin_zipf_splits.argtypes = [sz, i, i, C.POINTER(sz)]
        lib.purlin_skew_splits.argtypes = [sz, i, i, u64, C.POINTER(sz)]
        lib.purlin_sparse_matrix.argtypes = [i, i, sz, u64, C.POINTER(sz)]
        lib.purlin_hotring_matrix.argtypes = [i, sz, i, C.POINTER(sz)]
        _declared = True
    return lib


def zipf_exponent_eighths() -> int:
    """0.125 unless BENCH_ZIPF_EXPONENT selects 0 (uniform), 0.25, 0.5 or 1."""
    text = os.environ.get("BENCH_ZIPF_EXPONENT", "") or "0.125"
    if text not in _ZIPF:
        raise ValueError("BENCH_ZIPF_EXPONENT must be 0, 0.125, 0.25, 0.5 or 1")
    return _ZIPF[text]


def split_unit(total: int, world: int) -> int:
    lib = _lib()
    unit = int(lib.purlin_split_unit(total, world))
    if unit == 0:
        raise ValueError(_native.last_error(lib))
    return unit


def zipf_splits(total: int, world: int, eighths: int | None = None) -> List[int]:
    lib = _lib()
    out = (C.c_size_t * world)()
    if lib.purlin_zipf_splits(total, world, zipf_exponent_eighths() if eighths is None else eighths, out) != 0:
        raise ValueError(_native.last_error(lib))
    return [int(v) for v in out]


def skew_splits(total: int, world: int, percent: int, seed: int = 0) -> List[int]:
    lib = _lib()
    out = (C.c_size_t * world)()
    if lib.purlin_skew_splits(total, world, percent, seed, out) != 0:
        raise ValueError(_native.last_error(lib))
    return [int(v) for v in out]


def _matrix(out, world):
    return [[int(out[r * world + d]) for d in range(world)] for r in range(world)]


def sparse_matrix(world: int, active: int, nbytes: int = 64 << 10, seed: int = 0) -> List[List[int]]:
    lib = _lib()
    out = (C.c_size_t * (world * world))()
    if lib.purlin_sparse_matrix(world, active, nbytes, seed, out) != 0:
        raise ValueError(_native.last_error(lib))
    return _matrix(out, world)


def hot_ring_matrix(world: int, bytes_per_rank: int, percent: int = 90) -> List[List[int]]:
    lib = _lib()
    out = (C.c_size_t * (world * world))()
    if lib.purlin_hotring_matrix(world, bytes_per_rank, percent, out) != 0:
        raise ValueError(_native.last_error(lib))
    return _matrix(out, world)


def offsets(sizes: List[int]) -> List[int]:
    out, acc = [], 0
    for s in sizes:
        out.append(acc)
        acc += s
    return out


def uniform_counts(world: int, base_elems: int = 4 << 20, seed: int = 7, multiple: int = 16) -> List[int]:
    """Element counts uniform in [0.5, 1.5] x base, rounded down to ``multiple`` elements (32 bytes of bf16)."""
    import torch
    g = torch.Generator().manual_seed(seed)
    u = torch.rand(world, generator=g, dtype=torch.float64)
    return [max(int(base_elems * (0.5 + float(x))) // multiple * multiple, multiple) for x in u]
