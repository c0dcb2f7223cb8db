"""Measured codesign tables: load, install into the native policy table, save.

The reference freezes its tuning into compile-time structs per architecture and world size
(csrc/include/purlin/host/codesign.cuh).  Here a table is data produced by the tuner
(``bench_collectives.py --tune``) on the machine: for every collective and message size it records the policy
(regime, variant, chunk size, CTA counts, NVLS on/off) that measured fastest.  Tables live in
``purlin_b200/tuning_tables/<gpu>_w<world>.json``; ``initialize`` installs the one that matches the GPU name and
world size.  A world size that was never swept borrows the table of the nearest measured world size of the same GPU
(the larger one on a tie): protocol choice and chunk sizes depend far more on the message size than on the number of
ranks, the layout engine re-fits CTA counts to the world, and a borrowed policy that does not fit a call falls back to
the built-in bands like any other.  With no table at all the built-in bands apply.  ``PURLIN_TUNING_TABLE`` names a
file to use instead; ``PURLIN_NO_TUNING_TABLE=1`` disables loading.
"""
from __future__ import annotations

import ctypes as C
import json
import math
import os
from pathlib import Path
from typing import Optional

from . import _native

TABLE_DIR = Path(__file__).resolve().parent / "tuning_tables"
_installed: set = set()


def table_path(gpu_name: str, world: int) -> Path:
    tag = "".join(ch if ch.isalnum() else "_" for ch in gpu_name).strip("_")
    return TABLE_DIR / f"{tag}_w{world}.json"


def bands(entries):
    """Turns point measurements into size bands: each measured size owns everything up to the geometric mean with
    the next measured size of the same collective; the largest owns the rest."""
    out = []
    by_coll = {}
    for e in entries:
        by_coll.setdefault(int(e["collective"]), []).append(e)
    for coll, es in by_coll.items():
        es.sort(key=lambda e: int(e["bytes"]))
        for i, e in enumerate(es):
            if i + 1 < len(es):
                upper = int(math.sqrt(int(e["bytes"]) * int(es[i + 1]["bytes"])))
            else:
                upper = (1 << 62)
            out.append((coll, int(e["world"]), upper, e["policy"]))
    return out


def install(table: dict, lib=None) -> int:
    """Adds every band of ``table`` to the native policy table; returns how many were added."""
    lib = lib or _native.host()
    n = 0
    for coll, world, upper, pol in bands(table.get("entries", [])):
        p = _native.Policy.from_dict(pol)
        lib.purlin_tuning_add(coll, world, C.c_uint64(upper), C.byref(p))
        n += 1
    return n


def nearest_table(gpu_name: str, world: int) -> Optional[Path]:
    """The table of the same GPU measured at the world size closest to ``world`` (the larger one on a tie), if any."""
    stem = table_path(gpu_name, 0).name[:-len("0.json")]       # "<gpu>_w"
    best = None
    for p in sorted(TABLE_DIR.glob(stem + "*.json")):
        try:
            w = int(p.name[len(stem):-len(".json")])
        except ValueError:
            continue
        rank = (abs(w - world), -w)
        if best is None or rank < best[0]:
            best = (rank, p)
    return best[1] if best else None


def load_for(gpu_name: str, world: int, lib=None) -> Optional[Path]:
    """Installs the table for this GPU and world size once per process; returns the file used, if any."""
    if os.environ.get("PURLIN_NO_TUNING_TABLE"):
        return None
    override = os.environ.get("PURLIN_TUNING_TABLE")
    path = Path(override) if override else table_path(gpu_name, world)
    if not override and not path.exists():
        path = nearest_table(gpu_name, world) or path          # never swept at this world size: borrow the neighbour's
    key = (str(path), world)
    if key in _installed:
        return path
    if not path.exists():
        return None
    with open(path) as f:
        table = json.load(f)
    if int(table.get("world", world)) != world:
        if override:
            return None                                        # an explicit file must match
        table = dict(table, world=world, entries=[dict(e, world=world) for e in table.get("entries", [])])
    install(table, lib)
    _installed.add(key)
    return path


def save(table: dict, gpu_name: str, world: int) -> Path:
    TABLE_DIR.mkdir(parents=True, exist_ok=True)
    path = table_path(gpu_name, world)
    tmp = path.with_suffix(".tmp")
    with open(tmp, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    tmp.replace(path)
    return path


def clear(lib=None):
    (lib or _native.host()).purlin_tuning_clear()
    _installed.clear()
