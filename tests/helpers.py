"""Shared test helpers: seeded inputs, reference results and the CPU interpreter wrapper."""
import ctypes as C

import numpy as np
import torch

import purlin_b200 as P
from purlin_b200 import _native

AR, AG, AGV, RS, RSV, A2A, A2AV = range(7)
TORCH_DT = {0: torch.bfloat16, 1: torch.float16, 2: torch.float8_e4m3fn, 3: torch.float8_e5m2, 4: torch.float32}
ELEM = {0: 2, 1: 2, 2: 1, 3: 1, 4: 4}


def ints(n_elems, dtype, seed, lo=-2, hi=2):
    """Small integers: any summation order is exact in every element type."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n_elems,), generator=g).to(torch.float32).to(TORCH_DT[dtype])


def in_out_bytes(coll, world, rank, nbytes, sizes):
    """(input bytes, output bytes) of one rank. `sizes`: list[world] for AGV/RSV, matrix [world][world] for A2AV."""
    if coll == AR:
        return nbytes, nbytes
    if coll == AG:
        return nbytes, nbytes * world
    if coll == AGV:
        return sizes[rank], sum(sizes)
    if coll == RS:
        return nbytes * world, nbytes
    if coll == RSV:
        return sum(sizes), sizes[rank]
    if coll == A2A:
        return nbytes * world, nbytes * world
    return sum(sizes[rank]), sum(sizes[q][rank] for q in range(world))


def reduce_ref(parts, op=0):
    acc = parts[0].to(torch.float32).clone()
    for p in parts[1:]:
        x = p.to(torch.float32)
        acc = acc + x if op == 0 else acc * x if op == 1 else torch.maximum(acc, x)
    return acc


def expected(coll, world, rank, inputs, nbytes, sizes, dtype, op=0):
    """Reference output of `rank` from all ranks' typed inputs (fp32 accumulate, ascending rank order)."""
    e = ELEM[dtype]
    td = TORCH_DT[dtype]
    if coll == AR:
        return reduce_ref(inputs, op).to(td)
    if coll in (AG, AGV):
        return torch.cat(inputs)
    if coll == RS:
        n = nbytes // e
        return reduce_ref([x[rank * n:(rank + 1) * n] for x in inputs], op).to(td)
    if coll == RSV:
        off = sum(sizes[:rank]) // e
        n = sizes[rank] // e
        return reduce_ref([x[off:off + n] for x in inputs], op).to(td)
    if coll == A2A:
        n = nbytes // e
        return torch.cat([inputs[q][rank * n:(rank + 1) * n] for q in range(world)])
    out = []
    for q in range(world):
        off = sum(sizes[q][:rank]) // e
        out.append(inputs[q][off:off + sizes[q][rank] // e])
    return torch.cat(out) if out else torch.empty(0, dtype=td)


def flat_sizes(coll, world, sizes):
    if sizes is None:
        return None
    if coll == A2AV:
        return _native.size_array([sizes[r][q] for r in range(world) for q in range(world)])
    return _native.size_array(sizes)


def sim(coll, world, nbytes=0, sizes=None, dtype=4, op=0, staging=1 << 20, policy=None, drop=-1, seed=0):
    """Runs the CPU interpreter on seeded integer inputs; returns (status, outputs, expected outputs)."""
    lib = _native.host()
    e = ELEM[dtype]
    ins, outs, keep = [], [], []
    for r in range(world):
        ib, ob = in_out_bytes(coll, world, r, nbytes, sizes)
        ins.append(ints(ib // e, dtype, seed * 100 + r))
        outs.append(torch.full((max(ob // e, 1),), 7, dtype=torch.float32).to(TORCH_DT[dtype])[: ob // e].clone())
    srcs = (C.c_void_p * world)(*[t.data_ptr() if t.numel() else None for t in ins])
    dsts = (C.c_void_p * world)(*[t.data_ptr() if t.numel() else None for t in outs])
    status = (C.c_uint32 * 4)()
    rc = lib.purlin_sim_run(coll, world, nbytes, flat_sizes(coll, world, sizes), dtype, op, 0, staging,
                            C.byref(policy) if policy is not None else None, srcs, dsts, drop, status)
    if rc != 0:
        raise RuntimeError(_native.last_error(lib))
    exp = [expected(coll, world, r, ins, nbytes, sizes, dtype, op) for r in range(world)]
    return list(status), outs, exp


def sim_sequence(calls, world, dtype=4, op=0, staging=1 << 20, policy=None, seed=0, quantum=1, multicast=False, in_place_ar=False):
    """Runs a list of calls [(collective, nbytes, sizes), ...] through the interpreter with no barrier between calls and a
    seeded random schedule; returns (status, outputs[call][rank], expected[call][rank]). ``in_place_ar``: all-reduce calls
    get one buffer as source and destination."""
    lib = _native.host()
    lib.purlin_sim_run_overlapped.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.POINTER(C.c_void_p), C.c_int, C.c_int,
                                              C.c_int, C.c_int, C.c_size_t, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                              C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_uint32)]
    e = ELEM[dtype]
    n = len(calls)
    ins, outs, keep = [], [], []
    for c, (coll, nbytes, sizes) in enumerate(calls):
        row_in, row_out = [], []
        for r in range(world):
            ib, ob = in_out_bytes(coll, world, r, nbytes, sizes)
            row_in.append(ints(ib // e, dtype, seed * 7919 + c * 101 + r))
            if in_place_ar and coll == AR:
                row_out.append(row_in[-1].clone())      # the work buffer: input now, result afterwards
            else:
                row_out.append(torch.full((max(ob // e, 1),), 7, dtype=torch.float32).to(TORCH_DT[dtype])[: ob // e].clone())
        ins.append(row_in)
        outs.append(row_out)
    colls = (C.c_int * n)(*[c[0] for c in calls])
    nb = (C.c_size_t * n)(*[c[1] for c in calls])
    mats = []
    for coll, _, sizes in calls:
        m = flat_sizes(coll, world, sizes)
        keep.append(m)
        mats.append(C.cast(m, C.c_void_p) if m is not None else None)
    mat_arr = (C.c_void_p * n)(*mats)
    src_rows = [outs[c] if (in_place_ar and calls[c][0] == AR) else ins[c] for c in range(n)]
    srcs = (C.c_void_p * (n * world))(*[t.data_ptr() if t.numel() else None for row in src_rows for t in row])
    dsts = (C.c_void_p * (n * world))(*[t.data_ptr() if t.numel() else None for row in outs for t in row])
    status = (C.c_uint32 * 4)()
    rc = lib.purlin_sim_run_overlapped(n, colls, nb, mat_arr, world, dtype, op, 0, staging,
                                       C.byref(policy) if policy is not None else None, srcs, dsts, seed, quantum, int(multicast), status)
    if rc != 0:
        raise RuntimeError(_native.last_error(lib))
    exp = [[expected(coll, world, r, ins[c], nbytes, sizes, dtype, op) for r in range(world)] for c, (coll, nbytes, sizes) in enumerate(calls)]
    return list(status), outs, exp


def policy(**kw):
    p = _native.Policy()
    base = dict(regime=1, threads=256, putBlocks=4, localBlocks=2, consumeBlocks=8, gatherBlocks=8, lrBlocks=2, memType=0,
                mmDepth=4, unroll=4, stageDepth=0, arPath=1, lrMulticast=0, weighted=1, chunkBytes=0, perStreamThreshold=0)
    base.update(kw)
    for k, v in base.items():
        setattr(p, k, v)
    return p
