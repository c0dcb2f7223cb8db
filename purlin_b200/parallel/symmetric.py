"""Symmetric-memory providers: where the per-rank workspace block and its peer mappings come from.

The reference abstracts this as the ``SymmetricMemoryProvider`` concept with an
NVSHMEM implementation for C++ (csrc/contrib/symm_mem.cuh:10-59) and torch
symmetric memory for Python (purlin/__init__.py:73-85).  Four providers exist here:

``torch``     ``torch.distributed._symmetric_memory`` (CUDA VMM + NVLS multicast alias when the fabric offers it)
``ipc``       the native CUDA-IPC provider of libpurlin (peer mappings only, no multicast); handles travel over the process group
``vmm``       the native virtual-memory provider of libpurlin (cuMemCreate blocks, POSIX-fd handles duplicated between the
              ranks' processes, NVLS multicast alias when every device supports it); needs no torch symmetric memory
``emulated``  ``world`` blocks on one GPU, for single-GPU emulation of a multi-rank collective

All return ``(owner, handle, peer_pointers, multicast_pointer)`` where ``owner`` keeps the memory alive.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Tuple

import torch


class RawBuffer:
    """A device pointer dressed as ``__cuda_array_interface__`` so torch can view symmetric memory without a copy."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


def allocate_symmetric(nbytes: int, device: torch.device, group=None, provider: str | None = None):
    provider = provider or os.environ.get("PURLIN_PROVIDER", "torch")
    if provider == "torch":
        return _torch_provider(nbytes, device, group)
    if provider == "ipc":
        return _ipc_provider(nbytes, device, group)
    if provider == "vmm":
        return _vmm_provider(nbytes, device, group)
    raise ValueError(f"unknown symmetric memory provider {provider!r}")


def _torch_provider(nbytes: int, device: torch.device, group):
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    if group is None:
        group = dist.group.WORLD
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    try:
        hdl = symm_mem.rendezvous(buf, group)
    except TypeError:
        hdl = symm_mem.rendezvous(buf, group.group_name)
    peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
    mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
    torch.cuda.synchronize(device)
    dist.barrier(group)   # every rank's zero-fill is complete before any peer writes a flag
    return buf, hdl, peer_ptrs, mc


class _IpcMapping:
    """Keeps the local allocation and the opened peer mappings alive; closes them on deletion."""

    def __init__(self, lib, local, opened):
        self.lib, self.local, self.opened = lib, local, opened

    def close(self):
        for p in self.opened:
            self.lib.purlin_ipc_close(C.c_void_p(p))
        self.opened = []
        if self.local:
            self.lib.purlin_ipc_free(C.c_void_p(self.local))
            self.local = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ipc_provider(nbytes: int, device: torch.device, group):
    import torch.distributed as dist
    from .. import _native
    lib = _native.cuda()
    lib.purlin_ipc_export.argtypes = [C.c_void_p, C.c_char_p]
    lib.purlin_ipc_open.restype = C.c_void_p
    lib.purlin_ipc_open.argtypes = [C.c_char_p]
    lib.purlin_ipc_close.argtypes = [C.c_void_p]
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    # a dedicated cudaMalloc block (not a slice of torch's caching allocator), so the handle maps offset 0
    lib.purlin_ipc_alloc.restype = C.c_void_p
    lib.purlin_ipc_alloc.argtypes = [C.c_size_t]
    lib.purlin_ipc_free.argtypes = [C.c_void_p]
    with torch.cuda.device(device):
        local = lib.purlin_ipc_alloc(nbytes)
    if not local:
        raise RuntimeError("purlin: " + _native.last_error(lib))
    handle = C.create_string_buffer(64)
    _native.check(lib, lib.purlin_ipc_export(C.c_void_p(local), handle))
    handles: List[bytes] = [b""] * world
    dist.all_gather_object(handles, handle.raw, group=group)
    peer_ptrs, opened = [], []
    for q in range(world):
        if q == rank:
            peer_ptrs.append(int(local))
            continue
        p = lib.purlin_ipc_open(handles[q])
        if not p:
            raise RuntimeError("purlin: " + _native.last_error(lib))
        opened.append(p)
        peer_ptrs.append(int(p))
    dist.barrier(group)
    mapping = _IpcMapping(lib, local, opened)
    return mapping, mapping, peer_ptrs, 0


class _VmmMapping:
    """Owns a native virtual-memory block; releases it collectively (barrier, detach, barrier, destroy)."""

    def __init__(self, lib, block, group):
        self.lib, self.block, self.group = lib, block, group

    def close(self):
        import torch.distributed as dist
        if not self.block:
            return
        collective = dist.is_initialized()
        if collective:
            dist.barrier(self.group)
        self.lib.purlin_vmm_detach(C.c_void_p(self.block))
        if collective:
            dist.barrier(self.group)
        self.lib.purlin_vmm_destroy(C.c_void_p(self.block))
        self.block = None

    def __del__(self):
        # a collective release cannot run from a finaliser; drop the local mappings only
        try:
            if self.block:
                self.lib.purlin_vmm_destroy(C.c_void_p(self.block))
                self.block = None
        except Exception:
            pass


def _vmm_provider(nbytes: int, device: torch.device, group):
    import torch.distributed as dist
    from .. import _native
    lib = _native.cuda()
    lib.purlin_vmm_create.restype = C.c_void_p
    lib.purlin_vmm_create.argtypes = [C.c_int, C.c_size_t, C.c_int, C.c_int]
    lib.purlin_vmm_local_handle.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.purlin_vmm_map_peers.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.purlin_vmm_peer_ptr.restype = C.c_uint64
    lib.purlin_vmm_peer_ptr.argtypes = [C.c_void_p, C.c_int]
    lib.purlin_vmm_multicast_create.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    lib.purlin_vmm_multicast_join.argtypes = [C.c_void_p, C.c_int, C.c_int]
    lib.purlin_vmm_multicast_bind.argtypes = [C.c_void_p]
    lib.purlin_vmm_multicast_ptr.restype = C.c_uint64
    lib.purlin_vmm_multicast_ptr.argtypes = [C.c_void_p]
    lib.purlin_vmm_detach.argtypes = [C.c_void_p]
    lib.purlin_vmm_destroy.argtypes = [C.c_void_p]
    lib.purlin_vmm_multicast_supported.argtypes = [C.c_int]
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    index = device.index if device.index is not None else torch.cuda.current_device()

    def everyone(value):
        got = [None] * world
        dist.all_gather_object(got, value, group=group)
        return got

    block = lib.purlin_vmm_create(index, nbytes, rank, world)
    pid, fd = C.c_int(0), C.c_int(-1)
    if block:
        lib.purlin_vmm_local_handle(C.c_void_p(block), C.byref(pid), C.byref(fd))
    want_mc = bool(block) and world > 1 and not os.environ.get("PURLIN_DISABLE_MULTIMEM") and lib.purlin_vmm_multicast_supported(index) == 1
    hello = everyone((bool(block), pid.value, fd.value, want_mc))
    mapping = _VmmMapping(lib, block, group)

    def give_up(what):
        err = _native.last_error(lib)
        lib.purlin_vmm_exchange_done()
        if mapping.block:
            lib.purlin_vmm_destroy(C.c_void_p(mapping.block))
            mapping.block = None
        raise RuntimeError(f"purlin: {what}: {err}")

    if not all(h[0] for h in hello):
        give_up("symmetric allocation failed on some rank")
    pids = (C.c_int * world)(*[h[1] for h in hello])
    fds = (C.c_int * world)(*[h[2] for h in hello])
    ok = lib.purlin_vmm_map_peers(C.c_void_p(block), pids, fds) == 0
    if not all(everyone(ok)):
        give_up("mapping the peers' blocks failed on some rank")
    if all(h[3] for h in hello):
        mpid, mfd, made = C.c_int(0), C.c_int(-1), True
        if rank == 0:
            made = lib.purlin_vmm_multicast_create(C.c_void_p(block), C.byref(mpid), C.byref(mfd)) == 0
        first = everyone((made, mpid.value, mfd.value))[0]
        if first[0]:   # without a multicast object the block simply has no alias
            ok = lib.purlin_vmm_multicast_join(C.c_void_p(block), first[1], first[2]) == 0
            if not all(everyone(ok)):
                give_up("joining the multicast object failed on some rank")
            ok = lib.purlin_vmm_multicast_bind(C.c_void_p(block)) == 0
            if not all(everyone(ok)):
                give_up("binding the multicast object failed on some rank")
    dist.barrier(group)
    lib.purlin_vmm_exchange_done()   # every rank has duplicated what it needs: close the descriptor-sharing window
    peer_ptrs = [int(lib.purlin_vmm_peer_ptr(C.c_void_p(block), q)) for q in range(world)]
    mc = int(lib.purlin_vmm_multicast_ptr(C.c_void_p(block)))
    return mapping, mapping, peer_ptrs, mc


def allocate_emulated(nbytes: int, world: int, device: torch.device) -> Tuple[list, list]:
    """``world`` zeroed blocks on one device; every virtual rank sees the same pointer list."""
    blocks = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
    return blocks, [b.data_ptr() for b in blocks]


class HostSymmetricTensor:
    """CPU stand-in for ``SymmetricTensor``: the same methods over a gloo process group, so code written against the
    zero-copy API (gradient buckets, sharded parameters) runs and is tested without a GPU. Nothing is zero-copy here."""

    _OPS = None

    def __init__(self, shape, dtype, group=None):
        import math
        import torch.distributed as dist
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device("cpu")
        self.dtype = dtype
        numel = int(math.prod(shape)) if not isinstance(shape, int) else int(shape)
        self.nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if self.nbytes % 32:
            raise ValueError("symmetric tensors must be a multiple of 32 bytes")
        self.tensor = torch.zeros(shape, dtype=dtype)
        self.multicast_ptr = 0

    def _op(self, op: int):
        import torch.distributed as dist
        return {0: dist.ReduceOp.SUM, 1: dist.ReduceOp.PRODUCT, 2: dist.ReduceOp.MAX}[int(op)]

    def _reduced(self, op: int) -> torch.Tensor:
        import torch.distributed as dist
        acc = self.tensor.to(torch.float32) if self.dtype in (torch.bfloat16, torch.float16) else self.tensor.clone()
        dist.all_reduce(acc, op=self._op(op), group=self.group)      # fp32 accumulation, as on the device
        return acc.to(self.dtype)

    def all_reduce_(self, op: int = 0, mode: int = 0, blocks: int = 0, mm_depth: int = 8, timeout_ms: int = 10000):
        self.tensor.copy_(self._reduced(op))
        return self.tensor

    def _slice_elems(self) -> int:
        if self.nbytes % (32 * self.world):
            raise ValueError("the tensor must split into one 32-byte aligned slice per rank")
        return self.tensor.numel() // self.world

    def reduce_scatter(self, out: torch.Tensor, op: int = 0, mode: int = 0, blocks: int = 0, mm_depth: int = 8, timeout_ms: int = 10000):
        n = self._slice_elems()
        if out.numel() != n or out.dtype != self.dtype:
            raise ValueError("the output must be a contiguous tensor of numel / world elements of the same dtype")
        out.copy_(self._reduced(op).reshape(-1)[self.rank * n:(self.rank + 1) * n].view_as(out))
        return out

    def all_gather_(self, via_switch=None, blocks: int = 0, timeout_ms: int = 10000):
        import torch.distributed as dist
        n = self._slice_elems()
        flat = self.tensor.view(-1)
        mine = flat[self.rank * n:(self.rank + 1) * n].clone().view(torch.uint8)     # gloo moves bytes of any element type
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        flat.view(torch.uint8).copy_(torch.cat(parts))
        return self.tensor

    def status(self) -> int:
        return 0


class SymmetricTensor:
    """A tensor in symmetric memory together with its peer mappings and the flag block the zero-copy collectives use.

    ``tensor`` is an ordinary torch view of this rank's memory; fill it with any kernel, then call
    ``purlin_b200.all_reduce_symm`` to reduce it in place across the group without staging copies.
    """

    def __init__(self, shape, dtype, device, group=None, provider: str | None = None):
        import math
        import torch.distributed as dist
        from .. import _native
        self.lib = _native.cuda()
        self.lib.purlin_symm_flag_bytes.restype = C.c_size_t
        self.lib.purlin_symm_flag_bytes.argtypes = [C.c_int]
        self.lib.purlin_symm_all_reduce.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(C.c_uint64),
                                                    C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_void_p]
        self.lib.purlin_symm_reduce_scatter.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(C.c_uint64),
                                                        C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_uint64, C.c_void_p]
        self.lib.purlin_symm_all_gather.argtypes = [C.c_int, C.c_int, C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(C.c_uint64),
                                                    C.c_size_t, C.c_int, C.c_int, C.c_uint64, C.c_void_p]
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.device(device)
        self.dtype = dtype
        numel = int(math.prod(shape)) if not isinstance(shape, int) else int(shape)
        self.nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if self.nbytes % 32:
            raise ValueError("symmetric tensors must be a multiple of 32 bytes")
        data_bytes = (self.nbytes + 255) // 256 * 256
        flag_bytes = int(self.lib.purlin_symm_flag_bytes(self.world))
        self._owner, self._hdl, ptrs, mc = allocate_symmetric(data_bytes + flag_bytes, self.device, group, provider)
        self.data_ptrs = (C.c_uint64 * self.world)(*ptrs)
        self.flag_ptrs = (C.c_uint64 * self.world)(*[p + data_bytes for p in ptrs])
        self.multicast_ptr = int(mc or 0)
        raw = torch.as_tensor(RawBuffer(ptrs[self.rank], (self.nbytes,), "|u1"), device=self.device)
        self.tensor = raw.view(dtype).view(shape)

    def all_reduce_(self, op: int = 0, mode: int = 0, blocks: int = 0, mm_depth: int = 8, timeout_ms: int = 10000):
        from .. import _native, buffer_type
        rc = self.lib.purlin_symm_all_reduce(self.rank, self.world, self.data_ptrs, self.multicast_ptr, self.flag_ptrs, self.nbytes,
                                             int(buffer_type(self.dtype)), int(op), int(mode), blocks, mm_depth,
                                             timeout_ms * 1_000_000, torch.cuda.current_stream().cuda_stream)
        _native.check(self.lib, rc)
        return self.tensor

    def _slice_bytes(self) -> int:
        if self.nbytes % (32 * self.world):
            raise ValueError("the tensor must split into one 32-byte aligned slice per rank")
        return self.nbytes // self.world

    def reduce_scatter(self, out: torch.Tensor, op: int = 0, mode: int = 0, blocks: int = 0, mm_depth: int = 8, timeout_ms: int = 10000):
        """``out`` (an ordinary tensor of numel / world elements) receives the reduction over ranks of slice ``rank``."""
        from .. import _native, buffer_type
        n = self._slice_bytes()
        if out.numel() * out.element_size() != n or not out.is_contiguous() or out.dtype != self.dtype:
            raise ValueError("the output must be a contiguous tensor of numel / world elements of the same dtype")
        rc = self.lib.purlin_symm_reduce_scatter(self.rank, self.world, self.data_ptrs, self.multicast_ptr, self.flag_ptrs, out.data_ptr(), n,
                                                 int(buffer_type(self.dtype)), int(op), int(mode), blocks, mm_depth,
                                                 timeout_ms * 1_000_000, torch.cuda.current_stream().cuda_stream)
        _native.check(self.lib, rc)
        return out

    def all_gather_(self, via_switch=None, blocks: int = 0, timeout_ms: int = 10000):
        """In place: slice ``rank`` of this rank's tensor is copied into slice ``rank`` of every rank's tensor."""
        from .. import _native
        sw = -1 if via_switch is None else int(bool(via_switch))
        rc = self.lib.purlin_symm_all_gather(self.rank, self.world, self.data_ptrs, self.multicast_ptr, self.flag_ptrs, self._slice_bytes(),
                                             sw, blocks, timeout_ms * 1_000_000, torch.cuda.current_stream().cuda_stream)
        _native.check(self.lib, rc)
        return self.tensor

    def status(self) -> int:
        """Synchronises and returns the status word of the flag block (0 = healthy)."""
        torch.cuda.synchronize(self.device)
        words = torch.as_tensor(RawBuffer(int(self.flag_ptrs[self.rank]), (2 * self.world + 4,), "<i8"), device=self.device)
        return int(words[2 * self.world + 2].item() & 0xffffffff)
