"""Sequence-parallel exchanges built on the collectives: Ulysses head<->sequence all-to-all, sequence gather, ring rotation.

The reference has no sequence- or context-parallel code; it names all2all as the primitive for the Ulysses exchange and
its push / pull copies as the primitive for ring rotation of keys and values (csrc/include/purlin/collective.cuh:32-36,
csrc/examples/p2p/push.cu).  These helpers are thin, allocation-light wrappers over ``all_to_all`` and ``all_gather``.

Ulysses: attention wants every token of a few heads, the rest of the layer wants every head of a few tokens.
    seq_to_heads   [S / W, H, D]  ->  [S, H / W, D]     (before attention)
    heads_to_seq   [S, H / W, D]  ->  [S / W, H, D]     (after attention)
Ring attention rotates key/value blocks one rank onward per step: ``ring_shift`` is an all-to-all-v whose only non-empty
stream goes to the next rank (the "hot ring" traffic pattern the variable-length protocol is stress-tested with).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import all_gather, all_to_all, all_to_all_v


def seq_to_heads(x: torch.Tensor, handle, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x``: this rank's [S / W, H, D] tokens with all heads. Returns [S, H / W, D]: all tokens, this rank's heads."""
    w = handle.world
    s_local, h, d = x.shape
    if h % w:
        raise ValueError("the number of heads must be divisible by the world size")
    # slice q of the send buffer = the heads that rank q will own
    send = x.view(s_local, w, h // w, d).permute(1, 0, 2, 3).contiguous()
    recv = torch.empty_like(send) if out is None else out.view(w, s_local, h // w, d)
    all_to_all(send, recv, handle)
    return recv.view(w * s_local, h // w, d)       # block q came from rank q = sequence chunk q


def heads_to_seq(x: torch.Tensor, handle, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of ``seq_to_heads``: [S, H / W, D] -> [S / W, H, D]."""
    w = handle.world
    s, h_local, d = x.shape
    if s % w:
        raise ValueError("the sequence length must be divisible by the world size")
    send = x.contiguous().view(w, s // w, h_local, d)      # slice q = the tokens rank q owns
    recv = torch.empty_like(send)
    all_to_all(send, recv, handle)
    # block q came from rank q = head group q; put the head groups back side by side
    res = recv.permute(1, 0, 2, 3).reshape(s // w, w * h_local, d)
    if out is not None:
        out.copy_(res)
        return out
    return res


def gather_sequence(x: torch.Tensor, handle, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All ranks' [S / W, ...] chunks side by side: the key/value gather of context-parallel attention."""
    w = handle.world
    x = x.contiguous()
    if out is None:
        out = torch.empty((w * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    all_gather(x, out, handle)
    return out


def ring_shift(x: torch.Tensor, handle, out: Optional[torch.Tensor] = None, step: int = 1) -> torch.Tensor:
    """Every rank sends ``x`` to rank ``(rank + step) % world`` and receives the block of rank ``(rank - step) % world``."""
    w, r = handle.world, handle.rank
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    n = x.numel() * x.element_size()
    if n % 32:
        raise ValueError("ring blocks must be a multiple of 32 bytes")
    step %= w
    if step == 0:
        out.copy_(x)
        return out
    in_splits = [n if q == (r + step) % w else 0 for q in range(w)]
    out_splits = [n if q == (r - step) % w else 0 for q in range(w)]
    all_to_all_v(x, out, in_splits + out_splits, handle)
    return out
