"""The allocation-free routing entry point, called through its exported C symbol.

Some callers may not allocate device memory when they need to route tokens (a server whose memory pool is frozen
after warm-up, an enqueue-style callback): `purlin_moe_route_noalloc` keeps its only scratch, the per-expert
counters, in a static device array of the library. This test calls the symbol with ctypes, twice in a row, and
compares each result with the context-based entry point: expert ids and gate weights must match exactly; slots
are handed out by atomics in whatever order warps run, so they are compared as what they must be, a numbering
0..count-1 of each expert's rows, with the same per-expert counts.  This file sorts last on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _slots_are_a_numbering(idx, slot, experts):
    flat_e, flat_s = idx.flatten().long().cpu(), slot.flatten().long().cpu()
    counts = torch.bincount(flat_e, minlength=experts)
    for e in torch.unique(flat_e).tolist():
        got = torch.sort(flat_s[flat_e == e]).values
        if not torch.equal(got, torch.arange(int(counts[e]))):
            return False, counts
    return True, counts


def test_route_noalloc_matches_context_route_twice():
    from purlin_b200 import _native
    from purlin_b200.parallel.expert_parallel import ExpertParallelContext
    lib = _native.cuda()
    fn = lib.purlin_moe_route_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    dev = torch.device("cuda", 0)
    tokens, experts, topk = 1024, 256, 8
    ep = ExpertParallelContext(None, dev, max_tokens=tokens, hidden=256, experts=experts, topk=topk)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):   # the second call reuses the scratch the first one left behind
        g = torch.Generator(device=dev).manual_seed(11 + call)
        logits = torch.randn(tokens, experts, generator=g, device=dev)
        ref_idx, ref_w = ep.route(logits)
        ref_slot = ep.slot[:tokens].clone()
        ref_idx, ref_w = ref_idx.clone(), ref_w.clone()
        idx = torch.full((tokens, topk), -1, dtype=torch.int32, device=dev)
        w = torch.zeros(tokens, topk, dtype=torch.float32, device=dev)
        slot = torch.full((tokens, topk), -1, dtype=torch.int32, device=dev)
        rc = fn(logits.data_ptr(), tokens, experts, topk, 1, idx.data_ptr(), w.data_ptr(), slot.data_ptr(), stream)
        assert rc == 0, _native.last_error(lib)
        torch.cuda.synchronize()
        # and against plain PyTorch: softmax, top-k, renormalised weights (ids as sets per token: equal logits may tie)
        tw, ti = torch.topk(torch.softmax(logits, dim=-1), topk, dim=-1)
        tw = tw / tw.sum(-1, keepdim=True)
        assert torch.equal(torch.sort(idx.long(), dim=-1).values, torch.sort(ti, dim=-1).values), f"call {call}: ids differ from torch.topk"
        assert torch.allclose(torch.sort(w, dim=-1).values, torch.sort(tw, dim=-1).values, atol=1e-5, rtol=1e-4)
        assert torch.equal(idx, ref_idx), f"call {call}: expert ids differ"
        assert torch.equal(w, ref_w), f"call {call}: gate weights differ"
        ok, counts = _slots_are_a_numbering(idx, slot, experts)
        ok_ref, counts_ref = _slots_are_a_numbering(ref_idx, ref_slot, experts)
        assert ok and ok_ref, f"call {call}: slots are not a numbering of each expert's rows"
        assert torch.equal(counts, counts_ref)
    ep.close()


def test_route_noalloc_rejects_sizes_beyond_its_scratch():
    from purlin_b200 import _native
    lib = _native.cuda()
    fn = lib.purlin_moe_route_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    x = torch.zeros(4, 1024, device="cuda")
    o = torch.zeros(4, 8, dtype=torch.int32, device="cuda")
    w = torch.zeros(4, 8, device="cuda")
    rc = fn(x.data_ptr(), 4, 1024, 8, 1, o.data_ptr(), w.data_ptr(), o.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "at most 512" in _native.last_error(lib)
