"""The MoE top-k selection on the host restatement of the routing kernels' arithmetic (csrc/include/purlin/moe_route.cuh).

The selection must be total: for any logits (NaN, +inf, -inf, rows with fewer than k usable values) every choice is a
distinct expert id inside [0, experts) and every weight is finite. The GPU kernels run the same code path; the GPU
tests compare them with this host function.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from purlin_b200 import _native


def route_host(logits: np.ndarray, topk: int, normalize: bool = True):
    lib = _native.host()
    lib.purlin_moe_route_host.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    t, e = logits.shape
    idx = np.full((t, topk), -7, dtype=np.int32)
    w = np.full((t, topk), np.nan, dtype=np.float32)
    rc = lib.purlin_moe_route_host(logits.ctypes.data, t, e, topk, int(normalize), idx.ctypes.data, w.ctypes.data)
    assert rc == 0, _native.last_error(lib)
    return idx, w


def test_matches_torch_softmax_topk_on_ordinary_rows():
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(257, 256, generator=g)
    idx, w = route_host(logits.numpy(), 8)
    tw, ti = torch.topk(torch.softmax(logits, -1), 8, dim=-1)
    tw = tw / tw.sum(-1, keepdim=True)
    assert np.array_equal(idx, ti.numpy().astype(np.int32))
    assert np.allclose(w, tw.numpy(), rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("fill", [float("nan"), float("inf"), float("-inf")])
def test_degenerate_rows_still_give_valid_distinct_experts(fill):
    experts, topk = 64, 8
    rows = np.full((5, experts), fill, dtype=np.float32)
    rows[1, 3] = 0.5                      # one usable value
    rows[2, :4] = [1.0, 2.0, 3.0, 4.0]    # fewer usable values than top-k
    rows[3, ::2] = 0.0
    rows[4] = np.linspace(-1, 1, experts)
    rows[4, 10] = fill
    idx, w = route_host(rows, topk)
    assert idx.min() >= 0 and idx.max() < experts
    for r in range(rows.shape[0]):
        assert len(set(idx[r].tolist())) == topk, f"row {r}: repeated expert"
    assert np.isfinite(w).all() and (w >= 0).all()
    # ties go to the lowest ids: an all-equal row picks experts 0..k-1 with equal weights
    assert idx[0].tolist() == list(range(topk))
    assert np.allclose(w[0], 1.0 / topk)


def test_usable_values_win_over_masked_ones():
    experts, topk = 32, 4
    row = np.full((1, experts), float("-inf"), dtype=np.float32)
    row[0, [7, 20]] = [1.0, 3.0]
    idx, w = route_host(row, topk)
    assert idx[0, 0] == 20 and idx[0, 1] == 7
    assert w[0, 2] == 0.0 and w[0, 3] == 0.0 and abs(w[0].sum() - 1.0) < 1e-6
    nan_row = np.zeros((1, experts), dtype=np.float32)
    nan_row[0, 5] = float("nan")
    idx, _ = route_host(nan_row, topk)
    assert 5 not in idx[0].tolist()
