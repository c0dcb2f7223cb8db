"""tcgen05 GEMM numerics against a plain fp32 PyTorch reference of the same operation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand(m, k, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(m, k, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("m,n,k,bn", [(128, 256, 64, 0), (256, 512, 512, 256), (384, 448, 1024, 224), (1024, 1024, 4096, 0),
                                       (200, 264, 72, 128), (128, 3584, 8192, 0), (4096, 7168, 1024, 0),
                                       (2560, 2048, 512, 0)])   # the last two leave a small final wave on 74 CTA pairs
def test_gemm_matches_fp32_reference(m, n, k, bn):
    from purlin_b200.ops.gemm import gemm
    a, w = _rand(m, k, 1), _rand(n, k, 2, 0.05)
    out = gemm(a, w, bn=bn)
    torch.cuda.synchronize()
    ref = a.float() @ w.float().t()
    err = (out.float() - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-3      # bf16 output rounding dominates
    assert err <= tol, f"max abs error {err} > {tol}"
    # a stricter check on a sample of entries in relative terms
    rel = ((out.float() - ref).abs() / (ref.abs() + 1.0)).max().item()
    assert rel < 2e-2


def test_gemm_exact_on_small_integers():
    # integer operands and K small enough that every partial sum is exact in fp32 and the result in bf16
    from purlin_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randint(-2, 3, (512, 256), generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randint(-1, 2, (768, 256), generator=g, device="cuda").to(torch.bfloat16)
    out = gemm(a, w)
    ref = (a.float() @ w.float().t())
    assert torch.equal(out.float(), ref.to(torch.bfloat16).float())


def test_partial_last_wave_is_exact_on_small_integers():
    # 10 x 8 tiles on 74 CTA pairs: a full wave and a last wave of six tiles
    from purlin_b200.ops.gemm import gemm
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randint(-2, 3, (2560, 256), generator=g, device="cuda").to(torch.bfloat16)
    w = torch.randint(-1, 2, (2048, 256), generator=g, device="cuda").to(torch.bfloat16)
    out = gemm(a, w)
    ref = (a.float() @ w.float().t())
    assert torch.equal(out.float(), ref.to(torch.bfloat16).float())


@pytest.mark.parametrize("m,i,k", [(256, 512, 256), (1024, 3584, 2048), (2560, 1024, 512)])
def test_swiglu_epilogue(m, i, k):
    from purlin_b200.ops.gemm import gemm_swiglu, interleave_gate_up
    a, wg, wu = _rand(m, k, 3), _rand(i, k, 4, 0.05), _rand(i, k, 5, 0.05)
    out = gemm_swiglu(a, interleave_gate_up(wg, wu))
    torch.cuda.synchronize()
    g = a.float() @ wg.float().t()
    u = a.float() @ wu.float().t()
    ref = torch.nn.functional.silu(g) * u
    err = (out.float() - ref).abs().max().item()
    assert err <= 2e-2 * ref.abs().max().item() + 1e-3


def test_repeated_calls_are_bitwise_stable():
    from purlin_b200.ops.gemm import gemm
    a, w = _rand(1024, 2048, 7), _rand(2048, 2048, 8, 0.05)
    first = gemm(a, w).clone()
    for _ in range(5):
        assert torch.equal(gemm(a, w), first)
