"""tcgen05 GEMM numerics against a plain fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_linear(x, w, bias=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias
    return y


def _close(got, want, atol=2e-2, rtol=2e-2):
    # tolerances of the reference's FFN qualification (src/xpool-dev/xtest/harness/support/ffn.py:20-28)
    got, want = got.float(), want.float()
    assert torch.isfinite(got).all()
    torch.testing.assert_close(got, want, atol=atol, rtol=rtol)
    nrmse = ((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt().clamp_min(1e-12)).item()
    assert nrmse <= 1e-2, nrmse


@pytest.mark.parametrize("rows", [1, 3, 16, 17, 64, 200, 1000])
@pytest.mark.parametrize("n,k", [(128, 64), (256, 256), (1024, 1024), (3072, 1024), (1024, 3072)])
def test_linear_matches_fp32(rows, n, k):
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(rows * 7 + n + k)
    x = (torch.randn(rows, k, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.05).bfloat16()
    y = gemm.linear(x, w)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    _close(y, _ref_linear(x, w))


@pytest.mark.parametrize("splits", [1, 2, 4])
@pytest.mark.parametrize("rows", [2, 48, 300])
def test_linear_split_k_and_bias_and_residual(rows, splits):
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(11 + rows + splits)
    n, k = 512, 2048
    x = (torch.randn(rows, k, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.03).bfloat16()
    b = torch.randn(n, device="cuda", generator=g)
    r = torch.randn(rows, n, device="cuda", generator=g).bfloat16()
    y = gemm.linear(x, w, bias=b, splits=splits)
    y2 = gemm.linear(x, w, resid=r, splits=splits)
    y3 = gemm.linear(x, w, out_fp32=True, splits=splits)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    ref = _ref_linear(x, w)
    _close(y, ref + b)
    _close(y2, ref.bfloat16().float() + r.float())
    _close(y3, ref, atol=1e-2, rtol=1e-2)


@pytest.mark.parametrize("bn", [16, 32, 64, 128])
def test_explicit_tile_widths(bn):
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(bn)
    x = (torch.randn(130, 512, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(384, 512, device="cuda", generator=g) * 0.05).bfloat16()
    y = gemm.linear(x, w, bn=bn)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    _close(y, _ref_linear(x, w))


@pytest.mark.parametrize("rows", [1, 5, 64, 129, 700])
@pytest.mark.parametrize("hidden,inter", [(256, 768), (1024, 3072)])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_gateup_swiglu(rows, hidden, inter, splits):
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(rows + hidden + splits)
    x = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(2 * inter, hidden, device="cuda", generator=g) * 0.05).bfloat16()
    y = gemm.gateup_swiglu(x, w, splits=splits)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    gu = _ref_linear(x, w).bfloat16().float()  # projection rounded to the payload dtype first
    ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
    _close(y, ref)


def test_repeated_calls_are_bitwise_stable():
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(5)
    x = (torch.randn(7, 4096, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(256, 4096, device="cuda", generator=g) * 0.05).bfloat16()
    a = gemm.linear(x, w, splits=4)
    b = gemm.linear(x, w, splits=4)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("rows", [4, 100, 600])
def test_tiled_weight_layout_gives_identical_results(rows):
    from crosspool_b200.ops import gemm

    g = torch.Generator(device="cuda").manual_seed(rows)
    x = (torch.randn(rows, 1024, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(768, 1024, device="cuda", generator=g) * 0.05).bfloat16()
    wt = gemm.tile_weight(w)
    assert torch.equal(wt.untiled(), w)
    assert torch.equal(gemm.linear(x, wt), gemm.linear(x, w))
    assert torch.equal(gemm.gateup_swiglu(x, wt), gemm.gateup_swiglu(x, w))
    gemm.check_status(x.device)
