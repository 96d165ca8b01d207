"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4, per-K-block scaling) against the fp32 product of the
dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,n,k", [(1, 128, 128), (7, 256, 512), (64, 1024, 4096), (130, 384, 1024), (512, 512, 2048)])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_fp8_linear_matches_dequantised_reference(rows, n, k, splits):
    from crosspool_b200.ops import gemm
    from crosspool_b200.quantization import Fp8Block

    if splits > k // 128:
        pytest.skip("more splits than K blocks")
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + n)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.05
    w[:128, :128] *= 30.0                      # one block with a very different scale
    x = (torch.randn(rows, k, device="cuda", generator=g) * 0.5).bfloat16()
    x[0, :128] *= 20.0
    st = Fp8Block().quantize(w)
    xq, xs = gemm.quantize_act_fp8(x)
    # activation quantisation: scale = amax / 448 per (row, 128 block); dequantised error within e4m3 resolution
    xd = xq.float() * xs[:, :rows].t().repeat_interleave(128, dim=1)
    assert ((xd - x.float()).abs() <= 0.0625 * x.float().abs() + 1e-3 * x.float().abs().amax()).all()
    out = gemm.linear_fp8(x, st["weight"], st["scale"].contiguous(), splits=splits)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    ref = xd @ Fp8Block().dequantize(st, torch.float32).t()
    err = (out.float() - ref).abs()
    assert (err <= 2e-2 * ref.abs() + 2e-2 * ref.abs().amax()).all(), err.max().item()
    nrmse = (err.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item()
    assert nrmse < 5e-3, nrmse                 # bf16 output rounding only


def test_fp8_linear_adds_the_residual_and_tracks_the_bf16_product():
    from crosspool_b200.ops import gemm
    from crosspool_b200.quantization import Fp8Block

    torch.manual_seed(3)
    rows, n, k = 48, 512, 1024
    w = torch.randn(n, k, device="cuda") * 0.03
    x = (torch.randn(rows, k, device="cuda") * 0.5).bfloat16()
    resid = torch.randn(rows, n, device="cuda").bfloat16()
    st = Fp8Block().quantize(w)
    out = gemm.linear_fp8(x, st["weight"], st["scale"].contiguous(), resid=resid)
    full = x.float() @ w.t() + resid.float()
    rel = ((out.float() - full).pow(2).mean().sqrt() / full.pow(2).mean().sqrt()).item()
    assert rel < 0.05, rel                     # two e4m3 roundings (about 3 % each) against exact bf16 math
