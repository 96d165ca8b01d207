import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_rmsnorm(x, w, eps):
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (n.bfloat16().float() * w.float())


@pytest.mark.parametrize("rows,hidden", [(1, 256), (3, 1024), (17, 2048), (64, 4096), (5, 5120), (2, 8192)])
def test_rmsnorm(rows, hidden):
    from crosspool_b200.ops import norm

    g = torch.Generator(device="cuda").manual_seed(rows + hidden)
    x = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16()
    y = norm.rmsnorm(x, w, 1e-6)
    torch.testing.assert_close(y.float(), _ref_rmsnorm(x, w, 1e-6), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("nparts", [1, 2, 4])
def test_add_rmsnorm_folds_partials_in_order(nparts):
    from crosspool_b200.ops import norm

    g = torch.Generator(device="cuda").manual_seed(nparts)
    rows, hidden = 9, 1024
    parts = [torch.randn(rows, hidden, device="cuda", generator=g).bfloat16() for _ in range(nparts)]
    resid = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).bfloat16()
    acc = torch.zeros(rows, hidden, device="cuda")
    for p in parts:
        acc += p.float()
    if nparts > 1:
        acc = acc.bfloat16().float()
    new_resid = (acc + resid.float()).bfloat16()
    r = resid.clone()
    y = norm.add_rmsnorm(parts, w, 1e-6, resid=r)
    assert torch.equal(r, new_resid)
    torch.testing.assert_close(y.float(), _ref_rmsnorm(new_resid, w, 1e-6), atol=2e-2, rtol=2e-2)


def test_publish_to_local_destinations_and_flag():
    from crosspool_b200.ops import norm

    rows, hidden = 33, 512
    x = torch.randn(rows, hidden, device="cuda").bfloat16()
    w = torch.ones(hidden, device="cuda").bfloat16()
    dst = [torch.zeros(rows, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    flags = torch.zeros(2, 8, device="cuda", dtype=torch.int32)
    meta = torch.zeros(2, 4, device="cuda", dtype=torch.int32)
    y = norm.add_rmsnorm(x, w, 1e-6, peer_ptrs=[d.data_ptr() for d in dst],
                         peer_flag_ptrs=[flags[i].data_ptr() for i in range(2)],
                         peer_meta_ptrs=[meta[i].data_ptr() for i in range(2)], publish_seq=7, meta=(3, 2, 99))
    torch.cuda.synchronize()
    for d in dst:
        assert torch.equal(d, y)
    assert flags[:, 0].tolist() == [7, 7]
    assert meta[0].tolist() == [rows, 3, 2, 99]


def test_wait_on_a_flag_that_nothing_sets_times_out_cleanly():
    """A bounded device wait runs out, the kernel poisons its output and reports a status."""
    from crosspool_b200.ops import gemm, norm

    x = torch.randn(2, 256, device="cuda").bfloat16()
    w = torch.ones(256, device="cuda").bfloat16()
    never = torch.zeros(4, device="cuda", dtype=torch.int32)
    y = norm.add_rmsnorm(x, w, 1e-6, wait_flag_ptrs=[never.data_ptr()], wait_seq=1, wait_ns=20_000_000)
    torch.cuda.synchronize()
    assert torch.isnan(y.float()).all()
    with pytest.raises(RuntimeError):
        gemm.check_status(x.device)
    # the context is still usable afterwards
    y2 = norm.rmsnorm(x, w)
    torch.cuda.synchronize()
    assert torch.isfinite(y2.float()).all()


def test_swiglu_unfused():
    from crosspool_b200.ops import norm

    gu = torch.randn(5, 512, device="cuda").bfloat16()
    y = norm.swiglu(gu)
    ref = torch.nn.functional.silu(gu[:, :256].float()) * gu[:, 256:].float()
    torch.testing.assert_close(y.float(), ref, atol=2e-2, rtol=2e-2)


def test_debug_options_round_trip_through_device_constant_memory():
    from crosspool_b200 import native

    before = native.get_debug_options()
    try:
        native.set_debug_options({"fabric_observer": True, "ffn_routing_observer": True})
        assert native.get_debug_options() == {"transport_observer": False, "fabric_observer": True, "graph_observer": False,
                                              "ffn_routing_observer": True}
    finally:
        native.set_debug_options(before)
