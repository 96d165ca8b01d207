"""MoE path (router top-k, route ordering, grouped tcgen05 GEMM, combine) against the dense-loop
PyTorch reference, including the expert-parallel partial sums."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(E=8, k=2, hidden=256, inter=128, **kw):
    from crosspool_b200.models.config import ModelConfig

    return ModelConfig(name="t", architecture="Qwen3MoeForCausalLM", hidden_size=hidden, num_layers=1, num_q_heads=4,
                       num_kv_heads=2, head_dim=64, intermediate_size=inter, vocab_size=128, num_experts=E,
                       num_experts_per_tok=k, moe_intermediate_size=inter, **kw)


@pytest.mark.parametrize("sigmoid,bias", [(False, False), (True, True)])
@pytest.mark.parametrize("E,k", [(8, 2), (128, 8), (64, 6)])
def test_router_topk_matches_reference_rules(E, k, sigmoid, bias):
    from crosspool_b200.models.reference import route_topk
    from crosspool_b200.ops import moe

    g = torch.Generator(device="cuda").manual_seed(E + k)
    rows = 37
    logits = torch.randn(rows, E, device="cuda", generator=g)
    logits[3, 5] = logits[3, 2]  # an exact tie
    cb = torch.randn(E, device="cuda", generator=g) * 0.1 if bias else None
    ids = torch.zeros(rows, k, dtype=torch.int32, device="cuda")
    w = torch.zeros(rows, k, device="cuda")
    moe.router_topk(logits, E, k, out_ids=ids, out_weights=w, sigmoid=sigmoid, renormalize=True, scale=2.5,
                    correction_bias=cb)
    rid, rw = route_topk(logits, k, True, "sigmoid" if sigmoid else "softmax", cb, 2.5)
    assert torch.equal(ids.long(), rid)
    torch.testing.assert_close(w, rw, atol=1e-4, rtol=1e-3)  # the reference's routing tolerances


@pytest.mark.parametrize("rows", [1, 9, 130])
@pytest.mark.parametrize("E,k,hidden,inter", [(8, 2, 256, 128), (128, 8, 2048, 768)])
def test_moe_forward_matches_dense_loop_reference(rows, E, k, hidden, inter):
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.models.weights import random_ffn_layer
    from crosspool_b200.ops import gemm, moe

    cfg = _cfg(E, k, hidden, inter)
    w = random_ffn_layer(cfg, 0, seed=5, device="cuda", dtype=torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(rows)
    x = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16()
    y = moe.moe_forward(x, w, cfg)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    ref = moe_ffn(x, w, cfg)
    err = (y.float() - ref.float()).abs()
    scale = ref.float().abs().max().clamp_min(1e-6)
    assert (err.max() / scale).item() < 0.05
    nrmse = (err.pow(2).mean().sqrt() / ref.float().pow(2).mean().sqrt().clamp_min(1e-9)).item()
    assert nrmse < 0.02, nrmse


def test_expert_parallel_partials_sum_to_the_full_result():
    from crosspool_b200.models.weights import FfnLayerWeights, random_ffn_layer
    from crosspool_b200.ops import moe

    cfg = _cfg(8, 2, 256, 128)
    w = random_ffn_layer(cfg, 0, seed=7, device="cuda", dtype=torch.bfloat16)
    x = (torch.randn(40, 256, device="cuda") * 0.5).bfloat16()
    full = moe.moe_forward(x, w, cfg).float()
    parts = []
    for lo, hi in ((0, 4), (4, 8)):
        shard = FfnLayerWeights(w.gate_up[lo:hi].contiguous(), w.down[lo:hi].contiguous(), router=w.router)
        parts.append(moe.moe_forward(x, shard, cfg, expert_range=(lo, hi)).float())
    torch.testing.assert_close(parts[0] + parts[1], full, atol=3e-2, rtol=3e-2)
    # a token routed only to the other rank's experts contributes exactly zero here
    logits = x.float() @ w.router.float().t()
    k = cfg.num_experts_per_tok
    vals, idx = logits.topk(k + 1, dim=-1)
    clear = (vals[:, k - 1] - vals[:, k]) > 0.05        # selection not within bf16 rounding of a tie
    top = idx[:, :k]
    only_hi, only_lo = (top >= 4).all(-1) & clear, (top < 4).all(-1) & clear
    assert only_hi.any() or only_lo.any()      # 40 tokens, top-2 of 8: some token lives on one rank only
    assert (parts[0][only_hi] == 0).all() and (parts[1][only_lo] == 0).all()


def _gpt_oss_like(w, E, hidden, inter, seed):
    """Adds what a GPT-OSS expert layer carries beyond plain SwiGLU experts: per-expert biases on both
    projections, a router bias, and the clamp / offset / sigmoid-slope of its activation."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    w.gate_up_bias = torch.randn(E, 2 * inter, device="cuda", generator=g) * 0.3
    w.down_bias = torch.randn(E, hidden, device="cuda", generator=g) * 0.3
    w.extra["router_bias"] = torch.randn(E, device="cuda", generator=g) * 0.5
    w.extra["gate_transform"] = (1.5, 1.0, 1.702)   # a tight limit so that the clamps bite at this scale
    return w


@pytest.mark.parametrize("rows", [3, 77])
def test_moe_forward_with_expert_biases_and_gate_transform(rows):
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.models.weights import random_ffn_layer
    from crosspool_b200.ops import gemm, moe
    from crosspool_b200.testing import assert_ffn_close

    E, k, hidden, inter = 8, 2, 256, 128
    cfg = _cfg(E, k, hidden, inter)
    w = _gpt_oss_like(random_ffn_layer(cfg, 0, seed=11, device="cuda", dtype=torch.bfloat16), E, hidden, inter, 1)
    x = (torch.randn(rows, hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(rows)) * 0.5).bfloat16()
    y = moe.moe_forward(x, w, cfg)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    ref = moe_ffn(x, w, cfg)
    assert_ffn_close(y.float(), ref.float())
    plain = moe_ffn(x, random_ffn_layer(cfg, 0, seed=11, device="cuda", dtype=torch.bfloat16), cfg)
    assert (plain.float() - ref.float()).abs().max() > 0.05       # the additions matter at this scale


@pytest.mark.parametrize("precision,scoring", [("fp32_logits", "softmax"), ("fp32", "sigmoid")])
@pytest.mark.parametrize("rows,E,hidden", [(5, 8, 256), (130, 64, 2048), (33, 160, 1536)])
def test_fp32_router_projection_matches_an_fp32_matmul(rows, E, hidden, precision, scoring):
    """The projection itself (fp32 accumulate, fp32 logits) within the reference's routing tolerances, and the routing
    decision of the whole layer equal to the oracle's."""
    from crosspool_b200.models.reference import moe_ffn, route_topk
    from crosspool_b200.models.weights import random_ffn_layer
    from crosspool_b200.ops import gemm, moe

    cfg = _cfg(E, min(4, E), hidden, 128, router_precision=precision, router_scoring=scoring)
    w = random_ffn_layer(cfg, 0, seed=9, device="cuda", dtype=torch.bfloat16)
    assert w.extra["router_precision"] == precision and (precision != "fp32" or w.extra["router_fp32"].dtype == torch.float32)
    g = torch.Generator(device="cuda").manual_seed(rows + E)
    x = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16()
    out = torch.full((rows, (E + 127) // 128 * 128), float("nan"), device="cuda")
    moe.router_project_fp32(x, w, out)
    rw = w.extra["router_fp32"] if precision == "fp32" else w.router.float()
    ref = x.double() @ rw.double().t()
    torch.testing.assert_close(out[:, :E].double(), ref, atol=1e-4, rtol=1e-3)
    ids = torch.zeros(rows, cfg.num_experts_per_tok, dtype=torch.int32, device="cuda")
    wt = torch.zeros(rows, cfg.num_experts_per_tok, device="cuda")
    moe.router_topk(out[:, :E] if E % 128 == 0 else out, E, cfg.num_experts_per_tok, out_ids=ids, out_weights=wt,
                    sigmoid=scoring == "sigmoid", renormalize=True)
    rid, rwt = route_topk(ref.float(), cfg.num_experts_per_tok, True, scoring)
    same = (ids.long().sort(-1).values == rid.sort(-1).values).all(-1).float().mean().item()
    assert same >= 0.97, same      # a near-tie may flip between fp32 and fp64 accumulation; nothing else may
    y = moe.moe_forward(x, w, cfg)
    torch.cuda.synchronize()
    gemm.check_status(x.device)
    r = moe_ffn(x, w, cfg).float()
    err = (y.float() - r).abs()
    assert (err.pow(2).mean().sqrt() / r.pow(2).mean().sqrt().clamp_min(1e-9)).item() < 0.03
