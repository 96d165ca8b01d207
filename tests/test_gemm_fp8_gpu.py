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


def test_engine_with_fp8_ffn_weights_stays_close_to_the_bf16_model():
    from crosspool_b200.engine.atn_engine import AttentionEngine, EngineConfig
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import ReferenceModel
    from crosspool_b200.models.weights import quantize_ffn_layer_fp8, random_attention_weights, random_ffn_weights
    from crosspool_b200.ops import gemm

    cfg = mc.preset("Qwen/Qwen3-0.6B").with_layers(2)
    aw = random_attention_weights(cfg, 1, "cuda", torch.bfloat16)
    fw = random_ffn_weights(cfg, 1, "cuda", torch.bfloat16)
    ref = ReferenceModel(cfg, aw, fw)
    fq = [quantize_ffn_layer_fp8(w) for w in random_ffn_weights(cfg, 1, "cuda", torch.bfloat16)]
    eng = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fq), EngineConfig(max_batch=4, prefill_chunk=128, max_seq_len=256))
    eng.warmup()
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(0)).tolist()
    s = eng.add_request(prompt, 3)
    first = None
    while eng.has_work:
        for i, (sq, _) in enumerate(eng.step()):
            first = eng.logits[i].float().clone() if first is None else first
    gemm.check_status(eng.device)
    _, rl = ref.generate(torch.tensor(prompt, device="cuda"), 1)
    p, q = rl[0].float().log_softmax(-1), first.log_softmax(-1)
    kl = (p.exp() * (p - q)).sum().item()
    assert kl < 0.05, kl       # fp8 weights and activations in the FFNs only
