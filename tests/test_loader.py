"""Architecture adapters, checkpoint coverage and TP-sharded loading from real safetensors files."""
import json

import pytest
import torch
from safetensors.torch import save_file

from crosspool_b200.engine import checkpoint as ck
from crosspool_b200.engine import loader
from crosspool_b200.ffn import ActivationKind, DenseFfnSpec, MoeFfnSpec, RouterAlgorithm
from crosspool_b200.models import adapters

QWEN3 = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "intermediate_size": 256, "num_hidden_layers": 2,
         "num_attention_heads": 4, "vocab_size": 100, "hidden_act": "silu", "torch_dtype": "bfloat16"}
QWEN3_MOE = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 64, "num_hidden_layers": 1, "num_experts": 4,
             "num_experts_per_tok": 2, "moe_intermediate_size": 128, "norm_topk_prob": True, "num_attention_heads": 4,
             "vocab_size": 100}


def _dense_ckpt(tmp_path, shards=2):
    g = torch.Generator().manual_seed(0)
    tensors = {"model.embed_tokens.weight": torch.randn(100, 64, generator=g)}
    for i in range(2):
        p = f"model.layers.{i}."
        tensors[p + "mlp.gate_proj.weight"] = torch.randn(256, 64, generator=g)
        tensors[p + "mlp.up_proj.weight"] = torch.randn(256, 64, generator=g)
        tensors[p + "mlp.down_proj.weight"] = torch.randn(64, 256, generator=g)
        tensors[p + "self_attn.q_proj.weight"] = torch.randn(64, 64, generator=g)
    keys = sorted(tensors)
    wm = {}
    for s in range(shards):
        part = {k: tensors[k] for k in keys[s::shards]}
        name = f"model-{s:05d}-of-{shards:05d}.safetensors"
        save_file(part, str(tmp_path / name))
        wm.update({k: name for k in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    (tmp_path / "config.json").write_text(json.dumps(QWEN3))
    return tensors


def test_dense_spec_coverage_and_sharded_load(tmp_path):
    tensors = _dense_ckpt(tmp_path)
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("q", QWEN3, view.keys())
    assert spec.num_layers == 2 and isinstance(spec.layers[0], DenseFfnSpec)
    assert spec.layers[0].activation == ActivationKind.SILU and spec.payload_dtype == "bfloat16"
    ck.validate_ffn_coverage(spec, view)
    full = loader.materialize_layer_weights(spec, view, 1, dtype=torch.float32)
    g, u, d = (tensors[f"model.layers.1.mlp.{n}_proj.weight"] for n in ("gate", "up", "down"))
    assert torch.equal(full.gate_up, torch.cat([g, u])) and torch.equal(full.down, d)
    parts = [loader.materialize_layer_weights(spec, view, 1, tp_rank=r, tp_size=4, dtype=torch.float32) for r in range(4)]
    for r, p in enumerate(parts):
        rows = slice(64 * r, 64 * (r + 1))
        assert torch.equal(p.gate_up, torch.cat([g[rows], u[rows]])) and torch.equal(p.down, d[:, rows])
    x = torch.randn(3, 64)
    ref = (torch.nn.functional.silu(x @ g.t()) * (x @ u.t())) @ d.t()
    tp = sum((torch.nn.functional.silu(x @ p.gate_up[:64].t()) * (x @ p.gate_up[64:].t())) @ p.down.t() for p in parts)
    torch.testing.assert_close(tp, ref, atol=1e-4, rtol=1e-4)
    assert spec.digest() == adapters.compile_ffn_spec("q", QWEN3, view.keys()).digest()


def test_coverage_rejects_missing_and_unexplained_tensors(tmp_path):
    _dense_ckpt(tmp_path, shards=1)
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("q", QWEN3)
    del view.key_to_file["model.layers.0.mlp.up_proj.weight"]
    with pytest.raises(ck.CheckpointError, match="misses 1"):
        ck.validate_ffn_coverage(spec, view)
    with pytest.raises(adapters.UnsupportedModel, match="misses"):
        adapters.compile_ffn_spec("q", QWEN3, view.keys())
    view = ck.read_checkpoint_key_view(tmp_path)
    view.key_to_file["model.layers.0.mlp.surprise.weight"] = "x"
    with pytest.raises(ck.CheckpointError, match="does not cover"):
        ck.validate_ffn_coverage(spec, view)


def test_moe_spec_and_expert_parallel_load(tmp_path):
    g = torch.Generator().manual_seed(1)
    t = {"model.layers.0.mlp.gate.weight": torch.randn(4, 64, generator=g)}
    for e in range(4):
        for n, shape in (("gate_proj", (128, 64)), ("up_proj", (128, 64)), ("down_proj", (64, 128))):
            t[f"model.layers.0.mlp.experts.{e}.{n}.weight"] = torch.randn(*shape, generator=g)
    save_file(t, str(tmp_path / "model.safetensors"))
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("m", QWEN3_MOE, view.keys())
    l = spec.layers[0]
    assert isinstance(l, MoeFfnSpec) and l.router_algorithm == RouterAlgorithm.SOFTMAX and l.effective_topk == 2
    ck.validate_ffn_coverage(spec, view)
    w = loader.materialize_layer_weights(spec, view, 0, dtype=torch.float32, tp_rank=1, tp_size=2, experts=range(2, 4))
    assert w.gate_up.shape == (2, 128, 64) and w.down.shape == (2, 64, 64) and w.router.shape == (4, 64)
    assert torch.equal(w.gate_up[0, :64], t["model.layers.0.mlp.experts.2.gate_proj.weight"][64:128])
    assert torch.equal(w.down[1], t["model.layers.0.mlp.experts.3.down_proj.weight"][:, 64:128])


@pytest.mark.parametrize("arch,cfg,check", [
    ("LlamaForCausalLM", {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 1, "mlp_bias": True},
     lambda s: s.layers[0].o_proj.bias_key == "model.layers.0.mlp.down_proj.bias"),
    ("OPTForCausalLM", {"hidden_size": 64, "ffn_dim": 256, "num_hidden_layers": 1, "activation_function": "relu"},
     lambda s: not s.layers[0].i_proj.gated and s.layers[0].activation == ActivationKind.RELU
     and s.layers[0].o_proj.weight_key == "model.decoder.layers.0.fc2.weight"),
    ("DeepseekV2ForCausalLM", {"hidden_size": 64, "intermediate_size": 256, "moe_intermediate_size": 32,
                               "num_hidden_layers": 3, "n_routed_experts": 8, "num_experts_per_tok": 2,
                               "first_k_dense_replace": 1, "n_shared_experts": 2, "routed_scaling_factor": 16.0},
     lambda s: isinstance(s.layers[0], DenseFfnSpec) and isinstance(s.layers[1], MoeFfnSpec)
     and s.layers[1].num_shared_experts == 2 and s.layers[1].routed_scaling_factor == 16.0
     and s.layers[1].router_precision.value == "fp32_logits"),
    ("Glm4MoeLiteForCausalLM", {"hidden_size": 64, "intermediate_size": 256, "moe_intermediate_size": 32,
                                "num_hidden_layers": 2, "n_routed_experts": 8, "num_experts_per_tok": 2,
                                "first_k_dense_replace": 1, "n_shared_experts": 1},
     lambda s: s.layers[1].router_algorithm == RouterAlgorithm.SIGMOID
     and s.layers[1].correction_bias_key.endswith("e_score_correction_bias")),
    ("GptOssForCausalLM", {"hidden_size": 64, "intermediate_size": 64, "num_hidden_layers": 1, "num_local_experts": 4,
                           "num_experts_per_tok": 2, "quantization_config": {"quant_method": "mxfp4"}},
     lambda s: s.quantization == "mxfp4" and s.layers[0].gate_transform.alpha == 1.702
     and s.layers[0].gate_transform.limit == 7.0 and s.layers[0].experts.packed_key.endswith("gate_up_proj_blocks")),
])
def test_architecture_adapters(arch, cfg, check):
    spec = adapters.compile_ffn_spec("x", {"architectures": [arch], **cfg})
    assert check(spec)


def test_unsupported_models_are_named():
    with pytest.raises(adapters.UnsupportedModel, match="no FFN adapter"):
        adapters.compile_ffn_spec("x", {"architectures": ["MambaForCausalLM"], "hidden_size": 8})
    with pytest.raises(adapters.UnsupportedModel, match="quantization"):
        adapters.compile_ffn_spec("x", {**QWEN3, "quantization_config": {"quant_method": "awq"}})
    with pytest.raises(adapters.UnsupportedModel, match="misses 'intermediate_size'"):
        adapters.compile_ffn_spec("x", {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 8, "num_hidden_layers": 1})


def test_gpt_oss_mxfp4_checkpoint_loads_dequantised_shards_with_biases(tmp_path):
    """Stacked MXFP4 expert tensors (blocks + e8m0 scales, interleaved gate/up rows, per-expert biases) become
    bf16 gate|up and down shards; the clamp/offset/alpha of the activation travel with the layer."""
    from crosspool_b200.quantization import Mxfp4

    E, H, I = 4, 64, 64
    cfg = {"architectures": ["GptOssForCausalLM"], "hidden_size": H, "intermediate_size": I, "num_hidden_layers": 1,
           "num_local_experts": E, "num_experts_per_tok": 2, "quantization_config": {"quant_method": "mxfp4"},
           "num_attention_heads": 4, "vocab_size": 100}
    g = torch.Generator().manual_seed(3)
    fmt = Mxfp4()
    gu_q, dn_q = fmt.quantize(torch.randn(E, 2 * I, H, generator=g)), fmt.quantize(torch.randn(E, H, I, generator=g))
    p = "model.layers.0.mlp."
    tensors = {p + "router.weight": torch.randn(E, H, generator=g).bfloat16(), p + "router.bias": torch.randn(E, generator=g).bfloat16(),
               p + "experts.gate_up_proj_blocks": gu_q["blocks"].reshape(E, 2 * I, H // 32, 16),
               p + "experts.gate_up_proj_scales": gu_q["scales"],
               p + "experts.gate_up_proj_bias": torch.randn(E, 2 * I, generator=g).bfloat16(),
               p + "experts.down_proj_blocks": dn_q["blocks"].reshape(E, H, I // 32, 16),
               p + "experts.down_proj_scales": dn_q["scales"],
               p + "experts.down_proj_bias": torch.randn(E, H, generator=g).bfloat16()}
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("oss", cfg, view.keys())
    ck.validate_ffn_coverage(spec, view)
    gu, dn = fmt.dequantize(gu_q), fmt.dequantize(dn_q)          # [E, 2I, H] rows interleaved gate, up, gate, ...
    gb = tensors[p + "experts.gate_up_proj_bias"].float()
    for rank in (0, 1):
        w = loader.materialize_layer_weights(spec, view, 0, tp_rank=rank, tp_size=2, experts=range(1, 3))
        rows = slice(32 * rank, 32 * (rank + 1))
        assert w.gate_up.shape == (2, 64, H) and w.down.shape == (2, H, 32)
        for i, e in enumerate((1, 2)):
            assert torch.equal(w.gate_up[i], torch.cat([gu[e, 0::2][rows], gu[e, 1::2][rows]]))
            assert torch.equal(w.down[i], dn[e][:, rows])
            assert torch.equal(w.gate_up_bias[i], torch.cat([gb[e, 0::2][rows], gb[e, 1::2][rows]]))
        assert (w.down_bias is not None) == (rank == 0)          # added once across the TP group
        assert w.extra["gate_transform"] == (7.0, 1.0, 1.702) and w.extra["router_bias"].shape == (E,)
    assert w.gate_up_bias.dtype == torch.float32


def test_an_fp32_router_checkpoint_keeps_its_router_weights_in_fp32(tmp_path):
    """A sigmoid-scored (GLM-style) router is projected in fp32: the loader keeps an fp32 copy of the router weights
    beside the payload copy and names the precision on the layer; a DeepSeek-V2 router keeps payload weights."""
    H, I, E = 64, 32, 4
    base = {"hidden_size": H, "intermediate_size": 128, "moe_intermediate_size": I, "num_hidden_layers": 1, "n_routed_experts": E,
            "num_experts_per_tok": 2, "first_k_dense_replace": 0, "num_attention_heads": 4, "vocab_size": 100}
    g = torch.Generator().manual_seed(5)
    p = "model.layers.0.mlp."
    router = torch.randn(E, H, generator=g)       # fp32 in the checkpoint
    tensors = {p + "gate.weight": router, p + "gate.e_score_correction_bias": torch.randn(E, generator=g)}
    for e in range(E):
        tensors[f"{p}experts.{e}.gate_proj.weight"] = torch.randn(I, H, generator=g).bfloat16()
        tensors[f"{p}experts.{e}.up_proj.weight"] = torch.randn(I, H, generator=g).bfloat16()
        tensors[f"{p}experts.{e}.down_proj.weight"] = torch.randn(H, I, generator=g).bfloat16()
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    view = ck.read_checkpoint_key_view(tmp_path)
    for arch, prec in (("Glm4MoeLiteForCausalLM", "fp32"), ("DeepseekV2ForCausalLM", "fp32_logits")):
        spec = adapters.compile_ffn_spec("m", {"architectures": [arch], **base}, view.keys())
        w = loader.materialize_layer_weights(spec, view, 0)
        assert w.extra["router_precision"] == prec and w.router.dtype == torch.bfloat16
        if prec == "fp32":
            assert torch.equal(w.extra["router_fp32"], router) and torch.equal(w.router, router.bfloat16())
        else:
            assert "router_fp32" not in w.extra


def test_block_scaled_fp8_checkpoint_loads_on_block_boundaries_and_keeps_the_stored_codes(tmp_path):
    """A ``*-FP8`` style checkpoint (e4m3 weights + ``weight_scale_inv`` per 128 x 128 block): the loader expands the
    local shard to the compute dtype for the Lanes and hands the stored codes and scales to the fp8 GEMM path; TP
    shards are cut on block boundaries and sum to the whole layer."""
    import json

    import pytest
    import torch
    from safetensors.torch import save_file

    from crosspool_b200.engine import checkpoint as ck
    from crosspool_b200.engine import loader
    from crosspool_b200.models import adapters, reference
    from crosspool_b200.models import config as mc
    from crosspool_b200.quantization import Fp8Block

    hidden, inter = 256, 512
    hf = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": hidden, "num_hidden_layers": 2, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": inter, "vocab_size": 512, "hidden_act": "silu",
          "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}
    g = torch.Generator().manual_seed(0)
    fmt, tensors, dense = Fp8Block(), {}, {}
    for l in range(2):
        for name, shape in (("gate_proj", (inter, hidden)), ("up_proj", (inter, hidden)), ("down_proj", (hidden, inter))):
            q = fmt.quantize(torch.randn(shape, generator=g) * 0.2)
            key = f"model.layers.{l}.mlp.{name}"
            tensors[key + ".weight"], tensors[key + ".weight_scale_inv"] = q["weight"], q["scale"]
            dense[key] = fmt.dequantize(q, torch.float32)
    (tmp_path / "config.json").write_text(json.dumps(hf))
    save_file(tensors, str(tmp_path / "model.safetensors"))
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("q8", hf, view.keys())
    assert spec.quantization == "fp8_block"
    ck.validate_ffn_coverage(spec, view)                         # the scales are FFN tensors too
    cfg = mc.from_hf_config(hf, "q8")
    x = torch.randn(9, hidden, generator=g) * 0.5
    p = "model.layers.1.mlp."
    want = (torch.nn.functional.silu(x @ dense[p + "gate_proj"].t()) * (x @ dense[p + "up_proj"].t())) @ dense[p + "down_proj"].t()
    whole = loader.materialize_layer_weights(spec, view, 1, dtype=torch.float32)
    torch.testing.assert_close(reference.ffn_forward(x, whole, cfg), want, rtol=1e-5, atol=1e-5)
    assert whole.extra["fp8"]["gate_up"].dtype == torch.float8_e4m3fn and whole.extra["fp8"]["gate_up_scale"].shape == (2 * inter // 128, hidden // 128)
    assert torch.equal(whole.extra["fp8"]["down"].view(torch.uint8), tensors[p + "down_proj.weight"].view(torch.uint8))
    parts = [reference.ffn_forward(x, loader.materialize_layer_weights(spec, view, 1, tp_rank=r, tp_size=2, dtype=torch.float32), cfg)
             for r in range(2)]
    torch.testing.assert_close(sum(parts), want, rtol=1e-5, atol=1e-5)
    half = loader.materialize_layer_weights(spec, view, 1, tp_rank=1, tp_size=2, dtype=torch.float32)
    assert half.gate_up.shape == (inter, hidden) and half.extra["fp8"]["down_scale"].shape == (hidden // 128, inter // 2 // 128)
    with pytest.raises(ValueError, match="whole 128-wide blocks"):
        loader.materialize_layer_weights(spec, view, 1, tp_rank=0, tp_size=8)          # 512 / 8 = 64 rows: not a block
    with pytest.raises(adapters.UnsupportedModel, match="multiples of 128"):
        adapters.compile_ffn_spec("q8", {**hf, "intermediate_size": 320})


def test_attention_side_of_a_block_scaled_fp8_checkpoint_is_dequantised_with_its_scales(tmp_path):
    """Published fp8 checkpoints quantise q/k/v/o as well (shapes need not be whole blocks: the last block is partial).
    The attention loader multiplies the codes by their block scales instead of casting the bare codes."""
    import json

    import pytest
    import torch
    from safetensors.torch import save_file

    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import load_attention_from_safetensors
    from crosspool_b200.quantization import Fp8Block

    hf = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 192, "num_hidden_layers": 1, "num_attention_heads": 4,
          "num_key_value_heads": 2, "head_dim": 48, "intermediate_size": 256, "vocab_size": 64,
          "quantization_config": {"quant_method": "fp8", "weight_block_size": [128, 128]}}
    g = torch.Generator().manual_seed(1)
    fmt, tensors, dense = Fp8Block(), {}, {}

    def fp8(key, n, k):
        w = torch.randn(n, k, generator=g) * 0.3
        np_, kp = (n + 127) // 128 * 128, (k + 127) // 128 * 128
        padded = torch.zeros(np_, kp)
        padded[:n, :k] = w
        q = fmt.quantize(padded)
        tensors[key] = q["weight"].view(torch.uint8)[:n, :k].contiguous().view(torch.float8_e4m3fn)
        tensors[key + "_scale_inv"] = q["scale"]
        dense[key] = fmt.dequantize(q, torch.float32)[:n, :k]

    p = "model.layers.0."
    for name, n in (("q", 192), ("k", 96), ("v", 96)):
        fp8(p + f"self_attn.{name}_proj.weight", n, 192)
    fp8(p + "self_attn.o_proj.weight", 192, 192)
    for key, shape in ((p + "input_layernorm.weight", 192), (p + "post_attention_layernorm.weight", 192), ("model.norm.weight", 192),
                       (p + "self_attn.q_norm.weight", 48), (p + "self_attn.k_norm.weight", 48)):
        tensors[key] = torch.ones(shape, dtype=torch.bfloat16)
    tensors["model.embed_tokens.weight"] = (torch.randn(64, 192, generator=g) * 0.1).to(torch.bfloat16)
    tensors["lm_head.weight"] = (torch.randn(64, 192, generator=g) * 0.1).to(torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(hf))
    save_file(tensors, str(tmp_path / "model.safetensors"))
    cfg = mc.from_hf_config(hf, "q8")
    aw = load_attention_from_safetensors(cfg, tmp_path, dtype=torch.float32)
    want = torch.cat([dense[p + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
    torch.testing.assert_close(aw.layers[0].qkv, want, rtol=0, atol=0)
    torch.testing.assert_close(aw.layers[0].o, dense[p + "self_attn.o_proj.weight"], rtol=0, atol=0)
    assert float(aw.layers[0].qkv.abs().max()) < 3.0              # bare codes would reach hundreds
    del tensors[p + "self_attn.o_proj.weight_scale_inv"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(ValueError, match="scale_inv"):
        load_attention_from_safetensors(cfg, tmp_path, dtype=torch.float32)
