"""Deployments load real-layout checkpoints: the FFN tier through the adapter + pinned loader, the attention
side through the safetensors reader; presets keep random init."""
import pytest
import torch

from crosspool_b200.testing import write_synthetic_checkpoint

DENSE = {"architectures": ["Qwen3ForCausalLM"], "hidden_size": 256, "intermediate_size": 512, "num_hidden_layers": 2,
         "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 512, "hidden_act": "silu",
         "torch_dtype": "bfloat16", "tie_word_embeddings": False, "rms_norm_eps": 1e-6, "rope_theta": 10000.0}
MOE = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 256, "num_hidden_layers": 1, "num_experts": 8,
       "num_experts_per_tok": 2, "moe_intermediate_size": 128, "norm_topk_prob": True, "num_attention_heads": 4,
       "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 512, "torch_dtype": "bfloat16"}


def _cfg_toml(path):
    return f"""
[daemon]
port = 18000
[atn]
devices = [0]
[ffn]
devices = [1]
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[[models]]
id = "tiny"
path = "{path}"
[[models]]
id = "Qwen/Qwen3-0.6B"
"""


def test_model_path_with_safetensors_selects_checkpoint_loading(tmp_path):
    from crosspool_b200.config import load_config
    from crosspool_b200.runtime.backends import checkpoint_dir_for, model_config_for

    write_synthetic_checkpoint(tmp_path / "tiny", DENSE)
    cfg = load_config(env={}, toml_text=_cfg_toml(tmp_path / "tiny"))
    assert checkpoint_dir_for(cfg, "tiny") == str(tmp_path / "tiny")
    assert checkpoint_dir_for(cfg, "Qwen/Qwen3-0.6B") is None           # a preset: random init
    mcfg = model_config_for(cfg, "tiny")
    assert (mcfg.hidden_size, mcfg.num_layers, mcfg.num_kv_heads, mcfg.head_dim) == (256, 2, 2, 64)


def test_checkpoint_source_shards_match_the_files(tmp_path):
    from crosspool_b200.parallel.fabric import CheckpointFfnSource

    t = write_synthetic_checkpoint(tmp_path, DENSE)
    src = CheckpointFfnSource("tiny", str(tmp_path))
    g, u, d = (t[f"model.layers.1.mlp.{n}_proj.weight"] for n in ("gate", "up", "down"))
    for r in range(2):
        w = src.layer(1, "cpu", tp_rank=r, tp_size=2)
        rows = slice(256 * r, 256 * (r + 1))
        assert torch.equal(w.gate_up, torch.cat([g[rows], u[rows]])) and torch.equal(w.down, d[:, rows])


def test_checkpoint_source_expert_ranges(tmp_path):
    from crosspool_b200.parallel.fabric import CheckpointFfnSource

    t = write_synthetic_checkpoint(tmp_path, MOE)
    src = CheckpointFfnSource("tiny-moe", str(tmp_path))
    w = src.layer(0, "cpu", expert_range=(4, 8))
    assert w.gate_up.shape == (4, 256, 256) and w.down.shape == (4, 256, 128) and w.router.shape == (8, 256)
    e5 = "model.layers.0.mlp.experts.5."
    assert torch.equal(w.gate_up[1], torch.cat([t[e5 + "gate_proj.weight"], t[e5 + "up_proj.weight"]]))
    assert torch.equal(w.router, t["model.layers.0.mlp.gate.weight"])


def test_attention_weights_from_checkpoint_match_the_files(tmp_path):
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import load_attention_from_safetensors

    t = write_synthetic_checkpoint(tmp_path, DENSE)
    cfg = mc.load(str(tmp_path))
    aw = load_attention_from_safetensors(cfg, tmp_path, "cpu", torch.bfloat16)
    p = "model.layers.1.self_attn."
    assert torch.equal(aw.layers[1].qkv, torch.cat([t[p + f"{n}_proj.weight"] for n in "qkv"]))
    assert torch.equal(aw.layers[1].o, t[p + "o_proj.weight"]) and torch.equal(aw.layers[1].q_norm, t[p + "q_norm.weight"])
    assert torch.equal(aw.lm_head, t["lm_head.weight"]) and torch.equal(aw.final_norm, t["model.norm.weight"])


@pytest.mark.gpu
def test_lane_runs_a_layer_loaded_from_a_checkpoint(tmp_path):
    """An FFN rank that loaded its shard from safetensors files produces the layer the files describe."""
    from crosspool_b200 import testing
    from crosspool_b200.models import config as mc
    from crosspool_b200.parallel import fabric as F

    t = write_synthetic_checkpoint(tmp_path, DENSE, scale=0.05)
    cfg = mc.load(str(tmp_path))
    place = F.InstancePlacement("tiny", cfg, seed=0, atn_rank=0, ffn_ranks=(1,), capacity_rows=64, checkpoint=str(tmp_path))
    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    st = ffn.add_instance(place, 0)
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    st.atn_base = buf.ptr
    ffn.install()
    try:
        x = (torch.randn(17, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        flay, alay = F.ffn_slot_layout(place), F.atn_slot_layout(place)
        st.slot.tensor(flay.input_offset, (place.capacity_rows, cfg.hidden_size), torch.bfloat16, "cuda")[:17] = x
        rec = st.slot.tensor(flay.record_offset, (64,), torch.int32, "cuda")
        rec[0], rec[1], rec[2], rec[3] = 17, 1, 2, 0      # rows, layer, mode, deadline
        rec[8] = 1                                        # InvocationRecord.sequence
        torch.cuda.synchronize()
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        out = buf.tensor(alay.output_offset, (place.capacity_rows, cfg.hidden_size), torch.bfloat16, "cuda")[:17].float()
        done = buf.tensor(alay.completion_offset, (64,), torch.int32, "cuda")
        assert (int(done[0]), int(done[1]), int(done[4])) == (0, 17, 1)      # result code, rows, sequence
        g, u, d = (t[f"model.layers.1.mlp.{n}_proj.weight"].cuda().float() for n in ("gate", "up", "down"))
        xf = x.float()
        ref = (torch.nn.functional.silu(xf @ g.t()) * (xf @ u.t())) @ d.t()
        testing.assert_ffn_close(out, ref)
    finally:
        ffn.close()
