"""Serving-engine integration surface with lightweight fakes (no engine installed): server-arg
rules, adapter discovery, shim installation and the ``xpool::ffn_shim`` op schema."""
import types

import pytest
import torch

from crosspool_b200.integrations.sglang import adapter as A
from crosspool_b200.integrations.sglang import plugin, server_args as S, shim
from crosspool_b200.native import runtime as rt


def test_server_arg_rules_name_every_offending_flag():
    ok = types.SimpleNamespace(tp_size=2, dp_size=1, cuda_graph_backend_decode="full", cuda_graph_backend_prefill="breakable")
    S.validate_server_args(ok, atn_tp_size=2)
    bad = types.SimpleNamespace(tp_size=2, dp_size=1, pp_size=2, speculative_algorithm="EAGLE", enable_lora=True,
                                enable_mlp_allreduce_fusion=True, cuda_graph_backend_prefill="full")
    with pytest.raises(S.ServerArgsError) as e:
        S.validate_server_args(bad, atn_tp_size=2)
    msg = str(e.value)
    for flag in ("--pp-size", "--speculative-algorithm", "--enable-lora", "--enable-mlp-allreduce-fusion",
                 "--cuda-graph-backend-prefill"):
        assert flag in msg
    with pytest.raises(S.ServerArgsError, match="enable-dp-attention"):
        S.validate_server_args(types.SimpleNamespace(tp_size=4, dp_size=4), atn_tp_size=1, atn_dp_size=4)
    with pytest.raises(S.ServerArgsError, match="tensor-parallel-size"):
        S.validate_server_args(types.SimpleNamespace(tp_size=1, dp_size=1), atn_tp_size=2)


def test_ffn_weights_are_filtered_from_the_attention_side():
    names = ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.gate_proj.weight",
             "model.layers.11.mlp.experts.3.down_proj.weight", "model.decoder.layers.2.fc1.weight", "lm_head.weight",
             "model.layers.0.post_attention_layernorm.weight"]
    kept = [n for n, _ in A.filter_decoder_ffn_weights((n, None) for n in names)]
    assert kept == ["model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "lm_head.weight",
                    "model.layers.0.post_attention_layernorm.weight"]


class _Layer(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.self_attn = torch.nn.Linear(4, 4)
        self.mlp = torch.nn.Linear(4, 4)


class _Model(torch.nn.Module):
    def __init__(self, n=3):
        super().__init__()
        self.model = torch.nn.Module()
        self.model.layers = torch.nn.ModuleList(_Layer() for _ in range(n))


def test_adapter_discovery_shim_installation_and_guards():
    runner = types.SimpleNamespace(model_config=types.SimpleNamespace(architecture="Qwen3MoeForCausalLM"))
    ad = A.find_adapter(runner)
    assert ad.name == "qwen3_moe" and ad.supports_dp_attention
    with pytest.raises(LookupError):
        A.find_adapter(types.SimpleNamespace(model_config=types.SimpleNamespace(architecture="Nope")))
    dense = A.find_adapter(types.SimpleNamespace(model_config=types.SimpleNamespace(architecture="Qwen3ForCausalLM")))
    with pytest.raises(ValueError, match="data parallelism"):
        dense.validate_before_load(runner, A.InstanceRankBinding("m", 0, 1, 4))
    model = _Model()
    with pytest.raises(RuntimeError, match="kept their MLP"):
        dense.require_ffn_shims(model, 3, shim.FfnShimModule)
    shims = dense.install_shims(model, lambda i, old: shim.FfnShimModule(i))
    assert [s.layer_ordinal for s in shims] == [0, 1, 2]
    assert dense.require_ffn_shims(model, 3, shim.FfnShimModule) == shims
    dense.require_no_ffn_parameters(model)  # the shims hold no parameters
    assert sum(p.numel() for s in shims for p in s.parameters()) == 0


def test_shim_forward_maps_modes_and_calls_the_op():
    calls = []

    def submit(h, rows, out, layer, mode, req, layout):
        calls.append((layer, mode, req, layout, rows is not None))
        out.copy_(h * 2)

    shim.bind_submit(submit)
    try:
        m = shim.FfnShimModule(5)
        x = torch.ones(3, 8)
        fb = types.SimpleNamespace(forward_mode=types.SimpleNamespace(name="DECODE"), dp_padding_mode=None)
        assert torch.equal(m(x, fb), x * 2)
        fb2 = types.SimpleNamespace(forward_mode=types.SimpleNamespace(name="EXTEND"),
                                    dp_padding_mode=types.SimpleNamespace(name="SUM_LEN"), mlp_reduce_scatter=True,
                                    global_num_tokens_gpu=torch.tensor([3, 1]))
        m(x, fb2)
        assert calls == [(5, rt.MODE_DECODE, rt.OUT_PER_RANK_COMPLETE, rt.DP_NONE, False),
                         (5, rt.MODE_PREFILL, rt.OUT_GROUP_SUM_COMPLETE, rt.DP_PACKED_BY_RANK, True)]
        with pytest.raises(RuntimeError, match="all-reduce"):
            m(x, types.SimpleNamespace(forward_mode="DECODE", fuse_mlp_allreduce=True))
        schema = str(torch.ops.xpool.ffn_shim.default._schema)
        assert "Tensor? dp_rank_payload_rows" in schema and "Tensor(a!) output" in schema
    finally:
        shim.bind_submit(None)
    with pytest.raises(RuntimeError, match="before an Instance runtime"):
        shim.FfnShimModule(0)(torch.ones(1, 2), types.SimpleNamespace(forward_mode="DECODE"))


def test_plugin_install_registers_hooks_and_sets_engine_switches():
    class Registry:
        def __init__(self, drop=None):
            self.reg, self.drop = [], drop

        def register(self, target, handler, kind):
            if target != self.drop:
                self.reg.append((target, kind))

        def applied_targets(self):
            return {t for t, _ in self.reg}

    env, checked = {}, []
    hooks = plugin.install(Registry(), check_config=lambda: checked.append(1), environ=env)
    assert checked == [1] and env["SGLANG_ENABLE_POST_CAPTURE_KV_SIZING"] == "True"
    assert any(h.target.endswith("ModelRunner.load_model") and h.kind == "around" for h in hooks)
    with pytest.raises(RuntimeError, match="not applied"):
        plugin.install(Registry(drop="sglang.srt.managers.scheduler.Scheduler.get_init_info"), environ={})
