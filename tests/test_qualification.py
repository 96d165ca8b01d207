"""Model qualification battery on CPU: every FFN architecture adapter against an evaluation made directly from
the raw checkpoint tensors, with TP and EP shard sums; and proof that the battery notices a wrong mapping."""
import dataclasses

import pytest
import torch

from crosspool_b200.devtools import qualification as Q
from crosspool_b200.ffn import GateUpOrder, MoeFfnSpec


@pytest.mark.parametrize("arch", sorted(Q.TINY_CONFIGS))
def test_every_architecture_qualifies(arch, tmp_path):
    rep = Q.qualify(Q.tiny_config(arch), tmp_path, rows=(5,))
    failed = [(c.name, c.detail) for c in rep.checks if not c.ok]
    assert rep.ok and not failed, failed
    names = " | ".join(c.name for c in rep.checks)
    assert "coverage" in names and "direct evaluation" in names and "TP2" in names
    if "moe" in rep.layers:
        assert "EP2" in names and "routing decisions" in names


def test_the_battery_notices_a_wrong_gate_up_order_and_a_wrong_scaling(tmp_path):
    from crosspool_b200.engine import checkpoint as ck
    from crosspool_b200.engine import loader
    from crosspool_b200.models import adapters, reference
    from crosspool_b200.models import config as mc

    cfg = Q.tiny_config("GptOssForCausalLM")
    spec = adapters.compile_ffn_spec("q", cfg)
    tensors = Q.synthesize_ffn_tensors(spec, 3)
    Q.write_ffn_checkpoint(tmp_path, cfg, tensors)
    view = ck.read_checkpoint_key_view(tmp_path)
    l = spec.layers[0]
    assert isinstance(l, MoeFfnSpec) and l.source_order == GateUpOrder.INTERLEAVED
    x = (torch.randn(9, l.hidden_size, generator=torch.Generator().manual_seed(1)) * 0.5).bfloat16()
    mcfg = mc.from_hf_config({"num_attention_heads": 4, "vocab_size": 256, **cfg}, "q")
    got = reference.ffn_forward(x, loader.materialize_layer_weights(spec, view, 0), mcfg).float()
    ok, _ = Q._close(got, Q.direct_ffn(l, tensors, x))
    assert ok
    wrong_order = dataclasses.replace(l, source_order=GateUpOrder.CONCATENATED)
    ok, d = Q._close(got, Q.direct_ffn(wrong_order, tensors, x))
    assert not ok and d["nrmse"] > 0.1
    wrong_scale = dataclasses.replace(l, routed_scaling_factor=1.25)
    ok, _ = Q._close(got, Q.direct_ffn(wrong_scale, tensors, x))
    assert not ok


def test_shrink_keeps_the_family_and_its_switches():
    real = {"architectures": ["Glm4MoeLiteForCausalLM"], "hidden_size": 4096, "n_routed_experts": 160, "scoring_func": "sigmoid",
            "routed_scaling_factor": 1.8, "norm_topk_prob": True}
    small = Q.shrink(real)
    assert small["architectures"] == ["Glm4MoeLiteForCausalLM"] and small["hidden_size"] == 64
    assert small["routed_scaling_factor"] == 1.8 and small["scoring_func"] == "sigmoid"
    with pytest.raises(KeyError):
        Q.tiny_config("MambaForCausalLM")


def test_cli_reports_pass_and_exit_code(capsys):
    assert Q.main(["--arch", "OPTForCausalLM"]) == 0
    assert "OPTForCausalLM: PASS" in capsys.readouterr().out
