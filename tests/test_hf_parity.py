"""Every architecture's FFN tier (and, where the oracle has the attention side, the whole model) against the
transformers implementation, through a checkpoint the library itself wrote."""

import pytest

from crosspool_b200.devtools import hf_parity
from crosspool_b200.devtools.qualification import TINY_CONFIGS

ARCHS = [a for a in sorted(TINY_CONFIGS) if "+" not in a]


@pytest.mark.parametrize("arch", ARCHS)
def test_loaded_ffn_and_oracle_equal_the_library_model(arch):
    if not hf_parity.available(arch):
        pytest.skip(f"the installed transformers has no {arch}")
    rep = hf_parity.parity(arch)
    failed = [(c.name, c.detail) for c in rep.checks if not c.ok]
    assert not failed, failed
    assert len(rep.checks) >= 5
    if arch in hf_parity.FULL_MODEL:
        assert any(c.name.startswith("whole model: logits") for c in rep.checks)


def test_unquantised_gpt_oss_experts_are_read_input_major(tmp_path):
    """The library stores unquantised GPT-OSS experts as [experts, in, out]; the loader returns [out, in] shards."""
    import json

    import torch

    from crosspool_b200.engine import checkpoint as ck
    from crosspool_b200.engine import loader
    from crosspool_b200.models import adapters

    arch = "GptOssForCausalLM"
    if not hf_parity.available(arch):
        pytest.skip("no GptOss in the installed transformers")
    model = hf_parity.build_tiny_model(arch)
    model.save_pretrained(tmp_path, safe_serialization=True)
    hf = json.loads((tmp_path / "config.json").read_text())
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec(arch, hf, view.keys())
    assert spec.layers[0].experts.input_major
    experts = hf_parity.decoder_layers(model)[0].mlp.experts
    e, h, i2 = experts.gate_up_proj.shape
    w = loader.materialize_layer_weights(spec, view, 0, dtype=torch.float32)
    assert w.gate_up.shape == (e, i2, h) and w.down.shape == (e, h, i2 // 2)
    torch.testing.assert_close(w.gate_up[1, : i2 // 2], experts.gate_up_proj[1, :, 0::2].t())      # gate rows
    torch.testing.assert_close(w.gate_up[1, i2 // 2:], experts.gate_up_proj[1, :, 1::2].t())       # up rows
    torch.testing.assert_close(w.down[2], experts.down_proj[2].t())
    half = loader.materialize_layer_weights(spec, view, 0, tp_rank=1, tp_size=2, dtype=torch.float32)
    q = i2 // 4
    torch.testing.assert_close(half.gate_up[0, :q], experts.gate_up_proj[0, :, 0::2].t()[q:])
    torch.testing.assert_close(half.down[0], experts.down_proj[0].t()[:, q:])
