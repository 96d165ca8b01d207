"""Every architecture's FFN tier (and, where the oracle has the attention side, the whole model) against the
transformers implementation, through a checkpoint the library itself wrote."""

import pytest

from crosspool_b200.devtools import hf_parity
from crosspool_b200.devtools.qualification import TINY_CONFIGS

ARCHS = [a for a in sorted(TINY_CONFIGS) if "+" not in a] + sorted(hf_parity.VARIANTS)


@pytest.mark.parametrize("arch", ARCHS)
def test_loaded_ffn_and_oracle_equal_the_library_model(arch):
    if not hf_parity.available(arch):
        pytest.skip(f"the installed transformers has no {arch}")
    rep = hf_parity.parity(arch)
    failed = [(c.name, c.detail) for c in rep.checks if not c.ok]
    assert not failed, failed
    assert any(c.name.startswith("whole model: logits") for c in rep.checks)
    assert any(c.name.startswith("whole model: prefill + token-by-token") for c in rep.checks)


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


@pytest.mark.parametrize("name,ranks,moe_parallel", [
    ("OPTForCausalLM", 2, "tp"), ("GptOssForCausalLM/window-yarn", 2, "ep"), ("DeepseekV2ForCausalLM/plain-q-yarn", 2, "ep"),
    ("Glm4MoeLiteForCausalLM/small-latent-yarn", 2, "tp"), ("Qwen3MoeForCausalLM", 2, "ep"), ("LlamaForCausalLM", 2, "tp")])
def test_disaggregated_processes_serve_a_library_checkpoint_with_the_librarys_logits(tmp_path, name, ranks, moe_parallel):
    """A checkpoint the library wrote, served by one attention process and two FFN processes (each loading only its
    shard through the production loader): greedy tokens and logits equal the library model's own."""
    import torch

    from crosspool_b200.engine import cpu_plumbing

    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    model = hf_parity.build_tiny_model(name)
    model.save_pretrained(tmp_path, safe_serialization=True)
    prompt_len, new_tokens = 12, 5
    got = cpu_plumbing.run_topology(str(tmp_path), ffn_ranks=ranks, moe_parallel=moe_parallel, requests=2, prompt_len=prompt_len,
                                    new_tokens=new_tokens)
    gen = torch.Generator().manual_seed(12345)          # the prompts run_topology drew (seed 0)
    for tokens, logits in zip(got.tokens, got.logits):
        prompt = torch.randint(0, model.config.vocab_size, (prompt_len,), generator=gen)
        ids = torch.cat([prompt, torch.tensor(tokens[:-1], dtype=torch.long)])
        with torch.no_grad():
            want = model(ids[None]).logits[0, prompt_len - 1:]
        assert want.argmax(-1).tolist() == tokens
        torch.testing.assert_close(logits, want, rtol=2e-4, atol=2e-4)
    assert got.invocations == 2 * (1 + new_tokens - 1) * model.config.num_hidden_layers


def test_mxfp4_expert_tensors_decode_to_what_the_librarys_dequantiser_gives(tmp_path):
    """The MXFP4 form of GPT-OSS experts (16-byte blocks of 32 four-bit values, one power-of-two scale per block)
    through the production loader, against the library's own dequantisation of the same bytes."""
    import torch

    from crosspool_b200.devtools import qualification as q
    from crosspool_b200.engine import checkpoint as ck
    from crosspool_b200.engine import loader
    from crosspool_b200.models import adapters

    try:
        from transformers.integrations.mxfp4 import convert_moe_packed_tensors
    except ImportError:
        pytest.skip("the installed transformers has no MXFP4 helpers")
    hf = q.tiny_config("GptOssForCausalLM+mxfp4")
    spec = adapters.compile_ffn_spec("mx", hf)
    tensors = q.synthesize_ffn_tensors(spec, seed=3)
    q.write_ffn_checkpoint(tmp_path, hf, tensors)
    view = ck.read_checkpoint_key_view(tmp_path)
    spec = adapters.compile_ffn_spec("mx", hf, view.keys())
    l = spec.layers[0]
    w = loader.materialize_layer_weights(spec, view, 0)
    stem = "model.layers.0.mlp.experts."
    gu = convert_moe_packed_tensors(tensors[stem + "gate_up_proj_blocks"], tensors[stem + "gate_up_proj_scales"])   # [E, in, out]
    dn = convert_moe_packed_tensors(tensors[stem + "down_proj_blocks"], tensors[stem + "down_proj_scales"])
    inter = l.moe_intermediate_size
    assert gu.shape == (l.num_experts, l.hidden_size, 2 * inter) and dn.shape == (l.num_experts, inter, l.hidden_size)
    rows = gu.transpose(1, 2)                                        # [E, 2I, H], gate and up rows interleaved
    assert torch.equal(w.gate_up[:, :inter].float(), rows[:, 0::2].float())
    assert torch.equal(w.gate_up[:, inter:].float(), rows[:, 1::2].float())
    assert torch.equal(w.down.float(), dn.transpose(1, 2).float())
    assert float(w.gate_up.float().abs().max()) > 0
