"""A transformers model as the attention side: its own forward / generate, FFNs served by the disaggregated tier."""

import pytest
import torch

from crosspool_b200.devtools import hf_parity


@pytest.mark.parametrize("name,ranks,moe_parallel", [
    ("Qwen3ForCausalLM", 2, "tp"), ("OPTForCausalLM", 2, "tp"), ("GptOssForCausalLM", 2, "ep"),
    ("DeepseekV2ForCausalLM/plain-q-yarn", 2, "tp"), ("Qwen3MoeForCausalLM", 2, "ep")])
def test_library_model_with_detached_ffns_generates_what_the_whole_model_generates(tmp_path, name, ranks, moe_parallel):
    from crosspool_b200.engine.cpu_plumbing import FfnTierProcesses
    from crosspool_b200.integrations import transformers as xhf

    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    model = hf_parity.build_tiny_model(name)
    model.save_pretrained(tmp_path, safe_serialization=True)
    ids = torch.randint(0, model.config.vocab_size, (2, 11), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want_logits = model(ids).logits
        want_tokens = model.generate(ids, max_new_tokens=6, do_sample=False)
    before = sum(p.numel() for p in model.parameters())
    rep = xhf.detach_ffn(model)
    assert len(rep.shims) == model.config.num_hidden_layers
    assert rep.freed_parameters > 0 and rep.kept_parameters == before - rep.freed_parameters
    assert not [n for n, _ in model.named_parameters() if ".mlp." in n or ".fc1." in n or ".fc2." in n]
    with pytest.raises(RuntimeError, match="before an Instance runtime was bound"):
        model(ids)                                    # nothing serves the FFNs yet
    with FfnTierProcesses(str(tmp_path), ranks, moe_parallel, max_rows=64, tag="hf") as tier:
        xhf.bind_cpu_tier(tier.shim)
        try:
            with torch.no_grad():
                got_logits = model(ids).logits
                got_tokens = model.generate(ids, max_new_tokens=6, do_sample=False)
        finally:
            xhf.unbind()
        # one prefill pass + (1 prefill + 5 decode) passes of generate, every layer each
        assert tier.shim.calls == 7 * model.config.num_hidden_layers
    torch.testing.assert_close(got_logits, want_logits, rtol=2e-4, atol=2e-4)
    assert got_tokens.tolist() == want_tokens.tolist()


def test_command_line_demo_generates_from_a_local_checkpoint_and_verifies_against_the_whole_model(tmp_path, capsys):
    from crosspool_b200.integrations.transformers import __main__ as demo

    name = "Qwen3MoeForCausalLM"
    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    hf_parity.build_tiny_model(name).save_pretrained(tmp_path, safe_serialization=True)
    rc = demo.main(["--checkpoint", str(tmp_path), "--ffn-ranks", "2", "--moe-parallel", "ep", "--ids", "5", "9", "11", "3",
                    "--max-new-tokens", "5", "--verify"])
    out = capsys.readouterr()
    assert rc == 0 and "same tokens as the whole model" in out.err
    assert len(out.out.split()) == 5 and "detached 2 FFN layers" in out.err


def test_served_qualification_brings_up_a_deployment_and_compares_its_answers_with_the_librarys(capsys):
    from crosspool_b200.devtools import served_qualification as sq

    name = "Glm4MoeLiteForCausalLM/small-latent-yarn"
    if not hf_parity.available(name):
        pytest.skip(f"the installed transformers has no {name}")
    assert sq.main(["--arch", name, "--prompts", "2", "--new-tokens", "4", "--json"]) == 0
    import json

    rep = json.loads([l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1])
    assert rep["ok"] and rep["architecture"] == "Glm4MoeLiteForCausalLM" and rep["ffn_ranks"] == 2
    assert [p["equal"] for p in rep["prompts"]] == [True, True] and all(len(p["served"]) == 4 for p in rep["prompts"])
