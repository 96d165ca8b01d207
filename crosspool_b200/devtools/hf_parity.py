"""Parity with the Hugging Face implementation of every supported architecture.

``qualification.py`` checks the FFN tier against a restatement written in this repository; this module checks it
against the model code that defines the checkpoints. For one architecture it

1. instantiates the ``transformers`` model class from the family's tiny configuration with random fp32 weights and
   writes it with ``save_pretrained`` (so tensor names, stacked / per-expert / input-major expert layouts and the
   ``config.json`` keys are whatever the library really produces);
2. reads that directory the way a deployment does: ``config.json`` -> FFN description (``models/adapters.py``), key
   view and coverage (``engine/checkpoint.py``), tensors through the production loader (``engine/loader.py``);
3. runs the library model on random token ids with forward hooks on every decoder layer's MLP, and evaluates the
   loaded layer on the captured input: outputs must agree to fp32 rounding;
4. for architectures whose attention side the oracle implements (``models/reference.py``), loads the attention
   tensors as well and compares the logits of the whole disaggregated model with the library's.

The reference keeps one qualification suite per model family (tests/suites/models/) that compares served output
with the serving engine's own; with no serving engine on this image the library model is the independent side.

    python -m crosspool_b200.devtools.hf_parity --arch all
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile

import torch

from .qualification import TINY_CONFIGS, Check, Report

FFN_ATOL = 2e-5        # fp32 on both sides: only summation order differs
LOGITS_ATOL = 2e-4

# architectures whose attention the oracle implements: the whole model is compared, not only its FFN layers
FULL_MODEL = ("Qwen2ForCausalLM", "Qwen3ForCausalLM", "LlamaForCausalLM", "Qwen3MoeForCausalLM", "OPTForCausalLM",
              "GptOssForCausalLM", "DeepseekV2ForCausalLM", "Glm4MoeLiteForCausalLM")


# harder settings of the same families: a window shorter than the sequence with YaRN-scaled rotary embeddings, latent
# attention with a plain query projection and YaRN magnitude correction, small latent ranks with a query bottleneck
_YARN = {"rope_type": "yarn", "factor": 32.0, "beta_fast": 32.0, "beta_slow": 1.0, "original_max_position_embeddings": 4096}
VARIANTS: dict[str, tuple[str, dict]] = {
    "GptOssForCausalLM/window-yarn": ("GptOssForCausalLM", {
        "sliding_window": 8, "max_position_embeddings": 131072,
        "rope_parameters": {**_YARN, "truncate": False, "rope_theta": 150000.0}}),
    "DeepseekV2ForCausalLM/plain-q-yarn": ("DeepseekV2ForCausalLM", {
        "q_lora_rank": None, "kv_lora_rank": 32, "qk_nope_head_dim": 16, "qk_rope_head_dim": 8, "v_head_dim": 16,
        "max_position_embeddings": 163840,
        # no mscale_all_dim: the library's port of this family omits the softmax-scale correction that comes with it
        "rope_parameters": {**_YARN, "factor": 40.0, "rope_theta": 10000.0}}),
    "Glm4MoeLiteForCausalLM/small-latent-yarn": ("Glm4MoeLiteForCausalLM", {
        "q_lora_rank": 24, "kv_lora_rank": 32, "qk_nope_head_dim": 16, "qk_rope_head_dim": 8, "v_head_dim": 24,
        "max_position_embeddings": 163840,
        "rope_parameters": {**_YARN, "factor": 40.0, "mscale": 1.0, "mscale_all_dim": 1.0, "rope_theta": 10000.0}}),
}


def resolve(name: str) -> tuple[str, dict]:
    """(architecture, tiny configuration fields) of an architecture name or one of :data:`VARIANTS`."""
    arch, extra = VARIANTS.get(name, (name, {}))
    return arch, {**{k: v for k, v in TINY_CONFIGS[arch].items() if k != "torch_dtype"}, **extra}


def available(arch: str) -> bool:
    arch = resolve(arch)[0] if arch in VARIANTS else arch
    try:
        import transformers
    except ImportError:
        return False
    return hasattr(transformers, arch)


def build_tiny_model(arch: str, seed: int = 0):
    """The library's model class for ``arch`` on the tiny configuration, fp32, with weights drawn wide enough that
    routing, clamping and biases all matter (norm weights around one, everything else N(0, 0.08))."""
    import transformers

    arch, fields = resolve(arch)
    cls = getattr(transformers, arch)
    torch.manual_seed(seed)
    model = cls(cls.config_class(**fields)).float().eval()
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for name, p in model.named_parameters():
            noise = torch.randn(p.shape, generator=g)
            p.copy_(1 + 0.1 * noise if "norm" in name and name.endswith("weight") else 0.08 * noise)
    return model


def decoder_layers(model):
    inner = model.model
    return inner.decoder.layers if hasattr(inner, "decoder") else inner.layers


def capture_ffn_io(model, ids: torch.Tensor) -> tuple[list[tuple[torch.Tensor, torch.Tensor]], torch.Tensor]:
    """Runs the library model once; returns (input, output) of every layer's FFN as 2-D tensors, and the logits."""
    got: dict[tuple[str, int], torch.Tensor] = {}
    handles = []
    for i, layer in enumerate(decoder_layers(model)):
        if hasattr(layer, "mlp"):
            def both(_m, args, out, i=i):
                got["x", i] = args[0].detach()
                got["y", i] = (out[0] if isinstance(out, tuple) else out).detach()
            handles.append(layer.mlp.register_forward_hook(both))
        else:   # OPT: two bare linear layers around the activation
            def first(_m, args, _out, i=i):
                got["x", i] = args[0].detach()

            def second(_m, _args, out, i=i):
                got["y", i] = out.detach()
            handles.append(layer.fc1.register_forward_hook(first))
            handles.append(layer.fc2.register_forward_hook(second))
    try:
        with torch.no_grad():
            logits = model(ids[None]).logits[0]
    finally:
        for h in handles:
            h.remove()
    n = len(decoder_layers(model))
    hidden = got["x", 0].shape[-1]
    return [(got["x", i].reshape(-1, hidden), got["y", i].reshape(-1, hidden)) for i in range(n)], logits


def parity(arch: str, *, tokens: int = 19, seed: int = 0, workdir: str | None = None) -> Report:
    from ..engine import checkpoint as ck
    from ..engine import loader
    from ..models import adapters, reference
    from ..models import config as mc
    from ..models import weights as mw

    model = build_tiny_model(arch, seed)
    arch = resolve(arch)[0]
    tmp = None
    if workdir is None:
        tmp = tempfile.TemporaryDirectory(prefix="xp-hf-parity-")
        workdir = tmp.name
    try:
        model.save_pretrained(workdir, safe_serialization=True)
        with open(f"{workdir}/config.json") as f:
            hf = json.load(f)
        view = ck.read_checkpoint_key_view(workdir)
        spec = adapters.compile_ffn_spec(arch, hf, view.keys())
        rep = Report(arch, spec.quantization, [l.kind.value for l in spec.layers])
        try:
            ck.validate_ffn_coverage(spec, view)
            rep.checks.append(Check("coverage: the description names exactly the FFN tensors the library wrote", True))
        except Exception as e:
            rep.checks.append(Check("coverage", False, {"error": repr(e)}))
            return rep
        cfg = mc.from_hf_config(hf, arch)
        ids = torch.randint(0, cfg.vocab_size, (tokens,), generator=torch.Generator().manual_seed(seed + 2))
        io, logits = capture_ffn_io(model, ids)
        layers = [loader.materialize_layer_weights(spec, view, i, dtype=torch.float32) for i in range(spec.num_layers)]
        for i, (x, y) in enumerate(io):
            out = reference.ffn_forward(x, layers[i], cfg)
            err = float((out - y).abs().max())
            rep.checks.append(Check(f"layer {i} ({spec.layers[i].kind.value}): loaded FFN equals the library's MLP on its own input",
                                    err <= FFN_ATOL * max(1.0, float(y.abs().max())), {"max_abs_err": err, "ref_max": float(y.abs().max())}))
            for tp in (2,):
                parts = [reference.ffn_forward(x, loader.materialize_layer_weights(spec, view, i, tp_rank=r, tp_size=tp,
                                                                                   dtype=torch.float32), cfg) for r in range(tp)]
                err = float((sum(parts) - y).abs().max())
                rep.checks.append(Check(f"layer {i}: TP{tp} shards sum to the library's output",
                                        err <= 4 * FFN_ATOL * max(1.0, float(y.abs().max())), {"max_abs_err": err}))
        if arch in FULL_MODEL:
            attn = mw.load_attention_from_safetensors(cfg, workdir, dtype=torch.float32)
            oracle = reference.ReferenceModel(cfg, attn, layers)
            with torch.no_grad():
                mine = oracle.forward(ids, torch.arange(tokens), oracle.new_cache())
            err = float((mine - logits).abs().max())
            rep.checks.append(Check("whole model: logits equal the library's", err <= LOGITS_ATOL * max(1.0, float(logits.abs().max())),
                                    {"max_abs_err": err, "ref_max": float(logits.abs().max())}))
            same = bool((mine.argmax(-1) == logits.argmax(-1)).all())
            rep.checks.append(Check("whole model: greedy tokens equal the library's", same))
            # the serving shape of the same computation: a prefill chunk, then one token at a time against the cache
            cache, cut = oracle.new_cache(), max(1, tokens * 2 // 3)
            with torch.no_grad():
                steps = [oracle.forward(ids[:cut], torch.arange(cut), cache)]
                steps += [oracle.forward(ids[t:t + 1], torch.tensor([t]), cache) for t in range(cut, tokens)]
            err = float((torch.cat(steps) - logits).abs().max())
            rep.checks.append(Check("whole model: prefill + token-by-token decode equals the library's full pass",
                                    err <= LOGITS_ATOL * max(1.0, float(logits.abs().max())), {"max_abs_err": err}))
        return rep
    finally:
        if tmp is not None:
            tmp.cleanup()


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.devtools.hf_parity")
    ap.add_argument("--arch", default="all")
    ap.add_argument("--json", action="store_true")
    ns = ap.parse_args(argv)
    archs = [a for a in sorted(TINY_CONFIGS) if "+" not in a] + sorted(VARIANTS) if ns.arch == "all" else [ns.arch]
    bad = 0
    for a in archs:
        if not available(a):
            print(f"{a}: SKIPPED (the installed transformers has no such class)")
            continue
        rep = parity(a)
        bad += 0 if rep.ok else 1
        if ns.json:
            print(json.dumps(rep.to_json()))
        else:
            print(f"{a}: {'PASS' if rep.ok else 'FAIL'} ({len(rep.checks)} checks{', whole model' if resolve(a)[0] in FULL_MODEL else ''})")
            for c in rep.checks:
                if not c.ok:
                    print(f"   FAILED {c.name}: {c.detail}")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
