"""Acceptance tolerances shared by the test-suite and by users validating a deployment.

The limits are the reference's (src/xpool-dev/xtest/harness/support/ffn.py:20-28,
docs/designs/qualification.md:86-89): FFN outputs within atol 0.02 / rtol 0.02 element-wise, normalised
RMSE <= 0.01 and max scaled error <= 0.10; routing weights atol 1e-4 / rtol 1e-3; logits against a stock
forward KL <= 0.05 nats for prefill and <= 0.001 nats for decode steps.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FFN_ATOL, FFN_RTOL, FFN_NRMSE, FFN_MAX_SCALED = 0.02, 0.02, 0.01, 0.10
ROUTING_ATOL, ROUTING_RTOL = 1e-4, 1e-3
KL_PREFILL, KL_DECODE = 0.05, 0.001


@dataclass
class FfnError:
    nrmse: float
    max_scaled: float
    frac_outside_elementwise: float

    @property
    def ok(self) -> bool:
        return self.nrmse <= FFN_NRMSE and self.max_scaled <= FFN_MAX_SCALED


def ffn_error(out: torch.Tensor, ref: torch.Tensor) -> FfnError:
    o, r = out.float(), ref.float()
    err = (o - r).abs()
    scale = r.abs().max().clamp_min(1e-12)
    nrmse = (err.pow(2).mean().sqrt() / r.pow(2).mean().sqrt().clamp_min(1e-12)).item()
    outside = (err > FFN_ATOL + FFN_RTOL * r.abs()).float().mean().item()
    return FfnError(nrmse, (err.max() / scale).item(), outside)


def assert_ffn_close(out: torch.Tensor, ref: torch.Tensor, what: str = "ffn output") -> FfnError:
    e = ffn_error(out, ref)
    if not e.ok:
        raise AssertionError(f"{what}: nrmse {e.nrmse:.4f} (limit {FFN_NRMSE}), max scaled error {e.max_scaled:.4f} (limit {FFN_MAX_SCALED})")
    return e


def kl_nats(p_logits: torch.Tensor, q_logits: torch.Tensor) -> torch.Tensor:
    """KL(p || q) per row, in nats."""
    p, q = p_logits.float().log_softmax(-1), q_logits.float().log_softmax(-1)
    return (p.exp() * (p - q)).sum(-1)


def assert_logits_close(ref_logits: torch.Tensor, got_logits: torch.Tensor, prefill_rows: int = 1) -> None:
    kl = kl_nats(ref_logits, got_logits)
    if kl[:prefill_rows].max().item() > KL_PREFILL:
        raise AssertionError(f"prefill KL {kl[:prefill_rows].max().item():.4f} nats exceeds {KL_PREFILL}")
    if kl.shape[0] > prefill_rows and kl[prefill_rows:].max().item() > KL_DECODE:
        raise AssertionError(f"decode KL {kl[prefill_rows:].max().item():.5f} nats exceeds {KL_DECODE}")


def write_synthetic_checkpoint(model_dir, hf_config: dict, seed: int = 0, shards: int = 2, scale: float = 0.02) -> dict:
    """Writes a random Hugging Face style checkpoint (``config.json``, sharded safetensors and their index) for a
    Qwen3 / Qwen3-MoE shaped ``hf_config`` and returns the tensors by key. Lets loading paths run against files
    of the real layout without model downloads."""
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    h, heads = int(hf_config["hidden_size"]), int(hf_config["num_attention_heads"])
    kvh = int(hf_config.get("num_key_value_heads") or heads)
    hd = int(hf_config.get("head_dim") or h // heads)
    n_exp = int(hf_config.get("num_experts") or 0)

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)

    def norm(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)

    t = {"model.embed_tokens.weight": rnd(int(hf_config["vocab_size"]), h), "model.norm.weight": norm(h)}
    if not hf_config.get("tie_word_embeddings", False):
        t["lm_head.weight"] = rnd(int(hf_config["vocab_size"]), h)
    for i in range(int(hf_config["num_hidden_layers"])):
        p = f"model.layers.{i}."
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = norm(h), norm(h)
        t[p + "self_attn.q_proj.weight"] = rnd(heads * hd, h)
        t[p + "self_attn.k_proj.weight"], t[p + "self_attn.v_proj.weight"] = rnd(kvh * hd, h), rnd(kvh * hd, h)
        t[p + "self_attn.o_proj.weight"] = rnd(h, heads * hd)
        if str(hf_config["architectures"][0]).startswith("Qwen3"):
            t[p + "self_attn.q_norm.weight"], t[p + "self_attn.k_norm.weight"] = norm(hd), norm(hd)
        if n_exp:
            inter = int(hf_config["moe_intermediate_size"])
            t[p + "mlp.gate.weight"] = rnd(n_exp, h)
            for e in range(n_exp):
                q = p + f"mlp.experts.{e}."
                t[q + "gate_proj.weight"], t[q + "up_proj.weight"] = rnd(inter, h), rnd(inter, h)
                t[q + "down_proj.weight"] = rnd(h, inter)
        else:
            inter = int(hf_config["intermediate_size"])
            t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"] = rnd(inter, h), rnd(inter, h)
            t[p + "mlp.down_proj.weight"] = rnd(h, inter)
    keys, wm = sorted(t), {}
    for s in range(shards):
        part = {k: t[k].contiguous() for k in keys[s::shards]}
        name = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, str(d / name))
        wm.update({k: name for k in part})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    (d / "config.json").write_text(json.dumps(hf_config))
    return t


def compare_generations(tokens, ref_tokens, logits, ref_logits, kl_limit: float = 0.005, tie_margin: float = 0.06):
    """Compares one greedy generation with an oracle run of the same prompt.

    Every step up to and including the first step whose token differs saw identical inputs, so on those
    steps the logit distributions must agree within ``kl_limit`` nats (the reference's decode bound is 0.001
    against its stock engine on trained weights, docs/designs/qualification.md:86-89; random-init logits are
    nearly flat, which makes bf16 argmax ties common and the KL bound the meaningful check). A differing
    token is accepted only as such a tie: the oracle's logits of the two candidates lie within
    ``tie_margin``. Returns ``(ok, agreeing_tokens, max_kl)``."""
    import torch

    n = 0
    while n < len(tokens) and n < len(ref_tokens) and tokens[n] == ref_tokens[n]:
        n += 1
    upto = min(n + 1, len(tokens), len(ref_tokens))
    a, b = torch.stack(list(logits[:upto])).float(), torch.stack(list(ref_logits[:upto])).float()
    p, q = a.log_softmax(-1), b.log_softmax(-1)
    kl = (p.exp() * (p - q)).sum(-1).max().item()
    ok = kl <= kl_limit and len(tokens) == len(ref_tokens)
    if n < len(tokens) and n < upto:
        gap = (b[n, ref_tokens[n]] - b[n, tokens[n]]).abs().item()
        ok = ok and gap <= tie_margin
    return ok, n, kl
