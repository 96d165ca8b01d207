"""What is supported for which architecture, derived from the code that implements it: the FFN adapters
(``models/adapters.py``), the attention forms of the GPU engine (``ModelConfig.gpu_attention_supported``) and of the
PyTorch oracle / CPU deployment, and the serving-engine shim adapters. ``xpool config models`` prints the table; the
user documentation embeds it and a test keeps the two equal. Reference: docs/supported-models.md."""

from __future__ import annotations

from dataclasses import dataclass

from . import adapters
from . import config as mc

# the smallest config.json of each family that the parsers accept (sizes are irrelevant here)
_PROBE = {"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
          "intermediate_size": 128, "moe_intermediate_size": 64, "num_experts": 4, "num_local_experts": 4, "n_routed_experts": 4,
          "num_experts_per_tok": 2, "ffn_dim": 128, "kv_lora_rank": 32, "qk_nope_head_dim": 16, "qk_rope_head_dim": 8,
          "v_head_dim": 16, "sliding_window": 128, "first_k_dense_replace": 1, "n_shared_experts": 1}
_LATENT = ("DeepseekV2ForCausalLM", "Glm4MoeLiteForCausalLM")


@dataclass(frozen=True)
class ArchitectureSupport:
    architecture: str
    ffn_kinds: tuple[str, ...]         # layer kinds of the family: dense, moe
    ffn_features: str
    attention_form: str
    gpu_attention: bool                # the repository's own GPU attention engine runs it
    engine_adapter: bool               # a serving-engine shim adapter exists (attention in the external engine)
    quantization: tuple[str, ...]


def _probe(arch: str) -> dict:
    cfg = {k: v for k, v in _PROBE.items() if arch in _LATENT or not k.startswith(("kv_lora", "qk_", "v_head"))}
    if not arch.startswith("GptOss"):
        cfg.pop("sliding_window")
    if arch.startswith("OPT"):
        cfg["activation_function"] = "relu"
    return {**cfg, "architectures": [arch]}


def _attention_form(c: mc.ModelConfig) -> str:
    if c.mla is not None:
        return "latent attention (MLA), interleaved rotary pairs, YaRN"
    parts = ["grouped-query" if c.num_kv_heads != c.num_q_heads else "multi-head"]
    parts.append("learned positions, LayerNorm" if c.positions == "learned" else "rotary")
    if c.qk_norm:
        parts.append("q/k RMSNorm")
    if c.attention_bias:
        parts.append("biases")
    if c.sliding_window:
        parts.append("alternating sliding window")
    if c.attention_sinks:
        parts.append("sinks, YaRN")
    return ", ".join(parts)


def _ffn_features(spec) -> str:
    from ..ffn import DenseFfnSpec, GateUpOrder, MoeFfnSpec, RouterAlgorithm, RouterProjectionPrecision

    out: list[str] = []
    for l in spec.layers:
        if isinstance(l, DenseFfnSpec):
            out.append("gated" if l.i_proj.gated else "ungated")
            out.append(l.activation.value)
            if l.o_proj.bias_key:
                out.append("biases")
        elif isinstance(l, MoeFfnSpec):
            out.append(f"top-k {'sigmoid' if l.router_algorithm == RouterAlgorithm.SIGMOID else 'softmax'} router")
            if l.router_precision != RouterProjectionPrecision.PAYLOAD:
                out.append(f"{l.router_precision.value} router projection")
            if l.correction_bias_key:
                out.append("selection bias")
            if l.num_shared_experts:
                out.append("shared experts")
            if l.routed_scaling_factor != 1.0 or "Deepseek" in spec.architecture or "Glm4" in spec.architecture:
                out.append("routed scaling")
            if l.experts.gate_bias_key:
                out.append("expert biases")
            if l.gate_transform.limit > 0:
                out.append("clamped activation")
            if l.source_order == GateUpOrder.INTERLEAVED:
                out.append("interleaved gate/up")
    seen: list[str] = []
    for o in out:
        if o not in seen:
            seen.append(o)
    return ", ".join(seen)


def supported_architectures() -> list[ArchitectureSupport]:
    from ..integrations.sglang import adapter as engine_adapters

    with_adapter = {a for ad in engine_adapters.ADAPTERS for a in ad.architectures}
    rows = []
    for arch in sorted(adapters.ADAPTERS):
        hf = _probe(arch)
        spec = adapters.compile_ffn_spec(arch, hf)
        c = mc.from_hf_config(hf, arch)
        kinds = tuple(dict.fromkeys(l.kind.value for l in spec.layers))
        # checkpoints in bf16 / fp16 / fp32 are all computed in bf16 (the payload and kernel dtype of this build)
        quant = ("bf16",) + (("mxfp4 (expanded to bf16 at load)",) if arch.startswith("GptOss") else ()) + \
            (("block fp8 checkpoints (expanded to bf16 for the Lanes; stored codes feed the decode-size fp8 GEMM)",)
             if kinds == ("dense",) and c.hidden_act == "silu" else ())
        rows.append(ArchitectureSupport(arch, kinds, _ffn_features(spec), _attention_form(c), c.gpu_attention_supported,
                                        arch in with_adapter, quant))
    return rows


def support_markdown() -> str:
    lines = ["| architecture | FFN tier | FFN features | attention form | GPU attention engine | engine shim adapter | "
             "library-attention engine process | CPU deployment and oracle | weight formats |",
             "| --- | --- | --- | --- | --- | --- | --- | --- | --- |"]
    for r in supported_architectures():
        lines.append(f"| `{r.architecture}` | {' + '.join(r.ffn_kinds)} | {r.ffn_features} | {r.attention_form} | "
                     f"{'yes' if r.gpu_attention else 'no'} | {'yes' if r.engine_adapter else 'no'} | yes | yes | {', '.join(r.quantization)} |")
    return "\n".join(lines) + "\n"
