"""Decoder model shapes: typed view of a Hugging Face ``config.json`` plus named presets.

The attention side needs heads / KV heads / head_dim / RoPE / norms; the FFN side needs the MLP or
MoE description (that part is compiled into an :class:`crosspool_b200.ffn.FfnModelSpec` by the
architecture adapters). The reference reads the same fields through ``FfnSourceConfig``
(src/xpool/runtime/ffnagent/architecture.py:133-215) and ``SglangModelShape.load``
(src/xpool/integrations/sglang/topology.py).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field, replace
from pathlib import Path
from typing import Any


@dataclass(frozen=True)
class MlaShape:
    """Multi-head latent attention (DeepSeek-V2, GLM-4-MoE-Lite): queries optionally through a rank-``q_lora_rank``
    bottleneck; keys and values expanded per head from one ``kv_lora_rank`` latent plus a ``qk_rope_head_dim`` rotary
    key shared by all heads."""

    q_lora_rank: int            # 0: a plain query projection
    kv_lora_rank: int
    qk_nope_head_dim: int
    qk_rope_head_dim: int
    v_head_dim: int

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim


@dataclass(frozen=True)
class ModelConfig:
    name: str
    architecture: str  # HF ``architectures[0]``
    hidden_size: int
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    max_position_embeddings: int = 40960
    # MoE (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    num_shared_experts: int = 0
    first_k_dense: int = 0
    routed_scaling_factor: float = 1.0
    router_scoring: str = "softmax"  # or "sigmoid"
    router_precision: str = "payload"  # "fp32_logits" (payload weights, fp32 logits) or "fp32" (fp32 weights too)
    dtype: str = "bfloat16"
    # attention forms beyond rotary GQA with RMSNorm (the only one the GPU attention engine runs; the PyTorch oracle and the
    # CPU deployment run all of them)
    norm: str = "rmsnorm"            # or "layernorm" (weights and biases, mean-centred): OPT
    positions: str = "rope"          # or "learned" (a position table added to the embeddings): OPT
    sliding_window: int = 0          # > 0: layers named "sliding_attention" in extra["layer_types"] see this many keys
    attention_sinks: bool = False    # one learned logit per head joins every softmax and takes no value: GPT-OSS
    o_bias: bool = False
    mla: MlaShape | None = None
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @property
    def gpu_attention_supported(self) -> bool:
        return (self.norm == "rmsnorm" and self.positions == "rope" and self.mla is None and not self.attention_sinks
                and not self.sliding_window and not self.o_bias and not self.extra.get("rope_scaling"))

    def layer_window(self, layer: int) -> int:
        """Keys a query of ``layer`` may look back over (itself included); 0 = all of them."""
        kinds = self.extra.get("layer_types")
        if not self.sliding_window or (kinds and kinds[layer] != "sliding_attention"):
            return 0
        return self.sliding_window

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_size(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def layer_is_moe(self, layer: int) -> bool:
        return self.is_moe and layer >= self.first_k_dense

    def attention_param_bytes(self) -> int:
        per_layer = (self.q_size + 2 * self.kv_size) * self.hidden_size + self.hidden_size * self.q_size
        per_layer += 2 * self.hidden_size + 2 * self.head_dim
        emb = self.vocab_size * self.hidden_size * (1 if self.tie_word_embeddings else 2)
        return 2 * (per_layer * self.num_layers + emb + self.hidden_size)

    def ffn_param_bytes_per_layer(self, layer: int = 0) -> int:
        if self.layer_is_moe(layer):
            e = self.num_experts * 3 * self.hidden_size * self.moe_intermediate_size
            e += self.num_experts * self.hidden_size
            e += self.num_shared_experts * 3 * self.hidden_size * self.moe_intermediate_size
            return 2 * e
        return 2 * 3 * self.hidden_size * self.intermediate_size

    def kv_bytes_per_token(self) -> int:
        return 2 * self.num_layers * self.kv_size * 2

    def with_layers(self, n: int) -> "ModelConfig":
        return replace(self, num_layers=n)


def _qwen3(name, layers, hidden, q, kv, inter, **kw) -> ModelConfig:
    return ModelConfig(name=name, architecture="Qwen3ForCausalLM", hidden_size=hidden, num_layers=layers,
                       num_q_heads=q, num_kv_heads=kv, head_dim=128, intermediate_size=inter, vocab_size=151936,
                       **kw)


PRESETS: dict[str, ModelConfig] = {
    # CPU plumbing shape of the acceptance configuration
    "tiny-qwen3": ModelConfig(name="tiny-qwen3", architecture="Qwen3ForCausalLM", hidden_size=256, num_layers=2,
                              num_q_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768, vocab_size=4096,
                              dtype="float32"),
    # the partner of Qwen3-0.6B in the reference's small benchmark pair (benches/benches.toml): 14 query / 2 KV heads
    # of 64, q/k/v biases, no q/k norm, rope theta 1e6
    "Qwen/Qwen2.5-0.5B": ModelConfig(name="Qwen/Qwen2.5-0.5B", architecture="Qwen2ForCausalLM", hidden_size=896, num_layers=24,
                                     num_q_heads=14, num_kv_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                                     rope_theta=1e6, qk_norm=False, attention_bias=True, tie_word_embeddings=True),
    "Qwen/Qwen3-0.6B": _qwen3("Qwen/Qwen3-0.6B", 28, 1024, 16, 8, 3072, tie_word_embeddings=True),
    "Qwen/Qwen3-1.7B": _qwen3("Qwen/Qwen3-1.7B", 28, 2048, 16, 8, 6144, tie_word_embeddings=True),
    "Qwen/Qwen3-8B": _qwen3("Qwen/Qwen3-8B", 36, 4096, 32, 8, 12288),
    "Qwen/Qwen3-14B": _qwen3("Qwen/Qwen3-14B", 40, 5120, 40, 8, 17408),
    "Qwen/Qwen3-32B": _qwen3("Qwen/Qwen3-32B", 64, 5120, 64, 8, 25600),
    "Qwen/Qwen3-30B-A3B": ModelConfig(name="Qwen/Qwen3-30B-A3B", architecture="Qwen3MoeForCausalLM", hidden_size=2048,
                                      num_layers=48, num_q_heads=32, num_kv_heads=4, head_dim=128,
                                      intermediate_size=6144, vocab_size=151936, num_experts=128,
                                      num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True),
    "tiny-qwen3-moe": ModelConfig(name="tiny-qwen3-moe", architecture="Qwen3MoeForCausalLM", hidden_size=256,
                                  num_layers=2, num_q_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=768,
                                  vocab_size=4096, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128),
}


def preset(name: str) -> ModelConfig:
    try:
        return PRESETS[name]
    except KeyError:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}") from None


def from_hf_config(cfg: dict[str, Any], name: str = "") -> ModelConfig:
    """Builds a :class:`ModelConfig` from a parsed ``config.json``."""
    arch = (cfg.get("architectures") or ["Qwen3ForCausalLM"])[0]
    hidden = int(cfg["hidden_size"])
    heads = int(cfg["num_attention_heads"])
    kv = heads if arch.startswith("OPT") else int(cfg.get("num_key_value_heads") or heads)   # OPT has no grouped KV heads
    head_dim = int(cfg.get("head_dim") or hidden // heads)
    n_exp = int(cfg.get("num_experts") or cfg.get("n_routed_experts") or cfg.get("num_local_experts") or 0)
    rope = dict(cfg.get("rope_parameters") or cfg.get("rope_scaling") or {})
    rope_type = rope.get("rope_type", rope.get("type", "default"))
    mla = None
    if cfg.get("kv_lora_rank"):
        mla = MlaShape(int(cfg.get("q_lora_rank") or 0), int(cfg["kv_lora_rank"]), int(cfg["qk_nope_head_dim"]),
                       int(cfg["qk_rope_head_dim"]), int(cfg["v_head_dim"]))
    opt = arch.startswith("OPT")
    if opt and (not cfg.get("do_layer_norm_before", True) or int(cfg.get("word_embed_proj_dim", hidden)) != hidden):
        raise ValueError("OPT variants with post-layer norms or a projected embedding width are not supported")
    gpt_oss = arch.startswith("GptOss")
    extra = {k: v for k, v in cfg.items() if k in ("swiglu_limit", "sliding_window", "quantization_config", "layer_types",
                                                   "rope_interleave")}
    if rope_type not in ("default", None):
        extra["rope_scaling"] = {**rope, "rope_type": rope_type}
    if gpt_oss and not extra.get("layer_types"):     # the family alternates, starting with a windowed layer
        extra["layer_types"] = ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(int(cfg["num_hidden_layers"]))]
    window = int(cfg.get("sliding_window") or 0) if "sliding_attention" in (extra.get("layer_types") or ()) else 0
    return ModelConfig(
        name=name or cfg.get("_name_or_path", arch),
        architecture=arch,
        hidden_size=hidden,
        num_layers=int(cfg["num_hidden_layers"]),
        num_q_heads=heads,
        num_kv_heads=kv,
        head_dim=head_dim,
        intermediate_size=int(cfg.get("intermediate_size") or cfg.get("ffn_dim") or 0),
        vocab_size=int(cfg["vocab_size"]),
        rms_norm_eps=float(cfg.get("rms_norm_eps", cfg.get("layer_norm_eps", 1e-5 if opt else 1e-6))),
        rope_theta=float(cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta") or 10000.0),
        qk_norm=arch.startswith("Qwen3"),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        attention_bias=bool(cfg.get("attention_bias", cfg.get("enable_bias", True) if opt else arch.startswith("Qwen2"))),
        mlp_bias=bool(cfg.get("mlp_bias", False)),
        hidden_act=str(cfg.get("hidden_act", cfg.get("activation_function", "silu"))),
        max_position_embeddings=int(cfg.get("max_position_embeddings", 32768)),
        num_experts=n_exp,
        num_experts_per_tok=int(cfg.get("num_experts_per_tok", 0) or 0),
        moe_intermediate_size=int(cfg.get("moe_intermediate_size", 0) or 0),
        norm_topk_prob=bool(cfg.get("norm_topk_prob", True)),
        num_shared_experts=int(cfg.get("n_shared_experts", 0) or 0),
        first_k_dense=int(cfg.get("first_k_dense_replace", 0) or 0),
        routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0) or 1.0),
        router_scoring=str(cfg.get("scoring_func", "softmax")),
        router_precision={"DeepseekV2ForCausalLM": "fp32_logits", "Glm4MoeLiteForCausalLM": "fp32"}.get(arch, "payload"),
        dtype=str(cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))),
        norm="layernorm" if opt else "rmsnorm",
        positions="learned" if opt else "rope",
        sliding_window=window,
        attention_sinks=gpt_oss,
        o_bias=bool(cfg.get("attention_bias", False)) and (gpt_oss or mla is not None) or opt and bool(cfg.get("enable_bias", True)),
        mla=mla,
        extra=extra,
    )


def load(path_or_preset: str) -> ModelConfig:
    """A preset name, a directory holding ``config.json``, or a path to one."""
    if path_or_preset in PRESETS:
        return PRESETS[path_or_preset]
    p = Path(path_or_preset)
    if p.is_dir():
        p = p / "config.json"
    if not p.exists():
        raise FileNotFoundError(f"{path_or_preset!r} is neither a preset nor a config.json")
    return from_hf_config(json.loads(p.read_text()), name=str(p.parent.name))
