"""Architecture adapters: Hugging Face ``config.json`` + checkpoint keys → :class:`FfnModelSpec`.

One adapter per supported architecture, discovered by ``architectures[0]`` — the same eight
families the reference serves (src/xpool/runtime/ffnagent/models/*.py, discovery in
src/xpool/runtime/ffnagent/architecture.py:175-215): Qwen2, Qwen3, Qwen3-MoE, Llama, OPT,
DeepSeek-V2, GLM-4 MoE Lite and GPT-OSS. Adapters only read the configuration and the *names* of
checkpoint tensors; no weight is opened here.
"""

from __future__ import annotations

from typing import Callable, Iterable, Mapping

from ..ffn import (ActivationKind, DenseFfnSpec, ExpertSource, FfnModelSpec, GatedProjectionSpec, GateTransform,
                   GateUpOrder, MoeFfnSpec, ProjectionSpec, RouterAlgorithm, RouterProjectionPrecision,
                   TopKWeightRounding)


class UnsupportedModel(ValueError):
    pass


class FfnSourceConfig:
    """Typed access to a parsed ``config.json``; a missing or mistyped field is an error that names it."""

    def __init__(self, cfg: Mapping):
        self.cfg = cfg

    def _get(self, key: str, typ, default=None, required=True):
        v = self.cfg.get(key, default)
        if v is None:
            if required:
                raise UnsupportedModel(f"config.json misses {key!r}")
            return None
        if typ is float and isinstance(v, int) and not isinstance(v, bool):
            v = float(v)
        if not isinstance(v, typ) or isinstance(v, bool) and typ is not bool:
            raise UnsupportedModel(f"config.json field {key!r} has type {type(v).__name__}, wanted {typ.__name__}")
        return v

    def int(self, key, default=None, required=True) -> int:
        return self._get(key, int, default, required)

    def int_any(self, *keys: str) -> int:
        """The first of ``keys`` the config holds (library versions write the same field under different names)."""
        for k in keys:
            if self.cfg.get(k) is not None:
                return self._get(k, int)
        raise UnsupportedModel(f"config.json misses {keys[0]!r}")

    def float(self, key, default=None, required=True) -> float:
        return self._get(key, float, default, required)

    def str(self, key, default=None, required=True) -> str:
        return self._get(key, str, default, required)

    def bool(self, key, default=False) -> bool:
        return bool(self._get(key, bool, default, False))

    @property
    def architecture(self) -> str:
        a = self.cfg.get("architectures") or []
        if not a:
            raise UnsupportedModel("config.json has no architectures")
        return a[0]

    @property
    def payload_dtype(self) -> str:
        dt = self.cfg.get("torch_dtype") or self.cfg.get("dtype") or "bfloat16"
        if dt not in ("bfloat16", "float16"):
            # payloads are 16-bit only (src/cext-include/xpool/ffn.hpp:83-85); fp32 checkpoints are served in bf16
            return "bfloat16"
        return dt

    @property
    def quantization(self) -> str:
        q = self.cfg.get("quantization_config") or {}
        method = q.get("quant_method")
        if method in (None, "none"):
            return "none"
        if method == "mxfp4":
            return "mxfp4"
        if method == "fp8" and list(q.get("weight_block_size") or []) == [128, 128]:
            return "fp8_block"
        raise UnsupportedModel(f"unsupported weight quantization method {method!r}")


_ACT = {"silu": ActivationKind.SILU, "swish": ActivationKind.SILU, "relu": ActivationKind.RELU,
        "gelu": ActivationKind.GELU, "gelu_new": ActivationKind.GELU, "gelu_pytorch_tanh": ActivationKind.GELU}


def _activation(name: str) -> ActivationKind:
    try:
        return _ACT[name]
    except KeyError:
        raise UnsupportedModel(f"unsupported activation {name!r}") from None


def _gated_dense(layer: int, hidden: int, inter: int, act: ActivationKind, prefix: str, bias: bool = False,
                 fp8_block: bool = False) -> DenseFfnSpec:
    """``fp8_block``: the checkpoint stores e4m3 weights with one ``weight_scale_inv`` per 128 x 128 block (the
    fine-grained fp8 layout of published ``*-FP8`` checkpoints); both dimensions must be whole blocks."""
    if fp8_block and (hidden % 128 or inter % 128):
        raise UnsupportedModel(f"block-scaled fp8 needs hidden ({hidden}) and intermediate ({inter}) sizes in multiples of 128")

    def proj(name, o, i):
        return ProjectionSpec(f"{prefix}.{name}.weight", o, i, f"{prefix}.{name}.bias" if bias else None,
                              f"{prefix}.{name}.weight_scale_inv" if fp8_block else None)

    return DenseFfnSpec(layer, hidden, inter, act,
                        GatedProjectionSpec(proj("gate_proj", inter, hidden), proj("up_proj", inter, hidden)),
                        proj("down_proj", hidden, inter))


def _llama_like(model_id: str, src: FfnSourceConfig, keys: Iterable[str]) -> FfnModelSpec:
    hidden, inter, n = src.int("hidden_size"), src.int("intermediate_size"), src.int("num_hidden_layers")
    act = _activation(src.str("hidden_act", "silu"))
    bias = src.bool("mlp_bias", False)
    fp8 = src.quantization == "fp8_block"
    layers = tuple(_gated_dense(i, hidden, inter, act, f"model.layers.{i}.mlp", bias, fp8) for i in range(n))
    return FfnModelSpec(model_id, src.architecture, src.payload_dtype, hidden, src.quantization, layers)


def _opt(model_id: str, src: FfnSourceConfig, keys: Iterable[str]) -> FfnModelSpec:
    hidden, inter, n = src.int("hidden_size"), src.int("ffn_dim"), src.int("num_hidden_layers")
    if src.int("word_embed_proj_dim", hidden) != hidden:
        raise UnsupportedModel("OPT variants with projected embeddings are not supported")
    act = _activation(src.str("activation_function", "relu"))
    layers = []
    for i in range(n):
        p = f"model.decoder.layers.{i}"
        up = ProjectionSpec(f"{p}.fc1.weight", inter, hidden, f"{p}.fc1.bias")
        layers.append(DenseFfnSpec(i, hidden, inter, act, GatedProjectionSpec(None, up),
                                   ProjectionSpec(f"{p}.fc2.weight", hidden, inter, f"{p}.fc2.bias")))
    return FfnModelSpec(model_id, src.architecture, src.payload_dtype, hidden, src.quantization, tuple(layers))


def _per_expert_source(prefix: str) -> ExpertSource:
    e = prefix + ".experts.{expert}"
    return ExpertSource(True, e + ".gate_proj.weight", e + ".up_proj.weight", None, e + ".down_proj.weight")


def _qwen3_moe(model_id: str, src: FfnSourceConfig, keys: Iterable[str]) -> FfnModelSpec:
    hidden, n = src.int("hidden_size"), src.int("num_hidden_layers")
    experts = src.int_any("num_experts", "num_local_experts")
    topk, minter = src.int("num_experts_per_tok"), src.int("moe_intermediate_size")
    if src.int("decoder_sparse_step", 1) != 1 or (src.cfg.get("mlp_only_layers") or []):
        raise UnsupportedModel("Qwen3-MoE with dense interleaving is not supported")
    act = _activation(src.str("hidden_act", "silu"))
    layers = tuple(
        MoeFfnSpec(i, hidden, minter, experts, topk, act, _per_expert_source(f"model.layers.{i}.mlp"),
                   router_weight_key=f"model.layers.{i}.mlp.gate.weight", router_algorithm=RouterAlgorithm.SOFTMAX,
                   router_precision=RouterProjectionPrecision.PAYLOAD, renormalize=src.bool("norm_topk_prob", True))
        for i in range(n))
    return FfnModelSpec(model_id, src.architecture, src.payload_dtype, hidden, src.quantization, layers)


def _deepseek_like(model_id: str, src: FfnSourceConfig, keys: Iterable[str], *, sigmoid: bool) -> FfnModelSpec:
    hidden, n = src.int("hidden_size"), src.int("num_hidden_layers")
    inter, minter = src.int("intermediate_size"), src.int("moe_intermediate_size")
    experts, topk = src.int("n_routed_experts"), src.int("num_experts_per_tok")
    first_dense = src.int("first_k_dense_replace", 0)
    shared = src.int("n_shared_experts", 0, required=False) or 0
    if src.int("moe_layer_freq", 1) != 1:
        raise UnsupportedModel("moe_layer_freq != 1 is not supported")
    if src.int("n_group", 1, required=False) not in (None, 1) or src.int("topk_group", 1, required=False) not in (None, 1):
        raise UnsupportedModel("grouped top-k routing is not supported")
    act = _activation(src.str("hidden_act", "silu"))
    scale = src.float("routed_scaling_factor", 1.0)
    layers = []
    for i in range(n):
        p = f"model.layers.{i}.mlp"
        if i < first_dense:
            layers.append(_gated_dense(i, hidden, inter, act, p))
            continue
        layers.append(MoeFfnSpec(
            i, hidden, minter, experts, topk, act, _per_expert_source(p), router_weight_key=f"{p}.gate.weight",
            router_algorithm=RouterAlgorithm.SIGMOID if sigmoid else RouterAlgorithm.SOFTMAX,
            router_precision=RouterProjectionPrecision.FP32 if sigmoid else RouterProjectionPrecision.FP32_LOGITS,
            renormalize=src.bool("norm_topk_prob", sigmoid), routed_scaling_factor=scale,
            correction_bias_key=f"{p}.gate.e_score_correction_bias" if sigmoid else None,
            num_shared_experts=shared, shared_intermediate_size=minter * shared,
            shared_gate_key=f"{p}.shared_experts.gate_proj.weight" if shared else None,
            shared_up_key=f"{p}.shared_experts.up_proj.weight" if shared else None,
            shared_down_key=f"{p}.shared_experts.down_proj.weight" if shared else None))
    return FfnModelSpec(model_id, src.architecture, src.payload_dtype, hidden, src.quantization, tuple(layers))


def _gpt_oss(model_id: str, src: FfnSourceConfig, keys: Iterable[str]) -> FfnModelSpec:
    hidden, n, inter = src.int("hidden_size"), src.int("num_hidden_layers"), src.int("intermediate_size")
    experts, topk = src.int("num_local_experts"), src.int("num_experts_per_tok")
    quant = src.quantization
    mx = quant == "mxfp4"
    limit = src.float("swiglu_limit", 7.0)
    layers = []
    for i in range(n):
        p = f"model.layers.{i}.mlp"
        ex = ExpertSource(False, None, None, f"{p}.experts.gate_up_proj" + ("_blocks" if mx else ""),
                          f"{p}.experts.down_proj" + ("_blocks" if mx else ""),
                          gate_bias_key=f"{p}.experts.gate_up_proj_bias", down_bias_key=f"{p}.experts.down_proj_bias",
                          scales_suffix="_scales" if mx else None, input_major=not mx)
        layers.append(MoeFfnSpec(
            i, hidden, inter, experts, topk, ActivationKind.SILU, ex, router_weight_key=f"{p}.router.weight",
            router_bias_key=f"{p}.router.bias", router_algorithm=RouterAlgorithm.SOFTMAX,
            router_precision=RouterProjectionPrecision.PAYLOAD, renormalize=True,
            topk_weight_rounding=TopKWeightRounding.LOGITS_DTYPE,
            gate_transform=GateTransform(limit=limit, up_offset=1.0, alpha=1.702),
            source_order=GateUpOrder.INTERLEAVED))
    return FfnModelSpec(model_id, src.architecture, src.payload_dtype, hidden, quant, tuple(layers))


ADAPTERS: dict[str, Callable[[str, FfnSourceConfig, Iterable[str]], FfnModelSpec]] = {
    "Qwen2ForCausalLM": _llama_like,
    "Qwen3ForCausalLM": _llama_like,
    "LlamaForCausalLM": _llama_like,
    "MistralForCausalLM": _llama_like,
    "Qwen3MoeForCausalLM": _qwen3_moe,
    "OPTForCausalLM": _opt,
    "DeepseekV2ForCausalLM": lambda m, s, k: _deepseek_like(m, s, k, sigmoid=False),
    "Glm4MoeLiteForCausalLM": lambda m, s, k: _deepseek_like(m, s, k, sigmoid=True),
    "GptOssForCausalLM": _gpt_oss,
}


def compile_ffn_spec(model_id: str, config: Mapping, checkpoint_keys: Iterable[str] | None = None) -> FfnModelSpec:
    """Compiles the FFN description and, when the checkpoint's key list is given, checks that every
    tensor the FFN side needs is present (exact coverage is validated by the loader)."""
    src = FfnSourceConfig(config)
    try:
        adapter = ADAPTERS[src.architecture]
    except KeyError:
        raise UnsupportedModel(f"no FFN adapter for architecture {src.architecture!r}; "
                               f"supported: {sorted(ADAPTERS)}") from None
    keys = list(checkpoint_keys) if checkpoint_keys is not None else None
    spec = adapter(model_id, src, keys or ())
    if keys is not None:
        missing = sorted(spec.required_keys() - set(keys))
        if missing:
            raise UnsupportedModel(f"checkpoint misses {len(missing)} FFN tensors, e.g. {missing[:3]}")
    return spec
