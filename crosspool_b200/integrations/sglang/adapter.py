"""Adapter surface between a serving engine's model classes and the FFN shim.

An adapter knows one architecture family: which module class is the decoder MLP, how to replace it
with a parameter-free :class:`FfnShimModule`, and which checkpoint tensors the attention side must
*not* load. The contract mirrors the reference's ``SglangShimAdapter``
(src/xpool/integrations/sglang/adapter.py:278-444).
"""

from __future__ import annotations

import re
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Iterable, Iterator

FFN_WEIGHT = re.compile(r"^model\.(decoder\.)?layers\.\d+\.(mlp|fc1|fc2|block_sparse_moe)\b")


def filter_decoder_ffn_weights(weights: Iterable[tuple[str, Any]]) -> Iterator[tuple[str, Any]]:
    """Drops decoder FFN tensors so that the attention side never materialises them
    (src/xpool/integrations/sglang/adapter.py:33-45)."""
    for name, tensor in weights:
        if not FFN_WEIGHT.match(name):
            yield name, tensor


_filter_depth = 0


class weight_filter_scope:
    """While active, every ``load_weights`` hook drops decoder-FFN tensors (the lifecycle hook opens it around the
    engine's ``load_model``; outside it the engine's own loaders are untouched)."""

    def __enter__(self):
        global _filter_depth
        _filter_depth += 1
        return self

    def __exit__(self, *exc):
        global _filter_depth
        _filter_depth -= 1
        return False


def filtering_active() -> bool:
    return _filter_depth > 0


def layer_ordinal_from_prefix(prefix: str, default: int = -1) -> int:
    """``model.layers.17.mlp`` -> 17 (engine modules are constructed with their parameter prefix)."""
    m = re.search(r"layers\.(\d+)", prefix or "")
    return int(m.group(1)) if m else default


@dataclass(frozen=True)
class Hook:
    target: str          # dotted path of the engine symbol
    handler: Any
    kind: str            # "replace" | "around" | "after"
    required: bool = True   # install fails when a required hook cannot be applied; the hooks of architecture adapters
                            # are optional there (an engine build need not ship every model) and checked at load time


@dataclass(frozen=True)
class InstanceRankBinding:
    model_id: str
    rank: int
    tp_size: int
    dp_size: int

    @classmethod
    def resolve(cls, server_args: Any, config) -> "InstanceRankBinding":
        path = getattr(server_args, "model_path", None)
        for m in config.models:
            if path in (m.id, m.path):
                return cls(m.id, int(getattr(server_args, "tp_rank", 0)), m.atn_tp_size, m.atn_dp_size)
        raise LookupError(f"model path {path!r} is not a configured model")


class ShimAdapter(ABC):
    name: str = ""
    architectures: tuple[str, ...] = ()
    supports_dp_attention: bool = False
    mlp_attribute: str = "mlp"

    def matches(self, model_runner: Any) -> bool:
        arch = getattr(getattr(model_runner, "model_config", None), "architecture", None)
        return arch in self.architectures

    @abstractmethod
    def hooks(self) -> list[Hook]: ...

    def validate_after_load(self, model: Any, expected_layers: int) -> list[Any]:
        raise NotImplementedError

    def validate_before_load(self, model_runner: Any, binding: InstanceRankBinding) -> None:
        if binding.dp_size > 1 and not self.supports_dp_attention:
            raise ValueError(f"adapter {self.name} does not support attention data parallelism")

    def decoder_layers(self, model: Any) -> list[Any]:
        inner = getattr(model, "model", model)
        return list(getattr(inner, "layers", getattr(getattr(inner, "decoder", None), "layers", [])))

    def install_shims(self, model: Any, make_shim) -> list[Any]:
        """Replaces every decoder MLP with a shim; returns the shims in layer order."""
        shims = []
        for ordinal, layer in enumerate(self.decoder_layers(model)):
            shim = make_shim(ordinal, getattr(layer, self.mlp_attribute))
            setattr(layer, self.mlp_attribute, shim)
            shims.append(shim)
        return shims

    def require_ffn_shims(self, model: Any, expected_layers: int, shim_type: type) -> list[Any]:
        shims = [getattr(l, self.mlp_attribute) for l in self.decoder_layers(model)]
        bad = [i for i, s in enumerate(shims) if not isinstance(s, shim_type)]
        if bad or len(shims) != expected_layers:
            raise RuntimeError(f"{len(bad)} decoder layers kept their MLP (first: {bad[:3]}); expected {expected_layers} shims")
        return shims

    def require_no_ffn_parameters(self, model: Any) -> None:
        named = getattr(model, "named_parameters", None)
        if named is None:
            return
        left = [n for n, _ in named() if FFN_WEIGHT.match(n)]
        if left:
            raise RuntimeError(f"attention side still holds FFN parameters, e.g. {left[:3]}")


class _ModuleAdapter(ShimAdapter):
    """An architecture described by where its classes live in the engine: the module, the model class whose
    ``load_weights`` is filtered, and the MLP / MoE-block classes that become shims. ``hooks()`` replaces each of those
    classes with a factory that builds an :class:`FfnShimModule` for the layer named by the ``prefix`` the engine passes,
    and wraps ``load_weights`` so that decoder-FFN tensors are never read on the attention side
    (reference: src/xpool/integrations/sglang/models/qwen2.py:28-137, qwen3_moe.py:24-109)."""

    module: str = ""
    model_class: str = ""
    mlp_classes: tuple[str, ...] = ()
    dense_prefix_layers: int = 0       # DeepSeek-style: this many leading layers are dense, the rest MoE blocks

    def shim_factory(self, class_name: str):
        from .shim import FfnShimModule

        def make(*args, prefix: str = "", layer_id: int | None = None, **kw):
            ordinal = layer_id if layer_id is not None else layer_ordinal_from_prefix(prefix)
            if ordinal < 0:
                raise ValueError(f"{class_name}: cannot tell the layer ordinal from prefix {prefix!r}")
            return FfnShimModule(ordinal)

        make.__name__ = f"{class_name}Shim"
        return make

    @staticmethod
    def load_weights_around(original, model, weights, *a, **kw):
        if filtering_active():
            weights = filter_decoder_ffn_weights(weights)
        return original(model, weights, *a, **kw)

    def hooks(self) -> list[Hook]:
        base = f"sglang.srt.models.{self.module}."
        out = [Hook(base + c, self.shim_factory(c), "replace", required=False) for c in self.mlp_classes]
        out.append(Hook(base + self.model_class + ".load_weights", self.load_weights_around, "around", required=False))
        return out

    def validate_after_load(self, model: Any, expected_layers: int) -> list[Any]:
        from .shim import FfnShimModule

        shims = self.require_ffn_shims(model, expected_layers, FfnShimModule)
        self.require_no_ffn_parameters(model)
        for i, sh in enumerate(shims):
            if sh.layer_ordinal != i:
                raise RuntimeError(f"decoder layer {i} carries the shim of layer {sh.layer_ordinal}")
        return shims


class Qwen2Adapter(_ModuleAdapter):
    name, architectures = "qwen2", ("Qwen2ForCausalLM",)
    module, model_class, mlp_classes = "qwen2", "Qwen2ForCausalLM", ("Qwen2MLP",)


class Qwen3Adapter(_ModuleAdapter):
    name, architectures = "qwen3", ("Qwen3ForCausalLM",)
    module, model_class, mlp_classes = "qwen3", "Qwen3ForCausalLM", ("Qwen3MLP",)


class LlamaAdapter(_ModuleAdapter):
    name, architectures = "llama", ("LlamaForCausalLM", "MistralForCausalLM")
    module, model_class, mlp_classes = "llama", "LlamaForCausalLM", ("LlamaMLP",)


class OptAdapter(_ModuleAdapter):
    """OPT keeps ``fc1`` / ``fc2`` directly on the decoder layer; the engine-side layer class is replaced by one whose
    two projections and activation are a single ``ffn`` shim."""

    name, architectures = "opt", ("OPTForCausalLM",)
    module, model_class, mlp_classes = "opt", "OPTForCausalLM", ("OPTDecoderMLP",)
    mlp_attribute = "ffn"


class Qwen3MoeAdapter(_ModuleAdapter):
    name, architectures, supports_dp_attention = "qwen3_moe", ("Qwen3MoeForCausalLM",), True
    module, model_class, mlp_classes = "qwen3_moe", "Qwen3MoeForCausalLM", ("Qwen3MoeSparseMoeBlock", "Qwen3MoeMLP")


class DeepseekV2Adapter(_ModuleAdapter):
    name, architectures = "deepseek_v2", ("DeepseekV2ForCausalLM",)
    module, model_class, mlp_classes = "deepseek_v2", "DeepseekV2ForCausalLM", ("DeepseekV2MoE", "DeepseekV2MLP")


class Glm4MoeLiteAdapter(_ModuleAdapter):
    name, architectures = "glm4_moe_lite", ("Glm4MoeLiteForCausalLM",)
    module, model_class, mlp_classes = "glm4_moe_lite", "Glm4MoeLiteForCausalLM", ("Glm4MoeLiteSparseMoeBlock", "Glm4MoeLiteMLP")


class GptOssAdapter(_ModuleAdapter):
    name, architectures = "gpt_oss", ("GptOssForCausalLM",)
    module, model_class, mlp_classes = "gpt_oss", "GptOssForCausalLM", ("GptOssSparseMoeBlock",)


ADAPTERS: tuple[ShimAdapter, ...] = (Qwen2Adapter(), Qwen3Adapter(), LlamaAdapter(), OptAdapter(), Qwen3MoeAdapter(),
                                     DeepseekV2Adapter(), Glm4MoeLiteAdapter(), GptOssAdapter())


def find_adapter(model_runner: Any) -> ShimAdapter:
    for a in ADAPTERS:
        if a.matches(model_runner):
            return a
    arch = getattr(getattr(model_runner, "model_config", None), "architecture", None)
    raise LookupError(f"no shim adapter for architecture {arch!r}")
