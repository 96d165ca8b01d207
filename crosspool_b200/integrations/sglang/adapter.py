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


@dataclass(frozen=True)
class Hook:
    target: str          # dotted path of the engine symbol
    handler: Any
    kind: str            # "replace" | "around" | "after"


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


class _Dense(ShimAdapter):
    def hooks(self) -> list[Hook]:
        return []


class Qwen2Adapter(_Dense):
    name, architectures = "qwen2", ("Qwen2ForCausalLM",)


class Qwen3Adapter(_Dense):
    name, architectures = "qwen3", ("Qwen3ForCausalLM",)


class LlamaAdapter(_Dense):
    name, architectures = "llama", ("LlamaForCausalLM", "MistralForCausalLM")


class OptAdapter(_Dense):
    name, architectures = "opt", ("OPTForCausalLM",)
    mlp_attribute = "ffn"


class Qwen3MoeAdapter(_Dense):
    name, architectures, supports_dp_attention = "qwen3_moe", ("Qwen3MoeForCausalLM",), True


class DeepseekV2Adapter(_Dense):
    name, architectures = "deepseek_v2", ("DeepseekV2ForCausalLM",)


class Glm4MoeLiteAdapter(_Dense):
    name, architectures = "glm4_moe_lite", ("Glm4MoeLiteForCausalLM",)


class GptOssAdapter(_Dense):
    name, architectures = "gpt_oss", ("GptOssForCausalLM",)


ADAPTERS: tuple[ShimAdapter, ...] = (Qwen2Adapter(), Qwen3Adapter(), LlamaAdapter(), OptAdapter(), Qwen3MoeAdapter(),
                                     DeepseekV2Adapter(), Glm4MoeLiteAdapter(), GptOssAdapter())


def find_adapter(model_runner: Any) -> ShimAdapter:
    for a in ADAPTERS:
        if a.matches(model_runner):
            return a
    arch = getattr(getattr(model_runner, "model_config", None), "architecture", None)
    raise LookupError(f"no shim adapter for architecture {arch!r}")
