"""Architecture-neutral description of a model's decoder FFNs (the "FFN spec IR").

An architecture adapter compiles a Hugging Face ``config.json`` plus the checkpoint's key list into
one :class:`FfnModelSpec`; everything downstream (placement, memory admission, weight loading, TP
slicing, executable signatures) works from this description and never looks at model names. The
vocabulary follows the reference's IR (src/xpool/ffn.py): projections are ``i_proj`` (gate and up
packed, or a single up projection) and ``o_proj``.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass, field
from enum import Enum


class ActivationKind(str, Enum):
    SILU = "silu"
    RELU = "relu"
    GELU = "gelu"


class GateUpOrder(str, Enum):
    CONCATENATED = "concatenated"  # gate rows then up rows
    INTERLEAVED = "interleaved"    # gate0, up0, gate1, up1, ...


class RouterAlgorithm(str, Enum):
    SOFTMAX = "softmax"
    SIGMOID = "sigmoid"


class RouterProjectionPrecision(str, Enum):
    PAYLOAD = "payload"          # logits GEMM in the payload dtype
    FP32 = "fp32"                # fp32 inputs and weights
    FP32_LOGITS = "fp32_logits"  # payload inputs, fp32 accumulate and logits


class TopKWeightRounding(str, Enum):
    NONE = "none"
    LOGITS_DTYPE = "logits_dtype"


class LayerKind(str, Enum):
    DENSE = "dense"
    MOE = "moe"


@dataclass(frozen=True)
class GateTransform:
    """``act(min(g, limit)) * (clamp(u, -limit, limit) + up_offset)``; ``limit <= 0`` disables clamping.
    ``alpha`` generalises SiLU to ``g * sigmoid(alpha * g)`` (GPT-OSS uses 1.702, limit 7, offset 1)."""

    limit: float = 0.0
    up_offset: float = 0.0
    alpha: float = 1.0


@dataclass(frozen=True)
class ProjectionSpec:
    """One linear map stored under ``weight_key`` (+ optional ``bias_key``) in the checkpoint."""

    weight_key: str
    out_features: int
    in_features: int
    bias_key: str | None = None
    scales_key: str | None = None  # block-scaled / MX formats


@dataclass(frozen=True)
class GatedProjectionSpec:
    """Gate and up projections, stored separately or packed in one tensor."""

    gate: ProjectionSpec | None
    up: ProjectionSpec
    packed: ProjectionSpec | None = None  # both in one tensor
    source_order: GateUpOrder = GateUpOrder.CONCATENATED

    @property
    def gated(self) -> bool:
        return self.gate is not None or self.packed is not None


@dataclass(frozen=True)
class DenseFfnSpec:
    layer: int
    hidden_size: int
    intermediate_size: int
    activation: ActivationKind
    i_proj: GatedProjectionSpec
    o_proj: ProjectionSpec
    gate_transform: GateTransform = GateTransform()
    kind: LayerKind = LayerKind.DENSE


@dataclass(frozen=True)
class ExpertSource:
    """Where expert tensors live: ``per_expert`` keys contain ``{expert}``; ``stacked`` tensors carry
    a leading expert dimension. ``input_major`` stacked tensors are stored ``[experts, in, out]`` (the unquantised
    GPT-OSS form, multiplied as ``x @ W``) instead of ``[experts, out, in]``."""

    per_expert: bool
    gate_key: str | None
    up_key: str | None
    packed_key: str | None
    down_key: str
    gate_bias_key: str | None = None
    down_bias_key: str | None = None
    scales_suffix: str | None = None
    input_major: bool = False


@dataclass(frozen=True)
class MoeFfnSpec:
    layer: int
    hidden_size: int
    moe_intermediate_size: int
    num_experts: int
    top_k: int
    activation: ActivationKind
    experts: ExpertSource
    router_weight_key: str
    router_bias_key: str | None = None
    router_algorithm: RouterAlgorithm = RouterAlgorithm.SOFTMAX
    router_precision: RouterProjectionPrecision = RouterProjectionPrecision.PAYLOAD
    renormalize: bool = True
    routed_scaling_factor: float = 1.0
    correction_bias_key: str | None = None
    topk_weight_rounding: TopKWeightRounding = TopKWeightRounding.NONE
    num_shared_experts: int = 0
    shared_intermediate_size: int = 0
    shared_gate_key: str | None = None
    shared_up_key: str | None = None
    shared_down_key: str | None = None
    gate_transform: GateTransform = GateTransform()
    source_order: GateUpOrder = GateUpOrder.CONCATENATED
    kind: LayerKind = LayerKind.MOE

    @property
    def effective_topk(self) -> int:
        return self.top_k + self.num_shared_experts


@dataclass(frozen=True)
class FfnModelSpec:
    model_id: str
    architecture: str
    payload_dtype: str  # "bfloat16" | "float16"
    hidden_size: int
    quantization: str   # "none" | "mxfp4" | "fp8_block"
    layers: tuple[DenseFfnSpec | MoeFfnSpec, ...] = field(default_factory=tuple)

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def required_keys(self) -> set[str]:
        """Every checkpoint key the FFN side must find (used for exact coverage validation)."""
        keys: set[str] = set()

        def add(p: ProjectionSpec | None):
            if p is None:
                return
            keys.add(p.weight_key)
            if p.bias_key:
                keys.add(p.bias_key)
            if p.scales_key:
                keys.add(p.scales_key)

        for l in self.layers:
            if isinstance(l, DenseFfnSpec):
                add(l.i_proj.gate), add(l.i_proj.up if l.i_proj.packed is None else None), add(l.i_proj.packed)
                add(l.o_proj)
            else:
                keys.add(l.router_weight_key)
                for k in (l.router_bias_key, l.correction_bias_key, l.shared_gate_key, l.shared_up_key,
                          l.shared_down_key):
                    if k:
                        keys.add(k)
                ex = l.experts
                names = [ex.gate_key, ex.up_key, ex.packed_key, ex.down_key, ex.gate_bias_key, ex.down_bias_key]
                for n in names:
                    if not n:
                        continue
                    if ex.per_expert:
                        keys.update(n.format(expert=e) for e in range(l.num_experts))
                    else:
                        keys.add(n)
                    if ex.scales_suffix and n in (ex.packed_key, ex.down_key, ex.gate_key, ex.up_key):
                        base = n.removesuffix("_blocks")
                        keys.add(base + ex.scales_suffix if not ex.per_expert else base)
        return keys

    def digest(self) -> str:
        def enc(o):
            if isinstance(o, Enum):
                return o.value
            raise TypeError(type(o))

        return hashlib.sha256(json.dumps(asdict(self), sort_keys=True, default=enc).encode()).hexdigest()
