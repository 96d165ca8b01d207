"""What the attention side of a served model looks like, and whether a requested attention TP / DP fits it.

``ModelShape.load`` reads a Hugging Face ``config.json`` dict (heads, KV heads, head dim, latent attention);
``validate_attention_tp`` applies the engine's sharding rule -- query heads split evenly, KV heads either split
evenly or are replicated a whole number of times -- and ``AttentionTopology`` refuses the combinations the Fabric
does not carry: attention TP together with attention DP
(reference: src/xpool/integrations/sglang/topology.py; src/cext/fabric/projection.cpp:27-28).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


class TopologyError(ValueError):
    pass


def _config_int(hf: dict[str, Any], key: str, default: int | None = None) -> int:
    """An integer field of ``config.json`` (integral floats and digit strings are accepted, nothing else)."""
    v = hf.get(key)
    if v is None:
        if default is None:
            raise TopologyError(f"model config.json lacks {key}")
        return default
    if isinstance(v, bool):
        raise TopologyError(f"model config.json field {key} must be an integer")
    if isinstance(v, int):
        return v
    if isinstance(v, float) and v.is_integer():
        return int(v)
    if isinstance(v, str) and v.strip().lstrip("-").isdigit():
        return int(v)
    raise TopologyError(f"model config.json field {key} must be an integer")


@dataclass(frozen=True)
class ModelShape:
    architecture: str
    hidden_size: int
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    latent_attention: bool = False      # MLA: one shared latent KV per token instead of per-head K/V
    kv_lora_rank: int = 0
    sliding_window: int = 0

    @property
    def attention_kind(self) -> str:
        """``mla`` (latent KV), ``mqa`` (one KV head), ``mha`` (as many KV heads as query heads) or ``gqa``."""
        if self.latent_attention:
            return "mla"
        if self.num_kv_heads == 1 and self.num_q_heads > 1:
            return "mqa"
        return "mha" if self.num_kv_heads == self.num_q_heads else "gqa"

    @classmethod
    def load(cls, hf: dict[str, Any]) -> "ModelShape":
        heads = _config_int(hf, "num_attention_heads")
        kv = _config_int(hf, "num_key_value_heads", heads)
        hidden = _config_int(hf, "hidden_size")
        if heads <= 0 or kv <= 0 or hidden <= 0 or kv > heads:
            raise TopologyError(f"implausible attention geometry: {heads} query heads, {kv} KV heads, hidden {hidden}")
        mla = bool(hf.get("kv_lora_rank"))
        return cls(architecture=(hf.get("architectures") or [""])[0], hidden_size=hidden,
                   num_layers=int(hf.get("num_hidden_layers", hf.get("num_layers", 0))), num_q_heads=heads, num_kv_heads=kv,
                   head_dim=int(hf.get("head_dim") or hidden // heads), latent_attention=mla,
                   kv_lora_rank=int(hf.get("kv_lora_rank") or 0), sliding_window=int(hf.get("sliding_window") or 0))

    def validate_attention_tp(self, tp: int) -> None:
        if tp < 1:
            raise TopologyError("attention TP size must be at least 1")
        if self.num_q_heads % tp:
            raise TopologyError(f"{self.num_q_heads} query heads do not split over attention TP {tp}")
        if not self.latent_attention and self.num_kv_heads % tp and tp % self.num_kv_heads:
            raise TopologyError(f"{self.num_kv_heads} KV heads neither split over nor replicate into attention TP {tp}")

    def kv_heads_per_rank(self, tp: int) -> int:
        return 1 if self.latent_attention else max(1, self.num_kv_heads // tp)


@dataclass(frozen=True)
class AttentionTopology:
    tp_size: int
    dp_size: int
    tp_rank: int = 0
    dp_rank: int = 0

    @classmethod
    def from_runtime(cls, server_args: Any, shape: ModelShape, *, atn_tp_size: int, atn_dp_size: int,
                     supports_dp_attention: bool) -> "AttentionTopology":
        """Checks the engine's launch arguments against the deployment's model entry."""
        for name, v in (("attention TP size", atn_tp_size), ("attention DP size", atn_dp_size)):
            if not isinstance(v, int) or isinstance(v, bool) or v < 1:
                raise TopologyError(f"{name} must be a positive integer, got {v!r}")
        cp = int(getattr(server_args, "attn_cp_size", 1) or 1)
        if cp != 1:
            raise TopologyError(f"attention context parallel size must be one, got {cp}")
        if atn_tp_size > 1 and atn_dp_size > 1:
            raise TopologyError("attention TP combined with attention DP is not supported by the Fabric")
        if atn_dp_size > 1 and not supports_dp_attention:
            raise TopologyError(f"{shape.architecture} has no data-parallel attention adapter")
        world = max(atn_tp_size, atn_dp_size)
        if int(getattr(server_args, "tp_size", 1)) != world:
            raise TopologyError(f"--tensor-parallel-size must be {world} (attention world size)")
        engine_dp = int(getattr(server_args, "dp_size", 1) or 1)
        if engine_dp != atn_dp_size:
            raise TopologyError(f"--data-parallel-size must be {atn_dp_size} (configured attention DP), got {engine_dp}")
        if bool(getattr(server_args, "enable_dp_attention", False)) != (atn_dp_size > 1):
            raise TopologyError(f"--enable-dp-attention must be {'set' if atn_dp_size > 1 else 'unset'} for attention DP size "
                                f"{atn_dp_size}")
        shape.validate_attention_tp(atn_tp_size)
        rank = int(getattr(server_args, "tp_rank", 0))
        return cls(atn_tp_size, atn_dp_size, tp_rank=rank if atn_tp_size > 1 else 0, dp_rank=rank if atn_dp_size > 1 else 0)

    @property
    def instance_rank(self) -> int:
        """Index of this rank among the Instance's attention ranks (``dp_rank * tp_size + tp_rank``, the reference's
        ``atnagent_index``, src/cext-include/xpool/fabric/layout.hpp:28-79)."""
        return self.dp_rank * self.tp_size + self.tp_rank
