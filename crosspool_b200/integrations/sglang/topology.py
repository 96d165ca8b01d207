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

    @classmethod
    def load(cls, hf: dict[str, Any]) -> "ModelShape":
        heads = int(hf["num_attention_heads"])
        kv = int(hf.get("num_key_value_heads") or heads)
        hidden = int(hf["hidden_size"])
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
        if atn_tp_size > 1 and atn_dp_size > 1:
            raise TopologyError("attention TP combined with attention DP is not supported by the Fabric")
        if atn_dp_size > 1 and not supports_dp_attention:
            raise TopologyError(f"{shape.architecture} has no data-parallel attention adapter")
        world = max(atn_tp_size, atn_dp_size)
        if int(getattr(server_args, "tp_size", 1)) != world:
            raise TopologyError(f"--tensor-parallel-size must be {world} (attention world size)")
        if atn_dp_size > 1 and not getattr(server_args, "enable_dp_attention", False):
            raise TopologyError("attention DP needs --enable-dp-attention")
        shape.validate_attention_tp(atn_tp_size)
        rank = int(getattr(server_args, "tp_rank", 0))
        return cls(atn_tp_size, atn_dp_size, tp_rank=rank if atn_tp_size > 1 else 0, dp_rank=rank if atn_dp_size > 1 else 0)

    @property
    def instance_rank(self) -> int:
        """Index of this rank among the Instance's attention ranks (``dp_rank * tp_size + tp_rank``, the reference's
        ``atnagent_index``, src/cext-include/xpool/fabric/layout.hpp:28-79)."""
        return self.dp_rank * self.tp_size + self.tp_rank
