"""Declarative validation of serving-engine launch arguments.

The attention/FFN split only works with a subset of an engine's features; anything that would move
FFN work back into the engine, change the MLP boundary, or reorder layers is refused up front with a
message naming the flag (reference: src/xpool/integrations/sglang/server_args.py:24-122).
Expert parallelism is *allowed* here (the reference rejects it): this system implements EP on the
FFN tier.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


@dataclass(frozen=True)
class ServerArgRule:
    name: str
    ok: Callable[[Any], bool]
    message: str


def _get(args: Any, name: str, default=None):
    return getattr(args, name, default) if not isinstance(args, dict) else args.get(name, default)


RULES: tuple[ServerArgRule, ...] = (
    ServerArgRule("pp_size", lambda v: v in (None, 1), "pipeline parallelism is not supported"),
    ServerArgRule("attention_context_parallel_size", lambda v: v in (None, 1), "attention context parallelism is not supported"),
    ServerArgRule("speculative_algorithm", lambda v: not v, "speculative decoding is not supported"),
    ServerArgRule("enable_lora", lambda v: not v, "LoRA adapters are not supported (they would add FFN-side weights)"),
    ServerArgRule("lora_paths", lambda v: not v, "LoRA adapters are not supported"),
    ServerArgRule("enable_two_batch_overlap", lambda v: not v, "two-batch overlap is not supported"),
    ServerArgRule("enable_torch_compile", lambda v: not v, "torch.compile is not supported on the attention side"),
    ServerArgRule("enable_mixed_chunk", lambda v: not v, "mixed prefill/decode chunks are not supported"),
    ServerArgRule("enable_layernorm_sp", lambda v: not v, "layernorm sequence parallelism is not supported"),
    ServerArgRule("enable_prefill_cp", lambda v: not v, "prefill context parallelism is not supported"),
    ServerArgRule("enable_mlp_allreduce_fusion", lambda v: not v, "MLP all-reduce fusion bypasses the FFN boundary"),
    ServerArgRule("cpu_offload_gb", lambda v: not v, "CPU offload is not supported"),
    ServerArgRule("disaggregation_mode", lambda v: v in (None, "null", "none"), "prefill/decode disaggregation is not supported"),
    ServerArgRule("enable_hierarchical_cache", lambda v: not v, "hierarchical KV cache is not supported"),
    ServerArgRule("cuda_graph_backend_decode", lambda v: v in (None, "disabled", "full"), "decode graphs must be 'full' or disabled"),
    ServerArgRule("cuda_graph_backend_prefill", lambda v: v in (None, "disabled", "breakable"),
                  "prefill graphs must be 'breakable' or disabled"),
)


class ServerArgsError(ValueError):
    pass


def validate_server_args(args: Any, atn_tp_size: int = 1, atn_dp_size: int = 1) -> None:
    problems = [f"--{r.name.replace('_', '-')}: {r.message}" for r in RULES if not r.ok(_get(args, r.name))]
    tp, dp = _get(args, "tp_size", atn_tp_size * atn_dp_size), _get(args, "dp_size", atn_dp_size)
    if tp != atn_tp_size * atn_dp_size:
        problems.append(f"--tensor-parallel-size {tp} does not match the configured attention world {atn_tp_size * atn_dp_size}")
    if dp != atn_dp_size:
        problems.append(f"--data-parallel-size {dp} does not match atn_dp_size {atn_dp_size}")
    if atn_dp_size > 1 and not _get(args, "enable_dp_attention", False):
        problems.append("--enable-dp-attention is required when atn_dp_size > 1")
    if problems:
        raise ServerArgsError("; ".join(problems))
