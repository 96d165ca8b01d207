"""The parameter-free module that stands where a decoder MLP was, and the ``xpool::ffn_shim`` op.

``FfnShimModule.forward`` maps the engine's forward mode and data-parallel padding mode to the FFN
ABI (src/xpool/integrations/sglang/shim.py:94-192): DECODE/EXTEND/IDLE -> Decode/Prefill/Idle;
``MAX_LEN`` padding -> ``UniformByRank``, ``SUM_LEN`` -> ``PackedByRank``; the output requirement is
``GroupSumComplete`` iff the engine will reduce-scatter the MLP output, else ``PerRankComplete``;
fused MLP all-reduce is refused. The op schema matches the reference's
(src/cext-bindings/ops.cpp:1-44): ``ffn_shim(Tensor hidden_states, Tensor? dp_rank_payload_rows,
Tensor(a!) output, int layer_ordinal, int forward_mode, int output_requirement, int dp_row_layout) -> ()``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from ...native import runtime as rt

_submit: Callable | None = None


def bind_submit(fn: Callable | None) -> None:
    """Installs the transport submit function ``fn(hidden, dp_rows, out, layer, mode, requirement, layout)``."""
    global _submit
    _submit = fn


def _ffn_shim_host(hidden_states, dp_rank_payload_rows, output, layer_ordinal, forward_mode, output_requirement, dp_row_layout):
    if _submit is None:
        raise RuntimeError("xpool::ffn_shim called before an Instance runtime was bound")
    _submit(hidden_states, dp_rank_payload_rows, output, layer_ordinal, forward_mode, output_requirement, dp_row_layout)


def _register_op() -> str:
    """Makes ``torch.ops.xpool.ffn_shim`` available. The native library (``csrc/bindings/torch_ops.cpp``) defines the
    schema and the CUDA implementation, which submits to the Instance transport on the current stream; Python adds
    the CPU key, which calls the function installed with :func:`bind_submit` (engine-less tests). Without the native
    library the whole operator is defined here and every device goes through ``bind_submit``."""
    from pathlib import Path

    native_lib = Path(__file__).resolve().parents[2] / "native" / "libxpool_torch_ops.so"
    try:
        if native_lib.exists():
            torch.ops.load_library(str(native_lib))
            lib = torch.library.Library("xpool", "IMPL")
            lib.impl("ffn_shim", _ffn_shim_host, "CPU")
            _keep.append(lib)
            return "native"
    except Exception:  # pragma: no cover - fall through to the Python definition
        pass
    try:
        lib = torch.library.Library("xpool", "FRAGMENT")
        lib.define("ffn_shim(Tensor hidden_states, Tensor? dp_rank_payload_rows, Tensor(a!) output, int layer_ordinal, "
                   "int forward_mode, int output_requirement, int dp_row_layout) -> ()")
        lib.impl("ffn_shim", _ffn_shim_host, "CompositeExplicitAutograd")
        _keep.append(lib)
        return "python"
    except Exception:  # pragma: no cover - already defined in this process
        return "existing"


_keep: list = []
OP_BACKEND = _register_op()


@dataclass(frozen=True)
class ShimMetadata:
    layer_ordinal: int
    forward_mode: int
    output_requirement: int
    dp_row_layout: int


def ffn_shim(hidden: torch.Tensor, dp_rows: torch.Tensor | None, meta: ShimMetadata) -> torch.Tensor:
    out = torch.empty_like(hidden)
    torch.ops.xpool.ffn_shim(hidden, dp_rows, out, meta.layer_ordinal, meta.forward_mode, meta.output_requirement,
                             meta.dp_row_layout)
    return out


def _mode_name(forward_mode: Any) -> str:
    n = getattr(forward_mode, "name", str(forward_mode)).upper()
    return n


def map_forward_mode(forward_mode: Any) -> int:
    n = _mode_name(forward_mode)
    if "IDLE" in n:
        return rt.MODE_IDLE
    if "DECODE" in n:
        return rt.MODE_DECODE
    if "EXTEND" in n or "PREFILL" in n:
        return rt.MODE_PREFILL
    raise ValueError(f"forward mode {n} is not supported by the FFN boundary")


def map_dp_layout(dp_padding_mode: Any) -> int:
    if dp_padding_mode is None:
        return rt.DP_NONE
    n = getattr(dp_padding_mode, "name", str(dp_padding_mode)).upper()
    if n == "MAX_LEN":
        return rt.DP_UNIFORM_BY_RANK
    if n == "SUM_LEN":
        return rt.DP_PACKED_BY_RANK
    raise ValueError(f"data-parallel padding mode {n} is not supported")


class FfnShimModule(torch.nn.Module):
    """Holds no parameters; ``forward`` ships the hidden states to the FFN tier."""

    def __init__(self, layer_ordinal: int):
        super().__init__()
        self.layer_ordinal = layer_ordinal

    def forward(self, hidden_states: torch.Tensor, forward_batch: Any = None, **kw) -> torch.Tensor:
        ctx = getattr(forward_batch, "forward_context", forward_batch)
        if getattr(ctx, "fuse_mlp_allreduce", False):
            raise RuntimeError("fused MLP all-reduce bypasses the FFN boundary")
        mode = map_forward_mode(getattr(forward_batch, "forward_mode", "DECODE"))
        layout = map_dp_layout(getattr(forward_batch, "dp_padding_mode", None))
        req = rt.OUT_GROUP_SUM_COMPLETE if getattr(ctx, "mlp_reduce_scatter", False) else rt.OUT_PER_RANK_COMPLETE
        rows = getattr(forward_batch, "global_num_tokens_gpu", None) if layout != rt.DP_NONE else None
        return ffn_shim(hidden_states, rows, ShimMetadata(self.layer_ordinal, mode, req, layout))
