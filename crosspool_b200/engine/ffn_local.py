"""Loopback FFN port: the layer's FFN runs in-stream on the attention GPU.

Used when one GPU hosts both roles (kernels that wait on one another must never be separate
launches on one GPU, so the loopback path is stream-ordered and flag-free). Dense layers are two
launches: gate/up GEMM with the SwiGLU epilogue, then the down projection.
"""

from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..models.weights import FfnLayerWeights
from ..ops import gemm
from .atn_engine import FfnPort


class LocalFfnPort(FfnPort):
    def __init__(self, cfg: ModelConfig, weights: list[FfnLayerWeights]):
        self.cfg, self.weights = cfg, weights
        self.act = None
        self.y = None

    def attach(self, engine) -> None:
        inter = max(w.gate_up.shape[-2] // 2 for w in self.weights)
        self.act = torch.zeros(engine.cap, inter, dtype=torch.bfloat16, device=engine.device)
        self.y = torch.zeros(engine.cap, self.cfg.hidden_size, dtype=torch.bfloat16, device=engine.device)
        self.moe_ws = None
        moe_layers = [w for w in self.weights if w.is_moe]
        if moe_layers:
            from ..ops import moe

            w = moe_layers[0]  # one scratch set sized for the engine's row capacity serves every layer and bucket
            self.moe_ws = moe.workspace(engine.device, engine.cap, self.cfg, w.gate_up.shape[1] // 2, w.gate_up.shape[0])

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> list[torch.Tensor]:
        w = self.weights[layer]
        if w.is_moe:
            from ..ops import moe

            return [moe.moe_forward(x, w, self.cfg, out=self.y[:rows], ws=self.moe_ws)]
        if "fp8" in w.extra:
            return [gemm.ffn_fp8(x, w.extra["fp8"], out=self.y[:rows])]
        inter = w.gate_up.shape[0] // 2
        act = self.act[:rows, :inter]
        lim, up_add, alpha = w.extra.get("gate_transform", (0.0, 0.0, 0.0))
        gemm.gateup_swiglu(x, w.gate_up, out=act, bias=w.gate_up_bias, gate_limit=lim, up_add=up_add, act_alpha=alpha)
        gemm.linear(act, w.down, out=self.y[:rows], bias=w.down_bias)
        return [self.y[:rows]]


class UnfusedFfnPort(FfnPort):
    """Baseline arm of the benchmarks: the layer's FFN as library calls -- cuBLAS GEMMs through ``torch.matmul``
    and a separate elementwise SwiGLU -- on the attention GPU's own memory. None of this repository's FFN kernels
    run on this path (MoE layers excepted, for which there is no library restatement here)."""

    def __init__(self, cfg: ModelConfig, weights: list[FfnLayerWeights]):
        self.cfg, self.weights = cfg, weights
        self._moe = LocalFfnPort(cfg, weights) if any(w.is_moe for w in weights) else None

    def attach(self, engine) -> None:
        dense = [w for w in self.weights if not w.is_moe]
        inter2 = max((w.gate_up.shape[0] for w in dense), default=2)
        dev, bf = engine.device, torch.bfloat16
        self.gu = torch.zeros(engine.cap, inter2, dtype=bf, device=dev)
        self.act = torch.zeros(engine.cap, inter2 // 2, dtype=bf, device=dev)
        self.y = torch.zeros(engine.cap, self.cfg.hidden_size, dtype=bf, device=dev)
        if self._moe is not None:
            self._moe.attach(engine)

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> list[torch.Tensor]:
        w = self.weights[layer]
        if w.is_moe:
            return self._moe.run(layer, x, rows, mode)
        return [unfused_dense_ffn(x, w, self.gu, self.act, self.y)]


def unfused_dense_ffn(x: torch.Tensor, w: FfnLayerWeights, gu: torch.Tensor, act: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """``down(silu(gate) * up)`` as library launches: two cuBLAS GEMMs, an elementwise SwiGLU, bias adds. The gate
    rows of ``gate_up`` come first, then the up rows."""
    rows, inter2 = x.shape[0], w.gate_up.shape[0]
    g = gu[:rows, :inter2]
    torch.matmul(x, w.gate_up.t(), out=g)
    if w.gate_up_bias is not None:
        g += w.gate_up_bias.to(g.dtype)
    a = act[:rows, :inter2 // 2]
    torch.mul(torch.nn.functional.silu(g[:, :inter2 // 2]), g[:, inter2 // 2:], out=a)
    out = y[:rows]
    torch.matmul(a, w.down.t(), out=out)
    if w.down_bias is not None:
        out += w.down_bias.to(out.dtype)
    return out
