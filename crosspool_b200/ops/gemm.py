"""Python face of the weight-stationary tcgen05 GEMM (``csrc/kernels/gemm.cu``).

``linear(x, w)`` computes ``x @ w.T`` for an ``nn.Linear``-layout weight; ``gateup_swiglu`` fuses the
gate and up projections with the SwiGLU epilogue (the reference's ``i_proj`` + activation,
src/xpool/runtime/ffnagent/operators/dense.py); ``linear(..., resid=r)`` fuses the residual add
(``o_proj``/down-projection followed by the add).

There is no eager fallback here: on CUDA tensors the native kernel runs or an error is raised.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import native

# Dynamic shared memory cap of decode-size GEMMs: 126 KB keeps three pipeline stages of the widest decode
# tile and fits beside one 98 KB decode-attention CTA of another stream on the same SM (227 KB per SM).
DECODE_SMEM_LIMIT = 126 * 1024
DECODE_ROWS = 256
# ... but only for weight matrices this small: streaming a larger one is bound by the bytes a CTA keeps in
# flight (measured: 5 stages of 24 KB per CTA reach 0.40 of the copy bandwidth on a 100 MB matrix), so it
# takes every stage the SM can hold.
DECODE_SMALL_WEIGHT_BYTES = 16 << 20
EPI_STORE = 0
EPI_SWIGLU = 1
EPI_RESIDUAL = 2
EPI_STORE_F32 = 3

_WS_BYTES = 96 << 20
_COUNTER_WORDS = 1 << 16


@dataclass
class _Scratch:
    ws: torch.Tensor
    counters: torch.Tensor
    status: torch.Tensor


_status: dict[int, torch.Tensor] = {}
_scratch: dict[tuple[int, int], _Scratch] = {}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_words(device: torch.device) -> torch.Tensor:
    """The device's four error words (one set per device, shared by every stream and kernel family)."""
    idx = _device_index(device)
    st = _status.get(idx)
    if st is None:
        st = _status[idx] = torch.zeros(4, dtype=torch.int32, device=device)
    return st


def scratch(device: torch.device) -> _Scratch:
    """Split-K workspace and tile counters of the GEMM kernels for the *current stream* of ``device``, and the
    device's error words. Workspace and counters are per stream: two engines of one GPU run their decode GEMMs
    concurrently on their own streams, and split-K calls that shared one workspace would fold each other's partial
    sums. The status words (``status[0]`` code, ``[1..3]`` detail) are one set per device, read by ``check_status``."""
    idx = _device_index(device)
    st = status_words(device)
    key = (idx, torch.cuda.current_stream(device).cuda_stream)
    s = _scratch.get(key)
    if s is None:
        s = _Scratch(
            ws=torch.empty(_WS_BYTES // 4, dtype=torch.float32, device=device),
            counters=torch.zeros(_COUNTER_WORDS, dtype=torch.int32, device=device),
            status=st,
        )
        _scratch[key] = s
    return s


def check_status(device: torch.device) -> None:
    """Raises if a kernel recorded a bounded-wait timeout since the last check (synchronises)."""
    status = status_words(device)
    words = status.tolist()
    code = words[0]
    if code != 0:
        status.zero_()
        idx = _device_index(device)
        for (d, _), sc in _scratch.items():
            if d == idx:
                sc.counters.zero_()   # a split-K call that gave up leaves tile counters behind: later calls must not fold stale partials
        detail = f" (detail {words[1]}, {words[2]:#x}, {words[3]})" if any(words[1:]) else ""
        raise RuntimeError(f"xpool kernel reported device status {code}{detail}")


class TiledWeight:
    """A weight matrix ``[n, k]`` stored as contiguous 128x64 tiles (tile index = row_tile * k_tiles +
    k_tile). One TMA box then reads one 16 KB run of HBM instead of 128 separate 128-byte pieces of
    128 different rows, which is what a weight-streaming (decode) GEMM needs to approach the
    memory roofline. Built once at load time with :func:`tile_weight`."""

    __slots__ = ("data", "shape", "dtype", "device")

    def __init__(self, data: torch.Tensor, n: int, k: int):
        self.data, self.shape, self.dtype, self.device = data, (n, k), data.dtype, data.device

    def data_ptr(self) -> int:
        return self.data.data_ptr()

    def untiled(self) -> torch.Tensor:
        n, k = self.shape
        return self.data.view(n // 128, k // 64, 128, 64).permute(0, 2, 1, 3).reshape(n, k)


def tile_weight(w: torch.Tensor) -> TiledWeight:
    n, k = w.shape
    if n % 128 or k % 64:
        raise ValueError(f"cannot tile a {n}x{k} weight into 128x64 blocks")
    t = w.view(n // 128, 128, k // 64, 64).permute(0, 2, 1, 3).contiguous()
    return TiledWeight(t.view(-1), n, k)


def _args(x, w, out, *, n_out, rows, epilogue, dual=0, up_offset=0, bias=None, resid=None, splits=0, bn=0,
          num_sms=0, evict_first=None, gate_limit=0.0, up_add=0.0, act_alpha=0.0) -> native.GemmArgs:
    tiled = isinstance(w, TiledWeight)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(-1) == 1 and out.stride(-1) == 1 and (tiled or w.stride(-1) == 1)
    k = x.shape[-1]
    assert w.shape[-1] == k, (w.shape, x.shape)
    s = scratch(x.device)
    a = native.GemmArgs()
    a.w = w.data_ptr()
    a.x = x.data_ptr()
    a.out = out.data_ptr()
    a.resid = resid.data_ptr() if resid is not None else None
    a.bias = bias.data_ptr() if bias is not None else None
    a.ws = s.ws.data_ptr()
    a.counters = s.counters.data_ptr()
    a.status = s.status.data_ptr()
    a.stream = torch.cuda.current_stream(x.device).cuda_stream
    a.ws_bytes = s.ws.numel() * 4
    a.counter_bytes = s.counters.numel() * 4
    a.w_rows_total = w.shape[0]
    a.n_out = n_out
    a.k = k
    a.rows = rows
    a.ldw = k if tiled else w.stride(0)
    a.w_tiled = int(tiled)
    a.ldx = x.stride(0)
    a.ld_out = out.stride(0)
    a.ld_resid = resid.stride(0) if resid is not None else 0
    a.epilogue = epilogue
    a.dual = dual
    a.up_offset = up_offset
    a.splits = splits
    a.bn = bn
    a.num_sms = num_sms
    # decode-sized calls stream the weights once: keep them from evicting activations in L2
    a.w_evict_first = int(rows <= 64) if evict_first is None else int(evict_first)
    a.gate_limit = gate_limit
    a.up_add = up_add
    a.act_alpha = act_alpha
    # decode-size calls leave room for a second kernel on the SM (the co-located Instance's attention)
    small = w.shape[0] * k * 2 <= DECODE_SMALL_WEIGHT_BYTES
    a.smem_limit = DECODE_SMEM_LIMIT if rows <= DECODE_ROWS and small else 0
    return a


def plan(a: native.GemmArgs) -> native.GemmPlan:
    p = native.GemmPlan()
    native.check(native.kernels().xp_gemm_plan(C.byref(a), C.byref(p)), "xp_gemm_plan")
    return p


def plan_shape(n_out: int, k: int, rows: int, dual: int = 0, num_sms: int = 148, ws_bytes: int = 96 << 20) -> dict:
    """Tile plan the kernel would pick for a shape; needs no device (used by the graph observer)."""
    a, p = native.GemmArgs(), native.GemmPlan()
    a.n_out, a.k, a.rows, a.dual, a.num_sms = n_out, k, rows, dual, num_sms
    a.ws, a.counters, a.ws_bytes, a.counter_bytes = 1, 1, ws_bytes, 1 << 16  # only tested for null by the planner
    native.check(native.kernels().xp_gemm_plan(C.byref(a), C.byref(p)), "xp_gemm_plan", 0)
    return {f: getattr(p, f) for f, _ in native.GemmPlan._fields_}


def linear(x: torch.Tensor, w: torch.Tensor, *, out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
           resid: torch.Tensor | None = None, out_fp32: bool = False, splits: int = 0, bn: int = 0,
           num_sms: int = 0, evict_first: bool | None = None) -> torch.Tensor:
    """``x[rows, k] @ w[n, k].T`` (+ fp32 ``bias``) (+ ``resid``) on the tcgen05 kernel."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, n = x2.shape[0], w.shape[0]
    if out is None:
        out = torch.empty(rows, n, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    epi = EPI_STORE_F32 if out.dtype == torch.float32 else (EPI_RESIDUAL if resid is not None else EPI_STORE)
    a = _args(x2, w, out, n_out=n, rows=rows, epilogue=epi, bias=bias, resid=resid, splits=splits, bn=bn,
              num_sms=num_sms, evict_first=evict_first)
    native.check(native.kernels().xp_gemm(C.byref(a)), "xp_gemm")
    return out.reshape(*x.shape[:-1], n) if x.dim() != 2 else out


def gateup_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, *, out: torch.Tensor | None = None,
                  bias: torch.Tensor | None = None, gate_limit: float = 0.0, up_add: float = 0.0,
                  act_alpha: float = 0.0, splits: int = 0, bn: int = 0, num_sms: int = 0) -> torch.Tensor:
    """``silu(x @ Wg.T) * (x @ Wu.T)`` with ``w_gate_up = cat([Wg, Wu])`` of shape ``[2*I, k]``."""
    x2 = x.reshape(-1, x.shape[-1])
    rows = x2.shape[0]
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty(rows, inter, dtype=torch.bfloat16, device=x.device)
    a = _args(x2, w_gate_up, out, n_out=inter, rows=rows, epilogue=EPI_SWIGLU, dual=1, up_offset=inter, bias=bias,
              splits=splits, bn=bn, num_sms=num_sms, gate_limit=gate_limit, up_add=up_add, act_alpha=act_alpha)
    native.check(native.kernels().xp_gemm(C.byref(a)), "xp_gemm(swiglu)")
    return out


# ---------------------------------------------------------------------------------------------- fp8

def quantize_act_fp8(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[rows, k]`` -> (e4m3 ``[rows, k]``, fp32 scales ``[k / 128, rows padded to 256]``): one
    scale per row and 128-element K block."""
    rows, k = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and k % 128 == 0
    xq = torch.empty(rows, k, dtype=torch.float8_e4m3fn, device=x.device)
    ld = (rows + 255) // 256 * 256
    scales = torch.empty(k // 128, ld, dtype=torch.float32, device=x.device)  # padding columns are never stored
    native.check(native.kernels().xp_quant_act_fp8(x.data_ptr(), xq.data_ptr(), scales.data_ptr(), rows, k, x.stride(0), k, ld,
                                                   torch.cuda.current_stream(x.device).cuda_stream), "xp_quant_act_fp8")
    return xq, scales


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, *, out: torch.Tensor | None = None,
               bias: torch.Tensor | None = None, resid: torch.Tensor | None = None, splits: int = 0, bn: int = 0) -> torch.Tensor:
    """``x @ dequant(wq, w_scale).T`` with block-scaled e4m3 operands on ``tcgen05.mma.kind::f8f6f4``.

    ``wq`` ``[n, k]`` e4m3 with ``w_scale`` ``[n / 128, k / 128]`` (:class:`~crosspool_b200.quantization.Fp8Block`);
    ``x`` bf16, quantised here per row and 128-element K block. Every K block is accumulated in TMEM on its
    own and folded into fp32 registers with ``w_scale * x_scale``, so the result equals the fp32 product of
    the dequantised operands up to summation order."""
    rows, k = x.shape
    n = wq.shape[0]
    assert wq.dtype == torch.float8_e4m3fn and wq.shape[1] == k and n % 128 == 0 and k % 128 == 0
    assert w_scale.dtype == torch.float32 and tuple(w_scale.shape) == (n // 128, k // 128) and w_scale.is_contiguous()
    xq, xs = quantize_act_fp8(x)
    if out is None:
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=x.device)
    s = scratch(x.device)
    a = native.GemmArgs()
    a.w, a.x, a.out = wq.data_ptr(), xq.data_ptr(), out.data_ptr()
    a.resid = resid.data_ptr() if resid is not None else None
    a.bias = bias.data_ptr() if bias is not None else None
    a.ws, a.counters, a.status = s.ws.data_ptr(), s.counters.data_ptr(), s.status.data_ptr()
    a.stream = torch.cuda.current_stream(x.device).cuda_stream
    a.ws_bytes, a.counter_bytes = s.ws.numel() * 4, s.counters.numel() * 4
    a.w_rows_total, a.n_out, a.k, a.rows = n, n, k, rows
    a.ldw, a.ldx, a.ld_out = wq.stride(0), k, out.stride(0)
    a.ld_resid = resid.stride(0) if resid is not None else 0
    a.epilogue = EPI_STORE_F32 if out.dtype == torch.float32 else (EPI_RESIDUAL if resid is not None else EPI_STORE)
    a.splits, a.bn = splits, bn
    a.w_evict_first = int(rows <= 64)
    a.fp8, a.w_scale, a.x_scale, a.ld_xscale = 1, w_scale.data_ptr(), xs.data_ptr(), xs.stride(0)
    native.check(native.kernels().xp_gemm(C.byref(a)), "xp_gemm(fp8)")
    return out


def ffn_fp8(x: torch.Tensor, q: dict, *, out: torch.Tensor | None = None) -> torch.Tensor:
    """Dense gated FFN with block-scaled fp8 weights: gate/up projection (one GEMM over the concatenated
    rows), SiLU-gate in bf16, down projection. ``q`` holds ``gate_up``/``down`` e4m3 tensors and their
    ``*_scale`` grids (see :func:`crosspool_b200.models.weights.quantize_ffn_layer_fp8`)."""
    from . import norm

    gu = linear_fp8(x, q["gate_up"], q["gate_up_scale"])
    act = norm.swiglu(gu)
    return linear_fp8(act, q["down"], q["down_scale"], out=out)
