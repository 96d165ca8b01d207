"""Mixture-of-experts FFN on the grouped tcgen05 GEMM.

Pipeline (all on the caller's stream, no host synchronisation, shapes independent of the routing):

    router logits GEMM -> top-k -> route ordering + tile tables -> row gather
    -> grouped gate/up GEMM with SwiGLU epilogue -> grouped down GEMM -> weighted combine

It replaces the reference's routing / bitmatrix / ordering / ragged-matmul / reduce chain
(src/xpool/runtime/ffnagent/operators/{routing,moe}.py). With ``expert_range=(lo, hi)`` only routes
to experts ``[lo, hi)`` are computed and the result is this rank's partial sum (expert parallelism);
``w.gate_up`` / ``w.down`` then hold just those experts.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import native
from ..models.config import ModelConfig
from ..models.weights import FfnLayerWeights
from . import gemm


@dataclass
class MoeWorkspace:
    cap_rows: int
    top_k: int
    logits: torch.Tensor
    ids: torch.Tensor
    weights: torch.Tensor
    counts: torch.Tensor
    offsets: torch.Tensor
    perm_token: torch.Tensor
    route_pos: torch.Tensor
    tiles_gu: torch.Tensor
    tiles_dn: torch.Tensor
    n_tiles: torch.Tensor
    xp: torch.Tensor
    act: torch.Tensor
    yp: torch.Tensor
    logits32: torch.Tensor | None = None   # fp32 router logits, allocated on first use by an fp32 router projection


ROUTER_PRECISIONS = {"payload": 0, "fp32_logits": 1, "fp32": 2}


def router_precision_code(w: FfnLayerWeights) -> int:
    """0: bf16 tensor-core projection with bf16 logits; 1: payload weights, fp32 accumulation and fp32 logits; 2: fp32
    weights (``w.extra["router_fp32"]``), fp32 accumulation and logits. Reference: ``RouterProjectionPrecision`` in
    src/xpool/ffn.py and its use in src/xpool/runtime/ffnagent/operators/routing.py."""
    p = w.extra.get("router_precision", "payload")
    p = getattr(p, "value", p)
    if p not in ROUTER_PRECISIONS:
        raise ValueError(f"unknown router projection precision {p!r}")
    if p == "fp32" and w.extra.get("router_fp32") is None:
        raise ValueError("router precision 'fp32' needs the fp32 router weights in extra['router_fp32']")
    return ROUTER_PRECISIONS[p]


def router_project_fp32(x: torch.Tensor, w: FfnLayerWeights, out: torch.Tensor) -> torch.Tensor:
    """``out[:, :num_experts] = x @ router^T`` accumulated and stored in fp32 (exact SIMT projection)."""
    code = router_precision_code(w)
    rw = w.extra["router_fp32"] if code == 2 else w.router
    assert rw.is_contiguous() and out.dtype == torch.float32 and x.stride(1) == 1
    assert rw.dtype == (torch.float32 if code == 2 else torch.bfloat16)
    native.check(native.kernels().xp_router_fp32(x.data_ptr(), x.stride(0), rw.data_ptr(), int(code == 2), out.data_ptr(),
                                                 out.stride(0), x.shape[0], x.shape[1], rw.shape[0], _stream(x.device)),
                 "xp_router_fp32")
    return out


_ws_cache: dict[tuple, MoeWorkspace] = {}


def workspace(device, cap_rows: int, cfg: ModelConfig, inter: int, n_local: int) -> MoeWorkspace:
    # one workspace per stream: Instances of one GPU that run concurrently must not share routing tables and scratch rows
    key = (str(device), torch.cuda.current_stream(device).cuda_stream if torch.device(device).type == "cuda" else 0,
           cap_rows, cfg.hidden_size, inter, cfg.num_experts_per_tok, n_local, cfg.num_experts)
    ws = _ws_cache.get(key)
    if ws is None:
        k, h = cfg.num_experts_per_tok, cfg.hidden_size
        routes = cap_rows * k
        e_pad = (cfg.num_experts + 127) // 128 * 128
        max_tiles = (max(inter, h) // 128) * (routes // 16 + n_local) + 8
        i32 = dict(dtype=torch.int32, device=device)
        bf = dict(dtype=torch.bfloat16, device=device)
        ws = MoeWorkspace(
            cap_rows, k, torch.zeros(cap_rows, e_pad, **bf), torch.zeros(cap_rows, k, **i32),
            torch.zeros(cap_rows, k, dtype=torch.float32, device=device), torch.zeros(n_local, **i32),
            torch.zeros(n_local + 1, **i32), torch.zeros(routes, **i32), torch.zeros(routes, **i32),
            torch.zeros(max_tiles, 4, **i32), torch.zeros(max_tiles, 4, **i32), torch.zeros(2, **i32),
            torch.zeros(routes, h, **bf), torch.zeros(routes, inter, **bf), torch.zeros(routes, h, **bf))
        _ws_cache[key] = ws
    return ws


def padded_router(w: FfnLayerWeights) -> torch.Tensor:
    """The layer's router weights with the expert dimension padded to a multiple of 128 rows (one UMMA
    tile); built once and kept with the layer."""
    router = w.router
    e = router.shape[0]
    if e % 128 == 0:
        return router
    t = w.extra.get("router_padded")
    if t is None or t.shape[1] != router.shape[1] or t.device != router.device:
        t = torch.zeros((e + 127) // 128 * 128, router.shape[1], dtype=router.dtype, device=router.device)
        t[:e] = router
        w.extra["router_padded"] = t
    return t


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def router_topk(logits: torch.Tensor, num_experts: int, top_k: int, *, out_ids: torch.Tensor, out_weights: torch.Tensor,
                sigmoid: bool = False, renormalize: bool = True, scale: float = 1.0,
                logit_bias: torch.Tensor | None = None, correction_bias: torch.Tensor | None = None,
                round_weights_bf16: bool = False) -> None:
    a = native.RouterArgs()
    a.logits = logits.data_ptr()
    a.logit_bias = logit_bias.data_ptr() if logit_bias is not None else None
    a.correction_bias = correction_bias.data_ptr() if correction_bias is not None else None
    a.topk_ids, a.topk_weights = out_ids.data_ptr(), out_weights.data_ptr()
    a.rows, a.num_experts, a.top_k, a.ld_logits = logits.shape[0], num_experts, top_k, logits.stride(0)
    a.logits_fp32 = int(logits.dtype == torch.float32)
    a.sigmoid, a.renormalize, a.round_weights_bf16, a.scale = int(sigmoid), int(renormalize), int(round_weights_bf16), scale
    native.check(native.kernels().xp_router_topk(C.byref(a), _stream(logits.device)), "xp_router_topk")


def _tile_width(rows: int, top_k: int, n_local: int) -> int:
    avg = max(1, rows * top_k // max(1, n_local))
    bn = 16
    while bn < avg and bn < 128:
        bn <<= 1
    return bn


def _grouped(x, w2d, out, *, n_out, rows_cap, bn, dual, up_offset, tiles, n_tiles, rows_per_group, epilogue, bias=None,
             transform=(0.0, 0.0, 0.0)):
    """``bias``: fp32 ``[experts, rows_per_group]``, indexed by the weight row of the stacked tensor."""
    a = gemm._args(x, w2d, out, n_out=n_out, rows=rows_cap, epilogue=epilogue, dual=dual, up_offset=up_offset, splits=1, bn=bn,
                   bias=bias, gate_limit=transform[0], up_add=transform[1], act_alpha=transform[2])
    a.tile_table, a.n_tiles, a.w_rows_per_group = tiles.data_ptr(), n_tiles.data_ptr(), rows_per_group
    native.check(native.kernels().xp_gemm(C.byref(a)), "xp_gemm(grouped)")


def moe_forward(x: torch.Tensor, w: FfnLayerWeights, cfg: ModelConfig, out: torch.Tensor | None = None,
                expert_range: tuple[int, int] | None = None, ws: MoeWorkspace | None = None) -> torch.Tensor:
    """``x`` [rows, hidden] bf16 -> MoE output [rows, hidden] (this rank's partial under EP)."""
    rows, h = x.shape
    k, e_total = cfg.num_experts_per_tok, cfg.num_experts
    lo, hi = expert_range or w.extra.get("experts") or (0, e_total)
    n_local = hi - lo
    inter = w.gate_up.shape[1] // 2
    assert w.gate_up.shape[0] == n_local and w.down.shape[0] == n_local
    dev = x.device
    ws = ws or workspace(dev, max(rows, 1), cfg, inter, n_local)
    if out is None:
        out = torch.empty(rows, h, dtype=torch.bfloat16, device=dev)
    lib, s = native.kernels(), _stream(dev)
    # 1. router (payload precision: bf16 logits; fp32 precisions: exact fp32 logits; scores always fp32)
    if router_precision_code(w) == 0:
        logits = ws.logits[:rows]
        gemm.linear(x, padded_router(w), out=logits)
    else:
        if ws.logits32 is None:
            ws.logits32 = torch.zeros(ws.cap_rows, ws.logits.shape[1], dtype=torch.float32, device=dev)
        logits = router_project_fp32(x, w, ws.logits32[:rows])
    router_topk(logits, e_total, k, out_ids=ws.ids[:rows], out_weights=ws.weights[:rows],
                sigmoid=cfg.router_scoring == "sigmoid", renormalize=cfg.norm_topk_prob, scale=cfg.routed_scaling_factor,
                correction_bias=w.extra.get("correction_bias"), logit_bias=w.extra.get("router_bias"),
                round_weights_bf16=bool(w.extra.get("round_topk_weights")))
    # 2. order the routes of the local experts, build the tile tables
    bn = _tile_width(rows, k, n_local)
    r = native.RouteArgs()
    r.topk_ids, r.counts, r.offsets = ws.ids.data_ptr(), ws.counts.data_ptr(), ws.offsets.data_ptr()
    r.perm_token, r.route_pos = ws.perm_token.data_ptr(), ws.route_pos.data_ptr()
    r.tiles_gateup, r.tiles_down = ws.tiles_gu.data_ptr(), ws.tiles_dn.data_ptr()
    r.n_tiles_gateup, r.n_tiles_down = ws.n_tiles.data_ptr(), ws.n_tiles.data_ptr() + 4
    r.rows, r.top_k, r.expert_lo, r.expert_hi = rows, k, lo, hi
    r.tm_gateup, r.bn_gateup, r.tm_down, r.bn_down = inter // 128, bn, h // 128, bn
    native.check(lib.xp_moe_route(C.byref(r), s), "xp_moe_route", 3)
    # 3. gather rows into expert order
    routes = rows * k
    native.check(lib.xp_moe_gather(x.data_ptr(), ws.perm_token.data_ptr(), ws.offsets.data_ptr() + 4 * n_local,
                                   ws.xp.data_ptr(), routes, h, x.stride(0), s), "xp_moe_gather")
    # 4. grouped projections
    _grouped(ws.xp[:routes], w.gate_up.view(n_local * 2 * inter, h), ws.act[:routes], n_out=inter, rows_cap=routes, bn=bn,
             dual=1, up_offset=inter, tiles=ws.tiles_gu, n_tiles=ws.n_tiles[0:1], rows_per_group=2 * inter,
             epilogue=gemm.EPI_SWIGLU, bias=w.gate_up_bias, transform=w.extra.get("gate_transform", (0.0, 0.0, 0.0)))
    _grouped(ws.act[:routes], w.down.view(n_local * h, inter), ws.yp[:routes], n_out=h, rows_cap=routes, bn=bn, dual=0,
             up_offset=0, tiles=ws.tiles_dn, n_tiles=ws.n_tiles[1:2], rows_per_group=h, epilogue=gemm.EPI_STORE,
             bias=w.down_bias)
    # 5. weighted sum over the selected experts, fixed order
    native.check(lib.xp_moe_combine(ws.yp.data_ptr(), ws.route_pos.data_ptr(), ws.weights.data_ptr(), out.data_ptr(), rows, k,
                                    h, out.stride(0), s), "xp_moe_combine")
    if w.shared_gate_up is not None and (expert_range is None or lo == 0):
        sh = gemm.linear(gemm.gateup_swiglu(x, w.shared_gate_up), w.shared_down)
        out += sh
    return out
