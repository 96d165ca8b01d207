"""Monolithic plain-PyTorch forward of the supported decoder architectures.

This is the oracle: the disaggregated deployments (CPU loopback processes, single-GPU loopback,
attention/FFN split over several GPUs) must reproduce its logits. It is also what the CPU plumbing
roles compute with, split at the FFN boundary: ``attention_half`` produces the post-attention-norm
hidden states that cross to the FFN role and ``ffn_forward`` is the FFN role's math. The boundary is
the reference's: the FFN receives the output of ``post_attention_layernorm`` and returns the MLP
output only; the residual stays on the attention side
(src/xpool/integrations/sglang/models/qwen2.py:104-127).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .config import ModelConfig
from .weights import AttentionWeights, AttnLayerWeights, FfnLayerWeights


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return n.to(x.dtype) * w


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x ``[T, heads, d]``, rotate-half convention, computed in fp32."""
    d = x.shape[-1]
    inv = theta ** (-torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d)
    ang = positions.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


def activation(name: str, g: torch.Tensor) -> torch.Tensor:
    if name in ("silu", "swish"):
        return F.silu(g)
    if name == "relu":
        return F.relu(g)
    if name in ("gelu", "gelu_new", "gelu_pytorch_tanh"):
        return F.gelu(g, approximate="tanh" if name != "gelu" else "none")
    raise ValueError(f"unsupported activation {name}")


def gated(g: torch.Tensor, u: torch.Tensor, act: str, transform: tuple[float, float, float] | None) -> torch.Tensor:
    """``act(g) * u``; with a gate transform ``(limit, up_offset, alpha)`` (GPT-OSS):
    ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``, ``g' * sigmoid(alpha * g') * (u' + up_offset)``
    (src/xpool/runtime/ffnagent/operators/activation.py:19-60)."""
    if transform is None:
        return activation(act, g.float()).to(g.dtype) * u
    limit, up_offset, alpha = transform
    gf, uf = g.float(), u.float()
    if limit > 0:
        gf, uf = gf.clamp(max=limit), uf.clamp(-limit, limit)
    return (gf * torch.sigmoid((alpha or 1.0) * gf) * (uf + up_offset)).to(g.dtype)


def dense_ffn(x: torch.Tensor, w: FfnLayerWeights, act: str = "silu") -> torch.Tensor:
    gu = F.linear(x, w.gate_up, w.gate_up_bias.to(x.dtype) if w.gate_up_bias is not None else None)
    if not w.extra.get("gated", True):       # a single up projection (OPT): act(x W1 + b1) W2 + b2
        h = activation(act, gu.float()).to(gu.dtype)
        return F.linear(h, w.down, w.down_bias.to(x.dtype) if w.down_bias is not None else None)
    inter = gu.shape[-1] // 2
    h = gated(gu[..., :inter], gu[..., inter:], act, w.extra.get("gate_transform"))
    return F.linear(h, w.down, w.down_bias.to(x.dtype) if w.down_bias is not None else None)


def route_topk(logits: torch.Tensor, k: int, renormalize: bool, scoring: str = "softmax",
               correction_bias: torch.Tensor | None = None, scaling: float = 1.0
               ) -> tuple[torch.Tensor, torch.Tensor]:
    """Router semantics of the reference (src/xpool/runtime/ffnagent/operators/routing.py:21-190):
    fp32 scores; selection on score (+ correction bias) with ties to the lower id for softmax and the
    higher id for sigmoid; weights from the original scores; normalise, then scale."""
    lf = logits.float()
    scores = lf.softmax(-1) if scoring == "softmax" else lf.sigmoid()
    sel = scores + correction_bias.float() if correction_bias is not None else scores
    n = sel.shape[-1]
    ids = torch.arange(n, device=sel.device)
    # stable tie-break by id: sort by (score desc, id asc|desc)
    order_key = ids if scoring == "softmax" else -ids
    idx = torch.argsort(order_key.expand_as(sel), dim=-1, stable=True)
    sel_sorted = sel.gather(-1, idx)
    top_in_sorted = torch.argsort(sel_sorted, dim=-1, descending=True, stable=True)[..., :k]
    top_ids = idx.gather(-1, top_in_sorted)
    top_w = scores.gather(-1, top_ids)
    if renormalize:
        s = top_w.sum(-1, keepdim=True)
        top_w = torch.where(s > 0, top_w / s, top_w)
    return top_ids, top_w * scaling


def moe_ffn(x: torch.Tensor, w: FfnLayerWeights, cfg: ModelConfig) -> torch.Tensor:
    prec = getattr(w.extra.get("router_precision", "payload"), "value", w.extra.get("router_precision", "payload"))
    if prec == "payload":
        logits = F.linear(x, w.router)
    else:   # fp32 accumulation and fp32 logits; "fp32" also keeps the router weights in fp32
        logits = F.linear(x.float(), w.extra["router_fp32"].float() if prec == "fp32" else w.router.float())
    if w.extra.get("router_bias") is not None:
        logits = logits.float() + w.extra["router_bias"].float()    # payload-precision logits, bias added in fp32
    ids, weights = route_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.router_scoring,
                              w.extra.get("correction_bias"), cfg.routed_scaling_factor)
    if w.extra.get("round_topk_weights"):
        weights = weights.to(x.dtype).float()
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    inter = w.gate_up.shape[1] // 2
    lo = (w.extra.get("experts") or (0, 0))[0]     # an expert-parallel shard holds experts lo .. lo + n: a partial sum
    for i in range(w.gate_up.shape[0]):
        e = lo + i
        tok, slot = (ids == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        gu = F.linear(xe, w.gate_up[i], w.gate_up_bias[i].to(x.dtype) if w.gate_up_bias is not None else None)
        h = gated(gu[:, :inter], gu[:, inter:], "silu", w.extra.get("gate_transform"))
        ye = F.linear(h, w.down[i], w.down_bias[i].to(x.dtype) if w.down_bias is not None else None)
        out.index_add_(0, tok, ye.float() * weights[tok, slot, None])
    if w.shared_gate_up is not None:
        out += dense_ffn(x, FfnLayerWeights(w.shared_gate_up, w.shared_down)).float()
    return out.to(x.dtype)


def ffn_forward(x: torch.Tensor, w: FfnLayerWeights, cfg: ModelConfig) -> torch.Tensor:
    return moe_ffn(x, w, cfg) if w.is_moe else dense_ffn(x, w, cfg.hidden_act)


class KvCacheRef:
    """Per-sequence contiguous K/V per layer (the oracle needs no paging)."""

    def __init__(self, cfg: ModelConfig):
        self.k = [None] * cfg.num_layers
        self.v = [None] * cfg.num_layers

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        self.k[layer] = k if self.k[layer] is None else torch.cat([self.k[layer], k], 0)
        self.v[layer] = v if self.v[layer] is None else torch.cat([self.v[layer], v], 0)
        return self.k[layer], self.v[layer]


def attention_core(cfg: ModelConfig, lw: AttnLayerWeights, x: torch.Tensor, positions: torch.Tensor,
                   cache: KvCacheRef, layer: int) -> torch.Tensor:
    """x ``[T, hidden]`` (already input-normalised) → attention output projected by ``o``."""
    T = x.shape[0]
    qkv = F.linear(x, lw.qkv, lw.qkv_bias.to(x.dtype) if lw.qkv_bias is not None else None)
    q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], -1)
    q = q.view(T, cfg.num_q_heads, cfg.head_dim)
    k = k.view(T, cfg.num_kv_heads, cfg.head_dim)
    v = v.view(T, cfg.num_kv_heads, cfg.head_dim)
    if lw.q_norm is not None:
        q, k = rmsnorm(q, lw.q_norm, cfg.rms_norm_eps), rmsnorm(k, lw.k_norm, cfg.rms_norm_eps)
    q, k = rope(q, positions, cfg.rope_theta), rope(k, positions, cfg.rope_theta)
    kk, vv = cache.append(layer, k, v)
    g = cfg.num_q_heads // cfg.num_kv_heads
    kf, vf = kk.float().repeat_interleave(g, 1), vv.float().repeat_interleave(g, 1)
    s = torch.einsum("thd,nhd->htn", q.float(), kf) * cfg.head_dim ** -0.5
    n = kk.shape[0]
    mask = torch.arange(n, device=x.device)[None, :] <= positions[:, None]
    s = s.masked_fill(~mask[None], float("-inf"))
    o = torch.einsum("htn,nhd->thd", s.softmax(-1), vf).to(x.dtype).reshape(T, cfg.q_size)
    return F.linear(o, lw.o)


class ReferenceModel:
    def __init__(self, cfg: ModelConfig, attn: AttentionWeights, ffn: list[FfnLayerWeights]):
        self.cfg, self.attn, self.ffn = cfg, attn, ffn

    def new_cache(self) -> KvCacheRef:
        return KvCacheRef(self.cfg)

    def attention_half(self, layer: int, resid: torch.Tensor, ffn_out: torch.Tensor | None,
                       positions: torch.Tensor, cache: KvCacheRef) -> tuple[torch.Tensor, torch.Tensor]:
        """Adds the previous layer's FFN output, runs attention, returns (residual, FFN input)."""
        cfg, lw = self.cfg, self.attn.layers[layer]
        if ffn_out is not None:
            resid = resid + ffn_out
        x = rmsnorm(resid, lw.input_norm, cfg.rms_norm_eps)
        resid = resid + attention_core(cfg, lw, x, positions, cache, layer)
        return resid, rmsnorm(resid, lw.post_attn_norm, cfg.rms_norm_eps)

    def logits(self, resid: torch.Tensor, ffn_out: torch.Tensor) -> torch.Tensor:
        h = rmsnorm(resid + ffn_out, self.attn.final_norm, self.cfg.rms_norm_eps)
        return F.linear(h, self.attn.lm_head)

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, cache: KvCacheRef, ffn=None) -> torch.Tensor:
        """One sequence; ``ffn(layer, x)`` overrides the FFN (used by disaggregated roles)."""
        resid = self.attn.embed[ids.long()]
        y = None
        for l in range(self.cfg.num_layers):
            resid, x = self.attention_half(l, resid, y, positions, cache)
            y = ffn(l, x) if ffn is not None else ffn_forward(x, self.ffn[l], self.cfg)
        return self.logits(resid, y)

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int, ffn=None) -> tuple[list[int], torch.Tensor]:
        """Greedy decoding; returns generated ids and the logits of every generated position."""
        cache = self.new_cache()
        dev = prompt.device
        logits = self.forward(prompt, torch.arange(prompt.numel(), device=dev), cache, ffn)[-1:]
        out, all_logits = [], []
        for i in range(new_tokens):
            all_logits.append(logits[-1])
            nxt = int(logits[-1].argmax())
            out.append(nxt)
            if i + 1 == new_tokens:
                break
            pos = torch.tensor([prompt.numel() + i], device=dev)
            logits = self.forward(torch.tensor([nxt], device=dev), pos, cache, ffn)
        return out, torch.stack(all_logits)
