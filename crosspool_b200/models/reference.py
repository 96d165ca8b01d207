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

import math

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


def layernorm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, eps: float) -> torch.Tensor:
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    n = (xf - mu) * torch.rsqrt((xf - mu).pow(2).mean(-1, keepdim=True) + eps)
    y = n.to(x.dtype) * w
    return y + b if b is not None else y


def block_norm(cfg: ModelConfig, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    """The decoder's normalisation: RMSNorm, or for ``cfg.norm == "layernorm"`` mean-centred with a bias."""
    return layernorm(x, w, b, cfg.rms_norm_eps) if cfg.norm == "layernorm" else rmsnorm(x, w, cfg.rms_norm_eps)


def rope_frequencies(cfg: ModelConfig, dim: int, device=None) -> tuple[torch.Tensor, float]:
    """Inverse frequencies of a ``dim``-wide rotary embedding and the factor its cos / sin are multiplied by.
    Without scaling: ``theta ** (-2i / dim)`` and 1. With YaRN (``extra["rope_scaling"]``): high-frequency pairs keep
    their frequency, low-frequency pairs are divided by ``factor``, with a linear ramp between the pairs that make
    ``beta_fast`` and ``beta_slow`` turns over the original context; the factor is ``0.1 ln(factor) + 1`` unless given."""
    pos = cfg.rope_theta ** (torch.arange(0, dim, 2, device=device, dtype=torch.float32) / dim)
    sc = cfg.extra.get("rope_scaling")
    if not sc:
        return 1.0 / pos, 1.0
    if sc["rope_type"] != "yarn":
        raise ValueError(f"rotary scaling {sc['rope_type']!r} is not supported")
    original = sc["original_max_position_embeddings"]
    factor = sc.get("factor") or cfg.max_position_embeddings / original

    def mscale(scale, m=1.0):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    att = sc.get("attention_factor")
    if att is None:
        m, m_all = sc.get("mscale"), sc.get("mscale_all_dim")
        att = mscale(factor, m) / mscale(factor, m_all) if m and m_all else mscale(factor)

    def pair_index(turns):   # the (fractional) pair whose wavelength fits `turns` times into the original context
        return dim * math.log(original / (turns * 2 * math.pi)) / (2 * math.log(cfg.rope_theta))

    low, high = pair_index(sc.get("beta_fast") or 32), pair_index(sc.get("beta_slow") or 1)
    if sc.get("truncate", True):
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, device=device, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
    inv = (1.0 / (factor * pos)) * ramp + (1.0 / pos) * (1 - ramp)
    return inv, float(att)


def rope_general(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, factor: float = 1.0,
                 interleaved: bool = False) -> torch.Tensor:
    """x ``[T, heads, d]``. ``interleaved``: pairs are ``(x[2i], x[2i+1])`` (DeepSeek-V2, GLM-4-MoE-Lite), else
    ``(x[i], x[i + d/2])``."""
    ang = positions.float()[:, None] * inv_freq[None, :]
    cos, sin = (ang.cos() * factor)[:, None, :], (ang.sin() * factor)[:, None, :]
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        return torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2).to(x.dtype)
    d = x.shape[-1]
    a, b = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(x.dtype)


def masked_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor, scale: float,
                             window: int = 0, sinks: torch.Tensor | None = None) -> torch.Tensor:
    """q ``[T, H, dq]``, k ``[N, H, dq]``, v ``[N, H, dv]`` (key ``n`` sits at position ``n``) -> ``[T, H, dv]``.
    Causal; ``window`` > 0 hides keys further back than ``window - 1``; ``sinks`` ``[H]`` adds one logit per head to
    the softmax denominator only."""
    n = k.shape[0]
    s = torch.einsum("thd,nhd->htn", q.float(), k.float()) * scale
    keys = torch.arange(n, device=q.device)[None, :]
    mask = keys <= positions[:, None]
    if window:
        mask &= keys > positions[:, None] - window
    s = s.masked_fill(~mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float()[:, None, None].expand(-1, s.shape[1], 1)], -1)
    p = s.softmax(-1)
    if sinks is not None:
        p = p[..., :-1]
    return torch.einsum("htn,nhd->thd", p, v.float())


def _latent_qkv(cfg: ModelConfig, lw: AttnLayerWeights, x: torch.Tensor, positions: torch.Tensor):
    """Latent attention in its expanded form: per-head keys ``[nope | rope]`` and values from the latent."""
    m, e, T, H = cfg.mla, lw.extra, x.shape[0], cfg.num_q_heads
    if m.q_lora_rank:
        qa = F.linear(x, e["q_a"], e["q_a_bias"].to(x.dtype) if "q_a_bias" in e else None)
        q = F.linear(rmsnorm(qa, e["q_a_norm"], cfg.rms_norm_eps), e["q_b"])
    else:
        q = F.linear(x, e["q"])
    q = q.view(T, H, m.qk_head_dim)
    q_nope, q_rope = q.split([m.qk_nope_head_dim, m.qk_rope_head_dim], -1)
    kv = F.linear(x, e["kv_a"], e["kv_a_bias"].to(x.dtype) if "kv_a_bias" in e else None)
    latent, k_rope = kv.split([m.kv_lora_rank, m.qk_rope_head_dim], -1)
    expanded = F.linear(rmsnorm(latent, e["kv_a_norm"], cfg.rms_norm_eps), e["kv_b"]).view(T, H, m.qk_nope_head_dim + m.v_head_dim)
    k_nope, v = expanded.split([m.qk_nope_head_dim, m.v_head_dim], -1)
    inv, factor = rope_frequencies(cfg, m.qk_rope_head_dim, x.device)
    inter = bool(cfg.extra.get("rope_interleave", True))
    q_rope = rope_general(q_rope, positions, inv, factor, inter)
    k_rope = rope_general(k_rope.view(T, 1, m.qk_rope_head_dim), positions, inv, factor, inter).expand(T, H, -1)
    return torch.cat([q_nope, q_rope], -1), torch.cat([k_nope, k_rope], -1), v


def attention_scale(cfg: ModelConfig) -> float:
    if cfg.mla is None:
        return cfg.head_dim ** -0.5
    scale = cfg.mla.qk_head_dim ** -0.5
    sc = cfg.extra.get("rope_scaling")
    if sc and sc.get("mscale_all_dim"):
        # Latent-attention families fold the YaRN magnitude correction into the softmax scale (the original DeepSeek-V2
        # model code and serving engines do; the transformers port of DeepSeek-V2 leaves it out, its GLM port has it).
        f = sc["factor"]
        m = 1.0 if f <= 1 else 0.1 * sc["mscale_all_dim"] * math.log(f) + 1.0
        scale *= m * m
    return scale


def attention_core(cfg: ModelConfig, lw: AttnLayerWeights, x: torch.Tensor, positions: torch.Tensor,
                   cache: KvCacheRef, layer: int) -> torch.Tensor:
    """x ``[T, hidden]`` (already input-normalised) -> attention output projected by ``o``. Grouped-query attention
    with rotary or learned positions, optional per-head q/k norms, biases, sliding windows and sinks; or latent
    attention (``cfg.mla``)."""
    T = x.shape[0]
    if cfg.mla is not None:
        q, k, v = _latent_qkv(cfg, lw, x, positions)
    else:
        qkv = F.linear(x, lw.qkv, lw.qkv_bias.to(x.dtype) if lw.qkv_bias is not None else None)
        q, k, v = qkv.split([cfg.q_size, cfg.kv_size, cfg.kv_size], -1)
        q = q.view(T, cfg.num_q_heads, cfg.head_dim)
        k = k.view(T, cfg.num_kv_heads, cfg.head_dim)
        v = v.view(T, cfg.num_kv_heads, cfg.head_dim)
        if lw.q_norm is not None:
            q, k = rmsnorm(q, lw.q_norm, cfg.rms_norm_eps), rmsnorm(k, lw.k_norm, cfg.rms_norm_eps)
        if cfg.positions == "rope":
            if cfg.extra.get("rope_scaling"):
                inv, factor = rope_frequencies(cfg, cfg.head_dim, x.device)
                q, k = rope_general(q, positions, inv, factor), rope_general(k, positions, inv, factor)
            else:
                q, k = rope(q, positions, cfg.rope_theta), rope(k, positions, cfg.rope_theta)
    kk, vv = cache.append(layer, k, v)
    g = cfg.num_q_heads // kk.shape[1]
    kf, vf = (kk.repeat_interleave(g, 1), vv.repeat_interleave(g, 1)) if g > 1 else (kk, vv)
    o = masked_softmax_attention(q, kf, vf, positions, attention_scale(cfg), cfg.layer_window(layer), lw.extra.get("sinks"))
    o = o.to(x.dtype).reshape(T, -1)
    return F.linear(o, lw.o, lw.extra["o_bias"].to(x.dtype) if "o_bias" in lw.extra else None)


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
        x = block_norm(cfg, resid, lw.input_norm, lw.extra.get("input_norm_bias"))
        resid = resid + attention_core(cfg, lw, x, positions, cache, layer)
        return resid, block_norm(cfg, resid, lw.post_attn_norm, lw.extra.get("post_attn_norm_bias"))

    def logits(self, resid: torch.Tensor, ffn_out: torch.Tensor) -> torch.Tensor:
        h = block_norm(self.cfg, resid + ffn_out, self.attn.final_norm, self.attn.extra.get("final_norm_bias"))
        return F.linear(h, self.attn.lm_head)

    def embed(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        h = self.attn.embed[ids.long()]
        if self.cfg.positions == "learned":      # OPT's table starts two rows in
            h = h + self.attn.extra["positions"][positions.long() + 2]
        return h

    def forward(self, ids: torch.Tensor, positions: torch.Tensor, cache: KvCacheRef, ffn=None) -> torch.Tensor:
        """One sequence; ``ffn(layer, x)`` overrides the FFN (used by disaggregated roles)."""
        resid = self.embed(ids, positions)
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
