"""Model weights split the way the deployment splits the model.

``AttentionWeights`` holds everything the attention devices keep (embedding, fused QKV, output
projection, norms, LM head); ``FfnLayerWeights`` holds one decoder layer's MLP or MoE tensors, the
only part FFN devices ever load. Random initialisation is N(0, 0.02) from a seed (benchmarks and
tests use it; there are no checkpoints on the build machines); Hugging Face safetensors
checkpoints load through :func:`load_attention_from_safetensors` and
:mod:`crosspool_b200.engine.loader` with the FFN tensors filtered out of the attention side, like
the reference's ``filter_decoder_ffn_weights`` (src/xpool/integrations/sglang/adapter.py:33-45).
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .config import ModelConfig
from ..utils.dtype import decode_dtype

FFN_KEY = re.compile(r"^model\.layers\.(\d+)\.mlp\.")
OPT_FFN_KEY = re.compile(r"^model\.decoder\.layers\.(\d+)\.fc[12]\.")


def _dtype(cfg: ModelConfig, override: torch.dtype | None) -> torch.dtype:
    if override is not None:
        return override
    return decode_dtype(cfg.dtype)


@dataclass
class AttnLayerWeights:
    input_norm: torch.Tensor        # [hidden]
    post_attn_norm: torch.Tensor    # [hidden]
    qkv: torch.Tensor               # [(q + 2kv) * d, hidden]
    o: torch.Tensor                 # [hidden, q * d]
    q_norm: torch.Tensor | None     # [d]
    k_norm: torch.Tensor | None
    qkv_bias: torch.Tensor | None = None
    # Other attention forms (oracle / CPU deployment): "input_norm_bias", "post_attn_norm_bias" (LayerNorm), "o_bias",
    # "sinks" [q heads]; latent attention leaves ``qkv`` None and holds "q" or ("q_a", "q_a_norm", "q_b"), "kv_a",
    # "kv_a_norm", "kv_b".
    extra: dict = field(default_factory=dict)


@dataclass
class AttentionWeights:
    embed: torch.Tensor             # [vocab, hidden]
    layers: list[AttnLayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor           # [vocab, hidden] (aliases embed when tied)
    extra: dict = field(default_factory=dict)   # "positions" [max + offset, hidden], "final_norm_bias" (OPT)


@dataclass
class FfnLayerWeights:
    """Dense: ``gate_up`` [2I, hidden] (gate rows then up rows) and ``down`` [hidden, I].
    MoE: ``router`` [E, hidden]; ``gate_up`` [E, 2I, hidden]; ``down`` [E, hidden, I]."""

    gate_up: torch.Tensor
    down: torch.Tensor
    router: torch.Tensor | None = None
    gate_up_bias: torch.Tensor | None = None
    down_bias: torch.Tensor | None = None
    shared_gate_up: torch.Tensor | None = None
    shared_down: torch.Tensor | None = None
    extra: dict = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.router is not None


def _generator(seed: int, device) -> torch.Generator:
    """CPU generator for CPU tensors (bit-identical everywhere); device generator on CUDA, where
    multi-gigabyte benchmark models are initialised in place instead of crossing PCIe."""
    dev = torch.device(device)
    g = torch.Generator(device=dev if dev.type == "cuda" else "cpu")
    g.manual_seed(seed)
    return g


def _randn(gen: torch.Generator, shape, dtype, device, std=0.02) -> torch.Tensor:
    if gen.device.type == "cuda":
        t = torch.empty(shape, dtype=dtype, device=gen.device)
        t.normal_(0.0, std, generator=gen)
        return t
    t = torch.empty(shape, dtype=torch.float32)
    t.normal_(0.0, std, generator=gen)
    return t.to(dtype=dtype, device=device)


def random_attention_weights(cfg: ModelConfig, seed: int = 0, device="cpu", dtype: torch.dtype | None = None
                             ) -> AttentionWeights:
    dt = _dtype(cfg, dtype)
    gen = _generator(seed * 1000003 + 1, device)
    embed = _randn(gen, (cfg.vocab_size, cfg.hidden_size), dt, device)
    layers = []
    if not cfg.gpu_attention_supported:
        return _random_attention_other_forms(cfg, gen, embed, dt, device)
    for _ in range(cfg.num_layers):
        layers.append(AttnLayerWeights(
            input_norm=torch.ones(cfg.hidden_size, dtype=dt, device=device),
            post_attn_norm=torch.ones(cfg.hidden_size, dtype=dt, device=device),
            qkv=_randn(gen, (cfg.q_size + 2 * cfg.kv_size, cfg.hidden_size), dt, device),
            o=_randn(gen, (cfg.hidden_size, cfg.q_size), dt, device),
            q_norm=torch.ones(cfg.head_dim, dtype=dt, device=device) if cfg.qk_norm else None,
            k_norm=torch.ones(cfg.head_dim, dtype=dt, device=device) if cfg.qk_norm else None,
            qkv_bias=(_randn(gen, (cfg.q_size + 2 * cfg.kv_size,), torch.float32, device) * 5.0) if cfg.attention_bias else None,
        ))
    final_norm = torch.ones(cfg.hidden_size, dtype=dt, device=device)
    lm_head = embed if cfg.tie_word_embeddings else _randn(gen, (cfg.vocab_size, cfg.hidden_size), dt, device)
    return AttentionWeights(embed, layers, final_norm, lm_head)


def _random_attention_other_forms(cfg: ModelConfig, gen, embed, dt, device) -> AttentionWeights:
    """Random tensors for the attention forms only the oracle runs (LayerNorm + learned positions, sinks, windows,
    latent attention); norm weights near one and small biases so every term matters."""
    h = cfg.hidden_size
    layernorm = cfg.norm == "layernorm"

    def norm_w(n):
        return (1 + _randn(gen, (n,), torch.float32, device, std=0.1)).to(dt)

    layers = []
    for _ in range(cfg.num_layers):
        extra: dict = {}
        if layernorm:
            extra["input_norm_bias"] = _randn(gen, (h,), dt, device)
            extra["post_attn_norm_bias"] = _randn(gen, (h,), dt, device)
        if cfg.attention_sinks:
            extra["sinks"] = _randn(gen, (cfg.num_q_heads,), torch.float32, device, std=1.0)
        qkv = qkv_bias = None
        if cfg.mla is not None:
            m = cfg.mla
            if m.q_lora_rank:
                extra["q_a"] = _randn(gen, (m.q_lora_rank, h), dt, device, std=0.08)
                extra["q_a_norm"] = norm_w(m.q_lora_rank)
                extra["q_b"] = _randn(gen, (cfg.num_q_heads * m.qk_head_dim, m.q_lora_rank), dt, device, std=0.08)
            else:
                extra["q"] = _randn(gen, (cfg.num_q_heads * m.qk_head_dim, h), dt, device, std=0.08)
            extra["kv_a"] = _randn(gen, (m.kv_lora_rank + m.qk_rope_head_dim, h), dt, device, std=0.08)
            extra["kv_a_norm"] = norm_w(m.kv_lora_rank)
            extra["kv_b"] = _randn(gen, (cfg.num_q_heads * (m.qk_nope_head_dim + m.v_head_dim), m.kv_lora_rank), dt, device, std=0.08)
            o_in = cfg.num_q_heads * m.v_head_dim
        else:
            qkv = _randn(gen, (cfg.q_size + 2 * cfg.kv_size, h), dt, device, std=0.08)
            if cfg.attention_bias:
                qkv_bias = _randn(gen, (cfg.q_size + 2 * cfg.kv_size,), torch.float32, device)
            o_in = cfg.q_size
        if cfg.o_bias:
            extra["o_bias"] = _randn(gen, (h,), torch.float32, device)
        layers.append(AttnLayerWeights(input_norm=norm_w(h), post_attn_norm=norm_w(h), qkv=qkv,
                                       o=_randn(gen, (h, o_in), dt, device, std=0.08), q_norm=None, k_norm=None,
                                       qkv_bias=qkv_bias, extra=extra))
    top: dict = {}
    if cfg.positions == "learned":
        top["positions"] = _randn(gen, (cfg.max_position_embeddings + 2, h), dt, device)
    if layernorm:
        top["final_norm_bias"] = _randn(gen, (h,), dt, device)
    lm_head = embed if cfg.tie_word_embeddings else _randn(gen, (cfg.vocab_size, h), dt, device)
    return AttentionWeights(embed, layers, norm_w(h), lm_head, extra=top)


def random_ffn_layer(cfg: ModelConfig, layer: int, seed: int = 0, device="cpu", dtype: torch.dtype | None = None,
                     tp_rank: int = 0, tp_size: int = 1, expert_range: tuple[int, int] | None = None
                     ) -> FfnLayerWeights:
    """One layer's FFN tensors, or the ``tp_rank`` shard of them.

    True tensor parallelism as in the reference (src/xpool/runtime/ffnagent/preparation.py:164-334):
    gate/up are split by output rows, down by input columns, for every expert alike. The full
    tensors are generated from the seed first so that shards of different ranks agree.
    ``expert_range`` keeps only experts ``[lo, hi)`` (expert parallelism).
    """
    dt = _dtype(cfg, dtype)
    gen = _generator(seed * 1000003 + 7919 * (layer + 1), device)
    h = cfg.hidden_size

    def shard_rows(t: torch.Tensor, inter: int) -> torch.Tensor:  # t [..., 2*inter, h]
        loc = inter // tp_size
        g = t[..., tp_rank * loc:(tp_rank + 1) * loc, :]
        u = t[..., inter + tp_rank * loc: inter + (tp_rank + 1) * loc, :]
        return torch.cat([g, u], dim=-2).contiguous()

    def shard_cols(t: torch.Tensor, inter: int) -> torch.Tensor:  # t [..., h, inter]
        loc = inter // tp_size
        return t[..., tp_rank * loc:(tp_rank + 1) * loc].contiguous()

    if cfg.layer_is_moe(layer):
        e, inter = cfg.num_experts, cfg.moe_intermediate_size
        router = _randn(gen, (e, h), dt, device)
        gate_up = _randn(gen, (e, 2 * inter, h), dt, device)
        down = _randn(gen, (e, h, inter), dt, device)
        if tp_size > 1:
            gate_up, down = shard_rows(gate_up, inter), shard_cols(down, inter)
        shared_gu = shared_dn = None
        if cfg.num_shared_experts > 0:
            # the shared experts act as one dense gated FFN of width num_shared * moe_intermediate
            si = cfg.num_shared_experts * inter
            shared_gu = _randn(gen, (2 * si, h), dt, device)
            shared_dn = _randn(gen, (h, si), dt, device)
            if tp_size > 1:
                shared_gu, shared_dn = shard_rows(shared_gu, si), shard_cols(shared_dn, si)
        if expert_range is not None:
            lo, hi = expert_range
            gate_up, down = gate_up[lo:hi].contiguous(), down[lo:hi].contiguous()
            if lo != 0:
                shared_gu = shared_dn = None   # the rank owning expert 0 adds the shared experts
        w = FfnLayerWeights(gate_up.to(device), down.to(device), router=router.to(device), shared_gate_up=shared_gu,
                            shared_down=shared_dn)
        if expert_range is not None:
            w.extra["experts"] = tuple(expert_range)
        if cfg.router_precision != "payload":
            w.extra["router_precision"] = cfg.router_precision
            if cfg.router_precision == "fp32":   # fp32 router weights; the payload copy is their rounding
                w.extra["router_fp32"] = (w.router.float() + _randn(gen, (e, h), torch.float32, device).to(device) * 2.0 ** -10
                                          ).contiguous()
                w.router = w.extra["router_fp32"].to(dt)
        return w
    inter = cfg.intermediate_size
    gate_up = _randn(gen, (2 * inter, h), dt, device)
    down = _randn(gen, (h, inter), dt, device)
    if tp_size > 1:
        gate_up, down = shard_rows(gate_up, inter), shard_cols(down, inter)
    return FfnLayerWeights(gate_up.to(device), down.to(device))


def quantize_ffn_layer_fp8(w: FfnLayerWeights) -> FfnLayerWeights:
    """Attaches block-scaled e4m3 copies of a dense layer's projections (128 x 128 weight blocks) under
    ``w.extra["fp8"]``; ports that find them run the fp8 GEMM path."""
    from ..quantization import Fp8Block

    if w.is_moe:
        raise NotImplementedError("fp8 expert weights are not supported")
    fmt = Fp8Block()
    gu, dn = fmt.quantize(w.gate_up), fmt.quantize(w.down)
    w.extra["fp8"] = {"gate_up": gu["weight"], "gate_up_scale": gu["scale"].contiguous(), "down": dn["weight"],
                      "down_scale": dn["scale"].contiguous()}
    return w


def random_ffn_weights(cfg: ModelConfig, seed: int = 0, device="cpu", dtype: torch.dtype | None = None,
                       tp_rank: int = 0, tp_size: int = 1) -> list[FfnLayerWeights]:
    return [random_ffn_layer(cfg, l, seed, device, dtype, tp_rank, tp_size) for l in range(cfg.num_layers)]


# ------------------------------------------------------------------ safetensors (attention side)

def attention_keys_filter(key: str) -> bool:
    """True for tensors the attention side loads: everything except the decoder FFNs (``model.layers.N.mlp.*``; for
    OPT ``model.decoder.layers.N.fc1/fc2.*``)."""
    return FFN_KEY.match(key) is None and OPT_FFN_KEY.match(key) is None


def load_attention_from_safetensors(cfg: ModelConfig, model_dir: str | Path, device="cpu",
                                    dtype: torch.dtype | None = None) -> AttentionWeights:
    from ..engine.checkpoint import read_checkpoint_key_view, open_tensor

    dt = _dtype(cfg, dtype)
    view = read_checkpoint_key_view(model_dir)

    def get(key: str) -> torch.Tensor:
        assert attention_keys_filter(key)
        t = open_tensor(view, key)
        if t.dtype == torch.float8_e4m3fn:
            # a block-scaled fp8 checkpoint quantises the attention projections too: codes x per-block scale
            scale_key = key + "_scale_inv"
            if scale_key not in view.key_to_file:
                raise ValueError(f"{key} holds e4m3 codes but the checkpoint has no {scale_key}")
            from ..quantization import Fp8Block

            n, k = t.shape
            pad = torch.zeros((n + 127) // 128 * 128, (k + 127) // 128 * 128, dtype=torch.uint8)
            pad[:n, :k] = t.view(torch.uint8)
            full = Fp8Block().dequantize({"weight": pad.view(torch.float8_e4m3fn), "scale": open_tensor(view, scale_key).float()}, torch.float32)
            return full[:n, :k].to(dtype=dt, device=device)
        return t.to(dtype=dt, device=device)

    def opt(key: str) -> torch.Tensor | None:
        return get(key) if key in view.key_to_file else None

    if cfg.positions == "learned":
        return _load_opt_attention(cfg, get, opt)
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        extra: dict = {}
        qkv = bias = None
        if cfg.mla is not None:
            if cfg.mla.q_lora_rank:
                extra.update(q_a=get(a + "q_a_proj.weight"), q_a_norm=get(a + "q_a_layernorm.weight"), q_b=get(a + "q_b_proj.weight"))
            else:
                extra["q"] = get(a + "q_proj.weight")
            extra.update(kv_a=get(a + "kv_a_proj_with_mqa.weight"), kv_a_norm=get(a + "kv_a_layernorm.weight"),
                         kv_b=get(a + "kv_b_proj.weight"))
            for name, key in (("q_a_bias", "q_a_proj.bias"), ("kv_a_bias", "kv_a_proj_with_mqa.bias")):
                if a + key in view.key_to_file:
                    extra[name] = get(a + key).float()
        else:
            qkv = torch.cat([get(a + f"{n}_proj.weight") for n in "qkv"], 0)
            if a + "q_proj.bias" in view.key_to_file:
                bias = torch.cat([get(a + f"{n}_proj.bias") for n in "qkv"], 0).float()
        if a + "o_proj.bias" in view.key_to_file:
            extra["o_bias"] = get(a + "o_proj.bias").float()
        if a + "sinks" in view.key_to_file:
            extra["sinks"] = get(a + "sinks").float()
        layers.append(AttnLayerWeights(
            input_norm=get(p + "input_layernorm.weight"),
            post_attn_norm=get(p + "post_attention_layernorm.weight"),
            qkv=qkv, o=get(a + "o_proj.weight"),
            q_norm=opt(a + "q_norm.weight"), k_norm=opt(a + "k_norm.weight"), qkv_bias=bias, extra=extra))
    embed = get("model.embed_tokens.weight")
    lm = opt("lm_head.weight")
    return AttentionWeights(embed, layers, get("model.norm.weight"), lm if lm is not None else embed)


def _load_opt_attention(cfg: ModelConfig, get, opt) -> AttentionWeights:
    """OPT: ``model.decoder.*`` names, LayerNorm with biases, biased projections, a learned position table."""
    layers = []
    for i in range(cfg.num_layers):
        p = f"model.decoder.layers.{i}."
        a = p + "self_attn."
        bias = None
        if opt(a + "q_proj.bias") is not None:
            bias = torch.cat([get(a + f"{n}_proj.bias") for n in "qkv"], 0).float()
        extra = {"input_norm_bias": get(p + "self_attn_layer_norm.bias"), "post_attn_norm_bias": get(p + "final_layer_norm.bias")}
        ob = opt(a + "out_proj.bias")
        if ob is not None:
            extra["o_bias"] = ob.float()
        layers.append(AttnLayerWeights(
            input_norm=get(p + "self_attn_layer_norm.weight"), post_attn_norm=get(p + "final_layer_norm.weight"),
            qkv=torch.cat([get(a + f"{n}_proj.weight") for n in "qkv"], 0), o=get(a + "out_proj.weight"),
            q_norm=None, k_norm=None, qkv_bias=bias, extra=extra))
    embed = get("model.decoder.embed_tokens.weight")
    lm = opt("lm_head.weight")
    top = {"positions": get("model.decoder.embed_positions.weight"), "final_norm_bias": get("model.decoder.final_layer_norm.bias")}
    return AttentionWeights(embed, layers, get("model.decoder.final_layer_norm.weight"), lm if lm is not None else embed, extra=top)
