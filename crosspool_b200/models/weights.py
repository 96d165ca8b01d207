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

FFN_KEY = re.compile(r"^model\.layers\.(\d+)\.mlp\.")


def _dtype(cfg: ModelConfig, override: torch.dtype | None) -> torch.dtype:
    if override is not None:
        return override
    return {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[cfg.dtype]


@dataclass
class AttnLayerWeights:
    input_norm: torch.Tensor        # [hidden]
    post_attn_norm: torch.Tensor    # [hidden]
    qkv: torch.Tensor               # [(q + 2kv) * d, hidden]
    o: torch.Tensor                 # [hidden, q * d]
    q_norm: torch.Tensor | None     # [d]
    k_norm: torch.Tensor | None
    qkv_bias: torch.Tensor | None = None


@dataclass
class AttentionWeights:
    embed: torch.Tensor             # [vocab, hidden]
    layers: list[AttnLayerWeights]
    final_norm: torch.Tensor
    lm_head: torch.Tensor           # [vocab, hidden] (aliases embed when tied)


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
    """True for tensors the attention side loads: everything except ``model.layers.N.mlp.*``."""
    return FFN_KEY.match(key) is None


def load_attention_from_safetensors(cfg: ModelConfig, model_dir: str | Path, device="cpu",
                                    dtype: torch.dtype | None = None) -> AttentionWeights:
    from ..engine.checkpoint import read_checkpoint_key_view, open_tensor

    dt = _dtype(cfg, dtype)
    view = read_checkpoint_key_view(model_dir)

    def get(key: str) -> torch.Tensor:
        assert attention_keys_filter(key)
        return open_tensor(view, key).to(dtype=dt, device=device)

    def opt(key: str) -> torch.Tensor | None:
        return get(key) if key in view.key_to_file else None

    layers = []
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        qkv = torch.cat([get(p + f"self_attn.{n}_proj.weight") for n in "qkv"], 0)
        bias = None
        if p + "self_attn.q_proj.bias" in view.key_to_file:
            bias = torch.cat([get(p + f"self_attn.{n}_proj.bias") for n in "qkv"], 0).float()
        layers.append(AttnLayerWeights(
            input_norm=get(p + "input_layernorm.weight"),
            post_attn_norm=get(p + "post_attention_layernorm.weight"),
            qkv=qkv, o=get(p + "self_attn.o_proj.weight"),
            q_norm=opt(p + "self_attn.q_norm.weight"), k_norm=opt(p + "self_attn.k_norm.weight"), qkv_bias=bias))
    embed = get("model.embed_tokens.weight")
    lm = opt("lm_head.weight")
    return AttentionWeights(embed, layers, get("model.norm.weight"), lm if lm is not None else embed)
