"""Model qualification: does the FFN tier compute what a model's checkpoint says?

For one architecture (a Hugging Face ``config.json``, usually shrunk by :func:`tiny_config`) the tool

1. compiles the FFN description (``models/adapters.py``) and synthesises a checkpoint that holds exactly the tensors
   the description names (per-expert or stacked experts, packed or separate gate/up, interleaved rows, biases, MXFP4
   blocks and scales, shared experts, correction bias);
2. checks coverage (``engine/checkpoint.py``) and loads every layer kind through the production loader: whole, as
   tensor-parallel shards and as expert-parallel ranges;
3. evaluates the layer twice in fp32: through the loader and the repository's oracle (``models/reference.py``,
   what every kernel test compares against), and *directly from the raw checkpoint tensors and the description*
   with code that shares nothing with either (:func:`direct_ffn`);
4. requires the two to agree within the reference's FFN tolerances (atol 0.02, rtol 0.02, normalised RMSE 0.01,
   max scaled error 0.10), the shard sums to equal the whole, and the routing decisions to be identical.

On a CUDA device the same inputs also go through the native kernels (``ops/gemm.py``, ``ops/moe.py``).

The reference qualifies its operators the same way, with deterministic structures and independent numerical
references (src/xpool-dev/xtest/harness/native/ffn/qualification.py:36-502; tolerances
src/xpool-dev/xtest/harness/support/ffn.py:20-28).

    python -m crosspool_b200.devtools.qualification --arch all
    python -m crosspool_b200.devtools.qualification --config /path/to/config.json --shrink
    python -m crosspool_b200.devtools.qualification --arch all --against hf     # the transformers model as the other side
    python -m crosspool_b200.devtools.qualification --arch all --against served # a CPU deployment per architecture, over HTTP
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from ..ffn import (ActivationKind, DenseFfnSpec, FfnModelSpec, GateUpOrder, MoeFfnSpec, RouterAlgorithm,
                   RouterProjectionPrecision, TopKWeightRounding)

ATOL, RTOL, NRMSE_MAX, SCALED_MAX = 0.02, 0.02, 0.01, 0.10

_BASE = {"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
         "torch_dtype": "bfloat16"}
TINY_CONFIGS: dict[str, dict] = {
    "Qwen2ForCausalLM": {**_BASE, "intermediate_size": 128, "hidden_act": "silu"},
    "Qwen3ForCausalLM": {**_BASE, "intermediate_size": 128, "hidden_act": "silu", "head_dim": 16},
    "LlamaForCausalLM": {**_BASE, "intermediate_size": 128, "hidden_act": "silu", "mlp_bias": True},
    "OPTForCausalLM": {**_BASE, "ffn_dim": 128, "activation_function": "relu", "max_position_embeddings": 128},
    "Qwen3MoeForCausalLM": {**_BASE, "intermediate_size": 128, "moe_intermediate_size": 64, "num_experts": 8,
                            "num_experts_per_tok": 2, "norm_topk_prob": True, "head_dim": 16},
    "DeepseekV2ForCausalLM": {**_BASE, "intermediate_size": 128, "moe_intermediate_size": 64, "n_routed_experts": 8,
                              "num_experts_per_tok": 2, "first_k_dense_replace": 1, "n_shared_experts": 2,
                              "routed_scaling_factor": 2.0, "norm_topk_prob": False},
    "Glm4MoeLiteForCausalLM": {**_BASE, "intermediate_size": 128, "moe_intermediate_size": 64, "n_routed_experts": 8,
                               "num_experts_per_tok": 2, "first_k_dense_replace": 1, "n_shared_experts": 1,
                               "routed_scaling_factor": 1.5, "norm_topk_prob": True, "scoring_func": "sigmoid", "rms_norm_eps": 1e-6},
    "GptOssForCausalLM": {**_BASE, "intermediate_size": 64, "num_local_experts": 4, "num_experts_per_tok": 2,
                          "swiglu_limit": 7.0},
    "GptOssForCausalLM+mxfp4": {**_BASE, "intermediate_size": 64, "num_local_experts": 4, "num_experts_per_tok": 2,
                                "swiglu_limit": 7.0, "quantization_config": {"quant_method": "mxfp4"}},
}


def tiny_config(arch: str) -> dict:
    """A small configuration of ``arch`` (``"GptOssForCausalLM+mxfp4"`` selects the quantised variant)."""
    if arch not in TINY_CONFIGS:
        raise KeyError(f"no tiny configuration for {arch!r}; known: {sorted(TINY_CONFIGS)}")
    return {"architectures": [arch.split("+")[0]], **TINY_CONFIGS[arch]}


def shrink(hf_config: dict) -> dict:
    """The architecture of a real ``config.json`` with every size replaced by the tiny one of its family."""
    arch = (hf_config.get("architectures") or ["?"])[0]
    key = arch + ("+mxfp4" if (hf_config.get("quantization_config") or {}).get("quant_method") == "mxfp4" else "")
    out = tiny_config(key)
    for k in ("hidden_act", "activation_function", "norm_topk_prob", "scoring_func", "routed_scaling_factor", "swiglu_limit",
              "mlp_bias"):
        if k in hf_config:
            out[k] = hf_config[k]
    return out


# ---------------------------------------------------------------------------------------------- synthetic checkpoint

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def _mx_decode(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """MXFP4 blocks ``[..., n/32, 16]`` (two codes per byte, low nibble first) and e8m0 scales ``[..., n/32]`` to fp32
    ``[..., n]`` through the E2M1 code book (independent of ``quantization/formats.py``)."""
    book = torch.tensor(_E2M1, dtype=torch.float32)
    b = blocks.to(torch.int64)
    codes = torch.stack((b & 15, b >> 4), dim=-1).flatten(-2)             # [..., n/32, 32]
    vals = book[codes] * torch.exp2(scales.to(torch.float32) - 127.0)[..., None]
    return vals.flatten(-2)


def synthesize_ffn_tensors(spec: FfnModelSpec, seed: int = 0, scale: float = 0.25) -> dict[str, torch.Tensor]:
    """Random tensors for every key ``spec`` names, in the layout the key's architecture stores them."""
    g = torch.Generator().manual_seed(seed)
    dt = torch.bfloat16

    def rnd(*shape, s=scale):
        return (torch.randn(*shape, generator=g) * s).to(dt)

    t: dict[str, torch.Tensor] = {}
    mx = spec.quantization == "mxfp4"
    for l in spec.layers:
        h = l.hidden_size
        if isinstance(l, DenseFfnSpec):
            ip, i = l.i_proj, l.intermediate_size
            if ip.packed is not None:
                t[ip.packed.weight_key] = rnd(2 * i, h)
                if ip.packed.bias_key:
                    t[ip.packed.bias_key] = rnd(2 * i)
            else:
                for p in (ip.gate, ip.up):
                    if p is not None:
                        t[p.weight_key] = rnd(i, h)
                        if p.bias_key:
                            t[p.bias_key] = rnd(i)
            t[l.o_proj.weight_key] = rnd(h, i)
            if l.o_proj.bias_key:
                t[l.o_proj.bias_key] = rnd(h)
            continue
        ex, e, i = l.experts, l.num_experts, l.moe_intermediate_size
        t[l.router_weight_key] = rnd(e, h, s=1.0) if l.router_precision == RouterProjectionPrecision.PAYLOAD else \
            torch.randn(e, h, generator=g)
        if l.router_bias_key:
            t[l.router_bias_key] = rnd(e)
        if l.correction_bias_key:
            t[l.correction_bias_key] = torch.randn(e, generator=g) * 0.05
        if ex.per_expert:
            for x in range(e):
                t[ex.gate_key.format(expert=x)], t[ex.up_key.format(expert=x)] = rnd(i, h), rnd(i, h)
                t[ex.down_key.format(expert=x)] = rnd(h, i)
        elif mx and ex.scales_suffix:
            from ..quantization import Mxfp4

            fmt = Mxfp4()
            for key, shape in ((ex.packed_key, (e, 2 * i, h)), (ex.down_key, (e, h, i))):
                q = fmt.quantize(torch.randn(*shape, generator=g) * scale)
                stem = key[: -len("_blocks")] if key.endswith("_blocks") else key
                t[key] = q["blocks"].reshape(*shape[:-1], shape[-1] // 32, 16)
                t[stem + ex.scales_suffix] = q["scales"]
        elif ex.input_major:         # stored for ``x @ W``: [experts, in, out]
            t[ex.packed_key], t[ex.down_key] = rnd(e, h, 2 * i), rnd(e, i, h)
        else:
            t[ex.packed_key], t[ex.down_key] = rnd(e, 2 * i, h), rnd(e, h, i)
        if ex.gate_bias_key:
            t[ex.gate_bias_key] = rnd(e, 2 * i)
        if ex.down_bias_key:
            t[ex.down_bias_key] = rnd(e, h)
        if l.num_shared_experts:
            si = l.shared_intermediate_size
            t[l.shared_gate_key], t[l.shared_up_key], t[l.shared_down_key] = rnd(si, h), rnd(si, h), rnd(h, si)
    return t


def write_ffn_checkpoint(model_dir: str | Path, hf_config: dict, tensors: dict[str, torch.Tensor], shards: int = 2) -> None:
    from safetensors.torch import save_file

    d = Path(model_dir)
    d.mkdir(parents=True, exist_ok=True)
    (d / "config.json").write_text(json.dumps(hf_config))
    keys = sorted(tensors)
    index = {}
    for s in range(shards):
        part = {k: tensors[k].contiguous() for k in keys[s::shards]}
        if not part:
            continue
        name = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, str(d / name))
        index.update({k: name for k in part})
    (d / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": index}))


# ---------------------------------------------------------------------------------------------- independent evaluation

def _act(kind: ActivationKind, g: torch.Tensor) -> torch.Tensor:
    if kind == ActivationKind.SILU:
        return g / (1.0 + torch.exp(-g))
    if kind == ActivationKind.RELU:
        return torch.where(g > 0, g, torch.zeros_like(g))
    c = 0.7978845608028654
    return 0.5 * g * (1.0 + torch.tanh(c * (g + 0.044715 * g ** 3)))    # tanh GELU


def _gate(kind: ActivationKind, gate: torch.Tensor | None, up: torch.Tensor, tr) -> torch.Tensor:
    if gate is None:
        return _act(kind, up)
    if tr.limit > 0 or tr.up_offset != 0 or tr.alpha != 1.0:
        if tr.limit > 0:
            gate, up = torch.minimum(gate, torch.tensor(tr.limit)), up.clamp(-tr.limit, tr.limit)
        return gate / (1.0 + torch.exp(-tr.alpha * gate)) * (up + tr.up_offset)
    return _act(kind, gate) * up


def _split(packed: torch.Tensor, order: GateUpOrder, dim: int = -2) -> tuple[torch.Tensor, torch.Tensor]:
    n = packed.shape[dim] // 2
    if order == GateUpOrder.INTERLEAVED:
        idx = torch.arange(0, 2 * n, 2)
        return packed.index_select(dim, idx), packed.index_select(dim, idx + 1)
    return packed.narrow(dim, 0, n), packed.narrow(dim, n, n)


def direct_routing(l: MoeFfnSpec, t: dict[str, torch.Tensor], x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k expert ids and combine weights straight from the description: payload-precision logits are rounded to
    the payload dtype, fp32 precisions are not; sigmoid routers select on score + correction bias and weigh by the
    score; weights are renormalised where the description says so and then scaled."""
    xr = x.to(torch.bfloat16)
    if l.router_precision == RouterProjectionPrecision.PAYLOAD:
        logits = (xr.float() @ t[l.router_weight_key].to(torch.bfloat16).float().t()).to(torch.bfloat16).float()
    elif l.router_precision == RouterProjectionPrecision.FP32_LOGITS:
        logits = xr.float() @ t[l.router_weight_key].to(torch.bfloat16).float().t()
    else:
        logits = xr.float() @ t[l.router_weight_key].float().t()
    if l.router_bias_key:
        logits = logits + t[l.router_bias_key].float()
    scores = torch.sigmoid(logits) if l.router_algorithm == RouterAlgorithm.SIGMOID else torch.softmax(logits, -1)
    sel = scores + t[l.correction_bias_key].float() if l.correction_bias_key else scores
    ids = sel.topk(l.top_k, dim=-1).indices
    w = scores.gather(-1, ids)
    if l.renormalize:
        w = w / w.sum(-1, keepdim=True)
    if l.topk_weight_rounding == TopKWeightRounding.LOGITS_DTYPE:
        w = w.to(torch.bfloat16).float()
    return ids, w * l.routed_scaling_factor


def direct_ffn(l: DenseFfnSpec | MoeFfnSpec, t: dict[str, torch.Tensor], x: torch.Tensor, mx: bool = False) -> torch.Tensor:
    """fp32 evaluation of one layer from the raw checkpoint tensors and its description (no loader, no oracle)."""
    xf = x.to(torch.bfloat16).float()

    def lin(v, w, b=None):
        y = v @ w.float().t()
        return y + b.float() if b is not None else y

    if isinstance(l, DenseFfnSpec):
        ip = l.i_proj
        if ip.packed is not None:
            gw, uw = _split(t[ip.packed.weight_key], ip.source_order)
            gb, ub = _split(t[ip.packed.bias_key], ip.source_order, -1) if ip.packed.bias_key else (None, None)
            gate, up = lin(xf, gw, gb), lin(xf, uw, ub)
        else:
            gate = lin(xf, t[ip.gate.weight_key], t.get(ip.gate.bias_key) if ip.gate.bias_key else None) if ip.gate else None
            up = lin(xf, t[ip.up.weight_key], t.get(ip.up.bias_key) if ip.up.bias_key else None)
        hcur = _gate(l.activation, gate, up, l.gate_transform)
        return lin(hcur, t[l.o_proj.weight_key], t.get(l.o_proj.bias_key) if l.o_proj.bias_key else None)

    ids, wts = direct_routing(l, t, x)
    ex = l.experts
    out = torch.zeros(x.shape[0], l.hidden_size)
    for e in range(l.num_experts):
        rows, slot = (ids == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        if ex.per_expert:
            gw, uw, dw = t[ex.gate_key.format(expert=e)], t[ex.up_key.format(expert=e)], t[ex.down_key.format(expert=e)]
        elif mx and ex.scales_suffix:
            stem_p = ex.packed_key[: -len("_blocks")] if ex.packed_key.endswith("_blocks") else ex.packed_key
            stem_d = ex.down_key[: -len("_blocks")] if ex.down_key.endswith("_blocks") else ex.down_key
            packed = _mx_decode(t[ex.packed_key][e], t[stem_p + ex.scales_suffix][e])
            gw, uw = _split(packed, l.source_order)
            dw = _mx_decode(t[ex.down_key][e], t[stem_d + ex.scales_suffix][e])
        elif ex.input_major:
            gw, uw = _split(t[ex.packed_key][e].t(), l.source_order)
            dw = t[ex.down_key][e].t()
        else:
            gw, uw = _split(t[ex.packed_key][e], l.source_order)
            dw = t[ex.down_key][e]
        gb = ub = db = None
        if ex.gate_bias_key:
            gb, ub = _split(t[ex.gate_bias_key][e], l.source_order, -1)
        if ex.down_bias_key:
            db = t[ex.down_bias_key][e]
        xe = xf[rows]
        hcur = _gate(l.activation, lin(xe, gw, gb), lin(xe, uw, ub), l.gate_transform)
        out.index_add_(0, rows, lin(hcur, dw, db) * wts[rows, slot, None])
    if l.num_shared_experts:
        hcur = _act(l.activation, lin(xf, t[l.shared_gate_key])) * lin(xf, t[l.shared_up_key])
        out = out + lin(hcur, t[l.shared_down_key])
    return out


# ---------------------------------------------------------------------------------------------- qualification run

@dataclass
class Check:
    name: str
    ok: bool
    detail: dict = field(default_factory=dict)


@dataclass
class Report:
    architecture: str
    quantization: str
    layers: list[str]
    checks: list[Check] = field(default_factory=list)

    @property
    def ok(self) -> bool:
        return all(c.ok for c in self.checks)

    def to_json(self) -> dict:
        return {"architecture": self.architecture, "quantization": self.quantization, "layers": self.layers, "ok": self.ok,
                "checks": [asdict(c) for c in self.checks]}


def _close(out: torch.Tensor, ref: torch.Tensor) -> tuple[bool, dict]:
    out, ref = out.float(), ref.float()
    err = (out - ref).abs()
    scale = ref.abs().max().clamp_min(1e-6)
    nrmse = (err.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-9)).item()
    elementwise = bool((err <= ATOL + RTOL * ref.abs()).all())
    scaled = (err.max() / scale).item()
    return (elementwise or (nrmse <= NRMSE_MAX and scaled <= SCALED_MAX)), {"nrmse": round(nrmse, 6), "max_scaled": round(scaled, 6),
                                                                         "elementwise": elementwise}


def qualify(hf_config: dict, workdir: str | Path | None = None, *, tp_sizes=(1, 2), ep_sizes=(1, 2), rows=(1, 7, 33),
            device: str = "cpu", seed: int = 0) -> Report:
    """Runs the battery for one configuration (see the module docstring). ``device="cuda"`` adds the native kernels."""
    from ..engine import checkpoint as ck
    from ..engine import loader
    from ..models import adapters, reference
    from ..models import config as mc

    spec = adapters.compile_ffn_spec("qualify", hf_config)
    tensors = synthesize_ffn_tensors(spec, seed)
    tmp = None
    if workdir is None:
        tmp = tempfile.TemporaryDirectory(prefix="xp-qualify-")
        workdir = tmp.name
    try:
        write_ffn_checkpoint(workdir, hf_config, tensors)
        view = ck.read_checkpoint_key_view(workdir)
        spec = adapters.compile_ffn_spec("qualify", hf_config, view.keys())
        rep = Report(spec.architecture, spec.quantization, [l.kind.value for l in spec.layers])
        try:
            ck.validate_ffn_coverage(spec, view)
            rep.checks.append(Check("coverage: the checkpoint holds exactly the FFN keys of the description", True))
        except Exception as e:
            rep.checks.append(Check("coverage", False, {"error": repr(e)}))
            return rep
        cfg = mc.from_hf_config({"num_attention_heads": 4, "vocab_size": 256, **hf_config}, "qualify")
        mx = spec.quantization == "mxfp4"
        seen: set[str] = set()
        g = torch.Generator().manual_seed(seed + 1)
        for l in spec.layers:
            if l.kind.value in seen:
                continue
            seen.add(l.kind.value)
            tag = f"layer {l.layer} ({l.kind.value})"
            whole = loader.materialize_layer_weights(spec, view, l.layer)
            for n in rows:
                x = (torch.randn(n, l.hidden_size, generator=g) * 0.5).to(torch.bfloat16)
                want = direct_ffn(l, tensors, x, mx)
                got = reference.ffn_forward(x, whole, cfg).float()
                ok, d = _close(got, want)
                rep.checks.append(Check(f"{tag}: loader + oracle equal the direct evaluation, {n} rows", ok, d))
                if isinstance(l, MoeFfnSpec):
                    ids, w = direct_routing(l, tensors, x)
                    logits = _oracle_logits(reference, x, whole)
                    rid, rw = reference.route_topk(logits, cfg.num_experts_per_tok, cfg.norm_topk_prob, cfg.router_scoring,
                                                   whole.extra.get("correction_bias"), cfg.routed_scaling_factor)
                    if whole.extra.get("round_topk_weights"):
                        rw = rw.to(torch.bfloat16)
                    same = bool((ids.sort(-1).values == rid.sort(-1).values).all())
                    wclose = bool(torch.allclose(w.sort(-1).values, rw.float().sort(-1).values, atol=1e-4, rtol=1e-3))
                    rep.checks.append(Check(f"{tag}: routing decisions and combine weights identical, {n} rows", same and wclose,
                                            {"ids_equal": same, "weights_close": wclose}))
                inter = l.intermediate_size if isinstance(l, DenseFfnSpec) else l.moe_intermediate_size
                for tp in tp_sizes:
                    if tp == 1 or inter % (tp * 16):
                        continue
                    parts = [reference.ffn_forward(x, loader.materialize_layer_weights(spec, view, l.layer, tp_rank=r, tp_size=tp),
                                                   cfg).float() for r in range(tp)]
                    ok, d = _close(sum(parts), want)
                    rep.checks.append(Check(f"{tag}: TP{tp} shard outputs sum to the whole, {n} rows", ok, d))
                if isinstance(l, MoeFfnSpec):
                    for ep in ep_sizes:
                        if ep == 1 or l.num_experts % ep:
                            continue
                        per = l.num_experts // ep
                        parts = []
                        for r in range(ep):
                            wr = loader.materialize_layer_weights(spec, view, l.layer, experts=range(r * per, (r + 1) * per))
                            if r != 0:
                                wr.shared_gate_up = wr.shared_down = None      # the rank of expert 0 adds the shared experts
                            parts.append(reference.moe_ffn(x, wr, cfg).float())   # the oracle restricts itself to the shard's range
                        ok, d = _close(sum(parts), want)
                        rep.checks.append(Check(f"{tag}: EP{ep} range outputs sum to the whole, {n} rows", ok, d))
                if device != "cpu":
                    rep.checks.append(_native_check(tag, spec, view, l, x, want, cfg, device))
        return rep
    finally:
        if tmp is not None:
            tmp.cleanup()


def _oracle_logits(reference, x, w):
    import torch.nn.functional as F

    prec = w.extra.get("router_precision", "payload")
    if prec == "payload":
        logits = F.linear(x, w.router)
    else:
        logits = F.linear(x.float(), w.extra["router_fp32"].float() if prec == "fp32" else w.router.float())
    if w.extra.get("router_bias") is not None:
        logits = logits.float() + w.extra["router_bias"].float()
    return logits


def _native_check(tag, spec, view, l, x, want, cfg, device) -> Check:
    from ..engine import loader
    from ..ops import gemm, moe

    try:
        w = loader.materialize_layer_weights(spec, view, l.layer, device=device)
        xd = x.to(device)
        if w.is_moe:
            got = moe.moe_forward(xd, w, cfg)
        else:
            if not w.extra.get("gated", True):
                return Check(f"{tag}: native kernels", True, {"skipped": "non-gated dense layers run on the oracle path only"})
            tr = w.extra.get("gate_transform") or (0.0, 0.0, 0.0)
            act = gemm.gateup_swiglu(xd, w.gate_up, bias=w.gate_up_bias, gate_limit=tr[0], up_add=tr[1], act_alpha=tr[2])
            got = gemm.linear(act, w.down, bias=w.down_bias)
        torch.cuda.synchronize()
        gemm.check_status(torch.device(device))
        ok, d = _close(got.float().cpu(), want)
        return Check(f"{tag}: native kernels equal the direct evaluation, {x.shape[0]} rows", ok, d)
    except Exception as e:
        return Check(f"{tag}: native kernels", False, {"error": repr(e)})


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.devtools.qualification")
    ap.add_argument("--arch", default="all", help="an architecture of the built-in tiny configurations, or 'all'")
    ap.add_argument("--config", default=None, help="a config.json (or its directory); use with --shrink for real models")
    ap.add_argument("--shrink", action="store_true", help="replace the sizes of --config by the family's tiny ones")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--against", choices=("direct", "hf", "served"), default="direct",
                    help="'hf': compare with the transformers implementation of the architecture (devtools/hf_parity.py); "
                         "'served': bring up a CPU deployment per architecture and compare its answers with the library's "
                         "(devtools/served_qualification.py)")
    ns = ap.parse_args(argv)
    if ns.against == "served":
        from . import served_qualification

        if ns.config:
            p = Path(ns.config)
            return served_qualification.main(["--checkpoint", str(p if p.is_dir() else p.parent)] + (["--json"] if ns.json else []))
        return served_qualification.main(["--arch", ns.arch] + (["--json"] if ns.json else []))
    if ns.against == "hf":
        from . import hf_parity

        return hf_parity.main(["--arch", ns.arch] + (["--json"] if ns.json else []))
    if ns.config:
        p = Path(ns.config)
        cfg = json.loads((p / "config.json" if p.is_dir() else p).read_text())
        configs = {cfg["architectures"][0]: shrink(cfg) if ns.shrink else cfg}
    else:
        configs = {a: tiny_config(a) for a in (sorted(TINY_CONFIGS) if ns.arch == "all" else [ns.arch])}
    bad = 0
    for name, cfg in configs.items():
        rep = qualify(cfg, device=ns.device)
        bad += 0 if rep.ok else 1
        if ns.json:
            print(json.dumps({"config": name, **rep.to_json()}))
        else:
            print(f"{name}: {'PASS' if rep.ok else 'FAIL'} ({len(rep.checks)} checks, layers {sorted(set(rep.layers))})")
            for c in rep.checks:
                if not c.ok:
                    print(f"   FAILED {c.name}: {c.detail}")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
