from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ...native import runtime as rt
from ..sglang import shim as op

# MLP blocks whose decoder layer unpacks two results (output, router scores)
_TUPLE_RESULT = ("GptOssMLP",)


class HfFfnShim(torch.nn.Module):
    """Stands where a decoder MLP was. Holds no parameters. Hidden states arrive as ``[batch, tokens, hidden]`` (or
    already flattened); one token per sequence is a decode step, anything longer a prefill chunk."""

    def __init__(self, layer_ordinal: int, returns_tuple: bool = False):
        super().__init__()
        self.layer_ordinal, self.returns_tuple = layer_ordinal, returns_tuple
        self.layer_kind = "dense"

    def forward(self, hidden_states: torch.Tensor, *_a, **_kw):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).contiguous()
        decode = hidden_states.dim() == 3 and shape[1] == 1
        meta = op.ShimMetadata(self.layer_ordinal, rt.MODE_DECODE if decode else rt.MODE_PREFILL, rt.OUT_PER_RANK_COMPLETE, rt.DP_NONE)
        y = op.ffn_shim(x, None, meta).view(shape)
        return (y, None) if self.returns_tuple else y


@dataclass
class DetachReport:
    shims: list[HfFfnShim] = field(default_factory=list)
    freed_parameters: int = 0          # elements of the FFN tensors the model no longer holds
    kept_parameters: int = 0


def _decoder_layers(model) -> list:
    inner = getattr(model, "model", model)
    if hasattr(inner, "decoder"):
        inner = inner.decoder
    return list(inner.layers)


def detach_ffn(model) -> DetachReport:
    """Replaces every decoder FFN of ``model`` by an :class:`HfFfnShim` (in place) and drops the FFN parameters."""
    rep = DetachReport()
    for ordinal, layer in enumerate(_decoder_layers(model)):
        if hasattr(layer, "mlp"):
            old = layer.mlp
            shim = HfFfnShim(ordinal, returns_tuple=type(old).__name__ in _TUPLE_RESULT)
            shim.layer_kind = "moe" if any("expert" in n for n, _ in old.named_parameters()) else "dense"
            rep.freed_parameters += sum(p.numel() for p in old.parameters())
            layer.mlp = shim
        elif hasattr(layer, "fc1") and hasattr(layer, "fc2"):
            # OPT computes fc2(act(fc1(x))) inline: the shim takes fc1's place and answers with the whole FFN
            if not getattr(layer, "do_layer_norm_before", True):
                raise NotImplementedError("OPT variants that normalise after the FFN are not supported")
            shim = HfFfnShim(ordinal)
            rep.freed_parameters += sum(p.numel() for m in (layer.fc1, layer.fc2) for p in m.parameters())
            layer.fc1, layer.activation_fn, layer.fc2 = shim, torch.nn.Identity(), torch.nn.Identity()
        else:
            raise NotImplementedError(f"decoder layer {ordinal} ({type(layer).__name__}) has no MLP this integration knows")
        rep.shims.append(shim)
    rep.kept_parameters = sum(p.numel() for p in model.parameters())
    return rep


def bind_cpu_tier(tier_shim) -> None:
    """Routes ``torch.ops.xpool.ffn_shim`` calls on CPU tensors to a CPU FFN tier (``RemoteFfnTier``: every rank gets
    the rows, partials are summed in rank order)."""

    def submit(hidden, _dp_rows, out, layer, mode, _requirement, _layout):
        out.copy_(tier_shim(int(layer), hidden.float(), int(mode)).to(out.dtype))

    op.bind_submit(submit)


def unbind() -> None:
    op.bind_submit(None)
