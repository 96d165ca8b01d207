"""Checkpoint index: which safetensors file holds which tensor, and FFN key coverage.

A Hugging Face checkpoint is either one ``model.safetensors`` or shards listed in
``model.safetensors.index.json``. The FFN side opens only ``model.layers.N.mlp.*`` tensors and checks
that the set it found is exactly the set its :class:`FfnModelSpec` needs; the attention side loads
everything else (reference: src/xpool/runtime/ffnagent/checkpoint.py:36-93).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..ffn import FfnModelSpec
from ..models.weights import FFN_KEY


class CheckpointError(ValueError):
    pass


@dataclass
class CheckpointKeyView:
    root: Path
    key_to_file: dict[str, str]

    def keys(self) -> list[str]:
        return sorted(self.key_to_file)

    def ffn_keys(self) -> list[str]:
        return sorted(k for k in self.key_to_file if FFN_KEY.match(k) or ".decoder.layers." in k and (".fc1." in k or ".fc2." in k))


def read_checkpoint_key_view(model_dir: str | Path) -> CheckpointKeyView:
    from safetensors import safe_open

    root = Path(model_dir)
    index = root / "model.safetensors.index.json"
    if index.exists():
        wm = json.loads(index.read_text()).get("weight_map")
        if not isinstance(wm, dict) or not wm:
            raise CheckpointError(f"{index} has no weight_map")
        missing = sorted({f for f in wm.values() if not (root / f).exists()})
        if missing:
            raise CheckpointError(f"index names missing shard files: {missing[:3]}")
        return CheckpointKeyView(root, dict(wm))
    files = sorted(root.glob("*.safetensors"))
    if not files:
        raise CheckpointError(f"no safetensors checkpoint under {root}")
    out: dict[str, str] = {}
    for f in files:
        with safe_open(str(f), framework="pt") as sf:
            for k in sf.keys():
                if k in out:
                    raise CheckpointError(f"tensor {k} appears in {out[k]} and {f.name}")
                out[k] = f.name
    return CheckpointKeyView(root, out)


def validate_ffn_coverage(spec: FfnModelSpec, view: CheckpointKeyView) -> None:
    """Exact coverage: every tensor the spec needs exists, and no FFN tensor of the checkpoint is
    left unexplained (an unexplained tensor means the adapter does not understand this model)."""
    need = spec.required_keys()
    have = set(view.key_to_file)
    missing = sorted(need - have)
    if missing:
        raise CheckpointError(f"checkpoint misses {len(missing)} FFN tensors, e.g. {missing[:3]}")
    extra = sorted(set(view.ffn_keys()) - need)
    if extra:
        raise CheckpointError(f"checkpoint has {len(extra)} FFN tensors the spec does not cover, e.g. {extra[:3]}")


def open_tensor(view: CheckpointKeyView, key: str) -> torch.Tensor:
    from safetensors import safe_open

    with safe_open(str(view.root / view.key_to_file[key]), framework="pt") as sf:
        return sf.get_tensor(key)
