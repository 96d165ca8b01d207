"""Names of tensor element types on the wire and in configuration files. Reference: src/xpool/utils/dtype.py."""

from __future__ import annotations

import torch

_BY_NAME = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
            "float8_e4m3fn": torch.float8_e4m3fn, "uint8": torch.uint8, "int32": torch.int32, "int64": torch.int64}
_ALIASES = {"fp32": "float32", "float": "float32", "bf16": "bfloat16", "fp16": "float16", "half": "float16",
            "fp8": "float8_e4m3fn", "e4m3": "float8_e4m3fn"}
_BY_DTYPE = {v: k for k, v in _BY_NAME.items()}


def decode_dtype(value: object) -> torch.dtype:
    """``torch.bfloat16``, ``"bfloat16"``, ``"torch.bfloat16"`` or a short alias (``bf16``) -> the dtype."""
    if isinstance(value, torch.dtype):
        if value not in _BY_DTYPE:
            raise ValueError(f"unsupported element type {value}")
        return value
    if not isinstance(value, str):
        raise TypeError(f"an element type is a name or a torch.dtype, not {type(value).__name__}")
    name = value.strip().lower().removeprefix("torch.")
    name = _ALIASES.get(name, name)
    try:
        return _BY_NAME[name]
    except KeyError:
        raise ValueError(f"unknown element type {value!r}; known: {sorted(_BY_NAME)}") from None


def encode_dtype(value: torch.dtype | str) -> str:
    """The canonical name (``"bfloat16"``) written to wire models, manifests and configuration."""
    return _BY_DTYPE[decode_dtype(value)]


def element_bytes(value: torch.dtype | str) -> int:
    return decode_dtype(value).itemsize
