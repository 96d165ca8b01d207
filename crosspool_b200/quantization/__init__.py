"""Weight quantization formats of FFN shards.

``resolve(method)`` maps a checkpoint's ``quantization_config.quant_method`` to a format object:
``None`` -> :class:`Unquantized`, ``"mxfp4"`` -> :class:`Mxfp4` (packed e2m1 values with e8m0 block
scales, as GPT-OSS ships its experts), ``"fp8_block"`` -> :class:`Fp8Block` (e4m3 with one fp32 scale
per 128 x 128 block); anything else is refused with the reference's message
(src/xpool/quantization/__init__.py:48-50).
"""

from __future__ import annotations

from .formats import Fp8Block, Mxfp4, Quantization, Unquantized

__all__ = ["Quantization", "Unquantized", "Mxfp4", "Fp8Block", "resolve"]


def resolve(method: str | None) -> Quantization:
    if method in (None, "", "none"):
        return Unquantized()
    if method == "mxfp4":
        return Mxfp4()
    if method in ("fp8_block", "fp8"):
        return Fp8Block()
    raise ValueError(f"unsupported weight quantization method: {method}")
