"""Quantization formats: storage layout, tensor-parallel slicing rules, and reference (de)quantizers.

A format answers three questions for the loader and the layer preparation step
(reference: src/xpool/quantization/{base,mxfp4,unquantized}.py): which tensors store a weight, how a
row/column range of the logical weight maps onto them (the *TP stride quantum*: a shard boundary must
not cut a scale block), and how to turn the stored tensors back into bf16.
"""

from __future__ import annotations

from abc import ABC, abstractmethod

import torch

# e2m1 code points (sign bit is the fourth bit)
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


class Quantization(ABC):
    name: str = ""
    #: a shard boundary along the contraction (input) axis must be a multiple of this many elements
    k_quantum: int = 1
    #: ... and along the output axis of this many rows
    n_quantum: int = 1

    @abstractmethod
    def quantize(self, w: torch.Tensor) -> dict[str, torch.Tensor]: ...

    @abstractmethod
    def dequantize(self, stored: dict[str, torch.Tensor], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor: ...

    @abstractmethod
    def stored_bytes(self, n: int, k: int) -> int: ...

    def check_shard(self, n0: int, n1: int, k0: int, k1: int) -> None:
        if (n0 % self.n_quantum or n1 % self.n_quantum or k0 % self.k_quantum or k1 % self.k_quantum):
            raise ValueError(f"{self.name}: shard [{n0}:{n1}, {k0}:{k1}] cuts a scale block "
                             f"(quanta {self.n_quantum} x {self.k_quantum})")

    def slice(self, stored: dict[str, torch.Tensor], n0: int, n1: int, k0: int, k1: int) -> dict[str, torch.Tensor]:
        """The stored tensors of the logical sub-matrix ``[n0:n1, k0:k1]``."""
        self.check_shard(n0, n1, k0, k1)
        return self._slice(stored, n0, n1, k0, k1)

    @abstractmethod
    def _slice(self, stored, n0, n1, k0, k1): ...


class Unquantized(Quantization):
    name = "unquantized"

    def quantize(self, w):
        return {"weight": w}

    def dequantize(self, stored, dtype=torch.bfloat16):
        return stored["weight"].to(dtype)

    def stored_bytes(self, n, k):
        return 2 * n * k

    def _slice(self, stored, n0, n1, k0, k1):
        return {"weight": stored["weight"][..., n0:n1, k0:k1]}


class Mxfp4(Quantization):
    """OCP microscaling fp4: 32 consecutive elements along k share one e8m0 scale (a power of two);
    two e2m1 values are packed per byte, low nibble first."""

    name = "mxfp4"
    k_quantum = 32

    def quantize(self, w):
        *lead, n, k = w.shape
        assert k % 32 == 0
        blocks = w.float().reshape(*lead, n, k // 32, 32)
        amax = blocks.abs().amax(-1).clamp_min(2.0 ** -126)
        exp = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)            # smallest power of two with amax/scale <= 6
        scaled = blocks / torch.exp2(exp)[..., None]
        table = _E2M1[:8].to(w.device)
        mag = (scaled.abs()[..., None] - table).abs().argmin(-1)             # nearest magnitude code
        code = (mag + (scaled < 0) * 8).to(torch.uint8).reshape(*lead, n, k)
        packed = code[..., 0::2] | (code[..., 1::2] << 4)
        return {"blocks": packed.contiguous(), "scales": (exp + 127).to(torch.uint8)}

    def dequantize(self, stored, dtype=torch.bfloat16):
        packed, scales = stored["blocks"], stored["scales"]
        lo, hi = packed & 0xF, packed >> 4
        code = torch.stack([lo, hi], dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2).long()
        vals = _E2M1.to(packed.device)[code]
        scale = torch.exp2(scales.float() - 127.0).repeat_interleave(32, dim=-1)
        return (vals * scale).to(dtype)

    def stored_bytes(self, n, k):
        return n * k // 2 + n * k // 32

    def _slice(self, stored, n0, n1, k0, k1):
        return {"blocks": stored["blocks"][..., n0:n1, k0 // 2:k1 // 2], "scales": stored["scales"][..., n0:n1, k0 // 32:k1 // 32]}


class Fp8Block(Quantization):
    """e4m3 values with one fp32 scale per 128 x 128 block (the layout block-scaled fp8 GEMMs read)."""

    name = "fp8_block"
    k_quantum = 128
    n_quantum = 128
    FP8_MAX = 448.0

    def quantize(self, w):
        *lead, n, k = w.shape
        assert n % 128 == 0 and k % 128 == 0
        b = w.float().reshape(*lead, n // 128, 128, k // 128, 128)
        amax = b.abs().amax((-3, -1)).clamp_min(1e-12)                      # [.., n/128, k/128]
        scale = amax / self.FP8_MAX
        q = (b / scale[..., :, None, :, None]).reshape(*lead, n, k).to(torch.float8_e4m3fn)
        return {"weight": q, "scale": scale}

    def dequantize(self, stored, dtype=torch.bfloat16):
        q, scale = stored["weight"], stored["scale"]
        s = scale.repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)
        return (q.float() * s).to(dtype)

    def stored_bytes(self, n, k):
        return n * k + (n // 128) * (k // 128) * 4

    def _slice(self, stored, n0, n1, k0, k1):
        return {"weight": stored["weight"][..., n0:n1, k0:k1],
                "scale": stored["scale"][..., n0 // 128:n1 // 128, k0 // 128:k1 // 128]}
