"""Acceptance tolerances shared by the test-suite and by users validating a deployment.

The limits are the reference's (src/xpool-dev/xtest/harness/support/ffn.py:20-28,
docs/designs/qualification.md:86-89): FFN outputs within atol 0.02 / rtol 0.02 element-wise, normalised
RMSE <= 0.01 and max scaled error <= 0.10; routing weights atol 1e-4 / rtol 1e-3; logits against a stock
forward KL <= 0.05 nats for prefill and <= 0.001 nats for decode steps.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

FFN_ATOL, FFN_RTOL, FFN_NRMSE, FFN_MAX_SCALED = 0.02, 0.02, 0.01, 0.10
ROUTING_ATOL, ROUTING_RTOL = 1e-4, 1e-3
KL_PREFILL, KL_DECODE = 0.05, 0.001


@dataclass
class FfnError:
    nrmse: float
    max_scaled: float
    frac_outside_elementwise: float

    @property
    def ok(self) -> bool:
        return self.nrmse <= FFN_NRMSE and self.max_scaled <= FFN_MAX_SCALED


def ffn_error(out: torch.Tensor, ref: torch.Tensor) -> FfnError:
    o, r = out.float(), ref.float()
    err = (o - r).abs()
    scale = r.abs().max().clamp_min(1e-12)
    nrmse = (err.pow(2).mean().sqrt() / r.pow(2).mean().sqrt().clamp_min(1e-12)).item()
    outside = (err > FFN_ATOL + FFN_RTOL * r.abs()).float().mean().item()
    return FfnError(nrmse, (err.max() / scale).item(), outside)


def assert_ffn_close(out: torch.Tensor, ref: torch.Tensor, what: str = "ffn output") -> FfnError:
    e = ffn_error(out, ref)
    if not e.ok:
        raise AssertionError(f"{what}: nrmse {e.nrmse:.4f} (limit {FFN_NRMSE}), max scaled error {e.max_scaled:.4f} (limit {FFN_MAX_SCALED})")
    return e


def kl_nats(p_logits: torch.Tensor, q_logits: torch.Tensor) -> torch.Tensor:
    """KL(p || q) per row, in nats."""
    p, q = p_logits.float().log_softmax(-1), q_logits.float().log_softmax(-1)
    return (p.exp() * (p - q)).sum(-1)


def assert_logits_close(ref_logits: torch.Tensor, got_logits: torch.Tensor, prefill_rows: int = 1) -> None:
    kl = kl_nats(ref_logits, got_logits)
    if kl[:prefill_rows].max().item() > KL_PREFILL:
        raise AssertionError(f"prefill KL {kl[:prefill_rows].max().item():.4f} nats exceeds {KL_PREFILL}")
    if kl.shape[0] > prefill_rows and kl[prefill_rows:].max().item() > KL_DECODE:
        raise AssertionError(f"decode KL {kl[prefill_rows:].max().item():.5f} nats exceeds {KL_DECODE}")
