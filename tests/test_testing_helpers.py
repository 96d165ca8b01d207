import pytest
import torch

from crosspool_b200 import testing as T


def test_ffn_tolerances_and_kl_helpers():
    g = torch.Generator().manual_seed(0)
    ref = torch.randn(64, 128, generator=g)
    assert T.assert_ffn_close(ref + 0.003 * torch.randn(64, 128, generator=g), ref).nrmse < 0.01
    with pytest.raises(AssertionError, match="nrmse"):
        T.assert_ffn_close(ref + 0.05 * torch.randn(64, 128, generator=g), ref)
    spike = ref.clone()
    spike[0, 0] += 0.5 * ref.abs().max()
    with pytest.raises(AssertionError, match="max scaled"):
        T.assert_ffn_close(spike, ref)
    logits = torch.randn(3, 1000, generator=g)
    assert T.kl_nats(logits, logits).abs().max() < 1e-6
    T.assert_logits_close(logits, logits + 1e-3 * torch.randn(3, 1000, generator=g))
    with pytest.raises(AssertionError, match="decode KL"):
        T.assert_logits_close(logits, logits + 0.2 * torch.randn(3, 1000, generator=g))
