"""Acceptance configuration (a): tiny Qwen3-architecture decoder, fp32, attention role and FFN role
in separate processes over the shared-memory mailbox; logits must match the monolithic forward."""
import torch

from crosspool_b200.engine import cpu_plumbing


def test_disaggregated_logits_match_monolithic_forward():
    got = cpu_plumbing.run("tiny-qwen3", seed=0, requests=8, prompt_len=32, new_tokens=16)
    want = cpu_plumbing.run_monolithic("tiny-qwen3", seed=0, requests=8, prompt_len=32, new_tokens=16)
    assert got.tokens == want.tokens
    for a, b in zip(got.logits, want.logits):
        assert a.shape == (16, 4096)
        assert (a - b).abs().max().item() <= 1e-4
    # 2 layers x (1 prefill + 15 decode forwards) x 8 requests
    assert got.invocations == 2 * 16 * 8


def test_moe_model_through_the_same_plumbing():
    got = cpu_plumbing.run("tiny-qwen3-moe", seed=3, requests=2, prompt_len=16, new_tokens=4)
    want = cpu_plumbing.run_monolithic("tiny-qwen3-moe", seed=3, requests=2, prompt_len=16, new_tokens=4)
    assert got.tokens == want.tokens
    for a, b in zip(got.logits, want.logits):
        assert (a - b).abs().max().item() <= 1e-4
