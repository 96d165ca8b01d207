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


import pytest


@pytest.mark.parametrize("preset,ranks,moe_parallel", [("tiny-qwen3", 2, "tp"), ("tiny-qwen3-moe", 2, "tp"),
                                                       ("tiny-qwen3-moe", 4, "ep")])
def test_ffn_tier_of_several_processes_folds_rank_partials_to_the_monolithic_logits(preset, ranks, moe_parallel):
    """One process per FFN rank, each with its tensor-parallel shard or its expert range only; the attention side
    folds the partials in rank order. fp32 sums of shards differ from the unsharded sum by rounding only."""
    got = cpu_plumbing.run_topology(preset, ffn_ranks=ranks, moe_parallel=moe_parallel, seed=5, requests=2, prompt_len=12,
                                    new_tokens=4)
    want = cpu_plumbing.run_monolithic(preset, seed=5, requests=2, prompt_len=12, new_tokens=4)
    assert got.tokens == want.tokens
    for a, b in zip(got.logits, want.logits):
        assert (a - b).abs().max().item() <= 2e-4
    assert got.invocations == 2 * 4 * 2          # layers x forwards x requests, whatever the number of ranks


def test_expert_parallel_topology_refuses_a_dense_model():
    with pytest.raises(ValueError, match="expert parallelism"):
        cpu_plumbing.run_topology("tiny-qwen3", ffn_ranks=2, moe_parallel="ep")
