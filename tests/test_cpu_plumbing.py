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


@pytest.mark.parametrize("layout", ["packed", "uniform"])
def test_data_parallel_attention_ranks_meet_in_one_evaluation_per_layer(layout):
    """Two attention processes of one Instance with different requests; the FFN process evaluates each layer once
    per rendezvous over both ranks' rows (row table checked by the native dp_inspect_rows), ranks without work take
    part with Idle invocations, and every rank gets the logits of the undivided model."""
    got = cpu_plumbing.run_dp_topology(dp=2, layout=layout)
    want = cpu_plumbing.run_dp_monolithic(dp=2)
    for a, b in zip(got.ranks, want):
        assert a.tokens == b.tokens
        for x, y in zip(a.logits, b.logits):
            torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-4)
    # both ranks made the same number of layer calls although rank 1 had fewer requests
    assert got.ranks[0].invocations == got.ranks[1].invocations == got.merged_evaluations
    assert got.idle_participations > 0
    assert got.mixed_mode_evaluations > 0          # a prefill of one rank met a decode step of the other


def test_data_parallel_ranks_that_disagree_about_the_layer_both_see_a_protocol_mismatch():
    import multiprocessing as mp
    import os
    import threading

    from crosspool_b200.models import config as model_config
    from crosspool_b200.native import runtime as rt

    cfg = model_config.preset("tiny-qwen3")
    names = [f"/xpool-cpu-{os.getpid()}-mismatch-dp{r}" for r in range(2)]
    boxes = [rt.CpuMailbox.create(n, 4, cfg.hidden_size * 4) for n in names]
    ctx = mp.get_context("spawn")
    ready, stats = ctx.Event(), ctx.Array("q", 3, lock=False)
    proc = ctx.Process(target=cpu_plumbing.dp_ffn_main, args=(names, "tiny-qwen3", 0, 4, ready, rt.DP_PACKED_BY_RANK, stats), daemon=True)
    proc.start()
    try:
        assert ready.wait(120)
        for mb in boxes:
            assert mb.wait_status(rt.MBOX_IDLE, 10.0) == rt.WAIT_READY
        x = torch.zeros(2, cfg.hidden_size)
        codes = [None, None]

        def call(r, layer):
            y = torch.empty_like(x)
            codes[r] = boxes[r].submit(x.data_ptr(), y.data_ptr(), 2, layer, rt.MODE_DECODE, timeout_s=20.0)

        threads = [threading.Thread(target=call, args=(0, 0)), threading.Thread(target=call, args=(1, 1))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert codes == [rt.RESULT_PROTOCOL_MISMATCH, rt.RESULT_PROTOCOL_MISMATCH]
        assert stats[0] == 0
    finally:
        for mb in boxes:
            mb.shutdown()
        proc.join(10)
        if proc.is_alive():
            proc.kill()
        for mb in boxes:
            mb.close()
