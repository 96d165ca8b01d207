"""Attention tensor parallelism over 2 GPUs (one process per GPU): identical tokens on all ranks, logits
close to the unsharded engine."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch


gpu = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@gpu
@pytest.mark.parametrize("graph", [0, 1])
def test_two_attention_tp_ranks_match_the_unsharded_engine(graph):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29561", str(ROOT / "tests/multigpu/atn_tp_check.py"), "--graph", str(graph)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "ATN_TP_CHECK_OK" in r.stdout


def test_weight_sharding_partitions_heads_exactly():
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import random_attention_weights
    from crosspool_b200.parallel import atn_tp

    cfg = mc.preset("tiny-qwen3")
    aw = random_attention_weights(cfg, 1)
    x = torch.randn(3, cfg.hidden_size)
    shards = [atn_tp.shard_attention_weights(aw, cfg, r, 2) for r in (0, 1)]
    loc = atn_tp.local_config(cfg, 2)
    assert (loc.num_q_heads, loc.num_kv_heads) == (cfg.num_q_heads // 2, cfg.num_kv_heads // 2)
    full = x @ aw.layers[0].qkv.float().t()
    q = torch.cat([x @ s.layers[0].qkv.float()[:loc.q_size].t() for s in shards], dim=1)
    assert torch.equal(q, full[:, :cfg.q_size])
    attn = torch.randn(3, cfg.q_size)
    o_full = attn @ aw.layers[0].o.float().t()
    o_parts = sum(attn[:, r * loc.q_size:(r + 1) * loc.q_size] @ shards[r].layers[0].o.float().t() for r in (0, 1))
    torch.testing.assert_close(o_parts, o_full, atol=1e-5, rtol=1e-5)
    with pytest.raises(ValueError):
        atn_tp.local_config(cfg, 4)
