"""Attention rank + FFN rank(s) as separate processes on separate GPUs (needs >= 2 GPUs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch


pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(nproc, extra):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29541", str(ROOT / "tests/multigpu/fabric_check.py")] + extra
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "FABRIC_CHECK_OK" in r.stdout


def test_one_atn_one_ffn_matches_loopback_tokens():
    _run(2, ["--tp", "1"])


def test_one_atn_two_ffn_tensor_parallel():
    _run(3, ["--tp", "2"])


def test_moe_model_through_lanes_on_one_ffn_rank():
    _run(2, ["--tp", "1", "--model", "tiny-qwen3-moe", "--layers", "2"])


def test_moe_expert_parallel_over_two_ffn_ranks():
    _run(3, ["--tp", "2", "--model", "tiny-qwen3-moe", "--layers", "2"])


def test_attention_tp_pair_with_a_remote_ffn_rank():
    _run(3, ["--atn-tp", "2", "--tp", "1"])


def test_layer_split_placement_over_two_ffn_ranks():
    _run(3, ["--tp", "1", "--layer-split", "2"])


def test_a_failure_on_the_ffn_rank_cancels_the_attention_ranks_wait_in_the_same_call():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29547", str(ROOT / "tests/multigpu/failure_check.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "FAILURE_CHECK_OK" in r.stdout


def test_native_ffn_shim_operator_reaches_the_ffn_tier_eagerly_and_from_a_graph():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29549", str(ROOT / "tests/multigpu/shim_check.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "SHIM_CHECK_OK" in r.stdout
