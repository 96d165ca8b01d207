"""End to end with real processes: ``xpool daemon serve`` + ``xpool atnagent`` + ``xpool ffnagent`` on two
GPUs, requests over HTTP, graceful quiesce. Needs >= 2 GPUs."""
import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

import httpx
import pytest
import torch


pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

TOML = """
[daemon]
port = 9831
[atn]
devices = [0]
[ffn]
devices = [1]
[scheduler]
ffn_concurrency = 2
[scheduler.slo]
ttft_ms = 2000
tbt_ms = 50
[[models]]
id = "Qwen/Qwen3-0.6B"
ffn_tp_size = 1
"""


@pytest.mark.parametrize("elastic", [False, True])
def test_daemon_agents_serve_requests_and_retire(tmp_path, elastic):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _serve_and_retire(tmp_path, TOML.replace("devices = [0]", "devices = [0]\nelastic_kv = true") if elastic else TOML,
                      [("ffnagent", 1), ("atnagent", 0)])


@pytest.mark.parametrize("elastic", [False, True])
def test_attention_tp_pair_serves_through_the_daemon(tmp_path, elastic):
    """One Instance whose attention runs tensor-parallel over two agent processes (GPUs 0 and 1); the FFN tier
    is GPU 2. The first rank owns the HTTP endpoint and replicates requests to the other."""
    if torch.cuda.device_count() < 3:
        pytest.skip("needs 3 GPUs")
    toml = TOML.replace("devices = [0]", "devices = [0, 1]").replace("devices = [1]", "devices = [2]") \
               .replace("ffn_tp_size = 1", "ffn_tp_size = 1\natn_tp_size = 2")
    if elastic:      # capacity changes are agreed between the two ranks over their gloo group
        toml = toml.replace("devices = [0, 1]", "devices = [0, 1]\nelastic_kv = true")
    _serve_and_retire(tmp_path, toml, [("ffnagent", 2), ("atnagent", 0), ("atnagent", 1)])


def _serve_and_retire(tmp_path, toml, agents):
    cfgp = tmp_path / "xpool.toml"
    cfgp.write_text(toml)
    env = dict(os.environ, XPOOL_CONFIG=str(cfgp), PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0", XPOOL_MAX_ROWS="512",
               XPOOL_MAX_BATCH="16", XPOOL_MAX_SEQ_LEN="512")
    xp = [sys.executable, "-m", "crosspool_b200.cli.main"]
    procs = [subprocess.Popen(xp + ["daemon", "serve"], env=env)]
    try:
        for _ in range(100):
            try:
                if httpx.get("http://127.0.0.1:9831/health", timeout=1).status_code == 200:
                    break
            except httpx.HTTPError:
                time.sleep(0.2)
        for role, dev in agents:
            procs.append(subprocess.Popen(xp + [role, "--device", str(dev)], env=env))
        ready = False
        for _ in range(600):
            r = httpx.get("http://127.0.0.1:9831/ready", timeout=2).json()
            if r["system_ready"]:
                ready = True
                break
            assert r["failure"] is None, r
            time.sleep(0.5)
        assert ready
        assert subprocess.run(xp + ["daemon", "check"], env=env, capture_output=True).returncode == 0
        out = httpx.post("http://127.0.0.1:30000/generate", json={"input_ids": list(range(1, 40)), "max_new_tokens": 5},
                         timeout=60).json()
        assert len(out["output_ids"]) == 5
        again = httpx.post("http://127.0.0.1:30000/generate", json={"input_ids": list(range(1, 40)), "max_new_tokens": 5},
                           timeout=60).json()
        assert again["output_ids"] == out["output_ids"]  # greedy decoding is deterministic
        assert httpx.post("http://127.0.0.1:9831/fabric/quiesce", json={"reason": "test"}, timeout=5).status_code == 200
        for p in procs[1:]:
            assert p.wait(60) == 0
        plan = httpx.get("http://127.0.0.1:9831/fabric/plan", timeout=2).json()
        assert plan["phase"] == "stopped"
    finally:
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)
        for p in procs:
            try:
                p.wait(10)
            except subprocess.TimeoutExpired:
                p.kill()
