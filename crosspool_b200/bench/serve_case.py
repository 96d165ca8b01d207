"""Brings up a local deployment (daemon + one agent per GPU, as ``xpool`` child processes), runs one
serving benchmark case against it over HTTP and retires it in order.

    python -m crosspool_b200.bench.serve_case --case poisson-16 --models Qwen/Qwen3-0.6B --atn 0 --ffn 1 \
        --out serve_poisson16.json

The deployment is the one a user would start by hand with ``xpool daemon serve`` / ``xpool atnagent`` /
``xpool ffnagent``; the load generator is ``bench.serving`` (open-loop Poisson arrivals, streaming
``POST /generate``, client-side TTFT / TPOT / ITL).
"""

from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]


def toml_for(models: list[str], atn: list[int], ffn: list[int], port: int, ffn_tp: int, lanes: int, atn_tp: int = 1,
             elastic: bool = False, serving_port: int = 30000) -> str:
    t = [f"[daemon]\nport = {port}", f"[atn]\ndevices = {atn}" + ("\nelastic_kv = true" if elastic else ""), f"[ffn]\ndevices = {ffn}",
         f"[scheduler]\nffn_concurrency = {lanes}", "[scheduler.slo]\nttft_ms = 2000\ntbt_ms = 50", f"[serving]\nbase_port = {serving_port}"]
    for m in models:
        t.append(f'[[models]]\nid = "{m}"\nffn_tp_size = {ffn_tp}\natn_tp_size = {atn_tp}')
    return "\n".join(t) + "\n"


class LocalDeployment:
    def __init__(self, toml_text: str, atn: list[int], ffn: list[int], port: int, env: dict[str, str] | None = None,
                 backend: str = "gpu", serving_port: int = 30000):
        """``backend="cpu"``: the agents run the shared-memory data plane and the PyTorch oracle (no GPU needed)."""
        self.toml_text, self.atn, self.ffn, self.port = toml_text, atn, ffn, port
        self.backend, self.serving_port = backend, serving_port
        self.env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0", **(env or {}))
        self.procs: list[subprocess.Popen] = []
        self._dir = tempfile.TemporaryDirectory(prefix="xpool-deploy-")

    def _xp(self, *args: str) -> subprocess.Popen:
        p = subprocess.Popen([sys.executable, "-m", "crosspool_b200.cli.main", *args], env=self.env)
        self.procs.append(p)
        return p

    def __enter__(self) -> "LocalDeployment":
        import httpx

        cfgp = Path(self._dir.name) / "xpool.toml"
        cfgp.write_text(self.toml_text)
        self.env["XPOOL_CONFIG"] = str(cfgp)
        base = f"http://127.0.0.1:{self.port}"
        self._xp("daemon", "serve")
        for _ in range(150):
            try:
                if httpx.get(base + "/health", timeout=1).status_code == 200:
                    break
            except httpx.HTTPError:
                time.sleep(0.2)
        for d in self.ffn:
            self._xp("ffnagent", "--device", str(d), "--backend", self.backend)
        for d in self.atn:
            self._xp("atnagent", "--device", str(d), "--backend", self.backend)
        for _ in range(1200):
            r = httpx.get(base + "/ready", timeout=5).json()
            if r.get("failure"):
                raise RuntimeError(f"deployment failed: {r['failure']}")
            if r["system_ready"]:
                return self
            if any(p.poll() not in (None, 0) for p in self.procs):
                raise RuntimeError("a deployment process exited early")
            time.sleep(0.5)
        raise TimeoutError("deployment did not become ready")

    def targets(self, models: list[str]) -> dict[str, str]:
        return {m: f"http://127.0.0.1:{self.serving_port}" for m in models}   # all Instances of attention device 0 share one listener

    def __exit__(self, *exc) -> None:
        import httpx

        try:
            httpx.post(f"http://127.0.0.1:{self.port}/fabric/quiesce", json={"reason": "benchmark finished"}, timeout=5)
            for p in self.procs[1:]:
                try:
                    p.wait(60)
                except subprocess.TimeoutExpired:
                    pass
        except Exception:
            pass
        for p in self.procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)   # exact child PIDs only
        for p in self.procs:
            try:
                p.wait(15)
            except subprocess.TimeoutExpired:
                p.kill()
        # the daemon is ended by SIGTERM; an agent that did not retire with exit code 0 is worth a line
        for p in self.procs[1:]:
            if p.returncode not in (0, None):
                print(f"deployment process {' '.join(p.args[3:])} exited with code {p.returncode}", file=sys.stderr, flush=True)
        self._dir.cleanup()


def _vocab_sizes(models: list[str]) -> dict[str, int]:
    """Vocabulary of every model that is a preset or a checkpoint directory, so that random prompt ids are valid ones."""
    from ..models import config as mc

    out = {}
    for m in models:
        try:
            out[m] = mc.load(m).vocab_size
        except (FileNotFoundError, KeyError, ValueError):
            pass
    return out


def main(argv: list[str] | None = None) -> int:
    from . import suite

    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.serve_case")
    ap.add_argument("--case", default="poisson-16", help=f"one of {sorted(suite.CASES)} or a case of --catalogue")
    ap.add_argument("--catalogue", default="", help="TOML catalogue with further cases (configs/benches.toml)")
    ap.add_argument("--models", nargs="+", default=None, help="default: the case's deployment, else Qwen/Qwen3-0.6B")
    ap.add_argument("--atn", type=int, nargs="+", default=None)
    ap.add_argument("--ffn", type=int, nargs="+", default=None)
    ap.add_argument("--ffn-tp", type=int, default=None)
    ap.add_argument("--atn-tp", type=int, default=None, help="attention tensor-parallel degree (= number of --atn devices)")
    ap.add_argument("--elastic", action="store_true", default=None, help="elastic KV: co-located Instances lend physical KV memory")
    ap.add_argument("--lanes", type=int, default=None)
    ap.add_argument("--port", type=int, default=9841)
    ap.add_argument("--serving-port", type=int, default=30000, help="HTTP port of the first attention device's Instances")
    ap.add_argument("--backend", choices=("gpu", "cpu"), default="gpu", help="cpu: run the deployment on the CPU data plane")
    ap.add_argument("--max-rows", type=int, default=4096, help="row capacity of an FFN invocation")
    ap.add_argument("--max-batch", type=int, default=None)
    ap.add_argument("--max-seq-len", type=int, default=None)
    ap.add_argument("--prefill-chunk", type=int, default=4096, help="tokens per prefill step of the attention engines")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--duration", type=float, default=0.0, help="override the case's duration (seconds)")
    ap.add_argument("--rate", type=float, default=0.0, help="override the case's per-model request rate")
    ap.add_argument("--out", default="")
    ns = ap.parse_args(argv)
    cases = dict(suite.CASES)
    if ns.catalogue:
        cases.update(suite.load_catalogue(ns.catalogue))
    if ns.case not in cases:
        ap.error(f"unknown case {ns.case!r}; known: {sorted(cases)}")
    case = cases[ns.case]
    dep_defaults = {"models": ["Qwen/Qwen3-0.6B"], "atn": [0], "ffn": [1], "ffn_tp": 1, "atn_tp": 1, "elastic": False, "lanes": 2,
                    "max_batch": 256, "max_seq_len": 2624}
    dep_defaults.update({k: list(v) if isinstance(v, tuple) else v for k, v in case.deployment_dict().items()})
    for k, v in dep_defaults.items():          # command line > the case's deployment > defaults
        if getattr(ns, k) is None:
            setattr(ns, k, v)
    if ns.duration > 0 or ns.rate > 0:
        import dataclasses

        case = dataclasses.replace(case, duration_s=ns.duration or case.duration_s,
                                   rate_per_s=(ns.rate,) if ns.rate > 0 else case.rate_per_s)
    env = {"XPOOL_MAX_BATCH": str(ns.max_batch), "XPOOL_MAX_SEQ_LEN": str(ns.max_seq_len), "XPOOL_MAX_ROWS": str(ns.max_rows),
           "XPOOL_PREFILL_CHUNK": str(min(ns.prefill_chunk, ns.max_rows))}
    text = toml_for(ns.models, ns.atn, ns.ffn, ns.port, ns.ffn_tp, ns.lanes, ns.atn_tp, ns.elastic, ns.serving_port)
    with LocalDeployment(text, ns.atn, ns.ffn, ns.port, env, backend=ns.backend, serving_port=ns.serving_port) as dep:
        report = suite.default_runner(case, dep.targets(ns.models), ns.seed, vocab_sizes=_vocab_sizes(ns.models))
    report["case"] = ns.case
    report["deployment"] = {"models": ns.models, "atn": ns.atn, "ffn": ns.ffn, "ffn_tp": ns.ffn_tp, "atn_tp": ns.atn_tp, "lanes": ns.lanes,
                            "elastic_kv": ns.elastic, "backend": ns.backend}
    agg = report["aggregate"]
    line = {"case": ns.case, "output_tok_per_s": round(agg["output_tok_per_s"], 1), "completed": agg["completed"],
            "errors": agg["errors"], "tpot_p50_ms": round(agg["tpot_ms"]["p50"], 2), "tpot_p99_ms": round(agg["tpot_ms"]["p99"], 2),
            "ttft_p50_ms": round(agg["arrival_ttft_ms"]["p50"], 1), "ttft_p99_ms": round(agg["arrival_ttft_ms"]["p99"], 1),
            "slo": agg.get("slo")}
    print(json.dumps(line), flush=True)
    if ns.out:
        Path(ns.out).write_text(json.dumps(report, indent=1))
    return 0 if agg["errors"] == 0 else 3


if __name__ == "__main__":
    raise SystemExit(main())
