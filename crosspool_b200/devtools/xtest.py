"""Test runner over the case catalogue ``tests/tests.toml``.

A case names pytest targets, the marker expression, how many GPUs it needs and a time limit. ``xtest run`` takes the
cases in catalogue order, leases devices for each (cases that need more GPUs than the machine has are reported as
skipped, not failed), runs pytest as an owned child process with ``CUDA_VISIBLE_DEVICES`` set to the lease, and
prints one summary line per case plus a JSON report (reference: ``xtest run`` over ``tests/tests.toml`` with resource
groups, src/xpool-dev/xtest/harness/runner/*).

    python -m crosspool_b200.devtools.xtest run [--tier cpu|gpu|multigpu] [--case NAME ...] [--report out.json]
    python -m crosspool_b200.devtools.xtest list
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
import tomllib
from dataclasses import dataclass
from pathlib import Path

from .supervisor import DeviceLeases

ROOT = Path(__file__).resolve().parents[2]


@dataclass(frozen=True)
class TestCase:
    name: str
    tier: str               # cpu | gpu | multigpu
    targets: tuple[str, ...]
    marker: str = ""
    gpus: int = 0
    timeout_s: float = 900.0
    env: tuple = ()


def load_cases(path: Path | None = None) -> list[TestCase]:
    doc = tomllib.loads((path or ROOT / "tests" / "tests.toml").read_text())
    out = []
    for name, c in doc.get("cases", {}).items():
        unknown = set(c) - {"tier", "targets", "marker", "gpus", "timeout_s", "env"}
        if unknown:
            raise ValueError(f"case {name}: unknown keys {sorted(unknown)}")
        out.append(TestCase(name, c.get("tier", "cpu"), tuple(c["targets"]), c.get("marker", ""), int(c.get("gpus", 0)),
                            float(c.get("timeout_s", 900.0)), tuple(sorted((c.get("env") or {}).items()))))
    return out


def visible_gpus() -> list[int]:
    try:
        import torch

        return list(range(torch.cuda.device_count()))
    except Exception:
        return []


def run_case(case: TestCase, leases: DeviceLeases, runner=None, supervisor=None) -> dict:
    """``supervisor`` (a :class:`~crosspool_b200.devtools.supervisor.Supervisor`): the case runs as an owned process
    group; at its time limit the whole group is retired, and processes it orphaned are drained and reported (a case
    that leaves processes behind fails). ``runner``: a ``subprocess.run`` stand-in for tests of this function."""
    if runner is None and supervisor is None:
        runner = subprocess.run
    if case.gpus > len(leases.free) + sum(len(v) for v in leases.taken.values()):
        return {"case": case.name, "status": "skipped", "reason": f"needs {case.gpus} GPUs"}
    with leases.lease(case.name, case.gpus) as devs:
        env = dict(os.environ, PYTHONPATH=str(ROOT), **dict(case.env))
        if case.gpus:
            env["CUDA_VISIBLE_DEVICES"] = ",".join(str(d) for d in devs)
        cmd = [sys.executable, "-m", "pytest", "-q", "-x", *case.targets]
        if case.marker:
            cmd += ["-m", case.marker]
        t0 = time.monotonic()
        if supervisor is not None:
            c = supervisor.run(case.name, cmd, case.timeout_s, env=env, cwd=str(ROOT))
            lines = c.log_tail.strip().splitlines()
            status = "passed" if c.ok else "failed"
            summary = lines[-1] if lines else ""
            if c.kind == "timed_out":
                summary = f"timed out after {case.timeout_s:.0f} s"
            elif c.orphans:
                summary += f" (left {len(c.orphans)} process(es) behind)"
            return {"case": case.name, "status": status, "rc": c.exit_code, "seconds": round(c.elapsed_s, 1), "devices": devs,
                    "summary": summary, "ended": c.kind, "orphans": list(c.orphans)}
        try:
            r = runner(cmd, env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=case.timeout_s)
            rc, tail = r.returncode, (r.stdout or "").strip().splitlines()[-1:] or [""]
        except subprocess.TimeoutExpired:
            rc, tail = 124, [f"timed out after {case.timeout_s:.0f} s"]
        return {"case": case.name, "status": "passed" if rc == 0 else "failed", "rc": rc, "seconds": round(time.monotonic() - t0, 1),
                "devices": devs, "summary": tail[0]}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="xtest")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("list")
    r = sub.add_parser("run")
    r.add_argument("--tier", choices=["cpu", "gpu", "multigpu"], action="append")
    r.add_argument("--case", action="append")
    r.add_argument("--report", default="")
    r.add_argument("--catalogue", default="")
    ns = ap.parse_args(argv)
    cases = load_cases(Path(ns.catalogue) if getattr(ns, "catalogue", "") else None)
    if ns.cmd == "list":
        for c in cases:
            print(f"{c.name:32s} {c.tier:9s} gpus={c.gpus} {' '.join(c.targets)}")
        return 0
    chosen = [c for c in cases if (not ns.tier or c.tier in ns.tier) and (not ns.case or c.name in ns.case)]
    leases = DeviceLeases(visible_gpus())
    import tempfile

    from .supervisor import Supervisor

    with tempfile.TemporaryDirectory(prefix="xtest-logs-") as logs:
        sup = Supervisor(log_dir=logs, adopt_orphans=sys.platform.startswith("linux"))
        results = [run_case(c, leases, supervisor=sup) for c in chosen]
    for res in results:
        print(f"{res['status']:8s} {res['case']:32s} {res.get('seconds', '')} {res.get('summary', res.get('reason', ''))}", flush=True)
    if ns.report:
        Path(ns.report).write_text(json.dumps(results, indent=1))
    return 1 if any(r["status"] == "failed" for r in results) else 0


if __name__ == "__main__":
    raise SystemExit(main())
