"""Benchmark suite runner: named cases, repetitions, sealed manifests, continuation.

A *case* fixes the workload (streams, duration, SLOs); every *repetition* runs it with its own seed and
leaves ``<out>/<case>/rep<k>/repetition.json``; once all repetitions of a case are sealed,
``<out>/<case>/case.json`` aggregates them. A manifest is *sealed* by a SHA-256 over its canonical JSON;
``--continue`` skips repetitions whose seal verifies, ``--rerun-failure`` also re-runs sealed
repetitions that recorded errors (reference: ``xbench run --all --continue DIR [--rerun-failure]``,
docs/designs/benchmark.md:234; src/xpool-dev/xbench/harness/serving/measure.py:37-137).

    python -m crosspool_b200.bench.suite --targets m=http://127.0.0.1:30000 --out runs/ --cases poisson-16 --continue
"""

from __future__ import annotations

import argparse
import asyncio
import hashlib
import json
import statistics
import sys
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable

from . import serving as S
from ..utils.files import atomic_write_text


@dataclass(frozen=True)
class Case:
    name: str
    rate_per_s: tuple[float, ...]          # per target, in the order targets are given (cycled)
    duration_s: float
    prompt: S.LengthSpec
    output: S.LengthSpec
    repetitions: int = 3
    warmup_requests: int = 2
    burst: tuple[float, float, float] = (1.0, 0.0, 0.0)
    slo_ttft_ms: float = 2000.0
    slo_tpot_ms: float = 50.0
    base_seed: int = 0
    # where the case is meant to run (catalogue cases): models, atn / ffn devices, lanes, ffn_tp, atn_tp, elastic
    deployment: tuple = ()

    def deployment_dict(self) -> dict:
        return dict(self.deployment)


CASES: dict[str, Case] = {c.name: c for c in (
    # one model, Poisson arrivals, uniform lengths (the single-model deployment shape)
    Case("poisson-16", (16.0,), 32.0, S.LengthSpec("uniform", 128, 2048), S.LengthSpec("uniform", 128, 512)),
    # skewed two-model demand: long-context traffic against short-context traffic
    Case("skewed-pair", (4.0, 32.0), 60.0, S.LengthSpec("lognormal", 256, 32768, 8192.0, 1.0), S.LengthSpec("uniform", 128, 256)),
    # four-model mix with bursts: rates 1:2:4:4, 4x bursts for 30 s in every 120 s
    Case("four-model-mix", (1.0, 2.0, 4.0, 4.0), 120.0, S.LengthSpec("lognormal", 16, 8192, 1024.0, 1.0),
         S.LengthSpec("uniform", 128, 1024), burst=(4.0, 30.0, 120.0)),
    Case("smoke", (8.0,), 2.0, S.LengthSpec("uniform", 8, 32), S.LengthSpec("uniform", 4, 8), repetitions=2, warmup_requests=1),
)}


def _length(spec: dict | str) -> S.LengthSpec:
    """``{kind="uniform", lo=, hi=}`` / ``{kind="lognormal", median=, sigma=, lo=, hi=}`` or the CLI string form."""
    if isinstance(spec, str):
        p = spec.split(":")
        return S.LengthSpec("uniform", int(p[1]), int(p[2])) if p[0] == "uniform" else \
            S.LengthSpec("lognormal", int(p[3]), int(p[4]), float(p[1]), float(p[2]))
    if spec.get("kind", "uniform") == "uniform":
        return S.LengthSpec("uniform", int(spec["lo"]), int(spec["hi"]))
    return S.LengthSpec("lognormal", int(spec.get("lo", 1)), int(spec["hi"]), float(spec["median"]), float(spec.get("sigma", 1.0)))


def _deployment(case: str, named: dict, ref) -> tuple:
    """A case names its deployment (``deployment = "small-pair"`` -> ``[deployments.small-pair]``) or spells it out."""
    if ref is None:
        return ()
    d = named.get(ref) if isinstance(ref, str) else ref
    if not isinstance(d, dict):
        raise ValueError(f"case {case}: unknown deployment {ref!r}")
    unknown = set(d) - {"models", "atn", "ffn", "lanes", "ffn_tp", "atn_tp", "elastic", "max_batch", "max_seq_len"}
    if unknown:
        raise ValueError(f"case {case}: unknown deployment keys {sorted(unknown)}")
    return tuple(sorted((k, tuple(v) if isinstance(v, list) else v) for k, v in d.items()))


def load_catalogue(path: str | Path) -> dict[str, Case]:
    """Cases from a TOML catalogue (the counterpart of the reference's ``benches/benches.toml``):

        [defaults]                      # optional, merged into every case
        duration_s = 60
        [cases.small-pair-1rps]
        rate_per_s = [1.0, 1.0]
        prompt = {kind = "lognormal", median = 1024, sigma = 1.0, lo = 16, hi = 8192}
        output = {kind = "uniform", lo = 128, hi = 512}
    """
    import tomllib

    doc = tomllib.loads(Path(path).read_text())
    defaults = doc.get("defaults", {})
    out = {}
    for name, raw in doc.get("cases", {}).items():
        c = {**defaults, **raw}
        unknown = set(c) - {"rate_per_s", "duration_s", "prompt", "output", "repetitions", "warmup_requests", "burst",
                            "slo_ttft_ms", "slo_tpot_ms", "base_seed", "deployment"}
        if unknown:
            raise ValueError(f"case {name}: unknown keys {sorted(unknown)}")
        rates = c["rate_per_s"]
        out[name] = Case(name, tuple(float(r) for r in (rates if isinstance(rates, list) else [rates])), float(c["duration_s"]),
                         _length(c["prompt"]), _length(c["output"]), int(c.get("repetitions", 3)),
                         int(c.get("warmup_requests", 2)), tuple(float(x) for x in c.get("burst", (1.0, 0.0, 0.0))),
                         float(c.get("slo_ttft_ms", 2000.0)), float(c.get("slo_tpot_ms", 50.0)), int(c.get("base_seed", 0)),
                         _deployment(name, doc.get("deployments", {}), c.get("deployment")))
    return out


def seal(doc: dict) -> dict:
    body = {k: v for k, v in doc.items() if k != "seal"}
    doc["seal"] = hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    return doc


def sealed_ok(path: Path) -> dict | None:
    try:
        doc = json.loads(path.read_text())
    except (OSError, ValueError):
        return None
    want = doc.get("seal")
    return doc if want and seal(dict(doc))["seal"] == want else None


def default_runner(case: Case, targets: dict[str, str], seed: int, vocab_sizes: dict[str, int] | None = None) -> dict:
    """``vocab_sizes``: per model, the range random prompt ids are drawn from (default: the Qwen vocabulary; a model with
    a smaller one would refuse ids beyond it)."""
    models = list(targets)
    vocab = vocab_sizes or {}
    streams = [S.StreamSpec(m, case.rate_per_s[i % len(case.rate_per_s)], case.prompt, case.output, burst_factor=case.burst[0],
                            burst_seconds=case.burst[1], burst_period=case.burst[2],
                            **({"vocab_size": int(vocab[m])} if m in vocab else {})) for i, m in enumerate(models)]
    reqs = S.plan_workload(streams, case.duration_s, seed, case.warmup_requests)
    records, window = asyncio.run(S.run_client(targets, reqs))
    return {"digest": S.workload_digest(reqs), "window_s": window,
            "aggregate": S.summarize(records, window, case.slo_ttft_ms, case.slo_tpot_ms),
            "per_model": {m: S.summarize([r for r in records if r.model == m], window, case.slo_ttft_ms, case.slo_tpot_ms)
                          for m in models}}


@dataclass
class SuiteResult:
    ran: list[str] = field(default_factory=list)
    skipped: list[str] = field(default_factory=list)
    failed: list[str] = field(default_factory=list)


def run_suite(cases: list[Case], targets: dict[str, str], out: Path, *, cont: bool = False, rerun_failure: bool = False,
              runner: Callable[[Case, dict[str, str], int], dict] = default_runner) -> SuiteResult:
    res = SuiteResult()
    for case in cases:
        cdir = out / case.name
        reps = []
        for k in range(case.repetitions):
            rpath = cdir / f"rep{k}" / "repetition.json"
            tag = f"{case.name}/rep{k}"
            old = sealed_ok(rpath) if cont else None
            if old is not None and not (rerun_failure and old.get("errors", 0) > 0):
                res.skipped.append(tag)
                reps.append(old)
                continue
            rpath.parent.mkdir(parents=True, exist_ok=True)
            seed = case.base_seed + 1000 * k
            try:
                report = runner(case, targets, seed)
                errors = int(report.get("aggregate", {}).get("errors", 0))
                doc = seal({"case": case.name, "repetition": k, "seed": seed, "errors": errors, "report": report})
            except Exception as e:  # a crashed repetition is recorded, the suite goes on
                doc = seal({"case": case.name, "repetition": k, "seed": seed, "errors": 1, "exception": repr(e)})
            atomic_write_text(rpath, json.dumps(doc, indent=1))   # resumed runs skip repetitions whose file exists
            reps.append(doc)
            (res.failed if doc["errors"] else res.ran).append(tag)
        good = [r["report"]["aggregate"] for r in reps if "report" in r and not r["errors"]]
        summary = {"case": case.name, "spec": json.loads(json.dumps(asdict(case))), "repetitions": len(reps), "clean": len(good)}
        if good:
            tput = [g["output_tok_per_s"] for g in good]
            summary.update(output_tok_per_s_median=statistics.median(tput), output_tok_per_s_min=min(tput),
                           p99_tpot_ms_median=statistics.median(g["tpot_ms"]["p99"] for g in good),
                           p50_ttft_ms_median=statistics.median(g["arrival_ttft_ms"]["p50"] for g in good))
        cdir.mkdir(parents=True, exist_ok=True)
        atomic_write_text(cdir / "case.json", json.dumps(seal(summary), indent=1))
    return res


def rate_tag(rate: float) -> str:
    """``0.5`` -> ``0p5rps``, ``4`` -> ``4rps`` (the naming of the catalogue's rate sweeps)."""
    text = f"{rate:g}".replace(".", "p")
    return f"{text}rps"


def generate_cases(deployment: str, models: int, rates: list[float], *, split: tuple[float, ...] | None = None,
                   extra: dict | None = None) -> str:
    """TOML for one sweep of a catalogue: a case per rate for ``deployment`` with ``models`` co-located models.
    ``split`` skews the offered load between the models (fractions of ``models`` x rate, e.g. ``(0.8, 0.2)``);
    ``extra`` adds the same keys (``duration_s``, ``prompt``, ...) to every case. The reference generates its
    catalogue the same way (``xbench case-gen``)."""
    if models < 1 or not rates:
        raise ValueError("a sweep needs at least one model and one rate")
    if split is not None and (len(split) != models or abs(sum(split) - 1.0) > 1e-9 or min(split) < 0):
        raise ValueError("split needs one non-negative fraction per model, summing to 1")

    def value(v) -> str:
        if isinstance(v, dict):
            return "{" + ", ".join(f"{k} = {value(x)}" for k, x in v.items()) + "}"
        if isinstance(v, str):
            return json.dumps(v)
        if isinstance(v, bool):
            return "true" if v else "false"
        if isinstance(v, (list, tuple)):
            return "[" + ", ".join(value(x) for x in v) + "]"
        return repr(float(v)) if isinstance(v, float) else str(v)

    out = []
    for r in rates:
        per = [r] * models if split is None else [round(r * models * f, 6) for f in split]
        name = f"{deployment}-{rate_tag(r)}" + ("" if split is None else "-skew" + "-".join(f"{int(round(100 * f))}" for f in split))
        lines = [f"[cases.{name}]", f'deployment = "{deployment}"', f"rate_per_s = {value([float(x) for x in per])}"]
        lines += [f"{k} = {value(v)}" for k, v in (extra or {}).items()]
        out.append("\n".join(lines))
    return "\n\n".join(out) + "\n"


def _case_gen(argv: list[str]) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.suite case-gen")
    ap.add_argument("--deployment", required=True)
    ap.add_argument("--models", type=int, required=True)
    ap.add_argument("--rates", type=float, nargs="+", required=True)
    ap.add_argument("--split", type=float, nargs="*", default=None)
    ap.add_argument("--duration-s", type=float, default=None)
    ns = ap.parse_args(argv)
    extra = {"duration_s": ns.duration_s} if ns.duration_s else None
    print(generate_cases(ns.deployment, ns.models, ns.rates, split=tuple(ns.split) if ns.split else None, extra=extra), end="")
    return 0


def _list_cases(argv: list[str]) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.suite list")
    ap.add_argument("--catalogue", default="")
    ns = ap.parse_args(argv)
    cases = dict(CASES)
    if ns.catalogue:
        cases.update(load_catalogue(ns.catalogue))
    for name, c in sorted(cases.items()):
        dep = c.deployment_dict()
        where = f"{len(dep.get('models', ()))} models on atn {list(dep.get('atn', ()))} / ffn {list(dep.get('ffn', ()))}" if dep else "any deployment"
        print(f"{name:40s} rates {list(c.rate_per_s)} req/s  {c.duration_s:g} s x {c.repetitions}  {where}")
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["case-gen"]:
        return _case_gen(argv[1:])
    if argv[:1] == ["list"]:
        return _list_cases(argv[1:])
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.suite",
                                 epilog="other forms: `suite list [--catalogue F]`, `suite case-gen --deployment D --models N --rates ...`; "
                                        "reports: python -m crosspool_b200.bench.report")
    ap.add_argument("--targets", nargs="+", required=True, help="model=http://host:port ...")
    ap.add_argument("--out", required=True)
    ap.add_argument("--cases", nargs="*", default=[], help=f"subset of {sorted(CASES)} (default: all but smoke)")
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--catalogue", default="", help="TOML file with [cases.<name>] tables (adds to the built-in cases)")
    ap.add_argument("--vocab", nargs="*", default=[], help="model=N: vocabulary size random prompt ids are drawn from (default 151936)")
    ap.add_argument("--continue", dest="cont", action="store_true")
    ap.add_argument("--rerun-failure", action="store_true")
    ns = ap.parse_args(argv)
    if ns.catalogue:
        CASES.update(load_catalogue(ns.catalogue))
    names = ns.cases or [n for n in CASES if n != "smoke"]
    unknown = [n for n in names if n not in CASES]
    if unknown:
        ap.error(f"unknown cases {unknown}")
    targets = dict(t.split("=", 1) for t in ns.targets)
    vocab = {m: int(n) for m, n in (v.split("=", 1) for v in ns.vocab)}
    runner = (lambda c, t, seed: default_runner(c, t, seed, vocab)) if vocab else default_runner
    res = run_suite([CASES[n] for n in names], targets, Path(ns.out), cont=ns.cont, rerun_failure=ns.rerun_failure, runner=runner)
    print(json.dumps(asdict(res), indent=1))
    return 3 if res.failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
