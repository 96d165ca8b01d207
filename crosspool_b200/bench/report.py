"""Reports over the sealed results of a benchmark-suite run (``bench/suite.py``).

    python -m crosspool_b200.bench.report list RUN_DIR                 # sealed cases and repetitions, with verdicts
    python -m crosspool_b200.bench.report make RUN_DIR [--output DIR]  # summary.json, report.md, CSV tables, SVG chart per case
    python -m crosspool_b200.bench.report clean ROOT --keep 3          # drop all but the newest run directories

``make`` trusts nothing but sealed files: a ``repetition.json`` or ``case.json`` whose seal does not match its content
(edited by hand, or cut off by a crash) is reported as unsealed and left out, never repaired; a repetition that failed
keeps its verdict and is listed, not averaged. It reads no earlier report, and it never writes into the measurement
files. The reference's ``xbench report`` has the same contract (docs/designs/benchmark.md, "report validates retained
replay ... preserves measurement files and original execution verdicts"); figures here are plain SVG written by this
module, since no plotting library is a dependency.
"""

from __future__ import annotations

import argparse
import csv
import io
import json
import re
import shutil
import statistics
import sys
from dataclasses import dataclass, field
from pathlib import Path

from ..utils.files import atomic_write_text
from .suite import sealed_ok

METRICS = (("output_tok_per_s", "output tokens/s"), ("arrival_ttft_ms", "arrival TTFT ms"), ("http_ttft_ms", "HTTP TTFT ms"),
           ("tpot_ms", "TPOT ms"), ("itl_ms", "ITL ms"))
PERCENTILES = ("p50", "p90", "p95", "p99")


@dataclass
class Repetition:
    index: int
    path: Path
    doc: dict | None                 # None: not sealed (missing, cut off or edited)

    @property
    def verdict(self) -> str:
        if self.doc is None:
            return "unsealed"
        return "failed" if self.doc.get("errors") or "report" not in self.doc else "ok"


@dataclass
class CaseRun:
    name: str
    path: Path
    summary: dict | None
    repetitions: list[Repetition] = field(default_factory=list)

    @property
    def good(self) -> list[Repetition]:
        return [r for r in self.repetitions if r.verdict == "ok"]


def discover(run_dir: str | Path) -> list[CaseRun]:
    """Cases of a run directory, without recomputing any metric: seals are checked, nothing else is parsed."""
    root = Path(run_dir)
    if not root.is_dir():
        raise FileNotFoundError(f"{root} is not a run directory")
    out = []
    for cdir in sorted(p for p in root.iterdir() if p.is_dir()):
        reps = []
        rdirs = [(int(m.group(1)), p) for p in cdir.iterdir() if p.is_dir() and (m := re.fullmatch(r"rep(\d+)", p.name))]
        for index, rdir in sorted(rdirs):
            path = rdir / "repetition.json"
            reps.append(Repetition(index, path, sealed_ok(path) if path.exists() else None))
        if not reps and not (cdir / "case.json").exists():
            continue
        out.append(CaseRun(cdir.name, cdir, sealed_ok(cdir / "case.json") if (cdir / "case.json").exists() else None, reps))
    return out


def _median(vals: list[float]) -> float:
    vals = [v for v in vals if v == v]
    return statistics.median(vals) if vals else float("nan")


def aggregate(case: CaseRun) -> dict:
    """Recomputed from the sealed repetitions alone (the case's own summary is only compared, never copied)."""
    good = case.good
    models = sorted({m for r in good for m in r.doc["report"].get("per_model", {})})

    def block(pick) -> dict:
        aggs = [pick(r.doc["report"]) for r in good]
        aggs = [a for a in aggs if a]
        out: dict = {"repetitions": len(aggs)}
        if not aggs:
            return out
        out["output_tok_per_s"] = {"median": _median([a["output_tok_per_s"] for a in aggs]), "min": min(a["output_tok_per_s"] for a in aggs),
                                   "max": max(a["output_tok_per_s"] for a in aggs)}
        out["requests"] = sum(a["requests"] for a in aggs)
        out["errors"] = sum(a["errors"] for a in aggs)
        for key, _ in METRICS[1:]:
            out[key] = {p: _median([a[key][p] for a in aggs if key in a]) for p in PERCENTILES}
        slo = [a["slo"] for a in aggs if "slo" in a]
        if slo:
            out["slo"] = {"ttft_ms": slo[0]["ttft_ms"], "tpot_ms": slo[0]["tpot_ms"], "attained_min": min(s["attained"] for s in slo),
                          "goodput_tok_per_s_median": _median([s["goodput_tok_per_s"] for s in slo]),
                          "every_repetition_within_slo": all(s["p99_tpot_within_slo"] and s["p99_ttft_within_slo"] for s in slo)}
        return out

    doc = {"case": case.name, "verdicts": {f"rep{r.index}": r.verdict for r in case.repetitions},
           "digests": sorted({r.doc["report"].get("digest", "") for r in good}),
           "aggregate": block(lambda rep: rep.get("aggregate")),
           "per_model": {m: block(lambda rep, m=m: rep.get("per_model", {}).get(m)) for m in models}}
    if case.summary is not None and good and "output_tok_per_s_median" in case.summary:
        doc["agrees_with_case_summary"] = abs(case.summary["output_tok_per_s_median"] - doc["aggregate"]["output_tok_per_s"]["median"]) < 1e-6
    return doc


def _fmt(v) -> str:
    if isinstance(v, float):
        return "n/a" if v != v else (f"{v:.0f}" if abs(v) >= 100 else f"{v:.1f}")
    return str(v)


def markdown(doc: dict) -> str:
    lines = [f"# {doc['case']}", "", "Repetitions: " + ", ".join(f"{k} {v}" for k, v in doc["verdicts"].items()), ""]
    if not doc["aggregate"].get("repetitions"):
        return "\n".join(lines + ["No sealed successful repetition: nothing to aggregate.", ""])
    lines += ["| series | tok/s median (min-max) | arrival TTFT p50 / p99 ms | TPOT p50 / p99 ms | ITL p99 ms | requests | errors |",
              "| --- | --- | --- | --- | --- | --- | --- |"]
    for name, b in [("all models", doc["aggregate"])] + sorted(doc["per_model"].items()):
        if not b.get("repetitions"):
            continue
        t = b["output_tok_per_s"]
        lines.append(f"| {name} | {_fmt(t['median'])} ({_fmt(t['min'])}-{_fmt(t['max'])}) | {_fmt(b['arrival_ttft_ms']['p50'])} / "
                     f"{_fmt(b['arrival_ttft_ms']['p99'])} | {_fmt(b['tpot_ms']['p50'])} / {_fmt(b['tpot_ms']['p99'])} | "
                     f"{_fmt(b['itl_ms']['p99'])} | {b['requests']} | {b['errors']} |")
    slo = doc["aggregate"].get("slo")
    if slo:
        lines += ["", f"SLO (TTFT {_fmt(slo['ttft_ms'])} ms, TPOT {_fmt(slo['tpot_ms'])} ms): lowest attainment {slo['attained_min']:.3f}, "
                      f"goodput {_fmt(slo['goodput_tok_per_s_median'])} tok/s, "
                      f"{'every' if slo['every_repetition_within_slo'] else 'not every'} repetition inside both p99 gates."]
    lines += ["", "Latencies are medians over the successful repetitions of each repetition's percentile; failed or unsealed "
                  "repetitions keep their verdict above and are not averaged.", "", "![throughput](throughput.svg)", ""]
    return "\n".join(lines)


def _csv(rows: list[list]) -> str:
    buf = io.StringIO()
    csv.writer(buf, lineterminator="\n").writerows(rows)
    return buf.getvalue()


def percentiles_csv(doc: dict) -> str:
    rows = [["series", "metric"] + list(PERCENTILES)]
    for name, b in [("all", doc["aggregate"])] + sorted(doc["per_model"].items()):
        for key, _ in METRICS[1:]:
            if key in b:
                rows.append([name, key] + [b[key][p] for p in PERCENTILES])
    return _csv(rows)


def throughput_csv(case: CaseRun) -> str:
    rows = [["repetition", "series", "output_tok_per_s", "window_s"]]
    for r in case.good:
        rep = r.doc["report"]
        rows.append([r.index, "all", rep["aggregate"]["output_tok_per_s"], rep.get("window_s", "")])
        for m, a in sorted(rep.get("per_model", {}).items()):
            rows.append([r.index, m, a["output_tok_per_s"], rep.get("window_s", "")])
    return _csv(rows)


def throughput_svg(case: CaseRun, width: int = 640, height: int = 300) -> str:
    """Grouped bars: one group per repetition, one bar per model plus the aggregate. Distinguishable in grayscale:
    the bars differ in fill lightness and carry their series name in the legend."""
    good = case.good
    series = ["all"] + sorted({m for r in good for m in r.doc["report"].get("per_model", {})})
    vals = {(r.index, s): (r.doc["report"]["aggregate"] if s == "all" else r.doc["report"]["per_model"].get(s, {})).get("output_tok_per_s", 0.0)
            for r in good for s in series}
    top = max(vals.values(), default=1.0) or 1.0
    left, bottom, right, head = 56, 40, 12, 28
    pw, ph = width - left - right, height - bottom - head
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" viewBox="0 0 {width} {height}" font-family="serif" font-size="11">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<text x="{left}" y="16" font-size="12">{case.name}: output tokens/s per repetition</text>']
    for k in range(5):
        y = head + ph - ph * k / 4
        out.append(f'<line x1="{left}" y1="{y:.1f}" x2="{left + pw}" y2="{y:.1f}" stroke="#ccc" stroke-width="0.5"/>')
        out.append(f'<text x="{left - 4}" y="{y + 3:.1f}" text-anchor="end">{top * k / 4:.0f}</text>')
    n = max(1, len(good))
    gw = pw / n
    bw = gw * 0.8 / max(1, len(series))
    for gi, r in enumerate(good):
        for si, s in enumerate(series):
            v = vals[(r.index, s)]
            h = ph * v / top
            x = left + gi * gw + gw * 0.1 + si * bw
            shade = 40 + int(170 * si / max(1, len(series) - 1)) if len(series) > 1 else 90
            out.append(f'<rect x="{x:.1f}" y="{head + ph - h:.1f}" width="{bw * 0.92:.1f}" height="{h:.1f}" fill="rgb({shade},{shade},{shade})" '
                       f'stroke="black" stroke-width="0.4"><title>{s} rep{r.index}: {v:.1f} tok/s</title></rect>')
        out.append(f'<text x="{left + gi * gw + gw / 2:.1f}" y="{head + ph + 14}" text-anchor="middle">rep{r.index}</text>')
    for si, s in enumerate(series):
        shade = 40 + int(170 * si / max(1, len(series) - 1)) if len(series) > 1 else 90
        y = height - 8
        x = left + si * (pw / max(1, len(series)))
        out.append(f'<rect x="{x:.1f}" y="{y - 8}" width="9" height="9" fill="rgb({shade},{shade},{shade})" stroke="black" stroke-width="0.4"/>')
        out.append(f'<text x="{x + 13:.1f}" y="{y}">{s}</text>')
    out.append("</svg>")
    return "\n".join(out) + "\n"


def make_reports(run_dir: str | Path, output: str | Path | None = None) -> list[Path]:
    """Writes ``report/`` beside every case (or below ``output/<run name>/<case>/report``); returns the directories.
    Repeated calls overwrite the generated files and nothing else."""
    root = Path(run_dir)
    made = []
    for case in discover(root):
        doc = aggregate(case)
        dest = (Path(output) / root.name / case.name / "report") if output else case.path / "report"
        dest.mkdir(parents=True, exist_ok=True)
        atomic_write_text(dest / "summary.json", json.dumps(doc, indent=1))
        atomic_write_text(dest / "report.md", markdown(doc))
        atomic_write_text(dest / "percentiles.csv", percentiles_csv(doc))
        atomic_write_text(dest / "throughput.csv", throughput_csv(case))
        atomic_write_text(dest / "throughput.svg", throughput_svg(case))
        made.append(dest)
    return made


def clean(root: str | Path, keep: int) -> list[Path]:
    """Removes all but the ``keep`` most recently modified run directories below ``root`` (a run directory is one that
    holds at least one sealed ``case.json`` or ``repetition.json``; anything else is left alone)."""
    if keep < 0:
        raise ValueError("keep must not be negative")
    runs = []
    for p in Path(root).iterdir():
        if p.is_dir() and (any(p.glob("*/case.json")) or any(p.glob("*/rep[0-9]*/repetition.json"))):
            runs.append(p)
    runs.sort(key=lambda p: p.stat().st_mtime, reverse=True)
    gone = runs[keep:]
    for p in gone:
        shutil.rmtree(p)
    return gone


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.report")
    sub = ap.add_subparsers(dest="cmd", required=True)
    ls = sub.add_parser("list", help="sealed cases and repetitions of a run directory")
    ls.add_argument("run_dir")
    mk = sub.add_parser("make", help="write summary.json, report.md, CSV tables and an SVG chart per case")
    mk.add_argument("run_dir")
    mk.add_argument("--output", default=None, help="export below DIR/<run>/<case>/report instead of beside the measurements")
    cl = sub.add_parser("clean", help="drop all but the newest run directories below a root")
    cl.add_argument("root")
    cl.add_argument("--keep", type=int, required=True)
    ns = ap.parse_args(argv)
    try:
        if ns.cmd == "list":
            for case in discover(ns.run_dir):
                reps = " ".join(f"rep{r.index}:{r.verdict}" for r in case.repetitions)
                print(f"{case.name:32s} summary {'sealed' if case.summary is not None else 'unsealed'}  {reps}")
            return 0
        if ns.cmd == "make":
            for d in make_reports(ns.run_dir, ns.output):
                print(d)
            return 0
        for p in clean(ns.root, ns.keep):
            print(f"removed {p}")
        return 0
    except (FileNotFoundError, ValueError) as e:
        print(f"report: {e}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())
