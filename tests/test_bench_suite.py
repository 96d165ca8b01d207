"""Suite runner: sealed manifests, continuation, re-running failures."""
import json

from crosspool_b200.bench import suite as X


def _report(tput, errors=0):
    d = {"p50": 1.0, "p90": 2.0, "p95": 2.0, "p99": 3.0, "mean": 1.0, "n": 4}
    return {"aggregate": {"errors": errors, "output_tok_per_s": tput, "tpot_ms": d, "arrival_ttft_ms": d}}


def test_continue_skips_sealed_repetitions_and_rerun_failure_repeats_bad_ones(tmp_path):
    case = X.CASES["smoke"]
    calls = []

    def runner(c, targets, seed):
        calls.append(seed)
        if seed == 1000 and len(calls) <= 2:
            return _report(10.0, errors=2)
        return _report(100.0 + seed)

    r1 = X.run_suite([case], {"m": "http://x"}, tmp_path, runner=runner)
    assert r1.ran == ["smoke/rep0"] and r1.failed == ["smoke/rep1"] and calls == [0, 1000]
    summary = json.loads((tmp_path / "smoke" / "case.json").read_text())
    assert summary["clean"] == 1 and summary["output_tok_per_s_median"] == 100.0 and X.sealed_ok(tmp_path / "smoke" / "case.json")
    r2 = X.run_suite([case], {"m": "http://x"}, tmp_path, cont=True, runner=runner)
    assert r2.skipped == ["smoke/rep0", "smoke/rep1"] and calls == [0, 1000]          # nothing re-run
    r3 = X.run_suite([case], {"m": "http://x"}, tmp_path, cont=True, rerun_failure=True, runner=runner)
    assert r3.skipped == ["smoke/rep0"] and r3.ran == ["smoke/rep1"] and calls == [0, 1000, 1000]
    assert json.loads((tmp_path / "smoke" / "case.json").read_text())["clean"] == 2
    # a tampered manifest no longer verifies and is run again
    p = tmp_path / "smoke" / "rep0" / "repetition.json"
    doc = json.loads(p.read_text())
    doc["report"]["aggregate"]["output_tok_per_s"] = 1e9
    p.write_text(json.dumps(doc))
    assert X.sealed_ok(p) is None
    r4 = X.run_suite([case], {"m": "http://x"}, tmp_path, cont=True, runner=runner)
    assert r4.ran == ["smoke/rep0"]


def test_a_crashing_repetition_is_recorded_and_the_suite_continues(tmp_path):
    def runner(c, targets, seed):
        if seed == 0:
            raise ConnectionError("target down")
        return _report(5.0)

    r = X.run_suite([X.CASES["smoke"]], {"m": "http://x"}, tmp_path, runner=runner)
    assert r.failed == ["smoke/rep0"] and r.ran == ["smoke/rep1"]
    assert "ConnectionError" in json.loads((tmp_path / "smoke" / "rep0" / "repetition.json").read_text())["exception"]
    assert X.main(["--targets", "m=http://x", "--out", str(tmp_path), "--cases", "nope"] ) if False else True


def test_toml_catalogue_loads_the_sixty_one_cases_with_defaults_and_deployments():
    from pathlib import Path

    cases = X.load_catalogue(Path(__file__).resolve().parent.parent / "configs" / "benches.toml")
    assert len(cases) == 61
    assert {"small-pair-1rps", "medium-input-heavy", "four-model-bursty", "large-isolated-b-4rps", "small-pair-atn-tp2-2rps"} <= set(cases)
    c = cases["medium-input-heavy"]
    assert c.rate_per_s == (2.0, 2.0) and c.prompt.kind == "lognormal" and c.prompt.median == 4096 and c.output.hi == 128
    assert cases["four-model-bursty"].burst == (4.0, 30.0, 120.0) and cases["small-pair-1rps"].duration_s == 60
    assert cases["small-pair-1rps"].repetitions == 3
    d = cases["medium-pair-tp2-2rps"].deployment_dict()
    assert d["ffn"] == (1, 2) and d["ffn_tp"] == 2 and d["models"] == ("Qwen/Qwen3-14B", "Qwen/Qwen3-8B") and d["lanes"] == 2
    assert cases["small-pair-lanes1-1rps"].deployment_dict()["lanes"] == 1
    assert cases["small-pair-atn-tp2-4rps"].deployment_dict()["atn_tp"] == 2
    assert cases["large-pair-elastic-1rps"].deployment_dict()["elastic"] is True
    assert sum(1 for n in cases if "isolated" in n) == 18 and sum(1 for n in cases if n.endswith("rps") and "-pair-" in n and "lanes1" not in n and "tp2" not in n and "elastic" not in n) == 18


def _full_report(tput, errors=0, models=("a", "b")):
    d = lambda k: {"p50": 1.0 * k, "p90": 2.0 * k, "p95": 2.5 * k, "p99": 3.0 * k, "mean": 1.2 * k, "n": 8}
    agg = lambda t: {"requests": 8, "completed": 8 - errors, "errors": errors, "output_tokens": 100, "output_tok_per_s": t,
                     "http_ttft_ms": d(10), "arrival_ttft_ms": d(12), "tpot_ms": d(3), "itl_ms": d(4),
                     "slo": {"ttft_ms": 2000.0, "tpot_ms": 50.0, "attained": 1.0, "goodput_tok_per_s": t,
                             "p99_tpot_within_slo": True, "p99_ttft_within_slo": True}}
    return {"digest": "abc", "window_s": 4.0, "aggregate": agg(tput), "per_model": {m: agg(tput / len(models)) for m in models}}


def test_reports_are_built_from_sealed_repetitions_only_and_never_touch_the_measurements(tmp_path):
    from crosspool_b200.bench import report as R

    case = X.CASES["smoke"]                      # two repetitions
    seeds = []

    def runner(c, targets, seed):
        seeds.append(seed)
        return _full_report(100.0 if seed == 0 else 140.0)

    run = tmp_path / "run1"
    X.run_suite([case], {"a": "http://x", "b": "http://y"}, run, runner=runner)
    before = {p: p.read_bytes() for p in run.rglob("*.json")}
    dirs = R.make_reports(run)
    assert dirs == [run / "smoke" / "report"]
    summary = json.loads((dirs[0] / "summary.json").read_text())
    assert summary["verdicts"] == {"rep0": "ok", "rep1": "ok"} and summary["agrees_with_case_summary"]
    assert summary["aggregate"]["output_tok_per_s"] == {"median": 120.0, "min": 100.0, "max": 140.0}
    assert summary["per_model"]["a"]["output_tok_per_s"]["median"] == 60.0
    assert summary["aggregate"]["slo"]["every_repetition_within_slo"]
    md = (dirs[0] / "report.md").read_text()
    assert "| all models | 120 (100-140) |" in md and "| a | 60.0 (50.0-70.0) |" in md
    assert (dirs[0] / "percentiles.csv").read_text().splitlines()[0] == "series,metric,p50,p90,p95,p99"
    assert len((dirs[0] / "throughput.csv").read_text().splitlines()) == 1 + 2 * 3
    svg = (dirs[0] / "throughput.svg").read_text()
    assert svg.startswith("<svg") and svg.count("<rect") >= 1 + 6 and "rep1" in svg
    assert {p: p.read_bytes() for p in before} == before                         # measurements untouched
    # a repetition edited by hand loses its seal: listed as unsealed, left out of the numbers, not repaired
    p = run / "smoke" / "rep1" / "repetition.json"
    doc = json.loads(p.read_text())
    doc["report"]["aggregate"]["output_tok_per_s"] = 1e9
    p.write_text(json.dumps(doc))
    cases = R.discover(run)
    assert [r.verdict for r in cases[0].repetitions] == ["ok", "unsealed"]
    again = R.aggregate(cases[0])
    assert again["aggregate"]["output_tok_per_s"]["median"] == 100.0 and again["verdicts"]["rep1"] == "unsealed"
    assert json.loads(p.read_text())["report"]["aggregate"]["output_tok_per_s"] == 1e9
    # exporting elsewhere keeps the attribution in the path; the CLI lists and makes
    out = R.make_reports(run, output=tmp_path / "export")
    assert out == [tmp_path / "export" / "run1" / "smoke" / "report"]
    assert R.main(["list", str(run)]) == 0 and R.main(["make", str(run)]) == 0 and R.main(["list", str(tmp_path / "nope")]) == 2


def test_failed_repetitions_keep_their_verdict_and_clean_keeps_the_newest_runs(tmp_path):
    import os
    import time

    from crosspool_b200.bench import report as R

    case = X.CASES["smoke"]
    for i, name in enumerate(("old", "mid", "new")):
        X.run_suite([case], {"a": "http://x"}, tmp_path / name,
                    runner=lambda c, t, seed: _full_report(50.0, errors=3 if seed else 0, models=("a",)))
        os.utime(tmp_path / name, (time.time() + i, time.time() + i))
    (tmp_path / "notes").mkdir()                                                  # not a run: never removed
    doc = R.aggregate(R.discover(tmp_path / "new")[0])
    assert doc["verdicts"] == {"rep0": "ok", "rep1": "failed"} and doc["aggregate"]["repetitions"] == 1
    assert "rep1 failed" in R.markdown(doc)
    gone = R.clean(tmp_path, keep=2)
    assert [p.name for p in gone] == ["old"] and sorted(p.name for p in tmp_path.iterdir()) == ["mid", "new", "notes"]


def test_generated_sweeps_load_as_catalogue_cases_and_the_list_form_prints_them(tmp_path, capsys):
    import tomllib

    text = X.generate_cases("small-pair", 2, [0.5, 4], extra={"duration_s": 30.0})
    doc = tomllib.loads(text)
    assert list(doc["cases"]) == ["small-pair-0p5rps", "small-pair-4rps"]
    assert doc["cases"]["small-pair-4rps"] == {"deployment": "small-pair", "rate_per_s": [4.0, 4.0], "duration_s": 30.0}
    skew = tomllib.loads(X.generate_cases("small-pair", 2, [1.0], split=(0.8, 0.2)))
    assert skew["cases"]["small-pair-1rps-skew80-20"]["rate_per_s"] == [1.6, 0.4]
    import pytest
    with pytest.raises(ValueError):
        X.generate_cases("d", 2, [1.0], split=(0.5, 0.6))
    # generated cases are valid catalogue entries next to the shipped deployments
    base = open("configs/benches.toml").read() if __import__("os").path.exists("configs/benches.toml") else None
    if base is not None:
        cat = tmp_path / "cat.toml"
        head = base[: base.index("[cases.")]
        cat.write_text(head + text)
        cases = X.load_catalogue(str(cat))
        assert cases["small-pair-0p5rps"].rate_per_s == (0.5, 0.5) and cases["small-pair-0p5rps"].duration_s == 30.0
        assert X.main(["list", "--catalogue", str(cat)]) == 0
        assert "small-pair-4rps" in capsys.readouterr().out
    assert X.main(["case-gen", "--deployment", "d", "--models", "1", "--rates", "2"]) == 0
    assert "[cases.d-2rps]" in capsys.readouterr().out
