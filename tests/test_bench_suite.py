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
