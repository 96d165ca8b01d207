"""The served-throughput benchmark's planning, producer loop and aggregation against a CPU fake deployment."""
import argparse
import json
import time

import pytest

from crosspool_b200.bench import served
from crosspool_b200.bench.serving import PlannedRequest


class _Seq:
    def __init__(self, sid, n):
        self.seq_id, self.n, self.k = sid, n, 0

    @property
    def finished(self):
        return self.k >= self.n


class _Res:
    def __init__(self, tokens):
        self.tokens = tokens


class FakeDep:
    """Each step emits one token for every live request of every model and takes ``step_s``."""

    instances = []

    def __init__(self, step_s=0.002):
        self.live, self.nid, self.step_s = {}, 0, step_s
        self.counters = {"h2d_bytes": 0, "d2h_bytes": 0, "launches": 0, "decode_steps": 0, "prefill_steps": 0}

    def add_request(self, model_id, prompt, max_new_tokens, arrival=None):
        s = _Seq(self.nid, max_new_tokens)
        self.nid += 1
        self.live[(model_id, s.seq_id)] = s
        return s

    @property
    def has_work(self):
        return bool(self.live)

    def step(self):
        time.sleep(self.step_s)
        out = {}
        for (m, sid), s in list(self.live.items()):
            s.k += 1
            out.setdefault(m, []).append((s, 1))
            if s.finished:
                del self.live[(m, sid)]
        self.counters["decode_steps"] += 1
        self.counters["h2d_bytes"] += 100
        self.counters["d2h_bytes"] += 4
        self.counters["launches"] += 3
        return _Res(out)

    def stats(self):
        return self.counters


def _args(**kw):
    d = dict(steps=4, warmup=2, step_seconds=0.05, layers=0, impl="xpool", max_batch=0, kv_tokens=0)
    d.update(kw)
    return argparse.Namespace(**d)


def test_mixes_place_every_instance_and_plan_deterministically():
    for mix, world in (("b", 1), ("b", 2), ("c", 2), ("c", 4), ("e", 8), ("b", 8), ("d", 8), ("d", 4)):
        streams, info = served.build_mix(mix, world, 1.0)
        assert info["name"] == mix
        atn = {s.atn_rank for s in streams}
        ffn = {r for s in streams for r in s.ffn_ranks}
        assert not atn & ffn and (world == 1 or atn | ffn == set(range(world)))
        a = served.plan_streams(streams, 3.0, 1.0, seed=1)
        b = served.plan_streams(streams, 3.0, 1.0, seed=1)
        assert [(r.model, r.arrival_s, len(r.prompt)) for r in a] == [(r.model, r.arrival_s, len(r.prompt)) for r in b]
        assert all(x.arrival_s <= y.arrival_s for x, y in zip(a, a[1:]))
        for s in streams:
            lens = [len(r.prompt) for r in a if r.model == s.model_id]
            hi = max(s.prompt.hi, s.alt_prompt.hi if s.alt_prompt else 0)
            assert lens and max(lens) <= hi and max(lens) + max(s.output.hi, s.alt_output.hi if s.alt_output else 0) <= s.max_seq_len


def test_demand_swap_alternates_the_traffic_shapes_per_window():
    streams, _ = served.build_mix("c", 4, 1.0)
    s8 = next(s for s in streams if "8B" in s.model_id and s.atn_rank == 0)
    s06 = next(s for s in streams if "0.6B" in s.model_id and s.atn_rank == 0)
    reqs = served.plan_streams([s8, s06], 4.0, 1.0, seed=0)
    for w in range(4):
        in_w = [r for r in reqs if w <= r.arrival_s < w + 1]
        long_model = s8.model_id if w % 2 == 0 else s06.model_id
        assert all(r.max_new_tokens == (256 if r.model == long_model else 128) for r in in_w)
        assert all(len(r.prompt) == 256 for r in in_w if r.model != long_model)


def test_bursts_raise_the_rate_in_the_first_quarter_of_each_window():
    streams, _ = served.build_mix("e", 8, 4.0)
    reqs = served.plan_streams(streams[1:2], 40.0, 8.0, seed=0)
    burst = sum(1 for r in reqs if (r.arrival_s % 8.0) < 2.0)
    calm = len(reqs) - burst
    assert burst / 2.0 > 2.5 * (calm / 6.0)       # 4x the rate, within Poisson noise


def test_producer_loop_marks_windows_and_aggregates():
    args = _args()
    bounds, end_s, window_s = served.timeline(args)
    assert bounds == pytest.approx([0.1, 0.3, 0.5, 0.7]) and end_s == pytest.approx(0.7)
    reqs = [PlannedRequest("m", 0.01 * i, [1, 2, 3], 20) for i in range(60)]
    rs = served.RankServing(FakeDep(), reqs, "cpu")
    rs.run(time.perf_counter() + 0.01, bounds, end_s)
    summ = rs.summary(bounds)
    assert len(summ["windows"]) == served.WINDOWS and all(w["tokens"] > 0 and w["dev_ms"] > 0 for w in summ["windows"])
    streams = [served.ModelStream("m", "tiny-qwen3", 0, 0, (), 100.0, served._uniform(3, 3), served._uniform(20, 20), 8, 64, 1024)]
    agg = served.aggregate([summ, None], streams, args.steps, args.step_seconds, args.warmup)
    lat = agg["latency"]
    assert lat["finished"] > 0 and lat["slo_met"] and lat["tpot_ms"]["p99"] < 50
    out = served.result_json(args, 1, "xpool", {"layout": "fake", "name": "b"}, streams, agg, {}, "digest")
    assert out["steps"] == 4 and out["value"] > 0 and out["e2e"]["value"] > 0 and out["valid"]
    assert out["e2e"]["h2d_bytes_per_step"] > 0 and out["gpu_launches"] > 0
    # the two throughput figures come from different clocks and observation points but describe the same windows
    assert 0.5 < out["e2e"]["value"] / out["value"] < 2.0


def test_slo_violation_marks_the_result_invalid():
    recs = [{"model": "m", "arrival": 0.2, "n_prompt": 3, "n_out": 4, "done": True, "first": 3.0, "last": 3.3, "n": 4,
             "times": [3.0, 3.1, 3.2, 3.3]}]
    lat = served.latency_summary(recs, 0.0, 5.0)
    assert not lat["slo_met"] and lat["slo_attained"] == 0.0
    # a request that never got a token and has waited longer than the limit counts against the TTFT percentile
    recs.append({"model": "m", "arrival": 0.1, "n_prompt": 3, "n_out": 4, "done": False, "first": None, "last": None, "n": 0, "times": []})
    assert served.latency_summary(recs, 0.0, 5.0)["ttft_ms"]["n"] == 2


def test_vs_baseline_comes_from_the_recorded_library_arm_of_the_same_mix_and_load():
    import argparse

    base = argparse.Namespace(rate_scale=1.0, max_batch=0, kv_tokens=0, layers=0)
    rec = served.recorded_baseline("b", 1, base)
    assert rec is not None and rec["value"] > 0 and rec["slo_met"] is True and "--impl baseline" in rec["command"]
    assert served.recorded_baseline("b", 3, base) is None                               # never measured: no ratio
    assert served.recorded_baseline("b", 1, argparse.Namespace(rate_scale=1.5, max_batch=0, kv_tokens=0, layers=0)) is None
    assert served.recorded_baseline("b", 1, argparse.Namespace(rate_scale=1.0, max_batch=0, kv_tokens=0, layers=2)) is None


def test_progress_watchdog_ends_a_stuck_run_with_an_error_line_and_stays_quiet_when_cancelled():
    import subprocess
    import sys

    code = ("import time, json\n"
            "from crosspool_b200.bench.served import _ProgressWatchdog\n"
            "w = _ProgressWatchdog('baseline', 0)\n"
            "w.phase('a', 30.0); w.phase('b', 0.2)\n"
            "time.sleep(5)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "baseline" and "phase 'b'" in line["error"][0]
    ok = ("import time\n"
          "from crosspool_b200.bench.served import _ProgressWatchdog\n"
          "w = _ProgressWatchdog('xpool', 1)\n"
          "w.phase('a', 0.2); w.cancel(); time.sleep(0.6); print('done')\n")
    r = subprocess.run([sys.executable, "-c", ok], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == "done"
