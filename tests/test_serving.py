"""Serving loop + HTTP API + open-loop benchmark client against a fake (CPU) deployment."""
import asyncio
import random
import time

import httpx
import pytest

from crosspool_b200.bench import serving as B
from crosspool_b200.runtime.serving import EngineLoop, create_serving_app


class FakeSeq:
    def __init__(self, sid, n):
        self.seq_id, self.n, self.done = sid, n, 0

    @property
    def finished(self):
        return self.done >= self.n


class FakeResult:
    def __init__(self, tokens):
        self.tokens = tokens


class FakeDeployment:
    """Every step gives each live request one token (value = prompt length + index)."""

    def __init__(self, step_s=0.001):
        self.live, self.next_id, self.step_s = {}, 0, step_s

    def add_request(self, model_id, prompt, max_new_tokens, arrival=None):
        if not prompt:
            raise ValueError("empty prompt")
        s = FakeSeq(self.next_id, max_new_tokens)
        s.base = len(prompt)
        self.next_id += 1
        self.live[(model_id, s.seq_id)] = s
        return s

    @property
    def has_work(self):
        return bool(self.live)

    def step(self):
        time.sleep(self.step_s)
        out = {}
        for (m, sid), s in list(self.live.items()):
            s.done += 1
            out.setdefault(m, []).append((s, s.base + s.done))
            if s.finished:
                del self.live[(m, sid)]
        return FakeResult(out)


@pytest.fixture()
def served():
    loop = EngineLoop(FakeDeployment())
    loop.start()
    app = create_serving_app(loop, ["a", "b"])
    yield app, loop
    loop.stop()


def test_generate_plain_and_streaming(served):
    app, loop = served

    async def go():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=app), base_url="http://t") as c:
            r = await c.post("/generate", json={"model": "a", "input_ids": [1, 2, 3], "max_new_tokens": 4})
            assert r.status_code == 200 and r.json()["output_ids"] == [4, 5, 6, 7]
            assert (await c.post("/generate", json={"model": "zzz", "input_ids": [1]})).status_code == 404
            assert (await c.post("/generate", json={"model": "a", "input_ids": []})).status_code == 422
            toks = []
            async with c.stream("POST", "/generate", json={"model": "b", "input_ids": [9] * 10, "max_new_tokens": 3,
                                                         "stream": True}) as s:
                async for line in s.aiter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        toks.append(__import__("json").loads(line[6:]))
            assert [t["token_id"] for t in toks] == [11, 12, 13] and toks[-1]["finished"] is True
            assert (await c.get("/health")).json()["tokens"] >= 7

    asyncio.run(go())


def test_workload_is_deterministic_and_respects_distributions():
    s = [B.StreamSpec("a", 20.0, B.LengthSpec("lognormal", 16, 4096, 512, 1.0), B.LengthSpec("uniform", 8, 32),
                      vocab_size=1000, max_output_input_ratio=2.0),
         B.StreamSpec("b", 5.0, B.LengthSpec("uniform", 100, 200), B.LengthSpec("uniform", 4, 4), vocab_size=1000,
                      burst_factor=4.0, burst_seconds=2.0, burst_period=10.0)]
    w1, w2 = B.plan_workload(s, 20.0, seed=7, warmup_requests=2), B.plan_workload(s, 20.0, seed=7, warmup_requests=2)
    assert B.workload_digest(w1) == B.workload_digest(w2) != B.workload_digest(B.plan_workload(s, 20.0, seed=8))
    a = [r for r in w1 if r.model == "a" and not r.warmup]
    assert 300 < len(a) < 500  # Poisson, 20 req/s for 20 s
    lens = sorted(len(r.prompt) for r in a)
    assert 16 <= lens[0] and lens[-1] <= 4096 and 350 < lens[len(lens) // 2] < 750  # median near 512
    assert all(r.max_new_tokens <= 2 * len(r.prompt) for r in a)
    assert sum(r.warmup for r in w1) == 4 and all(r.arrival_s == 0 for r in w1 if r.warmup)
    b = [r.arrival_s for r in w1 if r.model == "b" and not r.warmup]
    in_burst = sum(1 for t in b if t % 10 < 2)
    assert in_burst / len(b) > 0.3  # 20% of the time, 4x the rate -> half of the arrivals
    assert [r.arrival_s for r in a] == sorted(r.arrival_s for r in a)


def test_open_loop_client_measures_ttft_tpot_and_percentiles(served):
    app, loop = served
    streams = [B.StreamSpec(m, 40.0, B.LengthSpec("uniform", 4, 8), B.LengthSpec("uniform", 5, 9), vocab_size=100)
               for m in ("a", "b")]
    reqs = B.plan_workload(streams, 1.0, seed=1, warmup_requests=1)
    recs, window = asyncio.run(B.run_client({"a": "http://t", "b": "http://t"}, reqs, transport=httpx.ASGITransport(app=app)))
    rep = B.summarize(recs, window, slo_ttft_ms=2000, slo_tpot_ms=50)
    assert rep["errors"] == 0 and rep["completed"] == len([r for r in reqs if not r.warmup])
    assert rep["output_tokens"] == sum(r.max_new_tokens for r in reqs if not r.warmup)
    assert 0 < rep["tpot_ms"]["p50"] < 50 and rep["http_ttft_ms"]["p99"] >= rep["http_ttft_ms"]["p50"] > 0
    assert rep["slo"]["attained"] > 0.9 and rep["output_tok_per_s"] > 100
    for r in recs:
        assert r.sent >= r.planned_arrival - 1e-3 and r.first_token >= r.sent


def test_percentile_is_linear_rank():
    from crosspool_b200.deployment import percentile

    assert percentile([1, 2, 3, 4], 50) == 2.5 and percentile([10], 99) == 10 and percentile([0, 10], 90) == 9.0


def test_metrics_are_prometheus_text_and_a_broken_statistic_cannot_stop_the_loop(served):
    import types

    from fastapi.testclient import TestClient

    from crosspool_b200.runtime.metrics import InstanceMetrics

    app, loop = served
    with TestClient(app) as http:
        assert http.post("/generate", json={"model": "a", "input_ids": [1, 2, 3], "max_new_tokens": 4}).status_code == 200
        text = http.get("/metrics").text
        # the fake sequences carry no timing: requests are counted, histograms stay empty, serving went on
        assert 'xpool_requests_finished_total{model="a"} 1' in text and "xpool_engine_steps_total" in text
        assert "xpool_requests_in_flight 0" in text and "xpool_engine_failed 0" in text
    m = InstanceMetrics()
    seq = types.SimpleNamespace(prompt=[1] * 10, generated=[5] * 5, arrival=100.0, first_token_time=100.03, finish_time=100.11)
    m.finished("x/y", seq)
    m.finished("x/y", types.SimpleNamespace(prompt=[1], generated=[2], arrival=1.0, first_token_time=1.5, finish_time=1.5))
    out = m.render()
    assert 'xpool_time_to_first_token_seconds_bucket{le="0.05",model="x/y"} 1' in out
    assert 'xpool_time_to_first_token_seconds_bucket{le="+Inf",model="x/y"} 2' in out
    assert 'xpool_time_per_output_token_seconds_bucket{le="0.02",model="x/y"} 1' in out          # (0.11 - 0.03) / 4 = 20 ms
    assert 'xpool_time_per_output_token_seconds_count{model="x/y"} 1' in out                      # one-token answers have no TPOT
    assert 'xpool_prompt_tokens_total{model="x/y"} 11' in out and out.endswith("\n")
    for line in out.splitlines():
        assert line.startswith("#") or len(line.rsplit(" ", 1)) == 2
