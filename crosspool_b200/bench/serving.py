"""Serving benchmark: deterministic open-loop workload, streaming client, latency metrics.

Mirrors the reference's xbench methodology (docs/designs/benchmark.md:111-193,
src/xpool-dev/xbench/harness/serving/{workload,client,measure}.py):

* per-(seed, model, purpose) RNGs derived with SHA-256; Poisson arrivals by ``expovariate(rate)`` until
  ``duration``; token counts from a truncated log-normal by inverse-CDF sampling inside the legal
  interval (or uniform); prompts are uniform random token ids;
* an open-loop producer releases each request at its planned arrival time; ``max_inflight`` workers
  stream ``POST /generate``;
* per request: HTTP TTFT (send -> first token), arrival TTFT (planned arrival -> first token), ITL
  samples, TPOT = (completion - first token) / (N - 1); percentiles by linear rank
  ``(n - 1) * p / 100``; output throughput attributed at observation time; warm-up requests are
  separate and excluded from the window.

``python -m crosspool_b200.bench.serving --targets model=http://127.0.0.1:30000 --rate 4 ...``
"""

from __future__ import annotations

import argparse
import asyncio
import hashlib
import json
import math
import random
import time
from dataclasses import dataclass, field
from statistics import NormalDist

from ..deployment import percentile


def derive_rng(seed: int, model: str, purpose: str) -> random.Random:
    h = hashlib.sha256(f"{seed}|{model}|{purpose}".encode()).digest()
    return random.Random(int.from_bytes(h[:8], "big"))


@dataclass(frozen=True)
class LengthSpec:
    """``kind`` = ``uniform`` (lo..hi) or ``lognormal`` (median, sigma, truncated to lo..hi)."""

    kind: str
    lo: int
    hi: int
    median: float = 0.0
    sigma: float = 1.0

    def sample(self, rng: random.Random) -> int:
        if self.kind == "uniform":
            return rng.randint(self.lo, self.hi)
        # inverse-CDF sampling of a log-normal truncated to [lo, hi]
        nd = NormalDist(math.log(self.median), self.sigma)
        a, b = nd.cdf(math.log(max(self.lo, 1))), nd.cdf(math.log(self.hi))
        u = a + (b - a) * rng.random()
        u = min(max(u, 1e-12), 1 - 1e-12)
        return int(min(self.hi, max(self.lo, round(math.exp(nd.inv_cdf(u))))))


@dataclass
class PlannedRequest:
    model: str
    arrival_s: float
    prompt: list[int]
    max_new_tokens: int
    warmup: bool = False


@dataclass
class StreamSpec:
    model: str
    rate_per_s: float
    prompt: LengthSpec
    output: LengthSpec
    vocab_size: int = 151936
    burst_factor: float = 1.0      # rate multiplier inside bursts
    burst_seconds: float = 0.0     # burst length ...
    burst_period: float = 0.0      # ... in every period
    max_output_input_ratio: float = 0.0


def plan_workload(streams: list[StreamSpec], duration_s: float, seed: int, warmup_requests: int = 0) -> list[PlannedRequest]:
    out: list[PlannedRequest] = []
    for s in streams:
        arr, plen, olen, tok = (derive_rng(seed, s.model, p) for p in ("arrivals", "prompt_len", "output_len", "tokens"))
        t = 0.0
        while True:
            rate = s.rate_per_s
            if s.burst_period > 0 and (t % s.burst_period) < s.burst_seconds:
                rate *= s.burst_factor
            t += arr.expovariate(rate)
            if t >= duration_s:
                break
            n_in = s.prompt.sample(plen)
            n_out = s.output.sample(olen)
            if s.max_output_input_ratio > 0:
                n_out = max(1, min(n_out, int(n_in * s.max_output_input_ratio)))
            out.append(PlannedRequest(s.model, t, [tok.randrange(s.vocab_size) for _ in range(n_in)], n_out))
        wr = derive_rng(seed, s.model, "warmup")
        for _ in range(warmup_requests):
            out.append(PlannedRequest(s.model, 0.0, [wr.randrange(s.vocab_size) for _ in range(s.prompt.sample(wr))],
                                      max(1, min(8, s.output.lo)), warmup=True))
    out.sort(key=lambda r: (r.warmup is False, r.arrival_s))
    return out


def workload_digest(reqs: list[PlannedRequest]) -> str:
    h = hashlib.sha256()
    for r in reqs:
        h.update(f"{r.model}|{r.arrival_s:.9f}|{r.max_new_tokens}|{len(r.prompt)}|{sum(r.prompt)}|{r.warmup}".encode())
    return h.hexdigest()


@dataclass
class RequestRecord:
    model: str
    planned_arrival: float
    sent: float = 0.0
    first_token: float = 0.0
    completed: float = 0.0
    token_times: list[float] = field(default_factory=list)
    n_prompt: int = 0
    error: str | None = None

    @property
    def ok(self) -> bool:
        return self.error is None and len(self.token_times) > 0

    @property
    def http_ttft(self) -> float:
        return self.first_token - self.sent

    @property
    def arrival_ttft(self) -> float:
        return self.first_token - self.planned_arrival

    @property
    def tpot(self) -> float | None:
        n = len(self.token_times)
        return (self.completed - self.first_token) / (n - 1) if n > 1 else None

    @property
    def itl(self) -> list[float]:
        return [b - a for a, b in zip(self.token_times, self.token_times[1:])]


def summarize(records: list[RequestRecord], window_s: float, slo_ttft_ms: float = 0.0, slo_tpot_ms: float = 0.0) -> dict:
    ok = [r for r in records if r.ok]

    def dist(vals: list[float]) -> dict:
        ms = [v * 1e3 for v in vals]
        return {"n": len(ms), "p50": percentile(ms, 50), "p90": percentile(ms, 90), "p95": percentile(ms, 95),
                "p99": percentile(ms, 99), "mean": sum(ms) / len(ms) if ms else float("nan")}

    tokens = sum(len(r.token_times) for r in ok)
    out = {"requests": len(records), "completed": len(ok), "errors": len(records) - len(ok), "output_tokens": tokens,
           "output_tok_per_s": tokens / window_s if window_s > 0 else float("nan"),
           "http_ttft_ms": dist([r.http_ttft for r in ok]), "arrival_ttft_ms": dist([r.arrival_ttft for r in ok]),
           "tpot_ms": dist([r.tpot for r in ok if r.tpot is not None]), "itl_ms": dist([x for r in ok for x in r.itl])}
    if slo_ttft_ms and slo_tpot_ms and ok:
        good = [r for r in ok if r.arrival_ttft * 1e3 <= slo_ttft_ms and (r.tpot is None or r.tpot * 1e3 <= slo_tpot_ms)]
        out["slo"] = {"ttft_ms": slo_ttft_ms, "tpot_ms": slo_tpot_ms, "attained": len(good) / len(ok),
                      "goodput_tok_per_s": sum(len(r.token_times) for r in good) / window_s,
                      "p99_tpot_within_slo": out["tpot_ms"]["p99"] <= slo_tpot_ms,
                      "p99_ttft_within_slo": out["arrival_ttft_ms"]["p99"] <= slo_ttft_ms}
    return out


async def _one(client, url: str, req: PlannedRequest, rec: RequestRecord, t0: float) -> None:
    rec.sent = time.perf_counter() - t0
    try:
        async with client.stream("POST", url + "/generate", json={"model": req.model, "input_ids": req.prompt,
                                                                "max_new_tokens": req.max_new_tokens, "stream": True}) as r:
            if r.status_code != 200:
                rec.error = f"HTTP {r.status_code}"
                return
            async for line in r.aiter_lines():
                if not line.startswith("data: "):
                    continue
                body = line[6:]
                if body == "[DONE]":
                    break
                ev = json.loads(body)
                if "error" in ev:
                    rec.error = ev["error"]
                    return
                now = time.perf_counter() - t0
                if not rec.token_times:
                    rec.first_token = now
                rec.token_times.append(now)
        rec.completed = rec.token_times[-1] if rec.token_times else 0.0
    except Exception as e:  # network failure is a failed request, not a crashed benchmark
        rec.error = f"{type(e).__name__}: {e}"


async def run_client(targets: dict[str, str], reqs: list[PlannedRequest], max_inflight: int = 1024, transport=None,
                     time_scale: float = 1.0) -> tuple[list[RequestRecord], float]:
    """Open-loop replay. ``targets`` maps model -> base URL. Returns (records of the measured
    requests, window seconds). ``time_scale`` < 1 compresses the planned timeline (tests)."""
    import httpx

    sem = asyncio.Semaphore(max_inflight)
    limits = httpx.Limits(max_connections=max_inflight, max_keepalive_connections=max_inflight)
    async with httpx.AsyncClient(timeout=httpx.Timeout(300.0, pool=None), transport=transport, limits=limits) as client:
        warm = [r for r in reqs if r.warmup]
        t0 = time.perf_counter()
        await asyncio.gather(*[_one(client, targets[r.model], r, RequestRecord(r.model, 0.0), t0) for r in warm])
        measured = [r for r in reqs if not r.warmup]
        records = [RequestRecord(r.model, r.arrival_s * time_scale, n_prompt=len(r.prompt)) for r in measured]
        t0 = time.perf_counter()

        async def launch(r: PlannedRequest, rec: RequestRecord):
            delay = rec.planned_arrival - (time.perf_counter() - t0)
            if delay > 0:
                await asyncio.sleep(delay)
            async with sem:
                await _one(client, targets[r.model], r, rec, t0)

        await asyncio.gather(*[launch(r, rec) for r, rec in zip(measured, records)])
        window = max([rec.completed for rec in records if rec.ok] + [1e-9])
    return records, window


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="xpool bench")
    ap.add_argument("--targets", nargs="+", required=True, help="model=http://host:port ...")
    ap.add_argument("--rate", type=float, nargs="+", default=[1.0], help="requests/s per model (one value or one per model)")
    ap.add_argument("--duration", type=float, default=60.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prompt", default="uniform:128:2048", help="uniform:lo:hi | lognormal:median:sigma:lo:hi")
    ap.add_argument("--output", default="uniform:128:512")
    ap.add_argument("--warmup-requests", type=int, default=2)
    ap.add_argument("--max-inflight", type=int, default=1024)
    ap.add_argument("--slo-ttft-ms", type=float, default=2000.0)
    ap.add_argument("--slo-tpot-ms", type=float, default=50.0)
    ap.add_argument("--burst", default="", help="factor:seconds:period, e.g. 4:30:120")
    ap.add_argument("--out", default="")
    ns = ap.parse_args(argv)

    def spec(s: str) -> LengthSpec:
        p = s.split(":")
        if p[0] == "uniform":
            return LengthSpec("uniform", int(p[1]), int(p[2]))
        return LengthSpec("lognormal", int(p[3]), int(p[4]), float(p[1]), float(p[2]))

    targets = dict(t.split("=", 1) for t in ns.targets)
    rates = ns.rate if len(ns.rate) == len(targets) else [ns.rate[0]] * len(targets)
    bf, bs, bp = (float(x) for x in ns.burst.split(":")) if ns.burst else (1.0, 0.0, 0.0)
    streams = [StreamSpec(m, r, spec(ns.prompt), spec(ns.output), burst_factor=bf, burst_seconds=bs, burst_period=bp)
               for m, r in zip(targets, rates)]
    reqs = plan_workload(streams, ns.duration, ns.seed, ns.warmup_requests)
    records, window = asyncio.run(run_client(targets, reqs, ns.max_inflight))
    report = {"digest": workload_digest(reqs), "window_s": window,
              "aggregate": summarize(records, window, ns.slo_ttft_ms, ns.slo_tpot_ms),
              "per_model": {m: summarize([r for r in records if r.model == m], window, ns.slo_ttft_ms, ns.slo_tpot_ms)
                            for m in targets}}
    text = json.dumps(report, indent=2)
    if ns.out:
        open(ns.out, "w").write(text)
    print(text)
    return 0 if report["aggregate"]["errors"] == 0 else 3


if __name__ == "__main__":
    raise SystemExit(main())
