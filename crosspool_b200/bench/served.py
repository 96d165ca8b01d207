"""Served-throughput benchmark: open-loop Poisson arrivals through the serving loop, SLO-gated.

This is what ``bench.py`` at the repository root runs. Every attention rank hosts its Instances in one
:class:`~crosspool_b200.deployment.Deployment` driven by an :class:`~crosspool_b200.runtime.serving.EngineLoop`
(admission, chunked prefill and decode interleaved, elastic KV where the mix says so); a producer on the same
rank releases each planned request at its arrival time with ``EngineLoop.submit`` -- the call the HTTP layer makes
for ``POST /generate`` -- and receives every token with the host time at which it left the engine. Workload
planning, length distributions and metric definitions are the ones of :mod:`crosspool_b200.bench.serving`
(the reference's xbench rules: src/xpool-dev/xbench/harness/serving/workload.py:162-197,328-341 and
measure.py:355-388,431-460).

A *step* of this benchmark is one scheduling interval of ``--step-seconds`` (0.5 s) of offered traffic, during
which every engine performs many iterations. ``--warmup W`` intervals of traffic bring the deployment to its
steady state (running batches filled, KV occupied); then three windows of exactly ``--steps K`` intervals each
are measured back to back, and the reported value is the median window.

Two measurements come from the same windows:

* ``value``: output tokens produced by the engines between the window's two boundary marks, divided by the device
  time between the CUDA events recorded at those marks (maximum over attention ranks);
* ``e2e.value``: output tokens *observed by the producer* (host clock, after the step's device-to-host copy of the
  sampled tokens and the loop's bookkeeping) inside the window, per second of wall time. TTFT is planned arrival to
  first observed token, TPOT is (last - first) / (n - 1) over finished requests.

Every engine step copies its inputs (token ids, positions, KV slots, lengths, block table) from pinned host memory
to the device and reads its sampled tokens back; both byte counts are reported per interval.
"""

from __future__ import annotations

import heapq
import json
import os
import statistics
import sys
import threading
import time
from dataclasses import dataclass, field

import torch

from ..deployment import Deployment, InstanceHandle, percentile
from ..engine.atn_engine import AttentionEngine, EngineConfig
from ..models import config as mc
from .decode_bench import ClockSampler
from .serving import LengthSpec, PlannedRequest, StreamSpec, plan_workload, workload_digest

PAGE = 64   # tokens per KV page: one TMA copy brings a whole 64-token K (or V) tile of the prefill attention
METRIC = "aggregate output tok/s across co-located models at p99 TPOT SLO; p50 TTFT"
SLO_TTFT_MS, SLO_TPOT_MS = 2000.0, 50.0
WINDOWS = 3


# ------------------------------------------------------------------------------------------- model mixes

@dataclass
class ModelStream:
    """One Instance of the mix: where it runs, how it is sized and what traffic it receives."""

    model_id: str
    preset: str
    seed: int
    atn_rank: int
    ffn_ranks: tuple[int, ...]
    rate: float
    prompt: LengthSpec
    output: LengthSpec
    max_batch: int
    max_seq_len: int
    kv_tokens: int                      # KV capacity in tokens (fixed cache) or reservation (elastic)
    prefill_chunk: int = 4096
    burst: tuple[float, float, float] = (1.0, 0.0, 0.0)   # factor, seconds, period
    elastic: bool = False
    # demand swap (two models trading places every ``swap_period`` seconds): the alternate traffic shape
    alt_rate: float = 0.0
    alt_prompt: LengthSpec | None = None
    alt_output: LengthSpec | None = None
    swap_phase: int = 0                 # 0: starts with the primary shape, 1: starts with the alternate
    weights_key: str | None = None      # Instances with the same key share one copy of the FFN weights per FFN rank
    preload_tokens: int = 0             # cap on the prompt tokens of the time-0 backlog (0: no cap)


def _uniform(lo, hi):
    return LengthSpec("uniform", lo, hi)


def _lognormal(median, lo, hi, sigma=1.0):
    return LengthSpec("lognormal", lo, hi, float(median), sigma)


def build_mix(name: str, world: int, scale: float, max_batch: int = 0, kv_tokens: int = 0) -> tuple[list[ModelStream], dict]:
    """The Instances and traffic of a named mix on ``world`` GPUs. ``scale`` multiplies every arrival rate;
    ``max_batch`` / ``kv_tokens`` override every Instance's running-request limit and KV capacity (0: the mix's own)."""
    streams, info = _build_mix(name, world, scale)
    for s in streams:
        s.max_batch = max_batch or s.max_batch
        s.kv_tokens = kv_tokens or s.kv_tokens
    return streams, info


def _build_mix(name: str, world: int, scale: float) -> tuple[list[ModelStream], dict]:
    b_prompt, b_out = _uniform(128, 2048), _uniform(128, 512)
    if name == "b":
        # Qwen3-0.6B, prompts uniform 128-2048, outputs uniform 128-512 (ignore-eos), Poisson arrivals;
        # one Instance per attention GPU. 1 GPU: loopback. N GPUs: N/2 attention + N/2 FFN ranks (N = 2: 1 + 1).
        n_atn = 1 if world <= 2 else world // 2
        n_ffn = world - n_atn
        out = []
        for a in range(n_atn):
            ffn = (n_atn + a % n_ffn,) if n_ffn else ()
            out.append(ModelStream(f"Qwen/Qwen3-0.6B#{a}", "Qwen/Qwen3-0.6B", a, a, ffn, 72.0 * scale, b_prompt, b_out,
                                   max_batch=768, max_seq_len=2048 + 512 + PAGE, kv_tokens=1152 * 1024))
        return out, {"name": "b", "layout": f"atn{n_atn}+ffn{n_ffn}" if n_ffn else "loopback",
                     "slo": {"ttft_ms": SLO_TTFT_MS, "tpot_ms": SLO_TPOT_MS}}
    if name == "c":
        # Qwen3-8B + Qwen3-0.6B sharing each attention GPU with elastic KV; FFN of the 8B tensor-parallel over the
        # 2-GPU FFN tier, the 0.6B on one rank of it. The two models trade long-context and short-context traffic
        # every window. On 2 GPUs the FFN tier is the one other GPU (8B untiled), a reduced form for bring-up.
        if world < 2:
            raise SystemExit("mix c needs at least 2 GPUs (1 attention + 1 FFN; 2 FFN from 3 GPUs on)")
        n_atn = max(1, world - 2)
        f0, f1 = n_atn, min(n_atn + 1, world - 1)
        long_p, long_o = _lognormal(8192, 256, 32768), _uniform(256, 256)
        short_p, short_o = _uniform(256, 256), _uniform(128, 128)
        out = []
        # 4 req/s of long-context and 32 req/s of short-context traffic for the whole deployment: every attention GPU
        # (each hosts its own pair of Instances) receives an equal share of both
        r_long, r_short = 4.0 * scale / n_atn, 32.0 * scale / n_atn
        for a in range(n_atn):
            common = dict(max_seq_len=32768 + 256 + PAGE, prefill_chunk=4096, elastic=True, alt_rate=r_short, alt_prompt=short_p,
                          alt_output=short_o, max_batch=128, kv_tokens=512 * 1024)
            out.append(ModelStream(f"Qwen/Qwen3-8B#{a}", "Qwen/Qwen3-8B", 10 + a, a, (f0, f1) if f1 != f0 else (f0,), r_long,
                                   long_p, long_o, swap_phase=0, preload_tokens=24 * 1024, **common))
            out.append(ModelStream(f"Qwen/Qwen3-0.6B#{a}", "Qwen/Qwen3-0.6B", 20 + a, a, (f0 if a % 2 == 0 else f1,), r_long,
                                   long_p, long_o, swap_phase=1, preload_tokens=96 * 1024, **common))
        return out, {"name": "c", "layout": f"atn{n_atn} (8B + 0.6B each, elastic KV) + ffn2 (8B TP2)",
                     "slo": {"ttft_ms": SLO_TTFT_MS, "tpot_ms": SLO_TPOT_MS}}
    if name == "d":
        # Qwen3-30B-A3B: attention data-parallel over half of the GPUs (one Instance rank each, requests spread evenly:
        # every rank has its own Poisson stream of a quarter of the load), experts expert-parallel over the other half
        # (one copy of the expert weights serves every data-parallel rank). Prompts uniform 512-4096, outputs 256-1024.
        if world < 2 or world % 2:
            raise SystemExit("mix d needs an even number of GPUs (half attention DP ranks, half expert-parallel FFN ranks)")
        n_atn = world // 2
        ffn = tuple(range(n_atn, world))
        out = [ModelStream(f"Qwen/Qwen3-30B-A3B#dp{a}", "Qwen/Qwen3-30B-A3B", 40, a, ffn, 6.0 * scale, _uniform(512, 4096),
                           _uniform(256, 1024), max_batch=256, max_seq_len=4096 + 1024 + PAGE, kv_tokens=768 * 1024,
                           weights_key="Qwen/Qwen3-30B-A3B", preload_tokens=64 * 1024) for a in range(n_atn)]
        return out, {"name": "d", "layout": f"attention DP{n_atn} + experts EP{n_atn} (128 experts, top-8)",
                     "slo": {"ttft_ms": SLO_TTFT_MS, "tpot_ms": SLO_TPOT_MS}}
    if name == "e":
        # Four models on 8 GPUs: attention on ranks 0-1 (elastic KV per GPU), FFN tier on ranks 2-7:
        # Qwen3-32B TP4 on 2-5, Qwen3-8B TP2 on 6-7, the two Qwen3-1.7B on 6 and 7. Rates 1:2:4:4, 4x bursts.
        if world != 8:
            raise SystemExit("mix e is defined for 8 GPUs")
        p, o = _lognormal(1024, 16, 8192), _uniform(128, 1024)
        common = dict(prompt=p, output=o, max_seq_len=8192 + 1024 + PAGE, elastic=True, burst=(4.0, 0.0, 0.0))
        r = 2.0 * scale
        out = [
            ModelStream("Qwen/Qwen3-32B#0", "Qwen/Qwen3-32B", 30, 0, (2, 3, 4, 5), r, max_batch=192, kv_tokens=320 * 1024, preload_tokens=16 * 1024, **common),
            ModelStream("Qwen/Qwen3-1.7B#0", "Qwen/Qwen3-1.7B", 31, 0, (6,), 4 * r, max_batch=256, kv_tokens=448 * 1024,
                        preload_tokens=96 * 1024, **common),
            ModelStream("Qwen/Qwen3-8B#0", "Qwen/Qwen3-8B", 32, 1, (6, 7), 2 * r, max_batch=256, kv_tokens=448 * 1024,
                        preload_tokens=32 * 1024, **common),
            ModelStream("Qwen/Qwen3-1.7B#1", "Qwen/Qwen3-1.7B", 33, 1, (7,), 4 * r, max_batch=256, kv_tokens=448 * 1024,
                        preload_tokens=96 * 1024, **common),
        ]
        return out, {"name": "e", "layout": "atn2 (32B + 1.7B | 8B + 1.7B, elastic KV) + ffn6 (32B TP4, 8B TP2, 1.7B x2)",
                     "burst": "4x for a quarter of every window", "slo": {"ttft_ms": SLO_TTFT_MS, "tpot_ms": SLO_TPOT_MS}}
    raise SystemExit(f"unknown mix {name!r} (b, c, d, e)")


def default_mix(world: int) -> str:
    return {1: "b", 2: "b", 4: "c", 8: "e"}.get(world, "b")


def _mean(spec: LengthSpec) -> float:
    if spec.kind == "uniform":
        return (spec.lo + spec.hi) / 2
    return min(spec.hi, spec.median * 1.65)     # log-normal with sigma 1: mean = median * e^0.5


def preload_requests(s: ModelStream, seed: int, tpot_estimate_s: float = 0.02, fraction: float = 0.8) -> list[PlannedRequest]:
    """Requests released at time 0 so that the warm-up intervals start near the steady state instead of an empty
    deployment: about ``fraction`` of the concurrency that Little's law gives for the stream (arrival rate x output
    length x time per token), each with a uniformly drawn share of its output still to produce, as requests caught
    mid-flight would have. They arrive before the first measured window, so they never enter the latency statistics."""
    from .serving import derive_rng

    rng = derive_rng(seed, s.model_id, "preload")
    vocab = mc.load(s.preset).vocab_size
    n = min(s.max_batch, int(fraction * s.rate * _mean(s.output) * tpot_estimate_s))
    out, tokens = [], 0
    for _ in range(n):
        n_in = s.prompt.sample(rng)
        if s.preload_tokens and tokens + n_in > s.preload_tokens:
            break       # a backlog that takes longer to prefill than the warm-up lasts would delay the measured arrivals
        tokens += n_in
        n_out = max(1, int(s.output.sample(rng) * rng.uniform(0.05, 1.0)))
        out.append(PlannedRequest(s.model_id, 0.0, [rng.randrange(vocab) for _ in range(n_in)], n_out, warmup=True))
    return out


def plan_streams(streams: list[ModelStream], total_s: float, window_s: float, seed: int, preload: bool = False
                 ) -> list[PlannedRequest]:
    """Planned arrivals for every Instance over ``total_s`` seconds. Bursts repeat every window; Instances with an
    alternate shape swap shapes every window. ``preload`` adds each stream's time-0 backlog (``preload_requests``)."""
    reqs: list[PlannedRequest] = []
    for s in streams:
        vocab = mc.load(s.preset).vocab_size
        if preload:
            reqs += preload_requests(s, seed)
        if s.alt_prompt is None:
            bf, bs, bp = s.burst
            if bf > 1.0 and bp <= 0:
                bs, bp = window_s / 4, window_s      # a burst for the first quarter of every window
            reqs += plan_workload([StreamSpec(s.model_id, s.rate, s.prompt, s.output, vocab_size=vocab, burst_factor=bf,
                                              burst_seconds=bs, burst_period=bp)], total_s, seed)
            continue
        # alternating shapes: plan both for the whole run, keep each only in its own windows
        prim = plan_workload([StreamSpec(s.model_id, s.rate, s.prompt, s.output, vocab_size=vocab)], total_s, seed)
        alt = plan_workload([StreamSpec(s.model_id, s.alt_rate, s.alt_prompt, s.alt_output, vocab_size=vocab)], total_s,
                            seed + 1)
        for r in prim:
            if (int(r.arrival_s // window_s) + s.swap_phase) % 2 == 0:
                reqs.append(r)
        for r in alt:
            if (int(r.arrival_s // window_s) + s.swap_phase) % 2 == 1:
                reqs.append(r)
    reqs.sort(key=lambda r: r.arrival_s)
    return reqs


# ------------------------------------------------------------------------------------------- rank-local serving

@dataclass
class Rec:
    model: str
    arrival: float            # planned arrival, seconds from the common start
    n_prompt: int
    n_out: int
    times: list[float] = field(default_factory=list)
    done: bool = False


class _HostEvent:
    """Stands in for a CUDA event when the deployment under test is a CPU fake."""

    def __init__(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other: "_HostEvent") -> float:
        return (other.t - self.t) * 1e3


@dataclass
class Mark:
    t_host: float
    event: object
    tokens: int
    stats: dict
    launches: int


class RankServing:
    """Plays the planned requests of this rank's Instances against its EngineLoop and records marks."""

    def __init__(self, dep: Deployment, reqs: list[PlannedRequest], device, on_tick=None):
        from ..runtime.serving import EngineLoop

        self.dep, self.reqs, self.device = dep, reqs, torch.device(device)
        self.loop = EngineLoop(dep, sink=self._sink)
        self.recs: list[Rec] = []
        self.tokens = 0
        self.marks: list[Mark] = []
        self._cuda = self.device.type == "cuda"
        self._tstream = torch.cuda.Stream(self.device) if self._cuda else None
        self._on_tick = on_tick
        self.t0 = 0.0

    def _sink(self, batch, now: float) -> None:
        t = now - self.t0
        for p, (tok, done) in batch:
            rec = p.tag
            rec.times.append(t)
            if done:
                rec.done = True
        self.tokens += len(batch)

    def _mark(self) -> None:
        if not self._cuda:
            self.marks.append(Mark(time.perf_counter() - self.t0, _HostEvent(), self.tokens, dict(self.dep.stats()), 0))
            return
        from .. import native

        ev = torch.cuda.Event(enable_timing=True)
        for i in self.dep.instances:           # between steps every engine stream is idle; order the event after them
            self._tstream.wait_stream(i.engine.stream)
        ev.record(self._tstream)
        self.marks.append(Mark(time.perf_counter() - self.t0, ev, self.tokens, dict(self.dep.stats()), native.launch_count()))

    def run(self, t0: float, boundaries: list[float], end_s: float) -> None:
        """``t0``: the common start on this host's ``perf_counter`` clock. Blocks until ``end_s``."""
        self.t0 = t0
        self.loop.start()
        events = [(r.arrival_s, 1, i) for i, r in enumerate(self.reqs)] + [(b, 0, -1) for b in boundaries]
        heapq.heapify(events)
        while events:
            at, kind, i = heapq.heappop(events)
            if at > end_s and kind == 1:
                break
            delay = t0 + at - time.perf_counter()
            if delay > 0:
                time.sleep(delay)
            if self.loop.error is not None:
                raise RuntimeError(f"engine loop failed: {self.loop.error!r}")
            if kind == 0:
                done = threading.Event()
                self.loop.call_between_steps(lambda d=done: (self._mark(), d.set()))
                if not done.wait(60):
                    raise RuntimeError("the engine loop did not reach a window boundary within 60 s")
                continue
            r = self.reqs[i]
            rec = Rec(r.model, r.arrival_s, len(r.prompt), r.max_new_tokens)
            self.recs.append(rec)
            self.loop.submit(r.model, r.prompt, r.max_new_tokens, queued=False, tag=rec)
        self.loop.stop()
        if self._cuda:
            torch.cuda.synchronize(self.device)
        if self.loop.error is not None:
            raise RuntimeError(f"engine loop failed: {self.loop.error!r}")

    def summary(self, boundaries: list[float]) -> dict:
        """Everything rank 0 needs from this rank (plain Python values)."""
        wins = []
        for a, b in zip(self.marks, self.marks[1:]):
            wins.append({"dev_ms": a.event.elapsed_time(b.event), "host_s": b.t_host - a.t_host, "tokens": b.tokens - a.tokens,
                         "h2d": b.stats["h2d_bytes"] - a.stats["h2d_bytes"], "d2h": b.stats["d2h_bytes"] - a.stats["d2h_bytes"],
                         "decode_steps": b.stats["decode_steps"] - a.stats["decode_steps"],
                         "prefill_steps": b.stats["prefill_steps"] - a.stats["prefill_steps"],
                         "launches": (b.launches - a.launches) + (b.stats["launches"] - a.stats["launches"]),
                         "t0": a.t_host, "t1": b.t_host})
        recs = [{"model": r.model, "arrival": r.arrival, "n_prompt": r.n_prompt, "n_out": r.n_out, "done": r.done,
                 "first": r.times[0] if r.times else None, "last": r.times[-1] if r.times else None, "n": len(r.times),
                 "times": r.times} for r in self.recs]
        return {"windows": wins, "recs": recs}


# ------------------------------------------------------------------------------------------- aggregation

def _dist(ms: list[float]) -> dict:
    return {"n": len(ms), "p50": percentile(ms, 50), "p90": percentile(ms, 90), "p99": percentile(ms, 99)}


def latency_summary(recs: list[dict], t_lo: float, t_hi: float) -> dict:
    """TTFT over requests that arrived inside [t_lo, t_hi); TPOT over those of them that finished. A request that
    arrived at least the TTFT limit before ``t_hi`` and never produced a token counts with the time it has waited."""
    ttft, tpot, good, total = [], [], 0, 0
    for r in recs:
        if not (t_lo <= r["arrival"] < t_hi):
            continue
        if r["first"] is None:
            waited = (t_hi - r["arrival"]) * 1e3
            if waited >= SLO_TTFT_MS:
                ttft.append(waited)
                total += 1
            continue
        t1 = (r["first"] - r["arrival"]) * 1e3
        ttft.append(t1)
        if r["done"] and r["n"] > 1:
            tp = (r["last"] - r["first"]) * 1e3 / (r["n"] - 1)
            tpot.append(tp)
            total += 1
            good += int(t1 <= SLO_TTFT_MS and tp <= SLO_TPOT_MS)
    out = {"ttft_ms": _dist(ttft), "tpot_ms": _dist(tpot), "requests": len(ttft), "finished": len(tpot),
           "slo_attained": good / total if total else float("nan")}
    out["slo_met"] = bool(tpot and ttft and out["tpot_ms"]["p99"] <= SLO_TPOT_MS and out["ttft_ms"]["p99"] <= SLO_TTFT_MS)
    return out


def aggregate(rank_summaries: list[dict], streams: list[ModelStream], K: int, dt: float, W: int) -> dict:
    """Combines the attention ranks' windows: device time = max over ranks, tokens = sum."""
    ranks = [s for s in rank_summaries if s]
    n_win = min(len(s["windows"]) for s in ranks)
    wins = []
    for w in range(n_win):
        dev_ms = max(s["windows"][w]["dev_ms"] for s in ranks)
        host_s = max(s["windows"][w]["host_s"] for s in ranks)
        tok = sum(s["windows"][w]["tokens"] for s in ranks)
        wins.append({"dev_ms": dev_ms, "host_s": host_s, "tokens": tok, "tok_per_s": tok / (dev_ms / 1e3),
                     **{k: sum(s["windows"][w][k] for s in ranks) for k in ("h2d", "d2h", "decode_steps", "prefill_steps", "launches")}})
    recs = [r for s in ranks for r in s["recs"]]
    t_lo, t_hi = W * dt, (W + n_win * K) * dt
    # producer-side (end to end) throughput per window: tokens observed inside the planned window
    e2e = []
    for w in range(n_win):
        a, b = (W + w * K) * dt, (W + (w + 1) * K) * dt
        n = sum(1 for r in recs for t in r["times"] if a <= t < b)
        e2e.append(n / (b - a))
    per_model = {}
    for s in streams:
        mine = [r for r in recs if r["model"] == s.model_id]
        toks = sum(1 for r in mine for t in r["times"] if t_lo <= t < t_hi)
        per_model[s.model_id] = {"output_tok_per_s": toks / (t_hi - t_lo), **latency_summary(mine, t_lo, t_hi)}
    order = sorted(range(n_win), key=lambda i: wins[i]["tok_per_s"])
    med = order[len(order) // 2]
    return {"windows": wins, "median_window": med, "e2e_windows": e2e, "latency": latency_summary(recs, t_lo, t_hi),
            "per_model": per_model, "requests": len(recs)}


def result_json(args, world: int, impl: str, mix_info: dict, streams: list[ModelStream], agg: dict, clocks: dict,
                digest: str, extra: dict | None = None) -> dict:
    K, dt = args.steps, args.step_seconds
    w = agg["windows"][agg["median_window"]]
    vals = [x["tok_per_s"] for x in agg["windows"]]
    lat = agg["latency"]
    e2e_med = statistics.median(agg["e2e_windows"])
    cfgd = {"model": " + ".join(s.model_id for s in streams), "mix": mix_info,
            "global_batch": {s.model_id: s.max_batch for s in streams},
            "seq_len": {s.model_id: f"prompt {s.prompt.kind} {s.prompt.lo}-{s.prompt.hi}, output {s.output.lo}-{s.output.hi}" for s in streams},
            "offered_req_per_s": {s.model_id: s.rate for s in streams},
            "parallelism": mix_info["layout"], "step": f"{dt} s scheduling interval of open-loop traffic",
            "windows": f"{len(vals)} x {K} steps after {args.warmup} warm-up steps; value = median window",
            "window_tok_per_s": [round(v, 1) for v in vals], "spread": round((max(vals) - min(vals)) / max(1e-9, statistics.median(vals)), 4),
            "engine_iterations_per_window": {"decode": w["decode_steps"], "prefill": w["prefill_steps"]},
            "slo": {"ttft_p99_ms_limit": SLO_TTFT_MS, "tpot_p99_ms_limit": SLO_TPOT_MS, "ttft_p99_ms": lat["ttft_ms"]["p99"],
                    "tpot_p99_ms": lat["tpot_ms"]["p99"], "met": lat["slo_met"], "attained": lat["slo_attained"]},
            "per_model": agg["per_model"], "workload_digest": digest,
            "l2": "weights and KV streamed per engine iteration exceed the 126 MB L2 (no flush needed)"}
    cfgd.update(extra or {})
    base = recorded_baseline(mix_info["name"], world, args) if impl == "xpool" else None
    vs = round(w["tok_per_s"] / base["value"], 4) if base and base.get("value") else None
    return {
        "metric": METRIC, "impl": impl, "value": w["tok_per_s"], "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": args.warmup, "ms_per_step": w["dev_ms"] / K, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": vs, "baseline_arm": base, "dtype": "bf16",
        "data": "synthetic: uniform random token ids, Poisson arrivals, lengths as listed under config.seq_len, random-init weights",
        "config": cfgd, "clocks": clocks,
        "e2e": {"value": e2e_med, "unit": "tok/s", "h2d_bytes_per_step": w["h2d"] // K, "d2h_bytes_per_step": w["d2h"] // K,
                "ttft_p50_ms": lat["ttft_ms"]["p50"], "ttft_p99_ms": lat["ttft_ms"]["p99"], "tpot_p50_ms": lat["tpot_ms"]["p50"],
                "tpot_p99_ms": lat["tpot_ms"]["p99"], "window_tok_per_s": [round(v, 1) for v in agg["e2e_windows"]],
                "clock": "host perf_counter at token delivery; TTFT from planned arrival"},
        "gpu_launches": w["launches"],
        "valid": bool(lat["slo_met"]) and args.layers == 0 and (extra or {}).get("correctness", {}).get("ok", True),
    }


def recorded_baseline(mix: str, world: int, args) -> dict | None:
    """The library-collective arm's (``--impl baseline``) measurement of the same mix, GPU count and offered load, as
    recorded in ``baseline_arm.json`` beside this file (value, latencies, whether it met the SLO, the command). The
    reference publishes no figure and does not build on this image, so this arm is the comparison the bench can print;
    a changed rate, batch limit or layer count has no recorded counterpart (None)."""
    if getattr(args, "rate_scale", 1.0) != 1.0 or getattr(args, "max_batch", 0) or getattr(args, "kv_tokens", 0) or args.layers:
        return None
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline_arm.json")
    try:
        with open(path, encoding="utf-8") as f:
            table = json.load(f)
    except (OSError, ValueError):
        return None
    return table.get(f"{mix}@{world}")


# ------------------------------------------------------------------------------------------- engine sizing

def engine_config(s: ModelStream) -> EngineConfig:
    return EngineConfig(max_batch=s.max_batch, prefill_chunk=s.prefill_chunk, max_seq_len=s.max_seq_len, page_size=PAGE,
                        num_pages=s.kv_tokens // PAGE, max_prefill_seqs=64)


def model_cfg(s: ModelStream, layers: int = 0):
    cfg = mc.load(s.preset)
    return cfg.with_layers(layers) if layers else cfg


class ElasticPool:
    """Elastic KV for the Instances of one attention GPU inside one process: VMM-backed caches, the seqlock
    control channel and the daemon's capacity policy ticking on a background thread every 10 ms (the deployed
    system runs the same policy in the daemon: service/daemon/ecs_service.py)."""

    def __init__(self, device, budget_bytes: int, granularity: int = 16 << 20):
        from ..ecs import vmm
        from ..native.runtime import EcsChannel

        self.device, self.budget, self.granularity = torch.device(device), budget_bytes, granularity
        self.driver, self.quota = vmm.Driver.real(), vmm.MemoryQuota(1 << 62)
        self._name = f"/xp-bench-ecs-{os.getpid()}-{self.device.index or 0}"
        self._EcsChannel = EcsChannel
        self.channel = None
        self.members: list[tuple[AttentionEngine, object, int]] = []
        self.caches = []
        self._stop = threading.Event()
        self._thread = None
        self.policy = None

    def make_cache(self, cfg, s: ModelStream, share: float):
        from ..ecs import vmm

        kv = vmm.elastic_kv_cache(cfg, s.kv_tokens // PAGE, PAGE, self.device, self.driver, self.quota, initial_bundles=1,
                                  granularity=self.granularity)
        bb = kv.backing.bundle_bytes
        want = max(1, min(kv.backing.bundle_count, int(self.budget * share) // bb))
        if want > 1:
            vmm.grow(kv, list(range(1, want)))
        self.caches.append((kv, want))
        return kv

    def attach(self, engines: list[AttentionEngine], ttft_slo_s: float) -> None:
        from ..ecs import reconciler as R
        from ..service.daemon.ecs import CapacityPolicy, Partition

        self.channel = self._EcsChannel.create(self._name, 1, len(engines), 1)
        parts = []
        for i, (eng, (kv, mapped)) in enumerate(zip(engines, self.caches)):
            rec = R.CapacityReconciler(kv, self.channel, i, gate_factory=lambda e=eng: R.cuda_event_gate(e.stream))
            eng.attach_capacity(rec, ttft_slo_s=ttft_slo_s)
            bb = rec.bundle_bytes
            parts.append(Partition(i, f"p{i}", 0, bb, kv.backing.bundle_count * bb, bb, mapped_bytes=mapped * bb))
        self.policy = CapacityPolicy(self.channel, parts, {0: 0}, utilization=1.0)
        mapped_total = sum(p.mapped_bytes for p in parts)
        self.channel.publish_report(0, max(0, self.budget - mapped_total), max(self.budget, mapped_total), 0)
        self.policy.freeze_pools()
        self._thread = threading.Thread(target=self._run, daemon=True, name="ecs-policy")
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.wait(0.01):
            self.policy.tick()

    def close(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join(5)
        kinds: dict[str, int] = {}
        for e in (self.policy.events if self.policy else []):
            kinds[e.kind] = kinds.get(e.kind, 0) + 1
        if self.channel is not None:
            self.channel.close()
        return kinds


# ------------------------------------------------------------------------------------------- correctness gate

def check_against_oracle(eng: AttentionEngine, make_oracle, vocab: int, n_new: int = 5) -> dict:
    """Runs three short prompts through ``eng`` and through the oracle engine built by ``make_oracle()``; the logits of
    every step up to the first differing token must agree (see ``testing.compare_generations``)."""
    from ..testing import compare_generations

    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (7, 41, 150)]

    def run(e):
        seqs = [e.add_request(p, n_new) for p in prompts]
        logits = {s.seq_id: [] for s in seqs}
        while e.has_work:
            for i, (s, _) in enumerate(e.step()):
                logits[s.seq_id].append(e.logits[i].float().clone())
        return seqs, logits

    seqs, logits = run(eng)
    oracle = make_oracle()
    oracle.warmup()
    rseqs, rlogits = run(oracle)
    ok, agree, worst = True, [], 0.0
    for s, r in zip(seqs, rseqs):
        good, n, kl = compare_generations(s.generated, r.generated, logits[s.seq_id], rlogits[r.seq_id])
        ok, worst = ok and good, max(worst, kl)
        agree.append(f"{n}/{len(s.generated)}")
    del oracle
    torch.cuda.empty_cache()
    return {"ok": bool(ok), "tokens_agree": agree, "max_kl": worst, "oracle": "loopback engine with the unsharded FFN"}


def check_against_reference_model(eng: AttentionEngine, cfg, aw, fw, n_new: int = 4) -> dict:
    """1-GPU gate: the engine against the plain PyTorch restatement of the model (``models.reference``)."""
    from ..models.reference import ReferenceModel
    from ..testing import compare_generations

    ref = ReferenceModel(cfg, aw, fw)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 41, 150)]
    seqs = [eng.add_request(p, n_new) for p in prompts]
    logits = {s.seq_id: [] for s in seqs}
    while eng.has_work:
        for i, (s, _) in enumerate(eng.step()):
            logits[s.seq_id].append(eng.logits[i].float().clone())
    ok, agree, worst = True, [], 0.0
    for s, p in zip(seqs, prompts):
        toks, rl = ref.generate(torch.tensor(p, device=eng.device), n_new)
        # the restatement runs in fp32 on bf16 weights: the reference's prefill bound applies (0.05 nats)
        good, n, kl = compare_generations(s.generated, list(toks), logits[s.seq_id], list(rl), kl_limit=0.05, tie_margin=0.25)
        ok, worst = ok and good, max(worst, kl)
        agree.append(f"{n}/{len(s.generated)}")
    return {"ok": bool(ok), "tokens_agree": agree, "max_kl": worst, "oracle": "fp32 PyTorch restatement of the model"}


# ------------------------------------------------------------------------------------------- 1 GPU

def timeline(args) -> tuple[list[float], float, float]:
    """(window boundaries, end of the run, window length), seconds from the start."""
    dt, K, W = args.step_seconds, args.steps, args.warmup
    bounds = [(W + i * K) * dt for i in range(WINDOWS + 1)]
    return bounds, bounds[-1], K * dt


def run_single_gpu(args) -> dict:
    from ..engine.ffn_local import LocalFfnPort, UnfusedFfnPort
    from ..models.weights import random_attention_weights, random_ffn_weights
    from ..ops import gemm

    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    streams, info = build_mix(args.mix or "b", 1, args.rate_scale, args.max_batch, args.kv_tokens)
    bounds, end_s, window_s = timeline(args)
    reqs = plan_streams(streams, end_s, window_s, args.seed, preload=True)
    insts, first = [], None
    for s in streams:
        cfg = model_cfg(s, args.layers)
        aw = random_attention_weights(cfg, s.seed, dev, torch.bfloat16)
        fw = random_ffn_weights(cfg, s.seed, dev, torch.bfloat16)
        port = LocalFfnPort(cfg, fw) if args.impl == "xpool" else UnfusedFfnPort(cfg, fw)
        eng = AttentionEngine(cfg, aw, port, engine_config(s), dev)
        insts.append(InstanceHandle(s.model_id, cfg, eng))
        first = first or (eng, cfg, aw, fw)
    dep = Deployment(insts)
    dep.warmup()
    correctness = check_against_reference_model(*first)
    gemm.check_status(dev)
    rs = RankServing(dep, reqs, dev)
    sampler = ClockSampler(0)
    torch.cuda.synchronize(dev)
    sampler.start()
    rs.run(time.perf_counter() + 0.05, bounds, end_s)
    clocks = sampler.stop()
    gemm.check_status(dev)
    agg = aggregate([rs.summary(bounds)], streams, args.steps, args.step_seconds, args.warmup)
    return result_json(args, 1, args.impl, info, streams, agg, clocks, workload_digest(reqs), extra={"correctness": correctness})


# ------------------------------------------------------------------------------------------- N GPUs

def run_multi_gpu(args) -> int:
    import torch.distributed as dist

    from ..models.weights import random_attention_weights, random_ffn_weights
    from ..native import runtime as rt
    from ..ops import gemm
    from ..parallel import fabric as F

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != args.gpus or world < 2:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE == {args.gpus} >= 2 (got {world})")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if args.impl == "baseline":
        # the library arm runs one communicator and stream per Instance: give every stream a hardware queue of its own
        os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
    watchdog = _ProgressWatchdog(args.impl, rank)
    watchdog.phase("setup", 420.0)
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    ctl = dist.new_group(backend="gloo")

    streams, info = build_mix(args.mix or default_mix(world), world, args.rate_scale, args.max_batch, args.kv_tokens)
    bounds, end_s, window_s = timeline(args)
    mine = [s for s in streams if s.atn_rank == rank]
    reqs = plan_streams(mine, end_s, window_s, args.seed, preload=True) if mine else []
    cfgs = {s.model_id: model_cfg(s, args.layers) for s in streams}
    ecfgs = {s.model_id: engine_config(s) for s in streams}
    placements = [F.InstancePlacement(s.model_id, cfgs[s.model_id], seed=s.seed, atn_rank=s.atn_rank, ffn_ranks=s.ffn_ranks,
                                      capacity_rows=max(s.max_batch, s.prefill_chunk), weights_key=s.weights_key) for s in streams]
    topo = F.Topology(world, placements)

    pools: list[ElasticPool] = []

    def kv_for(p: F.InstancePlacement):
        s = next(x for x in streams if x.model_id == p.model_id)
        if not s.elastic:
            return None
        if not pools:
            budget = sum(x.kv_tokens * _kv_bytes_per_token(cfgs[x.model_id]) for x in mine) // 2
            pools.append(ElasticPool(dev, budget))
        return pools[0].make_cache(cfgs[p.model_id], s, share=1.0 / (2 * len(mine)))

    if args.impl == "xpool":
        policy = {"fifo": rt.POLICY_FIFO, "random": rt.POLICY_RANDOM, "slo": rt.POLICY_SLO}[args.policy]
        ctx = F.build_rank(topo, rank, dev, ecfgs, group=ctl, n_lanes=args.lanes, policy=policy, kv_for=kv_for)
        if ctx.role == "ffn":
            if getattr(args, "trace_dir", ""):
                ctx.ffn.enable_trace(1 << 21)      # Lane events of the whole run (24 bytes each)
            ctx.ffn.start(lease_ms=20.0)
    else:
        from ..parallel import nccl_baseline as NB

        ctx = NB.build_rank(topo, rank, dev, ecfgs, ctl, kv_for=kv_for)
        if ctx.role == "ffn":
            ctx.ffn.start()
    dist.barrier(group=ctl)

    summary, clocks, correctness, ecs_events = None, None, None, None
    failure = None
    stage = "start"
    try:
        if ctx.role == "atn":
            insts = [InstanceHandle(s.model_id, cfgs[s.model_id], ctx.engines[s.model_id]) for s in mine]
            dep = Deployment(insts)
            for i in insts:          # one Instance at a time, so that a failed bring-up names it
                stage = f"warm-up of {i.model_id}"
                i.engine.warmup()
                torch.cuda.synchronize(dev)
                gemm.check_status(dev)
            stage = "correctness check"
            if pools:
                pools[0].attach([i.engine for i in insts], SLO_TTFT_MS / 1e3)
            if rank == 0:
                s = min(mine, key=lambda x: cfgs[x.model_id].hidden_size * cfgs[x.model_id].num_layers)
                cfg = cfgs[s.model_id]

                def make_oracle(s=s, cfg=cfg):
                    from ..engine.ffn_local import LocalFfnPort

                    aw = random_attention_weights(cfg, s.seed, dev, torch.bfloat16)
                    fw = random_ffn_weights(cfg, s.seed, dev, torch.bfloat16)
                    return AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), EngineConfig(max_batch=8, prefill_chunk=256, max_seq_len=512), dev)

                correctness = check_against_oracle(ctx.engines[s.model_id], make_oracle, cfg.vocab_size)
                correctness["instance"] = s.model_id
            gemm.check_status(dev)
    except Exception as e:  # report, then let every rank leave together
        failure = f"{stage}: {e!r}"
    flags = [None] * world
    dist.all_gather_object(flags, failure, group=ctl)
    if any(flags):
        # what every rank knows about the failed bring-up: the attention ranks' exceptions, the FFN ranks' Lane
        # statistics, replay-thread errors and canonical failure record
        note = {"rank": rank, "role": ctx.role, "failure": failure}
        try:
            if ctx.role == "ffn" and args.impl == "xpool":
                f = ctx.ffn.failure()
                note.update(lanes=ctx.ffn.stats(), errors=list(getattr(ctx.ffn, "errors", [])),
                            canonical=None if f is None else [f.result_code, f.origin_pe, f.invocation_sequence, f.layer_ordinal])
            elif ctx.role == "atn" and args.impl == "xpool":
                note["instances"] = {m: (None if (f := e.port.failure()) is None else
                                         [f.result_code, f.origin_pe, f.invocation_sequence, f.layer_ordinal])
                                     for m, e in ctx.engines.items() if hasattr(e.port, "failure")}
        except Exception as e:
            note["diagnostics_failed"] = repr(e)
        notes = [None] * world
        dist.all_gather_object(notes, note, group=ctl)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "impl": args.impl, "error": [f for f in flags if f], "ranks": notes}), flush=True)
        watchdog.cancel()
        _shutdown(ctx, ctl, pools)
        return 1

    # common start: every rank's producer counts from its own clock right after this barrier
    dist.barrier(group=ctl)
    watchdog.phase("measured run", end_s + 90.0)
    t0 = time.perf_counter() + 0.1
    try:
        if ctx.role == "atn":
            rs = RankServing(dep, reqs, dev)
            sampler = ClockSampler(local)
            sampler.start()
            rs.run(t0, bounds, end_s)
            clocks = sampler.stop()
            gemm.check_status(dev)
            summary = rs.summary(bounds)
        else:
            time.sleep(max(0.0, t0 + end_s - time.perf_counter()))
    except Exception as e:
        failure = repr(e)
    dist.barrier(group=ctl)
    watchdog.phase("gathering results", 60.0)
    if pools:
        ecs_events = pools[0].close()
    lane_stats = ctx.ffn.stats() if ctx.role == "ffn" else None
    if lane_stats is not None and getattr(args, "trace_dir", "") and args.impl == "xpool":
        from ..devkit.observers import FabricObserver, lane_busy_summary

        art = FabricObserver(ctx.ffn).collect()
        lane_stats["busy"] = lane_busy_summary(art.events, args.lanes)
        lane_stats["trace_dropped"] = art.dropped
        os.makedirs(args.trace_dir, exist_ok=True)
        with open(os.path.join(args.trace_dir, f"fabric.rank{rank}.json"), "w", encoding="utf-8") as f:
            json.dump({"rank": rank, "summary": lane_stats["busy"], "dropped": art.dropped, "events": art.events[:20000]}, f)
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "role": ctx.role, "summary": summary, "clocks": clocks, "lanes": lane_stats,
                                      "correctness": correctness, "ecs": ecs_events, "failure": failure}, group=ctl)
    rc = 0
    if rank == 0:
        fails = [g["failure"] for g in gathered if g["failure"]]
        if fails:
            print(json.dumps({"metric": METRIC, "impl": args.impl, "error": fails}), flush=True)
            rc = 1
        else:
            agg = aggregate([g["summary"] for g in gathered], streams, args.steps, args.step_seconds, args.warmup)
            lanes = [g["lanes"] for g in gathered if g["lanes"]]
            extra = {"correctness": gathered[0]["correctness"], "lane_stats": lanes, "lanes_per_ffn_gpu": args.lanes,
                     "elastic_kv_events": [g["ecs"] for g in gathered if g["ecs"]],
                     "transport": "peer-memory stores issued by kernels (CUDA IPC over NVLink)" if args.impl == "xpool"
                     else "NCCL broadcast / reduce around cuBLAS GEMMs and an unfused activation"}
            out = result_json(args, world, args.impl, info, streams, agg, gathered[0]["clocks"], workload_digest(reqs), extra)
            served = sum(sum(l["served"]) for l in lanes) if args.impl == "xpool" else 0
            out["gpu_launches"] += 0 if not lanes else int(served * 4 * args.steps * args.step_seconds / max(1e-9, end_s))
            print(json.dumps(out), flush=True)
    watchdog.cancel()
    _shutdown(ctx, ctl, pools)
    return rc


def _kv_bytes_per_token(cfg) -> int:
    return 2 * cfg.num_layers * cfg.num_kv_heads * cfg.head_dim * 2


class _ProgressWatchdog:
    """Ends a multi-GPU run that makes no progress: if the phase in force lasts longer than its allowance, rank 0's
    process prints an error line in the benchmark's format and every process that notices exits with code 3. A stuck
    communicator or a generation that never becomes ready must not hold a machine of GPUs until an outer limit."""

    def __init__(self, impl: str, rank: int):
        self.impl, self.rank = impl, rank
        self._timer: threading.Timer | None = None

    def phase(self, name: str, seconds: float) -> None:
        self.cancel()

        def fire():
            if self.rank == 0:
                print(json.dumps({"metric": METRIC, "impl": self.impl,
                                  "error": [f"no progress: phase '{name}' exceeded {seconds:.0f} s"]}), flush=True)
            sys.stdout.flush()
            os._exit(3)

        self._timer = threading.Timer(seconds, fire)
        self._timer.daemon = True
        self._timer.start()

    def cancel(self) -> None:
        if self._timer is not None:
            self._timer.cancel()
            self._timer = None


def _exit_watchdog(seconds: float, code: int = 0) -> None:
    """Ends the process if teardown has not finished after ``seconds`` (the result line is already printed): a
    library communicator that does not come down must not keep a GPU box busy."""
    def fire():
        sys.stdout.flush()
        os._exit(code)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()


def _shutdown(ctx, ctl, pools) -> None:
    import torch.distributed as dist

    _exit_watchdog(45.0)
    dist.barrier(group=ctl)
    for port in getattr(ctx, "ports", []):      # baseline arm: a zero-row header ends each FFN service thread
        port.shutdown()
    if ctx.role == "atn":
        torch.cuda.synchronize()
    if ctx.role == "ffn" and ctx.ffn is not None:
        ctx.ffn.stop()
        ctx.ffn.close()
    dist.barrier(group=ctl)
    if getattr(ctx, "ports", None) is not None:
        # baseline arm: its NCCL communicators were captured into CUDA graphs; leave them to process exit
        sys.stdout.flush()
        os._exit(0)
    dist.destroy_process_group()
