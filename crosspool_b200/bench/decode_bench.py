"""Steady-state decode benchmark shared by the 1-GPU (loopback) and multi-GPU (Fabric) layouts.

See ``bench.py`` at the repository root for the contract. This module builds the Instances for one
rank, fills their decode batches, and measures (a) K steps through the public ``Deployment.step`` API
with per-step pinned H2D metadata and D2H tokens, and (b) K back-to-back replays of the Instances'
decode-step graphs timed with CUDA events.
"""

from __future__ import annotations

import os
import statistics
import subprocess
import time
from dataclasses import dataclass

import torch

from ..deployment import Deployment, percentile
from ..engine.atn_engine import EngineConfig
from ..models.config import ModelConfig

PAGE = 16
SYNCS_PER_RUN = 4  # how often run_rank() calls its cross-rank barrier


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, f"/tmp/xpool_clocks_{os.getpid()}.csv"

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


@dataclass
class Workload:
    prompts: list[list[int]]
    new_tokens: int
    pages: int
    max_seq: int


def make_workload(cfg: ModelConfig, batch: int, min_prompt: int, max_prompt: int, steps: int, warmup: int, seed: int
                  ) -> Workload:
    """``batch`` prompts with lengths uniform in [min_prompt, max_prompt] and uniform random ids."""
    gen = torch.Generator().manual_seed(1234 + seed)
    lens = torch.randint(min_prompt, max_prompt + 1, (batch,), generator=gen).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    new_tokens = steps + warmup + 160  # the fill phase interleaves decode steps; nobody may finish early
    pages = sum((len(p) + new_tokens + PAGE) // PAGE + 1 for p in prompts) + 64
    return Workload(prompts, new_tokens, pages, max_prompt + new_tokens + PAGE)


def engine_config(batch: int, wl: Workload, prefill_chunk: int = 4096) -> EngineConfig:
    return EngineConfig(max_batch=batch, prefill_chunk=prefill_chunk, max_seq_len=wl.max_seq, page_size=PAGE,
                        num_pages=wl.pages, decode_buckets=[batch])


@dataclass
class RankResult:
    tokens_per_step: int
    e2e_s: float
    e2e_tokens: int
    step_ms: list[float]
    ttft_ms: list[float]
    dev_ms: float
    e2e_dev_ms: float
    h2d_per_step: int
    d2h_per_step: int
    launches_per_step: int
    clocks: dict


def run_rank(dep: Deployment, workloads: dict[str, Workload], batch: int, steps: int, warmup: int, gpu_index: int,
             sync=lambda: None) -> RankResult:
    """Fills, warms and measures the Instances of one attention rank. ``sync`` is a cross-rank
    barrier (no-op for one GPU) called on both sides of each timed region."""
    from ..ops import gemm

    dev = dep.instances[0].engine.device
    dep.warmup()
    t_add = time.monotonic()
    seqs = []
    for inst in dep.instances:
        wl = workloads[inst.model_id]
        for p in wl.prompts:
            seqs.append(dep.add_request(inst.model_id, p, wl.new_tokens, arrival=t_add))
    while any(e.engine.waiting or e.engine.prefilling for e in dep.instances):
        dep.step()
    ttft = [(s.first_token_time - s.arrival) * 1e3 for s in seqs if s.first_token_time]
    for _ in range(warmup):
        dep.step()
    torch.cuda.synchronize(dev)
    gemm.check_status(dev)

    # ---- end to end through the public API
    sampler = ClockSampler(gpu_index)
    sampler.start()
    stats0 = dep.stats()
    step_ms = []
    sync()
    torch.cuda.synchronize(dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(steps):
        ts = time.perf_counter()
        tokens += dep.step().num_tokens
        step_ms.append((time.perf_counter() - ts) * 1e3)
    ev1.record()
    torch.cuda.synchronize(dev)
    e2e_s = time.perf_counter() - t0
    sync()
    stats1 = dep.stats()

    # ---- device-timed: back-to-back replays of every Instance's decode-step graph
    engines = [i.engine for i in dep.instances]
    graphs = [e._graphs[batch] for e in engines]
    timing = torch.cuda.Stream(dev)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(max(warmup, 3)):
        for e, g in zip(engines, graphs):
            with torch.cuda.stream(e.stream):
                g.replay()
    torch.cuda.synchronize(dev)
    sync()
    with torch.cuda.stream(timing):
        start.record()
    for e in engines:
        e.stream.wait_event(start)
    for _ in range(steps):
        for e, g in zip(engines, graphs):
            with torch.cuda.stream(e.stream):
                g.replay()
    for e in engines:
        done = torch.cuda.Event()
        done.record(e.stream)
        timing.wait_event(done)
    with torch.cuda.stream(timing):
        end.record()
    torch.cuda.synchronize(dev)
    sync()
    dev_ms = start.elapsed_time(end)
    clocks = sampler.stop()
    gemm.check_status(dev)
    return RankResult(
        tokens_per_step=batch * len(engines), e2e_s=e2e_s, e2e_tokens=tokens, step_ms=step_ms, ttft_ms=ttft,
        dev_ms=dev_ms, e2e_dev_ms=ev0.elapsed_time(ev1),
        h2d_per_step=(stats1["h2d_bytes"] - stats0["h2d_bytes"]) // steps,
        d2h_per_step=(stats1["d2h_bytes"] - stats0["d2h_bytes"]) // steps,
        launches_per_step=sum(e._graph_launches[batch] for e in engines), clocks=clocks)


def result_json(args, cfg: ModelConfig, n_gpus: int, parallelism: str, n_instances: int, tokens_per_step: int,
                dev_ms: float, e2e_s: float, e2e_tokens: int, step_ms: list[float], ttft_ms: list[float],
                h2d: int, d2h: int, launches: int, clocks: dict, extra_config: dict | None = None) -> dict:
    K = args.steps
    tpot_p99 = percentile(step_ms, 99)
    cfgd = {"model": f"{n_instances}x {args.model} co-located", "global_batch": tokens_per_step,
            "phase": "steady-state decode, every Instance at its full running batch",
            "slo": {"tpot_p99_ms_limit": 50.0, "tpot_p99_ms": tpot_p99, "met": bool(tpot_p99 <= 50.0)},
            "seq_len": f"prompt {args.min_prompt}-{args.max_prompt} + decode", "parallelism": parallelism,
            "layers": cfg.num_layers, "l2": "weights and KV streamed per step exceed the 126 MB L2 (no flush needed)"}
    cfgd.update(extra_config or {})
    return {
        "metric": "aggregate output tok/s across co-located models at p99 TPOT SLO; p50 TTFT",
        "value": tokens_per_step * K / (dev_ms / 1e3),
        "unit": "tok/s",
        "n_gpus": n_gpus,
        "steps": K,
        "warmup": args.warmup,
        "ms_per_step": dev_ms / K,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, prompt lengths uniform [%d, %d], random-init weights" % (
            args.min_prompt, args.max_prompt),
        "config": cfgd,
        "clocks": clocks,
        "e2e": {"value": e2e_tokens / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s * 1e3 / K, "tpot_p50_ms": percentile(step_ms, 50),
                "tpot_p99_ms": percentile(step_ms, 99), "ttft_p50_ms": percentile(ttft_ms, 50)},
        "gpu_launches": launches * K,
        "valid": args.layers == 0,
    }
