#!/usr/bin/env python
"""Headline benchmark: aggregate output tok/s across co-located models in steady-state decode.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N > 1, one rank
per GPU). The workload is acceptance configuration (b) of BASELINE.json scaled by N: Instances of the
Qwen3-0.6B architecture in bf16 with random-init weights, two co-located Instances per attention GPU,
each with ``--batch`` in-flight requests whose prompt lengths are uniform in [128, 2048] (uniform random
token ids, outputs forced with ignore-eos semantics). N = 1 runs every role on one GPU (loopback);
N >= 2 puts attention on N/2 GPUs and the shared FFN tier on the other N/2.

A *step* is one decode iteration of every co-located Instance (every in-flight request gains one
token). Two measurements are reported:

* ``value``: K steps device-timed with CUDA events around back-to-back replays of the Instances' full
  decode-step graphs (all layers, LM head, sampling) — the kernel-only number;
* ``e2e``: the same K steps driven through the public API (``Deployment.step``), timed around the whole
  loop, which per step copies the step's metadata (token ids, positions, KV slots, lengths, block
  table) from pinned host memory to the device and reads the sampled tokens back.

``--impl reference`` reports why the reference cannot run here.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

BASELINE_PUBLISHED = None  # the reference publishes no number
REFERENCE_UNAVAILABLE = ("reference not installable offline: needs CUDA Toolkit >= 13.2 (image has 12.9), "
                         "NVSHMEM 3.7.2, cuda-bindings 13, sglang 0.5.20, torch 2.13")


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="xpool", choices=["xpool", "reference"])
    ap.add_argument("--batch", type=int, default=256, help="in-flight requests per Instance")
    ap.add_argument("--model", default="Qwen/Qwen3-0.6B")
    ap.add_argument("--instances-per-atn", type=int, default=2)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the result invalid)")
    return ap.parse_args(argv)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, f"/tmp/xpool_clocks_{os.getpid()}.csv"

    def start(self):
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


def run_single_gpu(args) -> dict:
    import torch

    from crosspool_b200 import native
    from crosspool_b200.deployment import build_loopback, percentile
    from crosspool_b200.engine.atn_engine import EngineConfig
    from crosspool_b200.models import config as mc
    from crosspool_b200.ops import gemm

    torch.cuda.set_device(0)
    cfg = mc.load(args.model)
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    K, W, B = args.steps, args.warmup, args.batch
    n_inst = args.instances_per_atn
    gen = torch.Generator().manual_seed(1234)
    page = 16
    prompts = []
    for i in range(n_inst):
        lens = torch.randint(args.min_prompt, args.max_prompt + 1, (B,), generator=gen).tolist()
        prompts.append([torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens])
    new_tokens = K + W + 160  # the fill phase interleaves decode steps; nobody may finish early
    max_seq = args.max_prompt + new_tokens + page
    handles = []
    for i in range(n_inst):
        pages = sum((len(p) + new_tokens + page) // page + 1 for p in prompts[i]) + 64
        handles.append((f"{args.model}#{i}", cfg, i, pages))
    dep = None
    engines_cfg = []
    from crosspool_b200.deployment import Deployment, InstanceHandle
    from crosspool_b200.engine.atn_engine import AttentionEngine
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    insts = []
    for model_id, c, seed, pages in handles:
        ecfg = EngineConfig(max_batch=B, prefill_chunk=4096, max_seq_len=max_seq, page_size=page, num_pages=pages,
                            decode_buckets=[B])
        aw = random_attention_weights(c, seed, "cuda", torch.bfloat16)
        fw = random_ffn_weights(c, seed, "cuda", torch.bfloat16)
        insts.append(InstanceHandle(model_id, c, AttentionEngine(c, aw, LocalFfnPort(c, fw), ecfg, "cuda")))
    dep = Deployment(insts)
    dep.warmup()

    # ---- fill the decode batches (untimed): every request is prefilled and produces its first token
    t_add = time.monotonic()
    seqs = []
    for i, inst in enumerate(dep.instances):
        for p in prompts[i]:
            seqs.append(dep.add_request(inst.model_id, p, new_tokens, arrival=t_add))
    while any(e.engine.waiting or e.engine.prefilling for e in dep.instances):
        dep.step()
    ttft = [(s.first_token_time - s.arrival) * 1e3 for s in seqs if s.first_token_time]
    for _ in range(W):
        dep.step()
    torch.cuda.synchronize()
    gemm.check_status(torch.device("cuda"))

    # ---- end-to-end through the public API
    sampler = ClockSampler(0)
    sampler.start()
    stats0 = dep.stats()
    step_ms = []
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    tokens = 0
    for _ in range(K):
        ts = time.perf_counter()
        tokens += dep.step().num_tokens
        step_ms.append((time.perf_counter() - ts) * 1e3)
    ev1.record()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    stats1 = dep.stats()

    # ---- device-timed: back-to-back replays of every Instance's decode-step graph
    engines = [i.engine for i in dep.instances]
    graphs = [e._graphs[B] for e in engines]
    timing = torch.cuda.Stream()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(max(W, 3)):
        for e, g in zip(engines, graphs):
            with torch.cuda.stream(e.stream):
                g.replay()
    torch.cuda.synchronize()
    with torch.cuda.stream(timing):
        start.record()
    for e in engines:
        e.stream.wait_event(start)
    for _ in range(K):
        for e, g in zip(engines, graphs):
            with torch.cuda.stream(e.stream):
                g.replay()
    for e in engines:
        done = torch.cuda.Event()
        done.record(e.stream)
        timing.wait_event(done)
    with torch.cuda.stream(timing):
        end.record()
    torch.cuda.synchronize()
    dev_ms = start.elapsed_time(end)
    clocks = sampler.stop()
    gemm.check_status(torch.device("cuda"))

    tok_per_step = B * n_inst
    value = tok_per_step * K / (dev_ms / 1e3)
    e2e_value = tokens / e2e_s
    launches_per_step = sum(e._graph_launches[B] for e in engines)
    return {
        "metric": "aggregate output tok/s across co-located models (steady-state decode)",
        "value": value,
        "unit": "tok/s",
        "n_gpus": 1,
        "steps": K,
        "warmup": W,
        "ms_per_step": dev_ms / K,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: uniform random token ids, prompt lengths uniform [%d, %d], random-init weights" % (
            args.min_prompt, args.max_prompt),
        "config": {"model": f"{n_inst}x {args.model} co-located", "global_batch": tok_per_step,
                   "seq_len": f"prompt {args.min_prompt}-{args.max_prompt} + decode", "parallelism": "loopback(atn+ffn on 1 GPU)",
                   "layers": cfg.num_layers, "l2": "weights streamed per step exceed the 126 MB L2 (no flush needed)"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": (stats1["h2d_bytes"] - stats0["h2d_bytes"]) // K,
                "d2h_bytes_per_step": (stats1["d2h_bytes"] - stats0["d2h_bytes"]) // K,
                "ms_per_step": e2e_s * 1e3 / K, "tpot_p50_ms": percentile(step_ms, 50), "tpot_p99_ms": percentile(step_ms, 99),
                "ttft_p50_ms": percentile(ttft, 50), "device_ms_per_step": ev0.elapsed_time(ev1) / K},
        "gpu_launches": launches_per_step * K,
        "valid": args.layers == 0,
    }


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus == 1 and world == 1:
        res = run_single_gpu(args)
        print(json.dumps(res))
        return 0
    from crosspool_b200.parallel import fabric_bench

    return fabric_bench.main(args)


if __name__ == "__main__":
    sys.exit(main())
