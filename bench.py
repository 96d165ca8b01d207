#!/usr/bin/env python
"""Headline benchmark: aggregate output tok/s across co-located models served under open-loop traffic, with the
p99 TPOT / p99 TTFT service-level objectives checked, and p50 TTFT.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N > 1, one rank per GPU).
The served path is measured: admission, chunked prefill and decode interleaved by each Instance's engine loop,
Poisson arrivals generated in-process and submitted through ``EngineLoop.submit`` (what ``POST /generate`` calls),
synthetic prompts of the named length distributions, random-init weights of the named architectures, bf16.

The model mix follows the acceptance configurations by GPU count (``--mix`` overrides):

* N = 1: Qwen3-0.6B, every role on one GPU (loopback: the FFN runs in-stream);
* N = 2: Qwen3-0.6B on 1 attention GPU + 1 FFN GPU over NVLink peer memory;
* N = 4: Qwen3-8B + Qwen3-0.6B sharing each of 2 attention GPUs with elastic KV lending, FFN on a shared 2-GPU
  tier (8B tensor-parallel over both), the two models trading long- and short-context traffic every window;
* N = 8: Qwen3-32B (FFN TP4) + Qwen3-8B (FFN TP2) + 2 x Qwen3-1.7B, attention on 2 GPUs with elastic KV, FFN tier
  on 6 GPUs, bursty Poisson streams with rates 1:2:4:4.

A *step* is one ``--step-seconds`` (0.5 s) scheduling interval of offered traffic. After W warm-up intervals,
three windows of exactly K intervals are measured back to back; ``value`` is the median window's output tokens
divided by its device time (CUDA events at the window boundaries, maximum over attention ranks); ``e2e`` is the
same windows seen by the request producer on the host clock, with TTFT and TPOT percentiles. ``valid`` is false
when an SLO is missed or the correctness gate (logits against an oracle engine) fails.

``--impl baseline`` runs the same deployment and workload with the FFN tier built from library calls (NCCL
broadcast / reduce, cuBLAS GEMMs, unfused SwiGLU). ``--impl reference`` reports why the reference itself cannot
run here. ``--decode-only`` runs the steady-state decode replay benchmark instead (every Instance at a full
running batch, no arrivals), a kernel-level figure.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

REFERENCE_UNAVAILABLE = ("reference not installable offline: needs CUDA Toolkit >= 13.2 (image has 12.9), "
                         "NVSHMEM 3.7.2, cuda-bindings 13, sglang 0.5.20, torch 2.13")


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="scheduling intervals per measured window")
    ap.add_argument("--warmup", type=int, default=5, help="untimed intervals of traffic before the first window")
    ap.add_argument("--impl", default="xpool", choices=["xpool", "baseline", "reference"])
    ap.add_argument("--step-seconds", type=float, default=0.5)
    ap.add_argument("--mix", default="", choices=["", "b", "c", "d", "e"], help="model mix (default: by GPU count)")
    ap.add_argument("--rate-scale", type=float, default=1.0, help="multiplies every arrival rate of the mix")
    ap.add_argument("--max-batch", type=int, default=0, help="override the running-request limit of every Instance")
    ap.add_argument("--kv-tokens", type=int, default=0, help="override the KV capacity (tokens) of every Instance")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the models (marks the result invalid)")
    ap.add_argument("--lanes", type=int, default=2, help="Executor Lanes per FFN device (multi-GPU only)")
    ap.add_argument("--policy", default="fifo", choices=["fifo", "random", "slo"], help="Lane scheduling policy")
    # steady-state decode replay (kernel-level)
    ap.add_argument("--decode-only", action="store_true")
    ap.add_argument("--batch", type=int, default=256, help="decode-only: in-flight requests per Instance")
    ap.add_argument("--model", default="Qwen/Qwen3-0.6B", help="decode-only: model preset")
    ap.add_argument("--instances-per-atn", type=int, default=2)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--ffn-tp", type=int, default=1)
    ap.add_argument("--trace-dir", default="")
    ap.add_argument("--ffn-ranks", type=int, default=0)
    return ap.parse_args(argv)


def run_decode_only_single_gpu(args) -> dict:
    import torch

    from crosspool_b200.bench import decode_bench as db
    from crosspool_b200.deployment import Deployment, InstanceHandle
    from crosspool_b200.engine.atn_engine import AttentionEngine
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    torch.cuda.set_device(0)
    cfg = mc.load(args.model)
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    insts, workloads = [], {}
    for i in range(args.instances_per_atn):
        model_id = f"{args.model}#{i}"
        wl = db.make_workload(cfg, args.batch, args.min_prompt, args.max_prompt, args.steps, args.warmup, seed=i)
        workloads[model_id] = wl
        aw = random_attention_weights(cfg, i, "cuda", torch.bfloat16)
        fw = random_ffn_weights(cfg, i, "cuda", torch.bfloat16)
        insts.append(InstanceHandle(model_id, cfg, AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw),
                                                                   db.engine_config(args.batch, wl), "cuda")))
    r = db.run_rank(Deployment(insts), workloads, args.batch, args.steps, args.warmup, gpu_index=0)
    return db.result_json(args, cfg, 1, "loopback (attention + FFN on one GPU)", len(insts), r.tokens_per_step, r.dev_ms,
                          r.e2e_s, r.e2e_tokens, r.step_ms, r.ttft_ms, r.h2d_per_step, r.d2h_per_step,
                          r.launches_per_step, r.clocks)


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:       # one line for the whole job, also under torch.distributed.run
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}), flush=True)
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.decode_only:
        if args.gpus == 1 and world == 1:
            print(json.dumps(run_decode_only_single_gpu(args)))
            return 0
        from crosspool_b200.bench import fabric_bench

        return fabric_bench.main(args)
    from crosspool_b200.bench import served

    if args.gpus == 1 and world == 1:
        print(json.dumps(served.run_single_gpu(args)))
        return 0
    return served.run_multi_gpu(args)


if __name__ == "__main__":
    sys.exit(main())
