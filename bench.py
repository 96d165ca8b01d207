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

``--impl reference`` reports why the reference cannot run here: its build needs a CUDA 13.2 toolkit,
NVSHMEM and a serving engine that this image does not carry.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

BASELINE_PUBLISHED = None  # the reference publishes no throughput or latency number
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
    ap.add_argument("--ffn-tp", type=int, default=1, help="FFN tensor-parallel degree (multi-GPU only)")
    ap.add_argument("--lanes", type=int, default=2, help="Executor Lanes per FFN device (multi-GPU only)")
    ap.add_argument("--trace-dir", default="", help="multi-GPU only: write the FFN ranks' Lane timelines (chrome trace JSON) here")
    ap.add_argument("--policy", default="fifo", choices=["fifo", "random", "slo"], help="Lane scheduling policy (multi-GPU only)")
    ap.add_argument("--ffn-ranks", type=int, default=0, help="GPUs in the shared FFN tier (0: max(1, N // 4); multi-GPU only)")
    return ap.parse_args(argv)


def run_single_gpu(args) -> dict:
    """Loopback: every role on GPU 0, FFNs in-stream."""
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
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus == 1 and world == 1:
        res = run_single_gpu(args)
        print(json.dumps(res))
        return 0
    from crosspool_b200.bench import fabric_bench

    return fabric_bench.main(args)


if __name__ == "__main__":
    sys.exit(main())
