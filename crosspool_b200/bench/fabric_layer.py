"""One FFN layer across GPUs: the fused Fabric path against an unfused NCCL baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m crosspool_b200.bench.fabric_layer --model Qwen/Qwen3-8B --rows 16 64 256 2048

Rank 0 is the attention side, ranks 1..tp are the FFN TP group (``--tp``, world = 1 + tp).

* fused: the add-RMSNorm kernel stores the normalised rows straight into every FFN rank's slot and
  releases the sequence word; a Lane picks the invocation up, runs gate/up + SwiGLU and the down
  projection whose epilogue stores the partial into rank 0's buffer; rank 0's wait kernel sees the
  completion words and the next add-RMSNorm folds the partials (``parallel/fabric.py``).
* baseline: add-RMSNorm, then NCCL broadcast of the rows to the FFN group, the same two tcgen05 GEMMs as
  ordinary stream launches, NCCL reduce of the partials to rank 0, then the residual add in the next
  norm -- what a framework built from library collectives does.

Both are timed on rank 0 with CUDA events over ``--iters`` layer round trips after ``--warmup``; rank 0
prints one JSON line per row count with microseconds per layer, the roofline
``max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s, weight bytes / measured HBM bandwidth)``
and achieved / roofline for both paths.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0  # measured peer copy bandwidth per direction on this class of machine


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="Qwen/Qwen3-8B")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--rows", type=int, nargs="+", default=[16, 64, 256, 2048])
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    ctl = dist.new_group(backend="gloo")

    from ..bench.kernels import peaks
    from ..engine.atn_engine import EngineConfig
    from ..models import config as mc
    from ..models.weights import random_ffn_layer
    from ..ops import gemm, norm
    from ..parallel import fabric as F

    assert world == 1 + args.tp, "world size must be 1 + tp"
    cfg = mc.preset(args.model).with_layers(args.layers)
    cap = max(args.rows)
    place = F.InstancePlacement("m0", cfg, seed=5, atn_rank=0, ffn_ranks=tuple(range(1, world)), capacity_rows=cap)
    ecfg = EngineConfig(max_batch=min(cap, 256), prefill_chunk=cap, max_seq_len=256, use_cuda_graph=False)
    ctx = F.build_rank(F.Topology(world, [place]), rank, dev, {"m0": ecfg}, group=ctl, n_lanes=2)
    h, inter = cfg.hidden_size, cfg.intermediate_size // args.tp
    pk = peaks()
    results = []

    # ---------------------------------------------------------------- fused path
    if ctx.role == "ffn":
        ctx.ffn.start(lease_ms=20.0)
    dist.barrier(group=ctl)
    if ctx.role == "atn":
        port = ctx.engines["m0"].port
        w = torch.ones(h, dtype=torch.bfloat16, device=dev)
        for rows in args.rows:
            resid = (torch.randn(rows, h, device=dev) * 0.1).bfloat16()
            o = (torch.randn(rows, h, device=dev) * 0.1).bfloat16()
            x2 = torch.empty(rows, h, dtype=torch.bfloat16, device=dev)

            def layer(l):
                norm.add_rmsnorm([o], w, 1e-6, resid=resid, out=x2, want_local=False, **port.publish_targets(l, rows, 2))
                return port.run(l, x2, rows, 2)

            for i in range(args.warmup):
                layer(i % args.layers)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for i in range(args.iters):
                layer(i % args.layers)
            b.record()
            torch.cuda.synchronize()
            gemm.check_status(dev)
            results.append({"rows": rows, "fused_us": a.elapsed_time(b) * 1e3 / args.iters})
    dist.barrier(group=ctl)
    if ctx.role == "ffn":
        ctx.ffn.stop()
    dist.barrier(group=ctl)

    # ---------------------------------------------------------------- NCCL baseline
    ffn_group = dist.new_group(ranks=list(range(world)), backend="nccl")
    weights = None
    if ctx.role == "ffn":
        weights = [random_ffn_layer(cfg, l, 5, dev, torch.bfloat16, rank - 1, args.tp) for l in range(args.layers)]
    for k, rows in enumerate(args.rows):
        x = torch.zeros(rows, h, dtype=torch.bfloat16, device=dev)
        y = torch.zeros(rows, h, dtype=torch.bfloat16, device=dev)
        act = torch.zeros(rows, inter, dtype=torch.bfloat16, device=dev)
        resid = (torch.randn(rows, h, device=dev) * 0.1).bfloat16()
        o = (torch.randn(rows, h, device=dev) * 0.1).bfloat16()
        wn = torch.ones(h, dtype=torch.bfloat16, device=dev)

        def layer(l):
            if rank == 0:
                norm.add_rmsnorm([o], wn, 1e-6, resid=resid, out=x)
            dist.broadcast(x, src=0, group=ffn_group)
            if rank != 0:
                gemm.gateup_swiglu(x, weights[l].gate_up, out=act)
                gemm.linear(act, weights[l].down, out=y)
            else:
                y.zero_()
            dist.reduce(y, dst=0, group=ffn_group)

        for i in range(args.warmup):
            layer(i % args.layers)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier(group=ctl)
        a.record()
        for i in range(args.iters):
            layer(i % args.layers)
        b.record()
        torch.cuda.synchronize()
        if rank == 0:
            results[k]["nccl_us"] = a.elapsed_time(b) * 1e3 / args.iters
    if rank == 0:
        for r in results:
            rows = r["rows"]
            flops = 6.0 * rows * h * inter                      # per FFN rank
            t_flops = flops / (pk["bf16_tflops"] * 1e6)         # us
            link_bytes = rows * h * 2 * (1 + 1)                 # in to each rank + partial back, per rank, per direction
            t_link = link_bytes / (NVLINK_GBS * 1e3)
            t_w = 3.0 * h * inter * 2 / (pk["hbm_gbs"] * 1e3)
            roof = max(t_flops, t_link, t_w)
            r.update(model=args.model, tp=args.tp, roofline_us=round(roof, 2),
                     bound="flops" if roof == t_flops else "nvlink" if roof == t_link else "hbm(weights)",
                     fused_frac_of_roofline=round(roof / r["fused_us"], 3), nccl_frac_of_roofline=round(roof / r["nccl_us"], 3),
                     speedup_vs_nccl=round(r["nccl_us"] / r["fused_us"], 2), peaks=pk["source"])
            r["fused_us"], r["nccl_us"] = round(r["fused_us"], 2), round(r["nccl_us"], 2)
            print(json.dumps(r), flush=True)
    dist.barrier(group=ctl)
    if ctx.role == "ffn":
        ctx.ffn.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
