"""Multi-GPU layout of the decode benchmark (``bench.py --gpus N`` under ``torch.distributed.run``).

The last ``max(1, N // 4)`` ranks (or ``--ffn-ranks``) form the shared FFN tier, the others are attention
ranks: decode is bound by KV reads on the attention side, and one FFN GPU keeps up with the FFN
invocations of about six co-located Instances of this size, so the pool is kept small (that is the
point of pooling FFNs). Every attention rank hosts ``--instances-per-atn`` co-located Instances;
Instance ``j`` keeps its FFN on FFN rank(s) ``(j .. j + tp - 1) mod n_ffn``, so every FFN GPU serves
Instances of several attention GPUs. Times are device times, maximum over ranks.
"""

from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist


def main(args) -> int:
    from ..deployment import Deployment, InstanceHandle
    from ..models import config as mc
    from ..native import runtime as rt
    from ..parallel import fabric as F
    from . import decode_bench as db

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    if world != args.gpus or world < 2:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE == {args.gpus} >= 2 (got {world})")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    ctl = dist.new_group(backend="gloo")

    cfg = mc.load(args.model)
    if args.layers:
        cfg = cfg.with_layers(args.layers)
    n_ffn = getattr(args, "ffn_ranks", 0) or max(1, world // 4)
    n_ffn = min(n_ffn, world - 1)
    n_atn = world - n_ffn
    tp = max(1, min(args.ffn_tp, n_ffn))
    placements, workloads, ecfgs = [], {}, {}
    j = 0
    for a in range(n_atn):
        for i in range(args.instances_per_atn):
            model_id = f"{args.model}#{j}"
            wl = db.make_workload(cfg, args.batch, args.min_prompt, args.max_prompt, args.steps, args.warmup, seed=j)
            workloads[model_id] = wl
            ecfgs[model_id] = db.engine_config(args.batch, wl)
            ffn = tuple(n_atn + (j + t) % n_ffn for t in range(tp))
            cap = max(ecfgs[model_id].max_batch, ecfgs[model_id].prefill_chunk)
            placements.append(F.InstancePlacement(model_id, cfg, seed=j, atn_rank=a, ffn_ranks=ffn, capacity_rows=cap))
            j += 1
    topo = F.Topology(world, placements)
    policy = {"fifo": rt.POLICY_FIFO, "random": rt.POLICY_RANDOM, "slo": rt.POLICY_SLO}[getattr(args, "policy", "fifo")]
    ctx = F.build_rank(topo, rank, f"cuda:{local}", ecfgs, group=ctl, n_lanes=args.lanes, policy=policy)
    if policy == rt.POLICY_SLO:
        for eng in ctx.engines.values():
            eng.port.slo_tbt_ms = 50.0
    trace_dir = getattr(args, "trace_dir", "")
    if ctx.role == "ffn":
        if trace_dir:
            ctx.ffn.enable_trace(1 << 18)   # fabric observer: Lane admissions / completions with device timestamps
        ctx.ffn.start(lease_ms=20.0)
    dist.barrier(group=ctl)

    def sync():
        dist.barrier(group=ctl)

    vals = torch.zeros(8, dtype=torch.float64)
    res = None
    if ctx.role == "atn":
        insts = [InstanceHandle(p.model_id, cfg, ctx.engines[p.model_id]) for p in placements if p.atn_rank == rank]
        res = db.run_rank(Deployment(insts), {i.model_id: workloads[i.model_id] for i in insts}, args.batch, args.steps,
                          args.warmup, gpu_index=local, sync=sync)
        vals[0], vals[1], vals[2] = res.dev_ms, res.e2e_s, res.e2e_tokens
        vals[3], vals[4] = res.tokens_per_step, res.launches_per_step
        vals[5], vals[6] = res.h2d_per_step, res.d2h_per_step
    else:
        # FFN ranks join the barriers that bracket the measured regions
        for _ in range(db.SYNCS_PER_RUN):
            sync()
    mx = vals.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=ctl)
    sm = vals.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=ctl)
    lane_stats = None
    if ctx.role == "ffn":
        lane_stats = ctx.ffn.stats()
        ctx.ffn.stop()
        if trace_dir:
            from .. import devkit

            os.makedirs(trace_dir, exist_ok=True)
            art = devkit.FabricObserver(ctx.ffn, role=f"FfnAgent-rank{rank}").collect()
            tail = art.events[-20000:]      # the timed region is at the end of the run
            art.events = tail
            with open(os.path.join(trace_dir, f"lanes_rank{rank}.chrome.json"), "w") as f:
                json.dump(devkit.chrome_trace([art]), f)
            lane_stats["trace"] = {"events": len(tail), "dropped": art.dropped}
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank, "role": ctx.role, "lanes": lane_stats,
                                      "step_ms": res.step_ms if res else None, "ttft_ms": res.ttft_ms if res else None,
                                      "clocks": res.clocks if res else None}, group=ctl)
    if rank == 0:
        step_ms = [max(v) for v in zip(*[g["step_ms"] for g in gathered if g["step_ms"]])]
        ttft = [t for g in gathered if g["ttft_ms"] for t in g["ttft_ms"]]
        out = db.result_json(
            args, cfg, world, f"atn{n_atn} (one Instance set per GPU) + ffn{n_ffn} shared tier, ffn_tp={tp}, lanes={args.lanes}",
            len(placements), int(sm[3]), float(mx[0]), float(mx[1]), int(sm[2]), step_ms, ttft, int(sm[5]), int(sm[6]),
            int(sm[4]) + 4 * len(placements) * cfg.num_layers * tp, res.clocks,
            extra_config={"lane_stats": [g["lanes"] for g in gathered if g["lanes"]]})
        print(json.dumps(out), flush=True)
    dist.barrier(group=ctl)
    if ctx.role == "ffn":
        ctx.ffn.close()
    dist.destroy_process_group()
    return 0
