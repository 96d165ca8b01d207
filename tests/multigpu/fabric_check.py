"""Self-check of the multi-GPU Fabric, run under ``torch.distributed.run`` (one rank per GPU).

Rank 0 is the attention rank, ranks 1..tp are the FFN TP group. A short generation goes through the
Fabric and, on rank 0, through a loopback engine that holds the unsharded FFN weights; the logits of
both must agree. Prints ``FABRIC_CHECK_OK`` on success (the multi-GPU test greps for it).
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))
from crosspool_b200.testing import compare_generations  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--model", default="Qwen/Qwen3-0.6B")
    ap.add_argument("--lanes", type=int, default=1)
    ap.add_argument("--layer-split", type=int, default=0, help="split the layers over this many FFN groups of --tp ranks each")
    ap.add_argument("--atn-tp", type=int, default=1, help="attention TP ranks (ranks 0 .. atn_tp - 1); FFN ranks follow")
    args = ap.parse_args()

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    ctl = dist.new_group(backend="gloo")

    from crosspool_b200.engine.atn_engine import AttentionEngine, EngineConfig
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights
    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import fabric as F

    n_groups = max(1, args.layer_split)
    assert world >= args.atn_tp + args.tp * n_groups
    cfg = mc.preset(args.model).with_layers(args.layers)
    ecfg = EngineConfig(max_batch=8, prefill_chunk=128, max_seq_len=256)
    ffn_ranks = tuple(range(args.atn_tp, args.atn_tp + args.tp * n_groups))
    groups = ()
    if n_groups > 1:
        per = cfg.num_layers // n_groups
        groups = tuple((g * per, cfg.num_layers if g == n_groups - 1 else (g + 1) * per,
                        ffn_ranks[g * args.tp:(g + 1) * args.tp]) for g in range(n_groups))
    place = F.InstancePlacement("m0", cfg, seed=3, atn_rank=0, ffn_ranks=ffn_ranks, capacity_rows=128,
                                atn_tp_followers=tuple(range(1, args.atn_tp)), layer_groups=groups)
    topo = F.Topology(world, [place])
    ctx = F.build_rank(topo, rank, f"cuda:{local}", {"m0": ecfg}, group=ctl, n_lanes=args.lanes)
    ok = True
    if ctx.role == "ffn":
        ctx.ffn.start(lease_ms=20.0)
    dist.barrier(group=ctl)
    if ctx.role == "atn":
        eng = ctx.engines["m0"]
        eng.warmup()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 37, 90)]
        seqs = [eng.add_request(p, 6) for p in prompts]
        logits = {s.seq_id: [] for s in seqs}
        while eng.has_work:
            for i, (s, _) in enumerate(eng.step()):
                logits[s.seq_id].append(eng.logits[i].float().clone())
        gemm.check_status(eng.device)
        # loopback oracle with the unsharded weights
        aw = random_attention_weights(cfg, 3, eng.device, torch.bfloat16)
        fw = random_ffn_weights(cfg, 3, eng.device, torch.bfloat16)
        ref = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), ecfg, eng.device)
        ref.warmup()
        rseqs = [ref.add_request(p, 6) for p in prompts]
        rlogits = {s.seq_id: [] for s in rseqs}
        while ref.has_work:
            for i, (s, _) in enumerate(ref.step()):
                rlogits[s.seq_id].append(ref.logits[i].float().clone())
        for s, r in zip(seqs, rseqs):
            good, n, kl = compare_generations(s.generated, r.generated, logits[s.seq_id], rlogits[r.seq_id])
            print(f"[fabric_check] seq {s.seq_id}: tokens agree {n}/{len(s.generated)} max KL {kl:.2e} ok {good}", flush=True)
            ok = ok and good
    dist.barrier(group=ctl)
    if ctx.role == "ffn":
        st = ctx.ffn.stats()
        ctx.ffn.stop()
        print(f"[fabric_check] rank {rank} lane stats {st} errors {ctx.ffn.errors}", flush=True)
        ok = ok and not ctx.ffn.errors and st["status"] == 0 and st["served"][0] > 0
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ctl)
    if rank == 0 and int(flag) == 1:
        print("FABRIC_CHECK_OK", flush=True)
    dist.barrier(group=ctl)
    if ctx.role == "ffn":
        ctx.ffn.close()
    dist.destroy_process_group()
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
