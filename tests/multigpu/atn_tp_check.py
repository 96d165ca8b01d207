"""Self-check of attention tensor parallelism, run under ``torch.distributed.run`` with one rank per GPU
(world size = TP size). Every rank holds its share of the heads and a replica of the FFN; all ranks run
the same requests. Rank 0 compares the result with an unsharded engine; every rank must produce the same
tokens. Prints ``ATN_TP_CHECK_OK`` on success.
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
    ap.add_argument("--model", default="Qwen/Qwen3-0.6B")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--graph", type=int, default=1)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    dist.init_process_group("gloo", rank=rank, world_size=world)

    from crosspool_b200.engine.atn_engine import AttentionEngine, EngineConfig
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights
    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import atn_tp

    cfg = mc.preset(args.model).with_layers(args.layers)
    ecfg = EngineConfig(max_batch=8, prefill_chunk=128, max_seq_len=256, use_cuda_graph=bool(args.graph))
    aw = random_attention_weights(cfg, 3, dev, torch.bfloat16)
    fw = random_ffn_weights(cfg, 3, dev, torch.bfloat16)
    tp = atn_tp.TpGroup(rank, world, max(ecfg.max_batch, ecfg.prefill_chunk), cfg.hidden_size, dev)
    handles = [None] * world
    dist.all_gather_object(handles, tp.handle())
    tp.connect(handles)
    dist.barrier()
    eng = AttentionEngine(atn_tp.local_config(cfg, world), atn_tp.shard_attention_weights(aw, cfg, rank, world),
                          LocalFfnPort(cfg, fw), ecfg, dev, tp=tp)
    eng.warmup()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 37, 90)]
    seqs = [eng.add_request(p, 6) for p in prompts]
    logits = {s.seq_id: [] for s in seqs}
    while eng.has_work:
        for i, (s, _) in enumerate(eng.step()):
            logits[s.seq_id].append(eng.logits[i].float().clone())
    torch.cuda.synchronize()
    gemm.check_status(dev)
    mine = [s.generated for s in seqs]
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    ok = all(e == mine for e in everyone)
    if rank == 0:
        print(f"[atn_tp_check] tokens identical on all ranks: {ok}", flush=True)
        ref = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), ecfg, dev)
        ref.warmup()
        rseqs = [ref.add_request(p, 6) for p in prompts]
        rlogits = {s.seq_id: [] for s in rseqs}
        while ref.has_work:
            for i, (s, _) in enumerate(ref.step()):
                rlogits[s.seq_id].append(ref.logits[i].float().clone())
        for s, r in zip(seqs, rseqs):
            good, n, kl = compare_generations(s.generated, r.generated, logits[s.seq_id], rlogits[r.seq_id])
            print(f"[atn_tp_check] seq {s.seq_id}: tokens agree {n}/{len(s.generated)} max KL {kl:.2e} ok {good}", flush=True)
            ok = ok and good
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag) == 1:
        print("ATN_TP_CHECK_OK", flush=True)
    dist.barrier()
    tp.close()
    dist.destroy_process_group()
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
