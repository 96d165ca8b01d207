"""Canonical generation failure across two GPUs, run under ``torch.distributed.run`` (rank 0: attention, rank 1: FFN).

The failure is made on the host: rank 0 publishes an invocation that names a layer the FFN rank does not hold. The
Lane refuses it, claims its device's failure slot and copies the payload into rank 0's slot; rank 0's completion wait,
which has a 5 s limit, is cancelled by that word within the same layer call instead of running out. Both ranks then
read the same payload (result code, origin PE, sequence, layer). Nothing on either GPU faults, traps or hangs: the
refused invocation is answered with a completion record like any other. Prints ``FAILURE_CHECK_OK`` on success.
"""

from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))


def _attention_side(ctx, cfg, devkit, gemm, norm) -> bool:
    ok = True
    port = ctx.engines["m0"].port
    port.enable_trace(256)
    dev = port.device
    rows, h = 4, cfg.hidden_size
    w = torch.ones(h, dtype=torch.bfloat16, device=dev)
    o = (torch.randn(rows, h, device=dev) * 0.1).bfloat16()
    resid = torch.zeros(rows, h, dtype=torch.bfloat16, device=dev)
    x2 = torch.empty(rows, h, dtype=torch.bfloat16, device=dev)

    def call(layer):
        norm.add_rmsnorm([o], w, 1e-6, resid=resid, out=x2, want_local=False, **port.publish_targets(layer, rows, 2))
        port.run(layer, x2, rows, 2)
        torch.cuda.synchronize(dev)

    call(0)                                     # a good invocation first
    status = gemm.status_words(dev)
    assert int(status[0]) == 0 and port.failure() is None
    # the completion of the refused invocation still arrives, so make the wait look for the one after it: only
    # the failure word can end it before its 5 s limit
    t0 = time.monotonic()
    bad = dict(port.publish_targets(0, rows, 2), meta=(999, 2, 0))    # layer 0's FFN rank, but a layer nobody holds
    norm.add_rmsnorm([o], w, 1e-6, resid=resid, out=x2, want_local=False, **bad)
    torch.cuda.synchronize(dev)
    port.seq += 1                               # wait for sequence 3, which nobody will ever publish
    port.run(999, x2, rows, 2)
    torch.cuda.synchronize(dev)
    elapsed = time.monotonic() - t0
    f = port.failure()
    code = int(status[0])
    status.zero_()
    print(f"[failure_check] rank 0: wait ended after {elapsed * 1e3:.1f} ms with status {code}, failure {f}", flush=True)
    ok = ok and code == 5 and elapsed < 2.0 and f is not None
    ok = ok and (f.result_code, f.origin_pe, f.invocation_sequence, f.layer_ordinal) == (2, 1, 2, 999)
    tl = devkit.AtnFabricObserver(port).collect()
    names = [e["name"] for e in tl.events]
    ok = ok and names.count("published") == 2 and "wait_cancelled" in names
    print(f"[failure_check] rank 0 events {names}", flush=True)
    return ok


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    from crosspool_b200 import devkit
    from crosspool_b200.engine.atn_engine import EngineConfig
    from crosspool_b200.models import config as mc
    from crosspool_b200.ops import gemm, norm
    from crosspool_b200.parallel import fabric as F

    assert world == 2
    cfg = mc.preset("Qwen/Qwen3-0.6B").with_layers(2)
    place = F.InstancePlacement("m0", cfg, seed=3, atn_rank=0, ffn_ranks=(1,), capacity_rows=128)
    ctx = F.build_rank(F.Topology(world, [place]), rank, f"cuda:{local}", {"m0": EngineConfig(max_batch=8, prefill_chunk=128, max_seq_len=256)},
                       n_lanes=1)
    ok = True
    if ctx.role == "ffn":
        ctx.ffn.enable_trace(256)
        ctx.ffn.start(lease_ms=5.0)
    dist.barrier()
    if ctx.role == "atn":
        try:
            ok = _attention_side(ctx, cfg, devkit, gemm, norm)
        except Exception:           # reported below; both ranks still leave together
            import traceback

            print("[failure_check] rank 0 raised:\n" + traceback.format_exc(), flush=True)
            ok = False
    dist.barrier()
    if ctx.role == "ffn":
        f = ctx.ffn.failure()
        names = [e["name"] for e in devkit.FabricObserver(ctx.ffn).collect().events]
        print(f"[failure_check] rank 1: failure {f}; events {[n for n in names if n != 'idle']}", flush=True)
        ok = ok and f is not None and (f.result_code, f.origin_pe, f.invocation_sequence, f.layer_ordinal) == (2, 1, 2, 999)
        ok = ok and "failure_claimed" in names
        ctx.ffn.stop()
        ok = ok and not ctx.ffn.errors
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag) == 1:
        print("FAILURE_CHECK_OK", flush=True)
    dist.barrier()
    if ctx.role == "ffn":
        ctx.ffn.close()
    dist.destroy_process_group()
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
