"""``torch.ops.xpool.ffn_shim`` end to end on two GPUs, run under ``torch.distributed.run`` (rank 0: the Instance of an
external engine, rank 1: the FFN tier). Rank 0 calls the native operator on CUDA tensors exactly as a replaced decoder
MLP would, eagerly and from a captured CUDA graph; the result must equal the layer's FFN computed locally from the
unsharded weights. Prints ``SHIM_CHECK_OK`` on success.
"""

from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    from crosspool_b200.engine.atn_engine import EngineConfig
    from crosspool_b200.integrations.sglang import shim
    from crosspool_b200.integrations.sglang.transport import FabricInstanceTransport
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import dense_ffn
    from crosspool_b200.models.weights import random_ffn_layer
    from crosspool_b200.native import runtime as rt
    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import fabric as F

    assert world == 2
    cfg = mc.preset("Qwen/Qwen3-0.6B").with_layers(3)
    place = F.InstancePlacement("m0", cfg, seed=3, atn_rank=0, ffn_ranks=(1,), capacity_rows=128)
    ctx = F.build_rank(F.Topology(world, [place]), rank, f"cuda:{local}", {"m0": EngineConfig(max_batch=8, prefill_chunk=128, max_seq_len=256)},
                       n_lanes=2)
    ok = True
    if ctx.role == "ffn":
        ctx.ffn.start(lease_ms=5.0)
    dist.barrier()
    if ctx.role == "atn":
        dev = torch.device(f"cuda:{local}")
        tr = FabricInstanceTransport.from_port(ctx.engines["m0"].port)
        tr.make_current()
        print(f"[shim_check] operator backend: {shim.OP_BACKEND}", flush=True)
        ok = ok and shim.OP_BACKEND == "native"
        for layer, rows in ((0, 5), (2, 64), (1, 1)):
            x = (torch.randn(rows, cfg.hidden_size, device=dev) * 0.5).bfloat16()
            out = torch.full_like(x, float("nan"))
            torch.ops.xpool.ffn_shim(x, None, out, layer, rt.MODE_DECODE, rt.OUT_PER_RANK_COMPLETE, rt.DP_NONE)
            torch.cuda.synchronize(dev)
            w = random_ffn_layer(cfg, layer, 3, dev, torch.bfloat16)
            ref = dense_ffn(x.float(), type(w)(w.gate_up.float(), w.down.float()))
            err = (out.float() - ref).abs().max().item()
            print(f"[shim_check] layer {layer} rows {rows}: max abs err {err:.4f}", flush=True)
            ok = ok and err < 3e-2 and bool(torch.isfinite(out.float()).all())
        # the operator inside a captured graph (what an engine's decode graphs do)
        x = (torch.randn(8, cfg.hidden_size, device=dev) * 0.5).bfloat16()
        out = torch.zeros_like(x)
        stream = torch.cuda.Stream(dev)
        with torch.cuda.stream(stream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                torch.ops.xpool.ffn_shim(x, None, out, 1, rt.MODE_DECODE, rt.OUT_PER_RANK_COMPLETE, rt.DP_NONE)
            for _ in range(3):
                x.copy_((torch.randn(8, cfg.hidden_size, device=dev) * 0.5).bfloat16())
                g.replay()
                stream.synchronize()
                w = random_ffn_layer(cfg, 1, 3, dev, torch.bfloat16)
                err = (out.float() - dense_ffn(x.float(), type(w)(w.gate_up.float(), w.down.float()))).abs().max().item()
                ok = ok and err < 3e-2
        print(f"[shim_check] graph replays ok: {ok}", flush=True)
        gemm.check_status(dev)
        ok = ok and tr.failure() is None
        tr.close()
    dist.barrier()
    if ctx.role == "ffn":
        st = ctx.ffn.stats()
        ctx.ffn.stop()
        print(f"[shim_check] rank 1 lane stats {st} errors {ctx.ffn.errors}", flush=True)
        ok = ok and not ctx.ffn.errors and st["status"] == 0 and st["served"][0] >= 6
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag) == 1:
        print("SHIM_CHECK_OK", flush=True)
    dist.barrier()
    if ctx.role == "ffn":
        ctx.ffn.close()
    dist.destroy_process_group()
    return 0 if int(flag) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
