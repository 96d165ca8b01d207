"""Baseline arm: the same attention/FFN disaggregation built from library calls.

What a framework assembled from host-launched collectives does for one decoder FFN: the attention rank
broadcasts the normalised hidden states to the Instance's FFN ranks with NCCL, every FFN rank runs its shard as
cuBLAS GEMMs (``torch.matmul``) with a separate elementwise SwiGLU, and NCCL reduces the partial outputs back to
the attention rank, whose next add-RMSNorm adds them to the residual stream. The benchmarks compare the Fabric
(kernels that store into peer memory, ``parallel/fabric.py``) against this arm on the same deployment and
workload. None of this repository's FFN kernels, Lanes or flag protocol run here.

One NCCL communicator per Instance holds its attention rank and its FFN ranks, beside a gloo group of the same
members. Per engine iteration the attention rank first announces the row count on the host (a gloo broadcast, made
right before the iteration's kernels are enqueued); the FFN rank's service thread waits for that announcement on the
host and then enqueues all layers' receive -> GEMMs -> reduce without further host synchronisation. An announcement
of 0 rows ends the service thread. No collective kernel therefore sits on an FFN GPU waiting for work that has not
been decided yet: a library kernel that waits indefinitely blocks every CUDA call of the process that synchronises
the device (an allocation, a handle creation), which is how an FFN rank serving several Instances stops for good.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass, field
from datetime import timedelta

import torch
import torch.distributed as dist

from ..engine.atn_engine import AttentionEngine, EngineConfig, FfnPort
from ..engine.ffn_local import unfused_dense_ffn
from ..models.weights import random_attention_weights, random_ffn_layer
from .fabric import InstancePlacement, Topology


class NcclFfnPort(FfnPort):
    def __init__(self, place: InstancePlacement, group, host_group, device):
        self.place, self.group, self.host_group, self.device = place, group, host_group, torch.device(device)
        self.me = place.atn_rank
        self._hdr_host = torch.zeros(4, dtype=torch.int64)
        self.y = None

    def attach(self, engine: AttentionEngine) -> None:
        self.y = torch.zeros(engine.cap, self.place.cfg.hidden_size, dtype=torch.bfloat16, device=self.device)

    def announce_forward(self, rows: int, mode: int) -> None:
        """Host side, before the iteration's kernels are enqueued: tells the FFN ranks how many rows are coming."""
        self._hdr_host[0], self._hdr_host[1] = rows, mode
        dist.broadcast(self._hdr_host, src=self.me, group=self.host_group)

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> list[torch.Tensor]:
        dist.broadcast(x[:rows], src=self.me, group=self.group)
        y = self.y[:rows]
        y.zero_()                                  # the attention rank contributes nothing to the sum
        dist.reduce(y, dst=self.me, group=self.group)
        return [y]

    def shutdown(self) -> None:
        self._hdr_host[0] = 0
        dist.broadcast(self._hdr_host, src=self.me, group=self.host_group)


@dataclass
class _Served:
    place: InstancePlacement
    group: object
    host_group: object
    tp_rank: int
    weights: list
    thread: threading.Thread | None = None
    iterations: int = 0


class NcclFfnRank:
    """FFN side of the baseline: one service thread and one stream per Instance."""

    def __init__(self, device):
        self.device = torch.device(device)
        self.served: list[_Served] = []
        self.errors: list[str] = []

    def add_instance(self, place: InstancePlacement, group, host_group, tp_rank: int) -> None:
        cfg = place.cfg
        weights = []
        for l in range(cfg.num_layers):
            if cfg.layer_is_moe(l) and place.expert_parallel:
                weights.append(random_ffn_layer(cfg, l, place.seed, self.device, torch.bfloat16,
                                                expert_range=place.expert_range(tp_rank)))
            else:
                weights.append(random_ffn_layer(cfg, l, place.seed, self.device, torch.bfloat16, tp_rank, place.tp))
        self.served.append(_Served(place, group, host_group, tp_rank, weights))

    def _serve(self, sv: _Served) -> None:
        try:
            torch.cuda.set_device(self.device)
            p, cfg, dev, bf = sv.place, sv.place.cfg, self.device, torch.bfloat16
            cap, src = p.capacity_rows, p.atn_rank
            stream = torch.cuda.Stream(dev)
            dense = [w for w in sv.weights if not w.is_moe]
            inter2 = max((w.gate_up.shape[0] for w in dense), default=2)
            moe_ws = None
            with torch.cuda.stream(stream):
                hdr_host = torch.zeros(4, dtype=torch.int64)
                x = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
                gu = torch.zeros(cap, inter2, dtype=bf, device=dev)
                act = torch.zeros(cap, inter2 // 2, dtype=bf, device=dev)
                y = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
                if any(w.is_moe for w in sv.weights):
                    from ..ops import moe

                    w0 = next(w for w in sv.weights if w.is_moe)
                    moe_ws = moe.workspace(dev, cap, cfg, w0.gate_up.shape[1] // 2, w0.gate_up.shape[0])
                while True:
                    dist.broadcast(hdr_host, src=src, group=sv.host_group)   # host-side wait for the announcement
                    rows = int(hdr_host[0])
                    if rows <= 0:
                        return
                    for w in sv.weights:
                        xr = x[:rows]
                        dist.broadcast(xr, src=src, group=sv.group)
                        if w.is_moe:
                            from ..ops import moe

                            out = moe.moe_forward(xr, w, cfg, out=y[:rows], ws=moe_ws,
                                                  expert_range=p.expert_range(sv.tp_rank) if p.expert_parallel else None)
                        else:
                            out = unfused_dense_ffn(xr, w, gu, act, y)
                        dist.reduce(out, dst=src, group=sv.group)
                    sv.iterations += 1
        except Exception as e:  # pragma: no cover - surfaced through .errors
            self.errors.append(f"{sv.place.model_id}: {e!r}")

    def start(self) -> None:
        for sv in self.served:
            sv.thread = threading.Thread(target=self._serve, args=(sv,), daemon=True, name=f"nccl-ffn-{sv.place.model_id}")
            sv.thread.start()

    def stats(self) -> dict:
        return {"served": [sv.iterations * sv.place.cfg.num_layers for sv in self.served], "idle_replays": [], "status": 0,
                "errors": list(self.errors)}

    def stop(self) -> None:
        for sv in self.served:
            if sv.thread is not None:
                sv.thread.join(20)

    def close(self) -> None:
        self.served.clear()


@dataclass
class BaselineContext:
    rank: int
    role: str
    engines: dict[str, AttentionEngine] = field(default_factory=dict)
    ffn: NcclFfnRank | None = None
    ports: list[NcclFfnPort] = field(default_factory=list)


def build_rank(topo: Topology, rank: int, device, ecfg_for: dict[str, EngineConfig], ctl_group, kv_for=None,
               timeout_s: float = 120.0) -> BaselineContext:
    """Collective over all ranks: one NCCL communicator per Instance (its attention rank + its FFN ranks), then
    this rank's engines or FFN services."""
    role = topo.role(rank)
    ctx = BaselineContext(rank, role)
    if role == "ffn":
        ctx.ffn = NcclFfnRank(device)
    for p in topo.instances:
        if p.layer_groups or p.atn_tp_followers:
            raise ValueError("the baseline arm covers one attention rank and one FFN TP group per Instance")
        members = [p.atn_rank, *p.ffn_ranks]
        g = dist.new_group(ranks=members, backend="nccl", timeout=timedelta(seconds=timeout_s))
        hg = dist.new_group(ranks=members, backend="gloo", timeout=timedelta(seconds=max(timeout_s, 600.0)))
        if rank in members:
            # Communicators are created on first use, and creation is itself a collective. Doing it here, on one thread
            # and in the same order on every rank, keeps the service threads of an FFN rank that serves several
            # Instances from creating theirs in different orders on different ranks (which never completes).
            t = torch.zeros(1, device=device)
            dist.all_reduce(t, group=g)
            torch.cuda.synchronize(device)
        if rank == p.atn_rank:
            port = NcclFfnPort(p, g, hg, device)
            aw = random_attention_weights(p.cfg, p.seed, device, torch.bfloat16)
            kv = kv_for(p) if kv_for is not None else None
            ctx.engines[p.model_id] = AttentionEngine(p.cfg, aw, port, ecfg_for[p.model_id], device, kv=kv)
            ctx.ports.append(port)
        elif rank in p.ffn_ranks:
            ctx.ffn.add_instance(p, g, hg, p.ffn_ranks.index(rank))
    dist.barrier(group=ctl_group)
    return ctx
