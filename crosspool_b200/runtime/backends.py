"""GPU backends of the agent roles: what ``prepare_join`` ... ``finalize`` do on a device.

Arena handles travel as hex strings through the daemon's plan (``slot_handles``):
``ffn:<model>:<atn rank>:<ffn pe>`` for an FFN rank's slot of one Instance rank and
``atn:<model>:<atn rank>`` for the attention-side slot (completion records + TP partial buffers).
"""

from __future__ import annotations

import threading
import zlib

import torch

from ..config import XpoolConfig
from ..engine.atn_engine import AttentionEngine, EngineConfig
from ..models.weights import load_attention_from_safetensors, random_attention_weights
from ..native import runtime as rt
from ..parallel import fabric as F
from ..service.wire import FabricPlan, InvocationFailure, ServingListener

_POLICY = {"fifo": rt.POLICY_FIFO, "random": rt.POLICY_RANDOM, "slo": rt.POLICY_SLO}


def model_config_for(cfg: XpoolConfig, model_id: str):
    """The model's shape: a preset named by ``path`` or ``id``, else the ``config.json`` under ``path``."""
    return cfg.model_shape(model_id)


def checkpoint_dir_for(cfg: XpoolConfig, model_id: str) -> str | None:
    """The model's checkpoint directory when its path (``XpoolConfig.model_path``) names one (``config.json`` plus
    safetensors files); None for presets, which run on random-init weights."""
    p = cfg.model_path(model_id)
    if p is not None and p.is_dir() and (p / "config.json").exists() and any(p.glob("*.safetensors")):
        return str(p)
    return None


def placement_for(cfg: XpoolConfig, plan: FabricPlan, model_id: str, atn_rank: int, capacity_rows: int) -> F.InstancePlacement:
    """The placement of one Instance rank as the plan states it: FFN ranks per layer group in TP order, the attention TP
    followers, seed or checkpoint. Every backend (GPU, CPU, an engine process of its own) derives it here."""
    shards = [s for s in plan.shards if s.model_id == model_id]
    ranges = sorted({(s.layer_begin, s.layer_end) for s in shards})
    groups = tuple((lo, hi, tuple(s.pe for s in sorted((x for x in shards if (x.layer_begin, x.layer_end) == (lo, hi)),
                                                        key=lambda x: x.tp_rank))) for lo, hi in ranges)
    tp = cfg.model(model_id).atn_tp_size
    leader = atn_rank - atn_rank % tp        # attention TP groups are runs of ``atn_tp_size`` consecutive Instance ranks
    by_rank = {r.rank: r for r in plan.instance_ranks if r.model_id == model_id}
    rank = by_rank[leader]
    followers = tuple(by_rank[leader + i].pe for i in range(1, tp))
    seed = zlib.crc32(model_id.encode()) % 1000  # random-init deployments: same seed on every rank of a model
    union = tuple(pe for g in groups for pe in g[2])
    return F.InstancePlacement(model_id, model_config_for(cfg, model_id), seed, rank.pe, union, capacity_rows,
                               layer_groups=groups if len(groups) > 1 else (),
                               checkpoint=checkpoint_dir_for(cfg, model_id), atn_tp_followers=followers)



class FfnBackend:
    def __init__(self, cfg: XpoolConfig, device: int, capacity_rows: int = 4096, local_index: int | None = None):
        self.cfg, self.device, self.capacity_rows = cfg, device, capacity_rows
        self.cuda = torch.device(f"cuda:{device if local_index is None else local_index}")
        self.rt: F.FfnRankRuntime | None = None
        self._keys: list[tuple[F.FfnInstanceState, str]] = []

    def prepare_join(self, plan: FabricPlan) -> dict[str, str]:
        torch.cuda.set_device(self.cuda)
        my_pe = len(plan.atn_devices) + plan.ffn_devices.index(self.device)
        self.rt = F.FfnRankRuntime(self.cuda, n_lanes=plan.lanes_per_ffn_device, policy=_POLICY[plan.policy],
                                   seed=self.cfg.scheduler_ffn_random_seed or 0, pe=my_pe)
        handles = {}
        for r in plan.instance_ranks:
            if r.rank % self.cfg.model(r.model_id).atn_tp_size:
                continue    # an attention TP follower: the group's first rank talks to the FFN tier for all of them
            place = placement_for(self.cfg, plan, r.model_id, r.rank, self.capacity_rows)
            if my_pe not in place.ffn_ranks:
                continue
            tp_rank, lo, hi = place.locate(my_pe)
            st = self.rt.add_instance(place, tp_rank, (lo, hi))
            self._keys.append((st, f"atn:{r.model_id}:{r.rank}"))
            handles[f"ffn:{r.model_id}:{r.rank}:{my_pe}"] = st.slot.handle().hex()
        return handles

    def join(self, plan: FabricPlan) -> None:
        for st, key in self._keys:
            st.atn_base = F.PeerBuffer.open(bytes.fromhex(plan.slot_handles[key]))

    def prepare_execution(self, plan: FabricPlan) -> None:
        self.rt.install()

    def activate(self, plan: FabricPlan) -> None:
        self.rt.start(lease_ms=20.0)

    def poll_health(self) -> InvocationFailure | None:
        if self.rt is None:
            return None
        if self.rt.errors:
            raise RuntimeError("; ".join(self.rt.errors))
        f = self.rt.failure()     # the canonical failure: who met it, for which Instance, sequence and layer
        if f is not None:
            return InvocationFailure(result_code=f.result_code, origin_pe=f.origin_pe, instance_index=f.instance_index,
                                     invocation_sequence=f.invocation_sequence, layer_ordinal=f.layer_ordinal)
        st = self.rt.stats()
        if st["status"] != 0:   # a kernel status outside any invocation (no slot to blame)
            return InvocationFailure(result_code=3, origin_pe=self.rt.pe, instance_index=0, invocation_sequence=0, layer_ordinal=0)
        return None

    def quiesce(self) -> None:
        if self.rt:
            self.rt.stop()

    def drain(self) -> bool:
        torch.cuda.synchronize(self.cuda)
        return True

    def finalize(self) -> None:
        if self.rt:
            self.rt.close()
            self.rt = None


class AtnBackend:
    def __init__(self, cfg: XpoolConfig, device: int, instances: list[tuple[str, int]], ecfg: EngineConfig,
                 capacity_rows: int = 4096, local_index: int | None = None, listen: tuple[str, int] | None = None,
                 external: list[tuple[str, int]] | None = None, publish_arenas=None):
        """``external``: Instance ranks of this device that run in processes of their own (``[[models]] external = true``).
        For them the agent allocates the attention-side slot, publishes its IPC handle to the FFN ranks (plan) and to
        the daemon's arena broker (``publish_arenas(generation, [TransportArenaBinding])``), and hosts no engine; the
        rank's process maps it with ``integrations.sglang.transport.FabricInstanceTransport.from_handles``. This half has
        run on the CPU data plane only (``runtime/cpu_backends.py``), not yet on GPUs."""
        self.cfg, self.device, self.instances, self.ecfg = cfg, device, instances, ecfg
        self.external, self.publish_arenas = list(external or ()), publish_arenas
        self.capacity_rows = max(capacity_rows, ecfg.max_batch, ecfg.prefill_chunk)
        self.cuda = torch.device(f"cuda:{device if local_index is None else local_index}")
        self.buffers: dict[tuple[str, int], F.PeerBuffer] = {}
        self.places: dict[tuple[str, int], F.InstancePlacement] = {}
        self.engines: dict[str, AttentionEngine] = {}
        self.tp_groups: dict[tuple[str, int], object] = {}
        self._agree = None
        self.loop = None
        self._server = None
        self._listen = listen
        self.listener: ServingListener | None = None
        self.ecs_ref = None          # callable(generation) -> EcsChannelRef, set by the launcher when elastic KV is on
        self._ecs_channel = None
        self._reconcilers = []

    def _tp(self, model_id: str, rank: int) -> tuple[int, int, int]:
        """(TP rank, TP size, Instance rank of the group's first member)."""
        t = self.cfg.model(model_id).atn_tp_size
        return rank % t, t, rank - rank % t

    def prepare_join(self, plan: FabricPlan) -> dict[str, str]:
        from ..parallel import atn_tp

        torch.cuda.set_device(self.cuda)
        handles = {}
        for model_id, rank in self.instances:
            place = placement_for(self.cfg, plan, model_id, rank, self.capacity_rows)
            self.places[(model_id, rank)] = place
            tpr, tps, _ = self._tp(model_id, rank)
            if tpr == 0:
                buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
                self.buffers[(model_id, rank)] = buf
                handles[f"atn:{model_id}:{rank}"] = buf.handle().hex()
            if tps > 1:
                g = atn_tp.TpGroup(tpr, tps, max(self.ecfg.max_batch, self.ecfg.prefill_chunk), place.cfg.hidden_size, self.cuda)
                self.tp_groups[(model_id, rank)] = g
                handles[f"atp:{model_id}:{rank}"] = g.handle().hex()
        if self.external:
            from ..service.wire import TransportArenaBinding

            arenas = []
            for model_id, rank in self.external:
                if self.cfg.model(model_id).atn_tp_size != 1:
                    raise NotImplementedError("external Instance ranks with attention tensor parallelism are not brokered")
                place = placement_for(self.cfg, plan, model_id, rank, self.capacity_rows)
                nbytes = F.atn_slot_layout(place).total_bytes
                buf = F.PeerBuffer(nbytes)
                self.buffers[(model_id, rank)] = buf                 # freed in finalize with the hosted ranks' slots
                handles[f"atn:{model_id}:{rank}"] = buf.handle().hex()
                arenas.append(TransportArenaBinding(model_id=model_id, rank=rank, handle_hex=buf.handle().hex(), nbytes=nbytes))
            if self.publish_arenas is not None:
                self.publish_arenas(plan.generation, arenas)
        return handles

    def join(self, plan: FabricPlan) -> None:
        self._bases, self._leader_base = {}, {}
        for (model_id, rank), place in self.places.items():
            tpr, tps, leader = self._tp(model_id, rank)
            if tpr == 0:
                self._bases[(model_id, rank)] = [F.PeerBuffer.open(bytes.fromhex(plan.slot_handles[f"ffn:{model_id}:{rank}:{pe}"]))
                                                 for pe in place.ffn_ranks]
            else:
                self._leader_base[(model_id, rank)] = F.PeerBuffer.open(bytes.fromhex(plan.slot_handles[f"atn:{model_id}:{leader}"]))
            g = self.tp_groups.get((model_id, rank))
            if g is not None:
                g.connect([bytes.fromhex(plan.slot_handles[f"atp:{model_id}:{leader + i}"]) for i in range(tps)])

    def prepare_execution(self, plan: FabricPlan) -> None:
        from ..parallel import atn_tp

        for (model_id, rank), place in self.places.items():
            tpr, tps, _ = self._tp(model_id, rank)
            if tpr == 0:
                port = F.FabricFfnPort(place, self.buffers[(model_id, rank)], self._bases[(model_id, rank)], self.cuda)
                port.slo_tbt_ms = self.cfg.slo_for(model_id).tbt_ms   # per-step deadline for the Lanes' SLO policy
            else:
                port = F.FabricFfnFollowerPort(place, self._leader_base[(model_id, rank)], self.cuda)
            if place.checkpoint:
                aw = load_attention_from_safetensors(place.cfg, place.checkpoint, self.cuda, torch.bfloat16)
            else:
                aw = random_attention_weights(place.cfg, place.seed, self.cuda, torch.bfloat16)
            cfg_local, g = place.cfg, self.tp_groups.get((model_id, rank))
            if g is not None:
                aw = atn_tp.shard_attention_weights(aw, place.cfg, tpr, tps)
                cfg_local = atn_tp.local_config(place.cfg, tps)
            kv = self._elastic_cache(plan, model_id, rank, cfg_local) if self.cfg.atn_elastic_kv and self.ecs_ref else None
            eng = AttentionEngine(cfg_local, aw, port, self.ecfg, self.cuda, kv=kv, tp=g)
            if kv is not None:
                self._attach_capacity(eng, model_id, rank, tp=g is not None)
            self.engines[model_id] = eng
        if self._ecs_channel is not None:
            free, total = torch.cuda.mem_get_info(self.cuda)
            self._ecs_channel.publish_report(self._ecs_ref.devices[str(self.device)], free, total, 1)

    # ------------------------------------------------------------------ elastic KV
    def _elastic_cache(self, plan: FabricPlan, model_id: str, rank: int, model_cfg):
        """A KV cache over VMM bundles with one bundle mapped; the Instance rank describes its partition
        (floor = one bundle, reservation = the whole range) in the daemon's control channel."""
        import time

        from ..ecs import vmm
        from ..native.runtime import EcsChannel

        if self._ecs_channel is None:
            for _ in range(200):                      # the daemon opens the channel on its next policy tick
                try:
                    self._ecs_ref = self.ecs_ref(plan.generation)
                    break
                except Exception:
                    time.sleep(0.05)
            else:
                raise RuntimeError("the daemon did not publish an ECS control channel")
            self._ecs_channel = EcsChannel.attach(self._ecs_ref.name)
            self._driver, self._quota = vmm.Driver.real(), vmm.MemoryQuota(1 << 62)
        e = self.ecfg
        max_blocks = (e.max_seq_len + e.page_size - 1) // e.page_size
        pages = e.num_pages or e.max_batch * max_blocks
        kv = vmm.elastic_kv_cache(model_cfg, pages, e.page_size, self.cuda, self._driver, self._quota, initial_bundles=1)
        idx = self._ecs_ref.partitions[f"{model_id}:{rank}"]
        bb = kv.backing.bundle_bytes
        self._ecs_channel.set_partition(idx, self.device, 0, rank, bb, kv.backing.bundle_count * bb)
        return kv

    def _attach_capacity(self, eng, model_id: str, rank: int, tp: bool = False) -> None:
        from ..ecs import reconciler as R

        idx = self._ecs_ref.partitions[f"{model_id}:{rank}"]
        gate = lambda e=eng: R.cuda_event_gate(e.stream)
        if tp:
            # the ranks of the TP group agree every capacity change over their gloo group, which exists from
            # warm_and_serve on (before the first engine step)
            rec = R.TpAgreedReconciler(eng.kv, self._ecs_channel, idx, gate_factory=gate, agree=lambda v: self._agree(v))
        else:
            rec = R.CapacityReconciler(eng.kv, self._ecs_channel, idx, gate_factory=gate)
        eng.attach_capacity(rec, ttft_slo_s=self.cfg.slo_for(model_id).ttft_ms / 1e3)
        self._reconcilers.append(rec)

    def activate(self, plan: FabricPlan) -> None:
        pass  # engines warm up once the whole Fabric is executable (their graphs invoke the FFN tier)

    def warm_and_serve(self) -> None:
        from ..deployment import Deployment, InstanceHandle
        from .serving import EngineLoop, create_serving_app

        if not self.engines:
            return                   # every Instance rank of this device runs in a process of its own
        tp_members = {self._tp(m, r) for m, r in self.instances if self._tp(m, r)[1] > 1}
        order = sorted(self.engines, key=lambda m: self.cfg.model(m).atn_tp_size == 1)   # TP engines warm up first, in step
        dep = Deployment([InstanceHandle(m, self.engines[m].cfg, self.engines[m]) for m in order])
        leader = True
        if tp_members:
            import torch.distributed as dist

            from .tp_replication import TpEngineLoop

            if len(tp_members) != 1:
                raise RuntimeError("the tensor-parallel Instances of one attention device must share one TP group")
            (tpr, tps, first), = tp_members
            leader = tpr == 0
            # the members of the group meet here before any of them runs a kernel that waits on a peer; they
            # share the host, so the loopback interface carries the group (the host name may not resolve)
            import os

            os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
            dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{self.cfg.serving_tp_rendezvous_base_port + first}",
                                    rank=tpr, world_size=tps)
            from ..ecs.reconciler import gloo_agreement

            self._agree = gloo_agreement(None)
            dep.warmup()
            self.loop = TpEngineLoop(dep, None, leader)
        else:
            dep.warmup()
            self.loop = EngineLoop(dep)
        self.loop.start()
        if self._listen is not None and leader:
            import uvicorn

            from .serving import load_tokenizers

            toks = load_tokenizers({m: place.checkpoint for (m, _), place in self.places.items()})
            app = create_serving_app(self.loop, list(self.engines), tokenizer=toks)
            conf = uvicorn.Config(app, host=self._listen[0], port=self._listen[1], log_level="warning")
            self._server = uvicorn.Server(conf)
            threading.Thread(target=self._server.run, daemon=True, name="serving-http").start()
            for _ in range(1000):                    # the listener is published only once it accepts connections
                if self._server.started:
                    break
                threading.Event().wait(0.01)
            self.listener = ServingListener(host=self._listen[0], port=self._listen[1])

    def poll_health(self) -> InvocationFailure | None:
        for eng in self.engines.values():
            probe = getattr(eng.port, "failure", None)
            f = probe() if probe is not None else None
            if f is not None:   # claimed by an FFN rank, or by this rank when its own wait ran out
                return InvocationFailure(result_code=f.result_code, origin_pe=f.origin_pe, instance_index=f.instance_index,
                                         invocation_sequence=f.invocation_sequence, layer_ordinal=f.layer_ordinal)
        if self.loop is not None and self.loop.error is not None:
            raise RuntimeError(f"engine loop failed: {self.loop.error!r}")
        return None

    def quiesce(self) -> None:
        if self._server is not None:
            self._server.should_exit = True
        if self.loop is not None:
            self.loop.stop()

    def drain(self) -> bool:
        torch.cuda.synchronize(self.cuda)
        return True

    def finalize(self) -> None:
        if self._agree is not None:
            # the TP group's gloo process group owns worker threads; leaving them to interpreter shutdown ends the
            # process with "terminate called without an active exception" (joinable threads destroyed at exit)
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
            self._agree = None
        if self._server is not None:
            self._server.should_exit = True
        self.engines.clear()
        for b in self.buffers.values():
            b.free()
        self.buffers.clear()
        for g in self.tp_groups.values():
            g.close()
        self.tp_groups.clear()
