"""CPU backends of the agent roles: the whole product without a GPU.

``xpool ffnagent --backend cpu`` and ``xpool atnagent --backend cpu`` go through the same control plane as the GPU
agents (registration, configuration digest, placement, generation phases, handle brokering, readiness, quiesce and
retirement) and serve ``POST /generate``. The data plane is the CPU one of ``engine/cpu_plumbing.py``: a Transport
arena in POSIX shared memory per (Instance rank, FFN rank), driven by the native mailbox state machine; the "arena
handle" that travels through the daemon is the arena's name. The FFN agent loads the shard the plan assigns to it
(tensor-parallel rows or a range of experts, for its range of layers) through the production loader and answers
invocations from one thread per arena; the attention agent runs the PyTorch oracle, which computes every supported
attention form, under a small continuous-batching engine, and folds the FFN ranks' partials in rank order.

It exists for two reasons: every architecture can be served end to end where no B200 is at hand, and the control
plane is exercised by real processes in the CPU test tier (``tests/test_cpu_deploy.py``). The reference tests its
daemon with stand-in owner processes (tests/suites/integration/); here the stand-ins also compute.
"""

from __future__ import annotations

import threading
import time
import zlib
from collections import deque

import torch

from ..config import XpoolConfig
from ..engine.atn_engine import Sequence
from ..engine.cpu_plumbing import RemoteFfn, arena_view
from ..engine.kv_cache import OutOfPages
from ..models import reference
from ..models.weights import load_attention_from_safetensors, random_attention_weights, random_ffn_layer
from ..native import runtime as rt
from ..service.wire import FabricPlan, InvocationFailure, ServingListener
from .backends import placement_for

CPU_MAX_ROWS = 512


def cpu_capacity_rows(cfg: XpoolConfig) -> int:
    """Row capacity of every arena of a CPU deployment: all processes size and map the arenas with this number."""
    return min(cfg.engine_max_rows, CPU_MAX_ROWS)


def arena_name(cfg: XpoolConfig, plan: FabricPlan, model_id: str, atn_rank: int, pe: int) -> str:
    """Deterministic shared-memory name of one (Instance rank, FFN rank) arena of one generation of one deployment."""
    return f"/xp{cfg.daemon_port}g{plan.generation}m{zlib.crc32(model_id.encode()):08x}r{atn_rank}p{pe}"


def load_ffn_shard(place, tp_rank: int, lo: int, hi: int) -> list:
    """Layers ``lo .. hi`` of one FFN rank's share of a model, in fp32: rows ``tp_rank`` of the TP group for dense
    layers, the rank's range of experts for MoE layers of an expert-parallel placement."""
    cfg, tp = place.cfg, place.tp
    ep = place.expert_parallel
    out = []
    if place.checkpoint:
        import json
        from pathlib import Path

        from ..engine import checkpoint as ck
        from ..engine import loader
        from ..models import adapters

        view = ck.read_checkpoint_key_view(place.checkpoint)
        spec = adapters.compile_ffn_spec(place.model_id, json.loads((Path(place.checkpoint) / "config.json").read_text()), view.keys())
        ck.validate_ffn_coverage(spec, view)
        for l in range(lo, hi):
            if cfg.layer_is_moe(l) and ep:
                e0, e1 = place.expert_range(tp_rank)
                w = loader.materialize_layer_weights(spec, view, l, dtype=torch.float32, experts=range(e0, e1))
                if tp_rank != 0:
                    w.shared_gate_up = w.shared_down = None       # shared experts ride with the rank that owns expert 0
            else:
                w = loader.materialize_layer_weights(spec, view, l, dtype=torch.float32, tp_rank=tp_rank, tp_size=tp)
            out.append(w)
        return out
    for l in range(lo, hi):
        if cfg.layer_is_moe(l) and ep:
            out.append(random_ffn_layer(cfg, l, place.seed, dtype=torch.float32, expert_range=place.expert_range(tp_rank)))
        else:
            out.append(random_ffn_layer(cfg, l, place.seed, dtype=torch.float32, tp_rank=tp_rank, tp_size=tp))
    return out


class CpuFfnBackend:
    def __init__(self, cfg: XpoolConfig, device: int, capacity_rows: int = CPU_MAX_ROWS):
        self.cfg, self.device, self.capacity_rows = cfg, device, capacity_rows
        self._arenas: list[dict] = []
        self._threads: list[threading.Thread] = []
        self.errors: list[str] = []
        self.served = 0

    def prepare_join(self, plan: FabricPlan) -> dict[str, str]:
        torch.set_num_threads(1)
        my_pe = len(plan.atn_devices) + plan.ffn_devices.index(self.device)
        handles = {}
        shards: dict[tuple, list] = {}
        for r in plan.instance_ranks:
            if r.rank % self.cfg.model(r.model_id).atn_tp_size:
                continue
            place = placement_for(self.cfg, plan, r.model_id, r.rank, self.capacity_rows)
            if my_pe not in place.ffn_ranks:
                continue
            tp_rank, lo, hi = place.locate(my_pe)
            key = (r.model_id, tp_rank, lo, hi)           # data-parallel attention ranks share one copy of the shard
            if key not in shards:
                shards[key] = load_ffn_shard(place, tp_rank, lo, hi)
            name = arena_name(self.cfg, plan, r.model_id, r.rank, my_pe)
            mb = rt.CpuMailbox.create(name, self.capacity_rows, place.cfg.hidden_size * 4)
            self._arenas.append({"mb": mb, "cfg": place.cfg, "weights": shards[key], "lo": lo, "hi": hi, "name": name})
            handles[f"ffn:{r.model_id}:{r.rank}:{my_pe}"] = name.encode().hex()
        return handles

    def join(self, plan: FabricPlan) -> None:
        pass

    def prepare_execution(self, plan: FabricPlan) -> None:
        pass

    def activate(self, plan: FabricPlan) -> None:
        for a in self._arenas:
            a["mb"].activate()
            t = threading.Thread(target=self._serve, args=(a,), daemon=True, name=f"cpu-lane{a['name']}")
            t.start()
            self._threads.append(t)

    def _serve(self, a: dict) -> None:
        mb, cfg = a["mb"], a["cfg"]
        try:
            while True:
                rc, req = mb.take(0.5)
                if rc == rt.WAIT_TIMED_OUT:
                    continue
                if rc != rt.WAIT_READY:
                    return
                rows, layer, mode, _seq = req
                if not a["lo"] <= layer < a["hi"] or rows > self.capacity_rows:
                    mb.complete(rt.RESULT_PROTOCOL_MISMATCH)
                    self.errors.append(f"{a['name']}: invocation for layer {layer} with {rows} rows refused")
                    return
                y = arena_view(mb.output_address, rows, cfg.hidden_size)
                if mode == rt.MODE_IDLE:
                    y.zero_()
                else:
                    with torch.no_grad():
                        y.copy_(reference.ffn_forward(arena_view(mb.input_address, rows, cfg.hidden_size), a["weights"][layer - a["lo"]], cfg))
                mb.complete(rt.RESULT_OK)
                self.served += 1
        except Exception as e:      # reported by poll_health, which fails the generation
            self.errors.append(f"{a['name']}: {e!r}")

    def poll_health(self) -> InvocationFailure | None:
        if self.errors:
            raise RuntimeError("; ".join(self.errors))
        return None

    def quiesce(self) -> None:
        for a in self._arenas:
            a["mb"].shutdown()

    def drain(self) -> bool:
        for t in self._threads:
            t.join(5)
        return not any(t.is_alive() for t in self._threads)

    def finalize(self) -> None:
        for a in self._arenas:
            a["mb"].close()
        self._arenas, self._threads = [], []


class CpuTierPort:
    """Attention-side handle on the FFN ranks of one Instance rank: picks the layer's group, hands every rank of the
    group the rows (one thread per rank; the native call releases the interpreter lock) and sums the partials in rank
    order."""

    def __init__(self, groups: list[tuple[int, int, list[RemoteFfn]]]):
        self.groups, self.calls = groups, 0

    def __call__(self, layer: int, x: torch.Tensor, mode: int | None = None) -> torch.Tensor:
        ranks = next(r for lo, hi, r in self.groups if lo <= layer < hi)
        parts: list = [None] * len(ranks)
        errors: list = []

        def one(i):
            try:
                parts[i] = ranks[i](layer, x, mode)
            except Exception as e:
                errors.append(e)

        if len(ranks) == 1:
            one(0)
        else:
            ts = [threading.Thread(target=one, args=(i,)) for i in range(len(ranks))]
            for t in ts:
                t.start()
            for t in ts:
                t.join()
        if errors:
            raise errors[0]
        self.calls += 1
        out = parts[0].clone()
        for p in parts[1:]:
            out += p
        return out


class CpuOracleEngine:
    """Continuous batching over the PyTorch oracle, with the interface the serving loop expects of an engine. One
    step admits waiting requests (a whole prompt is one prefill pass) up to ``max_batch`` running sequences, or
    advances every running sequence by one token."""

    def __init__(self, cfg, attn_weights, ffn, max_batch: int = 8, max_seq_len: int = 512, model=None):
        self.cfg, self.model, self.ffn = cfg, model or reference.ReferenceModel(cfg, attn_weights, ffn=[]), ffn
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self._caches: dict[int, object] = {}
        self._next_id = 0
        self.stats = {"prefill_steps": 0, "decode_steps": 0, "stalled_for_pages": 0}
        self.kv = None                  # page accounting (engine/kv_cache.py) when the deployment runs elastic KV
        self.capacity = None
        self.ttft_slo_s = 0.0
        self._demand_pages = 0

    def warmup(self) -> None:
        pass

    def attach_kv(self, kv, reconciler=None, ttft_slo_s: float = 0.0) -> None:
        """Accounts the sequences' KV in pages of ``kv`` (tensors stay the oracle's own): a prompt is admitted when its
        pages fit what is mapped, a decode step takes a page when it crosses a boundary, and when pages are missing
        the engine publishes demand through ``reconciler`` and waits for the daemon's grow command, exactly the loop
        the GPU engine runs (``AttentionEngine.attach_capacity``)."""
        self.kv, self.capacity, self.ttft_slo_s = kv, reconciler, ttft_slo_s

    def idle_tick(self) -> None:
        if self.capacity is not None:
            self.capacity.poll()

    def _demand(self, missing_pages: int, head: Sequence | None) -> None:
        if self.capacity is None or missing_pages == self._demand_pages:
            return
        self._demand_pages = missing_pages
        if missing_pages <= 0:
            self.capacity.withdraw_demand()
            return
        deadline = int((head.arrival + self.ttft_slo_s) * 1e9) if head is not None and self.ttft_slo_s > 0 else 0
        self.capacity.publish_demand(missing_pages, deadline)

    def add_request(self, prompt: list[int], max_new_tokens: int, arrival: float | None = None, deadline: float = 0.0,
                    temperature: float = 0.0, seed: int = 0) -> Sequence:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if len(prompt) + max_new_tokens > self.max_seq_len:
            raise ValueError("request exceeds max_seq_len")
        if min(prompt) < 0 or max(prompt) >= self.cfg.vocab_size:
            raise ValueError(f"token id outside [0, {self.cfg.vocab_size})")
        if temperature > 0:
            raise ValueError("the CPU engine decodes greedily")
        s = Sequence(self._next_id, list(prompt), max_new_tokens, arrival if arrival is not None else time.monotonic(), deadline)
        self._next_id += 1
        self.waiting.append(s)
        return s

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _emit(self, s: Sequence, logits: torch.Tensor, now: float, out: list) -> None:
        tok = int(logits[-1].argmax())
        s.generated.append(tok)
        if s.first_token_time is None:
            s.first_token_time = now
        s.token_times.append(now)
        out.append((s, tok))
        if s.finished:
            s.finish_time = now
            self._caches.pop(s.seq_id, None)
            if self.kv is not None:
                self.kv.release(s.seq_id)
            if s in self.running:
                self.running.remove(s)
        elif s not in self.running:
            self.running.append(s)

    @torch.no_grad()
    def step(self) -> list[tuple[Sequence, int]]:
        out: list[tuple[Sequence, int]] = []
        if self.capacity is not None:
            self.capacity.poll()
        admit = bool(self.waiting) and len(self.running) < self.max_batch
        if admit and self.kv is not None:
            head = self.waiting[0]
            missing = self.kv.pages_needed(head.seq_id, len(head.prompt) + 1) - self.kv.allocator.free_pages
            if missing > 0:
                self._demand(missing, head)              # wait for the daemon's grow command; running work goes on
                self.stats["stalled_for_pages"] += 1
                admit = False
            else:
                self._demand(0, None)
                self.kv.ensure(head.seq_id, len(head.prompt) + 1)
        if admit:
            s = self.waiting.popleft()
            cache = self._caches[s.seq_id] = self.model.new_cache()
            n = len(s.prompt)
            lg = self.model.forward(torch.tensor(s.prompt), torch.arange(n), cache, self.ffn)
            s.computed = n
            self.stats["prefill_steps"] += 1
            self._emit(s, lg, time.monotonic(), out)
            return out
        for s in list(self.running):
            if self.kv is not None:
                try:
                    self.kv.ensure(s.seq_id, s.total_len + 1)
                except OutOfPages:
                    self._demand(1, s)                   # this sequence skips the step until a page is mapped
                    self.stats["stalled_for_pages"] += 1
                    continue
            pos = s.total_len - 1
            lg = self.model.forward(torch.tensor([s.generated[-1]]), torch.tensor([pos]), self._caches[s.seq_id], self.ffn)
            self._emit(s, lg, time.monotonic(), out)
        self.stats["decode_steps"] += 1
        if not out:
            time.sleep(0.002)                            # everything waits for memory: do not spin on the channel
        return out


class TpOracle(reference.ReferenceModel):
    """The oracle on one attention tensor-parallel rank: its share of the heads (``parallel/atn_tp.py`` sharding), the
    output projections summed over the group after every attention block (a gloo all-reduce here; the GPU ranks fold the
    same sum into the norm kernel through peer memory)."""

    def attention_half(self, layer, resid, ffn_out, positions, cache):
        import torch.distributed as dist

        cfg, lw = self.cfg, self.attn.layers[layer]
        if ffn_out is not None:
            resid = resid + ffn_out
        x = reference.block_norm(cfg, resid, lw.input_norm, lw.extra.get("input_norm_bias"))
        part = reference.attention_core(cfg, lw, x, positions, cache, layer).contiguous()
        dist.all_reduce(part)
        resid = resid + part
        return resid, reference.block_norm(cfg, resid, lw.post_attn_norm, lw.extra.get("post_attn_norm_bias"))


def tp_ffn(port, leader: bool):
    """FFN of a tensor-parallel Instance: the group's first rank talks to the FFN tier for all of them and hands the
    result to the others (the GPU followers read it from the first rank's slot)."""
    import torch.distributed as dist

    def call(layer: int, x: torch.Tensor, mode: int | None = None) -> torch.Tensor:
        y = port(layer, x, mode).contiguous() if leader else torch.empty_like(x)
        dist.broadcast(y, src=0)
        return y

    return call


class CpuDeployment:
    """The stepped-deployment protocol of ``runtime/serving.py::EngineLoop`` over CPU engines."""

    def __init__(self, engines: dict[str, CpuOracleEngine]):
        import types

        self.engines = engines
        self.instances = [types.SimpleNamespace(model_id=m, engine=e) for m, e in engines.items()]   # what this device hosts

    def add_request(self, model_id: str, prompt: list[int], max_new_tokens: int, arrival: float | None = None, **sampling):
        return self.engines[model_id].add_request(prompt, max_new_tokens, arrival, **sampling)

    @property
    def has_work(self) -> bool:
        return any(e.has_work for e in self.engines.values())

    def step(self):
        from ..deployment import StepResult

        res = StepResult()
        for model_id, e in self.engines.items():
            if e.has_work:
                res.tokens[model_id] = e.step()
            else:
                e.idle_tick()
        return res

    def idle_tick(self) -> None:
        for e in self.engines.values():
            e.idle_tick()


class CpuAtnBackend:
    def __init__(self, cfg: XpoolConfig, device: int, instances: list[tuple[str, int]], listen: tuple[str, int] | None = None,
                 capacity_rows: int = CPU_MAX_ROWS, max_batch: int = 8, max_seq_len: int = 512,
                 external: list[tuple[str, int]] | None = None, publish_arenas=None):
        """``external``: Instance ranks of this device that live in other processes; for them the backend only brokers
        the Transport arena (``publish_arenas(generation, [TransportArenaBinding])`` hands it to the daemon, which
        leases it to the rank's own process) and hosts no engine."""
        self.cfg, self.device, self.instances, self.capacity_rows = cfg, device, instances, capacity_rows
        self.external, self.publish_arenas = list(external or ()), publish_arenas
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.places: dict[tuple[str, int], object] = {}
        self.ports: dict[str, CpuTierPort] = {}
        self.engines: dict[str, CpuOracleEngine] = {}
        self._boxes: list[rt.CpuMailbox] = []
        self._listen = listen
        self._server = None
        self.loop = None
        self.listener: ServingListener | None = None
        self._tp: tuple[int, int, int] | None = None     # (TP rank, TP size, first rank) when this device hosts a TP member
        self.ecs_ref = None              # callable(generation) -> EcsChannelRef, set by the launcher when elastic KV is on
        self.kv_budget_bytes = 64 << 20  # what this "device" reports as its memory to the capacity policy
        self._ecs_channel = None
        self.reconcilers: list = []

    def _attach_elastic_kv(self, plan: FabricPlan) -> None:
        """Elastic KV on the CPU data plane: page accounting over the fake VMM driver (no tensors behind it), the real
        seqlock channel, reconciler and daemon policy. Bundles are 16 KiB per buffer so that tiny models move memory
        in steps of a few pages."""
        from ..ecs import reconciler as R
        from ..ecs import vmm
        from ..ecs.profile import KvPartitionGeometry
        from ..native.runtime import EcsChannel

        ref = None
        for _ in range(400):                                  # the daemon opens the channel on its next policy tick
            try:
                ref = self.ecs_ref(plan.generation)
                break
            except Exception:
                time.sleep(0.05)
        if ref is None:
            raise RuntimeError("the daemon did not publish an ECS control channel")
        self._ecs_channel = EcsChannel.attach(ref.name)
        gran, page = 16 << 10, 16
        mapped = 0
        for (model_id, rank), place in self.places.items():
            eng = self.engines[model_id]
            pages = eng.max_batch * ((eng.max_seq_len + page - 1) // page)
            kv = vmm.elastic_kv_cache(place.cfg, pages, page, "cpu", vmm.Driver.fake(1 << 40, granularity=gran), None,
                                      initial_bundles=1, make_tensors=False, granularity=gran)
            idx = ref.partitions[f"{model_id}:{rank}"]
            geo = KvPartitionGeometry.of(kv, floor_bundles=1)
            bb = geo.bundle_bytes
            geo.describe(self._ecs_channel, idx, self.device, rank)
            if self.cfg.model(model_id).atn_tp_size > 1:
                # the ranks of a TP group change capacity in the same engine step: they agree every poll over their gloo
                # group, which exists from warm_and_serve on (before the first step)
                rec = R.TpAgreedReconciler(kv, self._ecs_channel, idx, floor_bundles=geo.floor_bundles,
                                           agree=lambda v: R.gloo_agreement(None)(v))
            else:
                rec = R.CapacityReconciler(kv, self._ecs_channel, idx, floor_bundles=geo.floor_bundles)
            eng.attach_kv(kv, rec, ttft_slo_s=self.cfg.slo_for(model_id).ttft_ms / 1e3)
            self.reconcilers.append(rec)
            mapped += bb
        self._ecs_channel.publish_report(ref.devices[str(self.device)], max(0, self.kv_budget_bytes - mapped), self.kv_budget_bytes, 1)

    def prepare_join(self, plan: FabricPlan) -> dict[str, str]:
        torch.set_num_threads(1)
        handles = {}
        for model_id, rank in self.instances:
            self.places[(model_id, rank)] = placement_for(self.cfg, plan, model_id, rank, self.capacity_rows)
            handles[f"atn:{model_id}:{rank}"] = b"cpu".hex()       # the attention side owns no arena on the CPU
        if self.external:
            from ..service.wire import TransportArenaBinding

            arenas = []
            for model_id, rank in self.external:
                handles[f"atn:{model_id}:{rank}"] = b"cpu".hex()
                arenas.append(TransportArenaBinding(model_id=model_id, rank=rank, handle_hex=b"cpu".hex(), nbytes=0))
            if self.publish_arenas is not None:
                self.publish_arenas(plan.generation, arenas)
        return handles

    def join(self, plan: FabricPlan) -> None:
        for (model_id, rank), place in self.places.items():
            if rank % self.cfg.model(model_id).atn_tp_size:
                continue                 # a tensor-parallel follower: the group's first rank talks to the FFN tier
            groups = []
            for lo, hi, pes in place.groups():
                ranks = []
                for pe in pes:
                    name = bytes.fromhex(plan.slot_handles[f"ffn:{model_id}:{rank}:{pe}"]).decode()
                    mb = rt.CpuMailbox.attach(name, self.capacity_rows, place.cfg.hidden_size * 4)
                    self._boxes.append(mb)
                    ranks.append(RemoteFfn(mb, place.cfg.hidden_size, timeout_s=30.0))
                groups.append((lo, hi, ranks))
            self.ports[model_id] = CpuTierPort(groups)

    def prepare_execution(self, plan: FabricPlan) -> None:
        for (model_id, rank), place in self.places.items():
            if place.checkpoint:
                aw = load_attention_from_safetensors(place.cfg, place.checkpoint, dtype=torch.float32)
            else:
                aw = random_attention_weights(place.cfg, place.seed, dtype=torch.float32)
            tps = self.cfg.model(model_id).atn_tp_size
            if tps > 1:
                from ..parallel import atn_tp

                tpr = rank % tps
                local = atn_tp.local_config(place.cfg, tps)
                model = TpOracle(local, atn_tp.shard_attention_weights(aw, place.cfg, tpr, tps), ffn=[])
                self.engines[model_id] = CpuOracleEngine(local, None, tp_ffn(self.ports.get(model_id), tpr == 0), self.max_batch,
                                                         min(self.max_seq_len, self.capacity_rows), model=model)
                self._tp = (tpr, tps, rank - tpr)
                continue
            self.engines[model_id] = CpuOracleEngine(place.cfg, aw, self.ports[model_id], self.max_batch,
                                                     min(self.max_seq_len, self.capacity_rows))
        if self.cfg.atn_elastic_kv and self.ecs_ref is not None:
            self._attach_elastic_kv(plan)       # also with no hosted engine: the agent reports the device's memory

    def activate(self, plan: FabricPlan) -> None:
        pass

    def warm_and_serve(self) -> None:
        from .serving import EngineLoop, create_serving_app, load_tokenizers

        for mb in self._boxes:                                   # the FFN agents have activated their arenas by now
            if mb.wait_status(rt.MBOX_IDLE, 30.0) != rt.WAIT_READY:
                raise RuntimeError("an FFN arena never became idle")
        if not self.engines:
            return                                               # every rank of this device is served by another process
        leader = True
        if self._tp is not None:
            # the ranks of the group meet before any of them runs a forward pass; they share the host
            import os

            import torch.distributed as dist

            from .tp_replication import TpEngineLoop

            tpr, tps, first = self._tp
            leader = tpr == 0
            os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
            dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{self.cfg.serving_tp_rendezvous_base_port + first}",
                                    rank=tpr, world_size=tps)
            replicated = {m.id for m in self.cfg.models if m.atn_tp_size > 1}
            self.loop = TpEngineLoop(CpuDeployment(self.engines), None, leader, replicated=replicated)
            serves_http = leader or any(m not in replicated for m in self.engines)   # a follower answers for its other Instances
        else:
            self.loop = EngineLoop(CpuDeployment(self.engines))
            serves_http = True
        self.loop.start()
        if self._listen is not None and serves_http:
            import uvicorn

            toks = load_tokenizers({m: place.checkpoint for (m, _), place in self.places.items()})
            app = create_serving_app(self.loop, list(self.engines), tokenizer=toks)
            self._server = uvicorn.Server(uvicorn.Config(app, host=self._listen[0], port=self._listen[1], log_level="warning"))
            threading.Thread(target=self._server.run, daemon=True, name="serving-http").start()
            for _ in range(1000):                    # the listener is published only once it accepts connections
                if self._server.started:
                    break
                time.sleep(0.01)
            self.listener = ServingListener(host=self._listen[0], port=self._listen[1])

    def poll_health(self) -> InvocationFailure | None:
        if self.loop is not None and self.loop.error is not None:
            raise RuntimeError(f"engine loop failed: {self.loop.error!r}")
        return None

    def quiesce(self) -> None:
        if self._server is not None:
            self._server.should_exit = True
        if self.loop is not None:
            self.loop.stop()

    def drain(self) -> bool:
        return True

    def finalize(self) -> None:
        for mb in self._boxes:
            mb.close()
        self._boxes = []
        self.engines.clear()
        if self._tp is not None:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
        if self._ecs_channel is not None:
            self._ecs_channel.close()
            self._ecs_channel = None


def attach_cpu_instance(cfg: XpoolConfig, plan: FabricPlan, model_id: str, rank: int) -> "CpuInstanceTransport":
    """What an Instance rank in a process of its own does once the fabric is executable and the daemon has leased it
    its arena: it maps the FFN ranks' arenas named in the plan and gets a handle that evaluates one layer
    (``CpuTierPort``). The GPU counterpart maps IPC handles (``integrations/sglang/transport.py::from_handles``)."""
    capacity_rows = cpu_capacity_rows(cfg)
    place = placement_for(cfg, plan, model_id, rank, capacity_rows)
    boxes, groups = [], []
    for lo, hi, pes in place.groups():
        ranks = []
        for pe in pes:
            name = bytes.fromhex(plan.slot_handles[f"ffn:{model_id}:{rank}:{pe}"]).decode()
            mb = rt.CpuMailbox.attach(name, capacity_rows, place.cfg.hidden_size * 4)
            boxes.append(mb)
            ranks.append(RemoteFfn(mb, place.cfg.hidden_size, timeout_s=30.0))
        groups.append((lo, hi, ranks))
    return CpuInstanceTransport(CpuTierPort(groups), boxes)


class CpuInstanceTransport:
    def __init__(self, port: CpuTierPort, boxes: list):
        self.port, self._boxes = port, boxes

    def failure(self):
        return None

    def close(self) -> None:
        for mb in self._boxes:
            mb.close()
        self._boxes = []
