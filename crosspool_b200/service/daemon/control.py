"""The daemon's control plane: one lock, one state machine.

Responsibilities (reference: src/xpool/service/daemon/control.py, fabric.py, registration.py,
transport.py, readiness.py):

* **startup admission / config check** — a joining process must run the daemon's ABI and resolve the
  same effective configuration digest;
* **registration tables** — AtnAgents and FfnAgents by device, Instance ranks by (model, rank); an
  owner is ``(pid, create_time)``; the same owner re-registering is idempotent, a different live
  owner is a conflict, a dead or stale one is replaced;
* **generation planning** — when every configured participant is registered the membership is
  frozen, FFN shards are placed with memory admission, a generation id/uid is issued and the plan is
  served;
* **generation barrier** — the generation advances PREPARING_JOIN → JOINING → PREPARING_EXECUTION →
  ACTIVATING → EXECUTABLE only when *all* participants reported the matching phase; a phase that
  lasts longer than its timeout aborts the generation;
* **watchdog** — owner loss (process exited, heartbeat stale, owner replaced) and reported invocation
  failures abort or quiesce the generation (fail-stop: no re-planning while serving);
* **transport brokering** — arena/slot handles are published by their owners and acquired by exactly
  one lessee; quiescing blocks new leases;
* **readiness** — Fabric Executable vs System Ready vs Serving Healthy.
"""

from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable

from ...config import XpoolConfig
from ..errors import DaemonError
from ..wire import (AgentStartupAdmission, AtnAgentRegistration, FabricPhase, FabricPlan, FfnAgentRegistration,
                    HeartbeatResponse, InstanceRankInitialized, InstanceRankRegistration, InstanceRankTopology,
                    OwnerFailureReason, ParticipantPhase, ParticipantReport, ProcessRef, ReadinessEntry,
                    ReadinessSnapshot, Role, ShardPlacement, TransportArenaBinding)
from .placement import DeviceSupply, ModelDemand, PlacementError, place_ffn_models

from ...native import EXPECTED_ABI as ABI_VERSION  # noqa: E402  (one number for native code and wire)

HEARTBEAT_STALE_SECONDS = 15.0       # reference registration.py:27
PHASE_TIMEOUT_SECONDS = 60.0         # reference control.py:81-86
INSTANCE_STARTUP_SECONDS = 600.0     # reference control.py:87

_NEXT_PHASE = {
    FabricPhase.PREPARING_JOIN: (ParticipantPhase.JOIN_READY, FabricPhase.JOINING),
    FabricPhase.JOINING: (ParticipantPhase.JOINED, FabricPhase.PREPARING_EXECUTION),
    FabricPhase.PREPARING_EXECUTION: (ParticipantPhase.EXECUTION_READY, FabricPhase.ACTIVATING),
    FabricPhase.ACTIVATING: (ParticipantPhase.ACTIVE, FabricPhase.EXECUTABLE),
    FabricPhase.QUIESCING: (ParticipantPhase.QUIESCED, FabricPhase.DRAINING),
    FabricPhase.ABORTING: (ParticipantPhase.QUIESCED, FabricPhase.DRAINING),
    FabricPhase.DRAINING: (ParticipantPhase.DRAINED, FabricPhase.FINALIZING),
    FabricPhase.FINALIZING: (ParticipantPhase.FINALIZED, FabricPhase.STOPPED),
}
_PHASE_ORDER = [ParticipantPhase.REGISTERED, ParticipantPhase.JOIN_READY, ParticipantPhase.JOINED,
                ParticipantPhase.EXECUTION_READY, ParticipantPhase.ACTIVE, ParticipantPhase.QUIESCED,
                ParticipantPhase.DRAINED, ParticipantPhase.FINALIZED]


def default_process_alive(ref: ProcessRef) -> bool:
    """Is the (pid, create_time) pair still the same live process? Detects PID reuse."""
    try:
        import psutil

        p = psutil.Process(ref.pid)
        if ref.create_time and abs(p.create_time() - ref.create_time) > 1.0:
            return False
        return p.is_running() and p.status() != psutil.STATUS_ZOMBIE
    except Exception:
        return False


@dataclass
class Registration:
    owner: ProcessRef
    payload: object
    registered_at: float
    last_heartbeat: float
    pe: int = -1
    phase: ParticipantPhase = ParticipantPhase.REGISTERED
    initialized: bool = False
    listener: tuple[str, int] | None = None


@dataclass
class Generation:
    number: int
    uid: str
    phase: FabricPhase
    phase_since: float
    plan: FabricPlan
    participants: dict[int, str] = field(default_factory=dict)  # pe -> registration key
    failure: str | None = None
    owner_failures: list[tuple[str, OwnerFailureReason]] = field(default_factory=list)


class ControlPlane:
    def __init__(self, config: XpoolConfig, *, clock: Callable[[], float] = time.monotonic,
                 process_alive: Callable[[ProcessRef], bool] = default_process_alive,
                 model_demand: Callable[[str], ModelDemand] | None = None, abi_version: int = ABI_VERSION):
        self.config, self.clock, self.process_alive = config, clock, process_alive
        self.abi_version = abi_version
        self._model_demand = model_demand
        self._lock = threading.RLock()
        self.atnagents: dict[int, Registration] = {}
        self.ffnagents: dict[int, Registration] = {}
        self.instances: dict[tuple[str, int], Registration] = {}
        self.admitted: dict[tuple[str, int], ProcessRef] = {}
        self.generation: Generation | None = None
        self._generation_counter = 0
        self.arenas: dict[tuple[str, int], TransportArenaBinding] = {}
        self.leases: dict[tuple[str, int], ProcessRef] = {}
        self.lease_quiesced: set[int] = set()
        self.warnings: list[str] = []
        self.failure: str | None = None
        self.closing = False

    # ------------------------------------------------------------------ admission
    def check_config(self, owner: ProcessRef, digest: str) -> None:
        self._check_abi(owner)
        if digest != self.config.digest():
            raise DaemonError("mismatch", "effective configuration differs from the daemon's")

    def _check_abi(self, owner: ProcessRef) -> None:
        if owner.abi_version != self.abi_version:
            raise DaemonError("mismatch", f"native ABI {owner.abi_version} != daemon ABI {self.abi_version}")

    def admit_agent(self, req: AgentStartupAdmission) -> None:
        with self._lock:
            self._check_abi(req.owner)
            devices = self.config.atn_devices if req.role == Role.ATNAGENT else self.config.ffn_devices
            if req.device not in devices:
                raise DaemonError("invalid", f"device {req.device} is not configured for {req.role.value}")
            key = (req.role.value, req.device)
            cur = self.admitted.get(key)
            if cur is not None and cur != req.owner and self.process_alive(cur):
                raise DaemonError("conflict", f"{req.role.value} for device {req.device} is already starting (pid {cur.pid})")
            self.admitted[key] = req.owner

    # ------------------------------------------------------------------ registration
    def _install(self, table: dict, key, owner: ProcessRef, payload, what: str) -> Registration:
        now = self.clock()
        cur = table.get(key)
        if cur is not None and cur.owner != owner:
            stale = now - cur.last_heartbeat > HEARTBEAT_STALE_SECONDS
            if self.process_alive(cur.owner) and not stale:
                raise DaemonError("conflict", f"{what} is owned by live pid {cur.owner.pid}")
            self._owner_lost(f"{what}", OwnerFailureReason.REPLACED)
        if cur is not None and cur.owner == owner:
            cur.payload, cur.last_heartbeat = payload, now
            return cur
        reg = Registration(owner, payload, now, now)
        table[key] = reg
        return reg

    def register_atnagent(self, r: AtnAgentRegistration) -> None:
        with self._lock:
            self._check_abi(r.owner)
            if r.device not in self.config.atn_devices:
                raise DaemonError("invalid", f"device {r.device} is not an attention device")
            self._install(self.atnagents, r.device, r.owner, r, f"atnagent:{r.device}")
            self._maybe_plan()

    def register_ffnagent(self, r: FfnAgentRegistration) -> None:
        with self._lock:
            self._check_abi(r.owner)
            if r.device not in self.config.ffn_devices:
                raise DaemonError("invalid", f"device {r.device} is not an FFN device")
            self._install(self.ffnagents, r.device, r.owner, r, f"ffnagent:{r.device}")
            self._maybe_plan()

    def register_instance(self, r: InstanceRankRegistration) -> None:
        with self._lock:
            self._check_abi(r.owner)
            try:
                m = self.config.model(r.model_id)
            except KeyError:
                raise DaemonError("invalid", f"model {r.model_id} is not configured") from None
            if not 0 <= r.rank < m.atn_world_size:
                raise DaemonError("invalid", f"rank {r.rank} outside the model's attention world {m.atn_world_size}")
            if r.device not in self.config.atn_devices:
                raise DaemonError("invalid", f"device {r.device} is not an attention device")
            self._install(self.instances, (r.model_id, r.rank), r.owner, r, f"instance:{r.model_id}:{r.rank}")
            self._maybe_plan()

    def deregister_instance(self, model_id: str, rank: int, owner: ProcessRef) -> None:
        with self._lock:
            reg = self.instances.get((model_id, rank))
            if reg is None or reg.owner != owner:
                raise DaemonError("not_found", "no such registration")
            del self.instances[(model_id, rank)]
            self.leases.pop((model_id, rank), None)
            if self.generation and self.generation.phase == FabricPhase.EXECUTABLE:
                self._begin_quiesce(f"instance {model_id}:{rank} departed")

    def heartbeat(self, table_name: str, key, owner: ProcessRef) -> HeartbeatResponse:
        with self._lock:
            table = {"atnagent": self.atnagents, "ffnagent": self.ffnagents, "instance": self.instances}[table_name]
            reg = table.get(key)
            if reg is None or reg.owner != owner:
                raise DaemonError("gone", "registration was lost or replaced; re-register")
            reg.last_heartbeat = self.clock()
            g = self.generation
            return HeartbeatResponse(warnings=list(self.warnings), generation=g.number if g else None,
                                     fabric_phase=g.phase if g else FabricPhase.IDLE)

    # ------------------------------------------------------------------ planning
    def _expected_instances(self) -> list[tuple[str, int]]:
        return [(m.id, r) for m in self.config.models for r in range(m.atn_world_size)]

    def membership_complete(self) -> bool:
        return (all(d in self.atnagents for d in self.config.atn_devices)
                and all(d in self.ffnagents for d in self.config.ffn_devices)
                and all(k in self.instances for k in self._expected_instances()))

    def _demand_for(self, model_id: str) -> ModelDemand:
        if self._model_demand is not None:
            return self._model_demand(model_id)
        m = self.config.model(model_id)
        cfg = self.config.model_shape(model_id)
        regs = [r.payload for (mid, _), r in self.instances.items() if mid == model_id]
        rows = max([max(p.ffn_profile.max_prefill_rows, p.ffn_profile.max_decode_rows) for p in regs] or [1])
        inter = cfg.moe_intermediate_size * max(1, cfg.num_experts_per_tok) if cfg.is_moe else cfg.intermediate_size
        return ModelDemand(model_id, tuple(cfg.ffn_param_bytes_per_layer(l) for l in range(cfg.num_layers)),
                           self.config.ffn_tp_for(model_id), cfg.hidden_size, rows, m.atn_world_size, inter)

    def _maybe_plan(self) -> None:
        if self.generation is not None and self.generation.phase not in (FabricPhase.STOPPED,):
            return
        if self.closing or not self.membership_complete():
            return
        try:
            self.ensure_fabric_plan()
        except DaemonError as e:
            self.failure = e.message

    def ensure_fabric_plan(self) -> FabricPlan:
        """Freezes membership, places the FFN shards and opens a new generation."""
        with self._lock:
            g = self.generation
            if g is not None and g.phase != FabricPhase.STOPPED:
                return g.plan
            if not self.membership_complete():
                raise DaemonError("not_ready", "not every configured participant is registered")
            atn, ffn = list(self.config.atn_devices), list(self.config.ffn_devices)
            supplies = [DeviceSupply(d, self.ffnagents[d].payload.device_free_memory_bytes,
                                     self.ffnagents[d].payload.device_total_memory_bytes) for d in ffn]
            demands = [self._demand_for(m.id) for m in self.config.models]
            try:
                placed = place_ffn_models(demands, supplies, margin_bytes=self.config.ffn_device_memory_extra_margin_bytes,
                                          lanes=self.config.scheduler_ffn_concurrency,
                                          timeout_seconds=self.config.ffn_placement_timeout_seconds)
            except PlacementError as e:
                raise DaemonError("invalid", f"memory admission failed: {e}") from None
            # PE numbering: attention agents first, then FFN agents (coordinator = first FFN PE)
            pe_of_atn = {d: i for i, d in enumerate(atn)}
            pe_of_ffn = {d: len(atn) + i for i, d in enumerate(ffn)}
            shards = [ShardPlacement(model_id=mid, layer_begin=lo, layer_end=hi, tp_rank=r, tp_size=tp, device=d,
                                     pe=pe_of_ffn[d], bytes=sum(dm.shard_bytes(l) for l in range(lo, hi)))
                      for (mid, lo, hi, r, tp, d) in placed.shards()
                      for dm in demands if dm.model_id == mid]
            ranks = []
            for idx, (mid, rank) in enumerate(self._expected_instances()):
                reg = self.instances[(mid, rank)]
                ranks.append(InstanceRankTopology(model_id=mid, rank=rank, device=reg.payload.device,
                                                  pe=pe_of_atn[reg.payload.device], instance_index=idx))
            self._generation_counter += 1
            n = self._generation_counter
            uid = f"xpg-{n:06d}-{abs(hash((n, tuple(atn), tuple(ffn)))) % (1 << 32):08x}"
            plan = FabricPlan(generation=n, uid=uid, phase=FabricPhase.PREPARING_JOIN, atn_devices=atn, ffn_devices=ffn,
                              lanes_per_ffn_device=self.config.scheduler_ffn_concurrency,
                              policy=self.config.scheduler_ffn_policy, shards=shards, instance_ranks=ranks)
            gen = Generation(n, uid, FabricPhase.PREPARING_JOIN, self.clock(), plan)
            for d in atn:
                gen.participants[pe_of_atn[d]] = f"atnagent:{d}"
                self.atnagents[d].pe, self.atnagents[d].phase = pe_of_atn[d], ParticipantPhase.REGISTERED
            for d in ffn:
                gen.participants[pe_of_ffn[d]] = f"ffnagent:{d}"
                self.ffnagents[d].pe, self.ffnagents[d].phase = pe_of_ffn[d], ParticipantPhase.REGISTERED
            for reg in self.instances.values():
                reg.initialized = False
            self.generation = gen
            self.arenas.clear()
            self.leases.clear()
            self.lease_quiesced.clear()
            self.failure = None
            return plan

    def fabric_plan(self) -> FabricPlan:
        with self._lock:
            if self.generation is None:
                raise DaemonError("not_ready", "no generation planned yet")
            self.generation.plan.phase = self.generation.phase
            return self.generation.plan

    # ------------------------------------------------------------------ barrier
    def _participant(self, key: str) -> Registration | None:
        kind, dev = key.split(":")
        return (self.atnagents if kind == "atnagent" else self.ffnagents).get(int(dev))

    def report_participant(self, rep: ParticipantReport) -> FabricPhase:
        with self._lock:
            g = self.generation
            if g is None or rep.generation != g.number:
                raise DaemonError("mismatch", "report is for another generation")
            key = g.participants.get(rep.pe)
            reg = self._participant(key) if key else None
            if reg is None or reg.owner != rep.owner:
                raise DaemonError("gone", "reporting process does not own this PE")
            if _PHASE_ORDER.index(rep.phase) < _PHASE_ORDER.index(reg.phase):
                raise DaemonError("invalid", f"phase moves backwards: {reg.phase.value} -> {rep.phase.value}")
            reg.phase = rep.phase
            reg.last_heartbeat = self.clock()
            if rep.invocation_failure is not None or rep.control_failure is not None:
                why = (f"invocation failure code {rep.invocation_failure.result_code} from PE {rep.invocation_failure.origin_pe}"
                       if rep.invocation_failure else f"control failure: {rep.control_failure}")
                self._abort(why)
            self._advance_barrier()
            return g.phase

    def _advance_barrier(self) -> None:
        g = self.generation
        while g is not None and g.phase in _NEXT_PHASE:
            need, nxt = _NEXT_PHASE[g.phase]
            regs = [self._participant(k) for k in g.participants.values()]
            live = [r for r in regs if r is not None]
            if g.phase in (FabricPhase.ABORTING, FabricPhase.QUIESCING, FabricPhase.DRAINING, FabricPhase.FINALIZING):
                # participants that are gone cannot report; the survivors must
                ok = all(_PHASE_ORDER.index(r.phase) >= _PHASE_ORDER.index(need) for r in live)
            else:
                ok = len(live) == len(regs) and all(_PHASE_ORDER.index(r.phase) >= _PHASE_ORDER.index(need) for r in live)
            if not ok:
                return
            g.phase, g.phase_since = nxt, self.clock()

    def _abort(self, why: str) -> None:
        g = self.generation
        if g is None or g.phase in (FabricPhase.ABORTING, FabricPhase.DRAINING, FabricPhase.FINALIZING, FabricPhase.STOPPED):
            return
        g.failure = g.failure or why
        self.failure = self.failure or why
        g.phase, g.phase_since = FabricPhase.ABORTING, self.clock()
        self.lease_quiesced.update(self.config.atn_devices)

    def _begin_quiesce(self, why: str) -> None:
        g = self.generation
        if g is None or g.phase != FabricPhase.EXECUTABLE:
            return
        g.phase, g.phase_since = FabricPhase.QUIESCING, self.clock()
        self.warnings.append(f"quiescing: {why}")
        self.lease_quiesced.update(self.config.atn_devices)

    def quiesce(self, reason: str = "operator") -> FabricPhase:
        with self._lock:
            if self.generation is None:
                raise DaemonError("not_ready", "no generation")
            if self.generation.phase == FabricPhase.EXECUTABLE:
                self._begin_quiesce(reason)
            elif self.generation.phase not in (FabricPhase.QUIESCING, FabricPhase.DRAINING, FabricPhase.FINALIZING,
                                               FabricPhase.STOPPED, FabricPhase.ABORTING):
                self._abort(f"quiesce requested during {self.generation.phase.value}: {reason}")
            return self.generation.phase

    def _owner_lost(self, key: str, reason: OwnerFailureReason) -> None:
        g = self.generation
        if g is None:
            return
        g.owner_failures.append((key, reason))
        if g.phase == FabricPhase.EXECUTABLE and key.startswith("instance:"):
            self._begin_quiesce(f"{key} {reason.value}")
        else:
            self._abort(f"{key} {reason.value}")

    # ------------------------------------------------------------------ forced termination
    def terminate_owner(self, owner: ProcessRef, terminate: Callable[[ProcessRef], list[int]] | None = None) -> list[int]:
        """Ends a registered participant process (and its children) on an operator's or a peer's request, e.g. an
        Instance host that stopped answering while it still holds GPU memory. Only an owner the daemon knows,
        with a matching creation time, is ever signalled (the reference terminates an MPS client the same way,
        ``POST /serving/mps/terminate-client``, src/xpool/utils/mps.py:514-588)."""
        with self._lock:
            known = [r.owner for t in (self.atnagents, self.ffnagents, self.instances) for r in t.values()]
        if not any(o.pid == owner.pid and abs(o.create_time - owner.create_time) < 1.0 for o in known):
            raise DaemonError("not_found", f"process {owner.pid} is not a registered participant")
        if terminate is None:
            from ...utils import procs

            def terminate(ref: ProcessRef) -> list[int]:
                return procs.kill_tree(procs.ProcUniqId(ref.pid, ref.create_time))

        return terminate(owner)

    # ------------------------------------------------------------------ watchdog
    def watchdog(self) -> list[tuple[str, OwnerFailureReason]]:
        """Runs every second: classify lost owners, expire phases."""
        with self._lock:
            now, lost = self.clock(), []
            tables = [("atnagent", self.atnagents), ("ffnagent", self.ffnagents), ("instance", self.instances)]
            for kind, table in tables:
                for key, reg in list(table.items()):
                    name = f"{kind}:{key}" if not isinstance(key, tuple) else f"{kind}:{key[0]}:{key[1]}"
                    reason = None
                    if not self.process_alive(reg.owner):
                        reason = OwnerFailureReason.EXITED
                    elif now - reg.last_heartbeat > HEARTBEAT_STALE_SECONDS:
                        reason = OwnerFailureReason.STALE
                    if reason is not None:
                        lost.append((name, reason))
                        del table[key]
                        if isinstance(key, tuple):
                            self.leases.pop(key, None)
                        self._owner_lost(name, reason)
            g = self.generation
            if g is not None and g.phase in (FabricPhase.PREPARING_JOIN, FabricPhase.JOINING,
                                             FabricPhase.PREPARING_EXECUTION, FabricPhase.ACTIVATING):
                if now - g.phase_since > PHASE_TIMEOUT_SECONDS:
                    self._abort(f"phase {g.phase.value} timed out after {PHASE_TIMEOUT_SECONDS:.0f} s")
            if g is not None and g.phase == FabricPhase.EXECUTABLE:
                for (mid, rank), reg in self.instances.items():
                    if not reg.initialized and now - reg.registered_at > INSTANCE_STARTUP_SECONDS:
                        self._abort(f"instance {mid}:{rank} did not initialise within {INSTANCE_STARTUP_SECONDS:.0f} s")
            self._advance_barrier()
            return lost

    # ------------------------------------------------------------------ transport brokering
    def upsert_arenas(self, device: int, owner: ProcessRef, generation: int, arenas: list[TransportArenaBinding]) -> None:
        with self._lock:
            reg = self.atnagents.get(device)
            if reg is None or reg.owner != owner:
                raise DaemonError("gone", "not the registered AtnAgent of this device")
            if self.generation is None or generation != self.generation.number:
                raise DaemonError("mismatch", "arenas are for another generation")
            for a in arenas:
                self.arenas[(a.model_id, a.rank)] = a

    def acquire_arena(self, model_id: str, rank: int, owner: ProcessRef, generation: int) -> TransportArenaBinding:
        with self._lock:
            reg = self.instances.get((model_id, rank))
            if reg is None or reg.owner != owner:
                raise DaemonError("gone", "not the registered owner of this Instance rank")
            if self.generation is None or generation != self.generation.number:
                raise DaemonError("mismatch", "lease is for another generation")
            if self.generation.phase != FabricPhase.EXECUTABLE:
                raise DaemonError("not_ready", f"fabric is {self.generation.phase.value}, not executable")
            if reg.payload.device in self.lease_quiesced:
                raise DaemonError("not_ready", "leases on this device are quiesced")
            arena = self.arenas.get((model_id, rank))
            if arena is None:
                raise DaemonError("not_ready", "arena not published yet")
            cur = self.leases.get((model_id, rank))
            if cur is not None and cur != owner:
                raise DaemonError("conflict", "arena is leased to another process")
            self.leases[(model_id, rank)] = owner
            return arena

    def quiesce_leases(self, device: int, owner: ProcessRef) -> list[tuple[str, int]]:
        with self._lock:
            reg = self.atnagents.get(device)
            if reg is None or reg.owner != owner:
                raise DaemonError("gone", "not the registered AtnAgent of this device")
            self.lease_quiesced.add(device)
            return [k for k, r in self.instances.items() if r.payload.device == device and k in self.leases]

    def publish_slot_handles(self, owner: ProcessRef, generation: int, handles: dict[str, str]) -> None:
        with self._lock:
            if self.generation is None or generation != self.generation.number:
                raise DaemonError("mismatch", "handles are for another generation")
            self.generation.plan.slot_handles.update(handles)

    def instance_initialized(self, model_id: str, req: InstanceRankInitialized) -> None:
        with self._lock:
            reg = self.instances.get((model_id, req.rank))
            if reg is None or reg.owner != req.owner:
                raise DaemonError("gone", "not the registered owner")
            if self.generation is None or req.generation != self.generation.number:
                raise DaemonError("mismatch", "initialised against another generation")
            reg.initialized = True
            if req.serving_listener:
                reg.listener = (req.serving_listener.host, req.serving_listener.port)

    # ------------------------------------------------------------------ readiness
    def readiness(self, listener_healthy: Callable[[tuple[str, int]], bool] | None = None) -> ReadinessSnapshot:
        with self._lock:
            g = self.generation
            phase = g.phase if g else FabricPhase.IDLE
            executable = phase == FabricPhase.EXECUTABLE
            expected = self._expected_instances()
            inst_entries = []
            for k in expected:
                r = self.instances.get(k)
                state = "missing" if r is None else ("initialized" if r.initialized else "registered")
                inst_entries.append(ReadinessEntry(key=f"{k[0]}:{k[1]}", state=state))
            system_ready = executable and all(e.state == "initialized" for e in inst_entries)
            healthy = system_ready
            if system_ready and listener_healthy is not None:
                healthy = all(listener_healthy(r.listener) for r in self.instances.values() if r.listener)
            return ReadinessSnapshot(
                fabric_executable=executable, system_ready=system_ready, serving_healthy=healthy,
                generation=g.number if g else None, phase=phase,
                atnagents=[ReadinessEntry(key=str(d), state=(self.atnagents[d].phase.value if d in self.atnagents else "missing"))
                           for d in self.config.atn_devices],
                ffnagents=[ReadinessEntry(key=str(d), state=(self.ffnagents[d].phase.value if d in self.ffnagents else "missing"))
                           for d in self.config.ffn_devices],
                instance_ranks=inst_entries, warnings=list(self.warnings), failure=self.failure or (g.failure if g else None))

    # ------------------------------------------------------------------ retirement
    def begin_close(self) -> None:
        with self._lock:
            self.closing = True
            if self.generation and self.generation.phase == FabricPhase.EXECUTABLE:
                self._begin_quiesce("daemon closing")
            elif self.generation and self.generation.phase not in (FabricPhase.STOPPED, FabricPhase.DRAINING,
                                                                   FabricPhase.FINALIZING, FabricPhase.QUIESCING):
                self._abort("daemon closing")

    @property
    def exit_code(self) -> int:
        """0 for a clean run, 20 when a failure was recorded (reference daemon.py:93-110)."""
        return 20 if self.failure else 0
