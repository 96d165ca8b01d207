"""Control plane with a fake clock and fake process table (no GPU, no real processes):
registration rules, generation planning with memory admission, the generation barrier, watchdog
classification of lost owners, transport brokering, readiness — and the HTTP face in-process."""
import pytest

from crosspool_b200 import config as C
from crosspool_b200.service.daemon.control import (ABI_VERSION, HEARTBEAT_STALE_SECONDS, PHASE_TIMEOUT_SECONDS,
                                                   ControlPlane)
from crosspool_b200.service.daemon.placement import ModelDemand
from crosspool_b200.service.errors import DaemonError
from crosspool_b200.service.wire import (AgentStartupAdmission, AtnAgentRegistration, FabricPhase, FfnAgentRegistration,
                                         InstanceFfnProfile, InstanceRankInitialized, InstanceRankRegistration,
                                         InvocationFailure, ParticipantPhase, ParticipantReport, ProcessRef, Role,
                                         TransportArenaBinding)

TOML = """
[atn]
devices = [0]
[ffn]
devices = [1, 2]
[scheduler]
ffn_concurrency = 2
[scheduler.slo]
ttft_ms = 1000
tbt_ms = 50
[[models]]
id = "Qwen/Qwen3-0.6B"
ffn_tp_size = 1
[[models]]
id = "Qwen/Qwen3-8B"
ffn_tp_size = 2
"""


class FakeClock:
    def __init__(self):
        self.t = 100.0

    def __call__(self):
        return self.t

    def advance(self, dt):
        self.t += dt


class World:
    def __init__(self, free=64 << 30):
        self.cfg = C.load_config(env={}, toml_text=TOML)
        self.clock = FakeClock()
        self.alive = set()
        self.cp = ControlPlane(self.cfg, clock=self.clock, process_alive=lambda ref: ref.pid in self.alive)
        self.free = free

    def ref(self, pid):
        self.alive.add(pid)
        return ProcessRef(abi_version=ABI_VERSION, pid=pid, create_time=1.0)

    def join_all(self):
        self.cp.register_atnagent(AtnAgentRegistration(owner=self.ref(10), device=0))
        for d in (1, 2):
            self.cp.register_ffnagent(FfnAgentRegistration(owner=self.ref(20 + d), device=d, device_free_memory_bytes=self.free,
                                                           device_total_memory_bytes=180 << 30))
        prof = InstanceFfnProfile(max_prefill_rows=2048, max_decode_rows=256, hidden_size=1024)
        self.cp.register_instance(InstanceRankRegistration(owner=self.ref(30), model_id="Qwen/Qwen3-0.6B", rank=0, device=0,
                                                           ffn_profile=prof))
        self.cp.register_instance(InstanceRankRegistration(owner=self.ref(31), model_id="Qwen/Qwen3-8B", rank=0, device=0,
                                                           ffn_profile=prof))

    def report_all(self, phase):
        g = self.cp.generation
        for pe, key in g.participants.items():
            kind, dev = key.split(":")
            pid = 10 if kind == "atnagent" else 20 + int(dev)
            self.cp.report_participant(ParticipantReport(owner=self.ref(pid), generation=g.number, pe=pe, phase=phase))

    def to_executable(self):
        self.join_all()
        for ph in (ParticipantPhase.JOIN_READY, ParticipantPhase.JOINED, ParticipantPhase.EXECUTION_READY,
                   ParticipantPhase.ACTIVE):
            self.report_all(ph)
        assert self.cp.generation.phase == FabricPhase.EXECUTABLE


def test_plan_is_made_only_when_membership_is_complete_and_places_tp_groups():
    w = World()
    w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(10), device=0))
    with pytest.raises(DaemonError, match="no generation"):
        w.cp.fabric_plan()
    w.join_all()
    plan = w.cp.fabric_plan()
    assert plan.generation == 1 and plan.phase == FabricPhase.PREPARING_JOIN
    assert plan.atn_devices == [0] and plan.ffn_devices == [1, 2] and plan.lanes_per_ffn_device == 2
    big = [s for s in plan.shards if s.model_id == "Qwen/Qwen3-8B"]
    assert sorted((s.tp_rank, s.device) for s in big) == [(0, 1), (1, 2)] and all(s.tp_size == 2 for s in big)
    small = [s for s in plan.shards if s.model_id == "Qwen/Qwen3-0.6B"]
    assert len(small) == 1 and small[0].layer_end == 28
    assert [r.pe for r in plan.instance_ranks] == [0, 0] and [s.pe for s in big] == [1, 2]


def test_memory_admission_failure_is_reported_not_planned():
    w = World(free=1 << 30)  # Qwen3-8B FFN shards need ~5.4 GB per device
    w.join_all()
    assert w.cp.generation is None and "memory admission failed" in w.cp.failure
    assert w.cp.exit_code == 20


def test_barrier_advances_only_when_everyone_reported():
    w = World()
    w.join_all()
    g = w.cp.generation
    w.cp.report_participant(ParticipantReport(owner=w.ref(10), generation=1, pe=0, phase=ParticipantPhase.JOIN_READY))
    assert g.phase == FabricPhase.PREPARING_JOIN
    w.report_all(ParticipantPhase.JOIN_READY)
    assert g.phase == FabricPhase.JOINING
    with pytest.raises(DaemonError, match="backwards"):
        w.cp.report_participant(ParticipantReport(owner=w.ref(10), generation=1, pe=0, phase=ParticipantPhase.REGISTERED))
    with pytest.raises(DaemonError, match="another generation"):
        w.cp.report_participant(ParticipantReport(owner=w.ref(10), generation=7, pe=0, phase=ParticipantPhase.JOINED))
    with pytest.raises(DaemonError, match="does not own"):
        w.cp.report_participant(ParticipantReport(owner=w.ref(99), generation=1, pe=0, phase=ParticipantPhase.JOINED))


def test_phase_timeout_aborts_and_retirement_reaches_stopped():
    w = World()
    w.join_all()
    w.clock.advance(PHASE_TIMEOUT_SECONDS - 1)
    for reg in list(w.cp.atnagents.values()) + list(w.cp.ffnagents.values()) + list(w.cp.instances.values()):
        reg.last_heartbeat = w.clock()
    w.cp.watchdog()
    assert w.cp.generation.phase == FabricPhase.PREPARING_JOIN
    w.clock.advance(2)
    for reg in list(w.cp.atnagents.values()) + list(w.cp.ffnagents.values()) + list(w.cp.instances.values()):
        reg.last_heartbeat = w.clock()
    w.cp.watchdog()
    assert w.cp.generation.phase == FabricPhase.ABORTING and "timed out" in w.cp.failure
    for ph in (ParticipantPhase.QUIESCED, ParticipantPhase.DRAINED, ParticipantPhase.FINALIZED):
        w.report_all(ph)
    assert w.cp.generation.phase == FabricPhase.STOPPED and w.cp.exit_code == 20


def test_watchdog_classifies_exited_stale_and_replaced_owners():
    w = World()
    w.to_executable()
    # an instance rank goes stale: generation quiesces (graceful), it is not aborted
    w.clock.advance(HEARTBEAT_STALE_SECONDS + 1)
    for k, reg in w.cp.instances.items():
        if k[0] != "Qwen/Qwen3-8B":
            reg.last_heartbeat = w.clock()
    for reg in list(w.cp.atnagents.values()) + list(w.cp.ffnagents.values()):
        reg.last_heartbeat = w.clock()
    lost = w.cp.watchdog()
    assert [(n, r.value) for n, r in lost] == [("instance:Qwen/Qwen3-8B:0", "stale")]
    assert w.cp.generation.phase == FabricPhase.QUIESCING
    # an FFN agent process exits: that is an abort-class loss (already retiring here, so it stays)
    w.alive.discard(21)
    lost = w.cp.watchdog()
    assert ("ffnagent:1", "exited") in [(n, r.value) for n, r in lost]
    # survivors can still drain the generation to STOPPED
    for ph in (ParticipantPhase.QUIESCED, ParticipantPhase.DRAINED, ParticipantPhase.FINALIZED):
        g = w.cp.generation
        for pe, key in g.participants.items():
            kind, dev = key.split(":")
            pid = 10 if kind == "atnagent" else 20 + int(dev)
            if pid in w.alive:
                w.cp.report_participant(ParticipantReport(owner=w.ref(pid), generation=g.number, pe=pe, phase=ph))
    assert w.cp.generation.phase == FabricPhase.STOPPED


def test_registration_conflicts_and_replacement():
    w = World()
    w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(10), device=0))
    w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(10), device=0))  # idempotent
    with pytest.raises(DaemonError, match="owned by live pid 10"):
        w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(11), device=0))
    w.alive.discard(10)  # the old owner died: a new one may take over
    w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(11), device=0))
    assert w.cp.atnagents[0].owner.pid == 11
    with pytest.raises(DaemonError, match="not an attention device"):
        w.cp.register_atnagent(AtnAgentRegistration(owner=w.ref(12), device=5))
    with pytest.raises(DaemonError, match="ABI"):
        w.cp.register_atnagent(AtnAgentRegistration(owner=ProcessRef(abi_version=1, pid=13), device=0))
    with pytest.raises(DaemonError, match="gone|lost"):
        w.cp.heartbeat("atnagent", 0, w.ref(10))
    w.cp.admit_agent(AgentStartupAdmission(owner=w.ref(40), role=Role.FFNAGENT, device=1))
    with pytest.raises(DaemonError, match="already starting"):
        w.cp.admit_agent(AgentStartupAdmission(owner=w.ref(41), role=Role.FFNAGENT, device=1))


def test_invocation_failure_report_aborts_generation():
    w = World()
    w.to_executable()
    w.cp.report_participant(ParticipantReport(
        owner=w.ref(21), generation=1, pe=1, phase=ParticipantPhase.ACTIVE,
        invocation_failure=InvocationFailure(result_code=3, origin_pe=1, instance_index=0, invocation_sequence=9, layer_ordinal=4)))
    assert w.cp.generation.phase == FabricPhase.ABORTING and "code 3" in w.cp.failure


def test_transport_brokering_and_readiness_levels():
    w = World()
    w.join_all()
    with pytest.raises(DaemonError, match="not executable"):
        w.cp.upsert_arenas(0, w.ref(10), 1, [TransportArenaBinding(model_id="Qwen/Qwen3-8B", rank=0, handle_hex="ab", nbytes=4)])
        w.cp.acquire_arena("Qwen/Qwen3-8B", 0, w.ref(31), 1)
    for ph in (ParticipantPhase.JOIN_READY, ParticipantPhase.JOINED, ParticipantPhase.EXECUTION_READY, ParticipantPhase.ACTIVE):
        w.report_all(ph)
    r = w.cp.readiness()
    assert r.fabric_executable and not r.system_ready
    a = w.cp.acquire_arena("Qwen/Qwen3-8B", 0, w.ref(31), 1)
    assert a.handle_hex == "ab"
    with pytest.raises(DaemonError, match="another process"):
        w.cp.instances[("Qwen/Qwen3-8B", 0)].owner = w.ref(77)
        w.cp.acquire_arena("Qwen/Qwen3-8B", 0, w.ref(77), 1)
    w.cp.instances[("Qwen/Qwen3-8B", 0)].owner = w.ref(31)
    for mid, pid in (("Qwen/Qwen3-0.6B", 30), ("Qwen/Qwen3-8B", 31)):
        w.cp.instance_initialized(mid, InstanceRankInitialized(owner=w.ref(pid), rank=0, generation=1))
    r = w.cp.readiness()
    assert r.system_ready and r.serving_healthy
    assert w.cp.quiesce_leases(0, w.ref(10)) == [("Qwen/Qwen3-8B", 0)]
    with pytest.raises(DaemonError, match="quiesced"):
        w.cp.acquire_arena("Qwen/Qwen3-0.6B", 0, w.ref(30), 1)


def test_http_face_in_process():
    from fastapi.testclient import TestClient

    from crosspool_b200.service.daemon.app import create_app

    w = World()
    app = create_app(w.cfg, w.cp, background=False)
    with TestClient(app) as http:
        assert http.get("/health").json()["status"] == "ok"
        assert http.get("/config").json()["digest"] == w.cfg.digest()
        bad = http.post("/config/check", json={"owner": {"abi_version": ABI_VERSION, "pid": 1}, "digest": "x"})
        assert bad.status_code == 409 and bad.json()["detail"]["code"] == "mismatch"
        assert http.get("/fabric/plan").status_code == 503
        w.alive.update({10, 21, 22, 30, 31})
        own = lambda pid: {"abi_version": ABI_VERSION, "pid": pid, "create_time": 1.0}
        assert http.post("/atnagent/register", json={"owner": own(10), "device": 0}).status_code == 200
        for d in (1, 2):
            http.post("/ffnagent/register", json={"owner": own(20 + d), "device": d, "device_free_memory_bytes": 64 << 30,
                                                  "device_total_memory_bytes": 180 << 30})
        prof = {"max_prefill_rows": 512, "max_decode_rows": 64, "hidden_size": 1024}
        for mid, pid in (("Qwen/Qwen3-0.6B", 30), ("Qwen/Qwen3-8B", 31)):
            r = http.post("/instance/register", json={"owner": own(pid), "model_id": mid, "rank": 0, "device": 0, "ffn_profile": prof})
            assert r.status_code == 200, r.text
        plan = http.get("/fabric/plan").json()
        assert plan["generation"] == 1 and len(plan["shards"]) == 3
        hb = http.post("/instance/Qwen/Qwen3-8B/heartbeat/0", json={"owner": own(31)}).json()
        assert hb["fabric_phase"] == "preparing_join"
        ready = http.get("/ready").json()
        assert ready["fabric_executable"] is False and ready["phase"] == "preparing_join"


def test_terminate_owner_only_signals_registered_participants():
    w = World()
    owner = w.ref(4242)
    w.cp.register_atnagent(AtnAgentRegistration(owner=owner, device=0))
    killed = []
    assert w.cp.terminate_owner(owner, terminate=lambda ref: killed.append(ref.pid) or [ref.pid]) == [4242]
    with pytest.raises(DaemonError):   # same PID, other creation time: a reused PID is never signalled
        w.cp.terminate_owner(ProcessRef(abi_version=ABI_VERSION, pid=4242, create_time=900.0), terminate=lambda r: [r.pid])
    with pytest.raises(DaemonError):
        w.cp.terminate_owner(ProcessRef(abi_version=ABI_VERSION, pid=1, create_time=1.0), terminate=lambda r: [r.pid])
    assert killed == [4242]


def test_thousand_instance_rank_leases_plan_join_and_become_ready():
    """Topology scale of the reference's qualification plan (docs/designs/qualification.md:134-147): 1,000 Transport
    arena leases (125 co-located models x 8 data-parallel ranks over 8 attention and 4 FFN devices) go through
    planning, the generation barrier, arena brokering and readiness in bounded time."""
    import time

    n_models, dp, atn, ffn = 125, 8, list(range(8)), [8, 9, 10, 11]
    toml = (f"[atn]\ndevices = {atn}\n[ffn]\ndevices = {ffn}\n[scheduler]\nffn_concurrency = 2\n"
            "[scheduler.slo]\nttft_ms = 1000\ntbt_ms = 50\n")
    for i in range(n_models):
        toml += f'[[models]]\nid = "org/m{i}"\npath = "Qwen/Qwen3-0.6B"\nffn_tp_size = 1\natn_dp_size = {dp}\n'
    alive = set()

    def ref(pid):
        alive.add(pid)
        return ProcessRef(abi_version=ABI_VERSION, pid=pid, create_time=1.0)

    cp = ControlPlane(C.load_config(env={}, toml_text=toml), clock=FakeClock(), process_alive=lambda r: r.pid in alive)
    t0 = time.monotonic()
    for d in atn:
        cp.register_atnagent(AtnAgentRegistration(owner=ref(10 + d), device=d))
    for d in ffn:
        cp.register_ffnagent(FfnAgentRegistration(owner=ref(10 + d), device=d, device_free_memory_bytes=170 << 30,
                                                  device_total_memory_bytes=180 << 30))
    prof = InstanceFfnProfile(max_prefill_rows=256, max_decode_rows=32, hidden_size=1024)
    owners = {}
    for i in range(n_models):
        for r in range(dp):
            owners[(f"org/m{i}", r)] = ref(1000 + i * dp + r)
            cp.register_instance(InstanceRankRegistration(owner=owners[(f"org/m{i}", r)], model_id=f"org/m{i}", rank=r,
                                                          device=r, ffn_profile=prof))
    g = cp.generation
    assert g is not None and len(g.plan.instance_ranks) == 1000 and len(g.plan.shards) == n_models
    per_device = {d: sum(1 for s in g.plan.shards if s.device == d) for d in ffn}
    assert max(per_device.values()) - min(per_device.values()) <= 1          # headroom objective balances the tier
    for ph in (ParticipantPhase.JOIN_READY, ParticipantPhase.JOINED, ParticipantPhase.EXECUTION_READY, ParticipantPhase.ACTIVE):
        for pe, key in g.participants.items():
            cp.report_participant(ParticipantReport(owner=ref(10 + int(key.split(":")[1])), generation=g.number, pe=pe, phase=ph))
    assert g.phase == FabricPhase.EXECUTABLE
    for d in atn:
        cp.upsert_arenas(d, ref(10 + d), g.number, [TransportArenaBinding(model_id=f"org/m{i}", rank=d, handle_hex=f"{i:04x}", nbytes=64)
                                                    for i in range(n_models)])
    for (mid, r), owner in owners.items():
        assert cp.acquire_arena(mid, r, owner, g.number).handle_hex == f"{int(mid[5:]):04x}"
        cp.instance_initialized(mid, InstanceRankInitialized(owner=owner, rank=r, generation=g.number))
    rd = cp.readiness()
    assert rd.system_ready and len(rd.instance_ranks) == 1000
    assert sorted(len(cp.quiesce_leases(d, ref(10 + d))) for d in atn) == [n_models] * 8
    assert time.monotonic() - t0 < 30.0
