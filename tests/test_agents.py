"""Agent lifecycle against an in-process daemon (ASGI transport, fake process table, fake backends):
the generation reaches EXECUTABLE only when every agent went through every phase; a backend failure
is reported and aborts the generation; retirement drains to STOPPED."""
import threading
import time

import httpx
import pytest
from fastapi.testclient import TestClient

from crosspool_b200 import config as C
from crosspool_b200.native import EXPECTED_ABI
from crosspool_b200.runtime.roles import AtnAgent, FfnAgent
from crosspool_b200.service.client import XpoolClient
from crosspool_b200.service.daemon.app import create_app
from crosspool_b200.service.daemon.control import ControlPlane
from crosspool_b200.service.wire import FabricPhase, InstanceFfnProfile, InvocationFailure, ParticipantPhase, ProcessRef

TOML = """
[atn]
devices = [0]
[ffn]
devices = [1, 2]
[scheduler.slo]
ttft_ms = 1000
tbt_ms = 50
[[models]]
id = "Qwen/Qwen3-0.6B"
ffn_tp_size = 2
"""


class FakeBackend:
    def __init__(self, name, fail_in=None):
        self.name, self.calls, self.fail_in, self.failure = name, [], fail_in, None

    def _do(self, what):
        self.calls.append(what)
        if self.fail_in == what:
            raise RuntimeError(f"{self.name} broke in {what}")

    def prepare_join(self, plan):
        self._do("prepare_join")
        return {f"slot:{self.name}": "ab" * 32}

    def join(self, plan):
        self._do("join")
        assert len(plan.slot_handles) == 3  # every participant's handle is visible before joining

    def prepare_execution(self, plan):
        self._do("prepare_execution")

    def activate(self, plan):
        self._do("activate")

    def poll_health(self):
        return self.failure

    def quiesce(self):
        self._do("quiesce")

    def drain(self):
        self._do("drain")
        return True

    def finalize(self):
        self._do("finalize")


class ClientOverTestClient(XpoolClient):
    def __init__(self, http):
        self._http = http


def _world(fail=None):
    cfg = C.load_config(env={}, toml_text=TOML)
    cp = ControlPlane(cfg, process_alive=lambda ref: True)
    http = TestClient(create_app(cfg, cp, background=False))
    http.__enter__()
    client = ClientOverTestClient(http)
    prof = InstanceFfnProfile(max_prefill_rows=512, max_decode_rows=64, hidden_size=1024)
    own = lambda pid: ProcessRef(abi_version=EXPECTED_ABI, pid=pid, create_time=1.0)
    agents = [AtnAgent(client, 0, FakeBackend("atn0", fail), [("Qwen/Qwen3-0.6B", 0, prof)], owner=own(10)),
              FfnAgent(client, 1, FakeBackend("ffn1"), 64 << 30, 180 << 30, owner=own(21)),
              FfnAgent(client, 2, FakeBackend("ffn2"), 64 << 30, 180 << 30, owner=own(22))]
    return cp, http, agents


def _spin(agents, rounds=12):
    for _ in range(rounds):
        for a in agents:
            if not a.failed:
                a.advance()


def test_generation_reaches_executable_then_retires_to_stopped():
    cp, http, agents = _world()
    for a in agents:
        a.register()
    _spin(agents)
    assert cp.generation.phase == FabricPhase.EXECUTABLE
    assert all(a.phase == ParticipantPhase.ACTIVE for a in agents)
    assert agents[1].backend.calls == ["prepare_join", "join", "prepare_execution", "activate"]
    assert cp.readiness().system_ready  # the AtnAgent reported its Instance initialised
    assert [a.pe for a in agents] == [0, 1, 2]
    cp.quiesce("test")
    _spin(agents)
    assert cp.generation.phase == FabricPhase.STOPPED
    assert agents[0].backend.calls[-3:] == ["quiesce", "drain", "finalize"]
    http.__exit__(None, None, None)


def test_backend_failure_is_reported_and_aborts_the_generation():
    cp, http, agents = _world(fail="prepare_execution")
    for a in agents:
        a.register()
    _spin(agents)
    assert agents[0].failed and "broke in prepare_execution" in agents[0].failed
    assert cp.generation.phase in (FabricPhase.ABORTING, FabricPhase.DRAINING, FabricPhase.FINALIZING, FabricPhase.STOPPED)
    assert "control failure" in cp.failure and cp.exit_code == 20
    http.__exit__(None, None, None)


def test_invocation_failure_seen_by_a_lane_aborts_the_generation():
    cp, http, agents = _world()
    for a in agents:
        a.register()
    _spin(agents)
    agents[2].backend.failure = InvocationFailure(result_code=3, origin_pe=2, instance_index=0, invocation_sequence=5,
                                                  layer_ordinal=1)
    agents[2].advance()
    assert cp.generation.phase == FabricPhase.ABORTING
    agents[2].backend.failure = None
    _spin(agents)
    assert cp.generation.phase == FabricPhase.STOPPED
    http.__exit__(None, None, None)


def test_an_agent_whose_daemon_disappears_retires_on_its_own_after_a_grace_period():
    """The daemon is the only authority of a deployment: when it stops answering, an agent keeps trying for a grace
    period (a restart of the HTTP server is survivable), then quiesces, drains and finalises locally and exits non-zero
    instead of dying with a traceback in the middle of serving."""
    from crosspool_b200.service.errors import ClientError

    cp, http, agents = _world()
    for a in agents:
        a.register()
    _spin(agents)
    assert cp.generation.phase == FabricPhase.EXECUTABLE
    ffn = agents[1]
    real_plan, state = ffn.client.fabric_plan, {"down": False, "calls": 0}

    class Flaky:
        def __getattr__(self, name):
            target = getattr(agents[0].client, name)

            def call(*a, **kw):
                if state["down"]:
                    state["calls"] += 1
                    if state.get("recover_after") and state["calls"] >= state["recover_after"]:
                        state["down"] = False           # the daemon is back for the next call
                    raise ClientError("daemon unreachable: connection refused")
                return target(*a, **kw)
            return call

    ffn.client = Flaky()
    ffn.register = lambda: None
    ffn.start_heartbeat = lambda *a, **kw: None
    ffn.daemon_lost_seconds = 0.3
    ffn._sleep = lambda s: time.sleep(0.02)
    # a short outage is survived: the loop keeps polling and carries on when the daemon is back
    state["down"], state["recover_after"] = True, 3
    rc = ffn.run(poll_seconds=0.01, until=lambda a, fp: not state["down"] and state["calls"] >= 3)
    assert rc == 0 and ffn.failed is None and "quiesce" not in ffn.backend.calls
    # a lasting one ends in an orderly local retirement
    ffn._stop.clear()
    state["down"], state["recover_after"] = True, 0
    rc = ffn.run(poll_seconds=0.01)
    assert rc == 1 and ffn.failed.startswith("daemon lost") and ffn.retained
    assert ffn.backend.calls[-3:] == ["quiesce", "drain", "finalize"]
    del real_plan
    http.__exit__(None, None, None)
