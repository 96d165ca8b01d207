"""The Instance rank as a role of its own: what a serving-engine process does towards the daemon and the transport.

An Instance rank that lives in another engine's worker process (the plugin path, ``integrations/sglang``) is not hosted
by an AtnAgent of this repository: it registers itself, keeps its own heartbeat, waits until the Fabric generation is
executable, acquires the transport arena the daemon brokers for it, binds the native submit path behind
``torch.ops.xpool.ffn_shim``, announces itself initialised once its graphs are captured, and watches the generation's
failure word. Reference: ``InstanceRankRuntime``, ``InstanceRankHeartbeat`` and ``InstanceRankFailureMonitor`` in
src/xpool/runtime/instance.py (start, wait_for_fabric_executable 600 s, publish_initialized, wait_for_ready,
attach_arena_from_daemon; failure poll every 0.1 s).
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable

from ..service.wire import (FabricPhase, InstanceFfnProfile, InstanceRankInitialized, InstanceRankRegistration, ProcessRef,
                            ServingListener, TransportArenaAcquire, TransportArenaBinding)
from ..utils.background import BackgroundThread

FABRIC_EXECUTABLE_TIMEOUT_S = 600.0   # src/xpool/service/daemon/control.py:87 (instance startup)
HEARTBEAT_INTERVAL_S = 5.0
FAILURE_POLL_INTERVAL_S = 0.1


class InstanceStartupError(RuntimeError):
    pass


@dataclass
class InstanceFailure:
    result_code: int
    origin_pe: int
    invocation_sequence: int
    layer_ordinal: int


class InstanceRankFailureMonitor:
    """Polls the arena's failure word every 0.1 s; the first failure is handed to ``on_failure`` exactly once (the
    reference then reports and terminates the serving process: generations are fail-stop)."""

    def __init__(self, read_failure: Callable[[], InstanceFailure | None], on_failure: Callable[[InstanceFailure], None],
                 interval_s: float = FAILURE_POLL_INTERVAL_S):
        self._read, self._on_failure, self.interval_s = read_failure, on_failure, interval_s
        self.failure: InstanceFailure | None = None
        self._thread: BackgroundThread | None = None

    def poll_once(self) -> InstanceFailure | None:
        if self.failure is None:
            f = self._read()
            if f is not None:
                self.failure = f
                self._on_failure(f)
        return self.failure

    def start(self) -> None:
        self._thread = BackgroundThread.periodic(self.poll_once, self.interval_s, "instance-failure-monitor").start()

    def stop(self) -> None:
        if self._thread is not None:
            self._thread.stop()
            self._thread = None


class InstanceRankRuntime:
    """``client``: an ``XpoolClient``. ``attach``: ``callable(binding, plan) -> object`` that maps the brokered arena and
    binds the native submit path (returns whatever must stay alive; it may offer ``failure()`` and ``close()``)."""

    def __init__(self, client, model_id: str, rank: int, device: int, profile: InstanceFfnProfile, attach: Callable | None = None,
                 owner: ProcessRef | None = None, clock: Callable[[], float] = time.monotonic, sleep: Callable[[float], None] = time.sleep):
        from ..native import EXPECTED_ABI
        from ..service.client import self_ref

        self.client, self.model_id, self.rank, self.device, self.profile = client, model_id, rank, device, profile
        self._attach = attach
        self.owner = owner or self_ref(EXPECTED_ABI)
        self.clock, self.sleep = clock, sleep
        self.generation: int | None = None
        self.transport = None
        self.binding: TransportArenaBinding | None = None
        self.monitor: InstanceRankFailureMonitor | None = None
        self._heartbeat: BackgroundThread | None = None
        self.state = "created"

    # ------------------------------------------------------------------ start-up
    def start(self) -> None:
        self.client.register_instance(InstanceRankRegistration(owner=self.owner, model_id=self.model_id, rank=self.rank,
                                                               device=self.device, ffn_profile=self.profile))
        self._heartbeat = BackgroundThread.periodic(lambda: self.client.heartbeat_instance(self.model_id, self.rank, self.owner),
                                                    HEARTBEAT_INTERVAL_S, "instance-heartbeat", run_first=False).start()
        self.state = "registered"

    def wait_for_fabric_executable(self, timeout_s: float = FABRIC_EXECUTABLE_TIMEOUT_S, poll_s: float = 0.1):
        """Blocks until the generation that contains this rank is executable; returns its plan."""
        deadline = self.clock() + timeout_s
        while True:
            snap = self.client.ready()
            if snap.failure:
                raise InstanceStartupError(f"the generation failed while this Instance rank was starting: {snap.failure}")
            if snap.fabric_executable and snap.phase == FabricPhase.EXECUTABLE:
                plan = self.client.fabric_plan()
                if any(r.model_id == self.model_id and r.rank == self.rank for r in plan.instance_ranks):
                    self.generation = plan.generation
                    self.state = "fabric_executable"
                    return plan
            if self.clock() >= deadline:
                raise InstanceStartupError(f"Fabric not executable after {timeout_s:.0f} s (phase {snap.phase.value})")
            self.sleep(poll_s)

    def attach_arena_from_daemon(self, plan=None):
        """Acquires this rank's transport arena lease and binds the submit path to it."""
        if self.generation is None:
            raise InstanceStartupError("wait_for_fabric_executable must succeed first")
        self.binding = self.client.acquire_arena(self.model_id, TransportArenaAcquire(owner=self.owner, rank=self.rank,
                                                                                     generation=self.generation))
        if self._attach is not None:
            self.transport = self._attach(self.binding, plan)
            probe = getattr(self.transport, "failure", None)
            if probe is not None:
                self.monitor = InstanceRankFailureMonitor(lambda: _as_failure(probe()), self._on_failure)
        self.state = "attached"
        return self.transport

    def publish_initialized(self, listener: tuple[str, int] | None = None) -> None:
        sl = ServingListener(host=listener[0], port=listener[1]) if listener else None
        self.client.instance_initialized(self.model_id, InstanceRankInitialized(owner=self.owner, rank=self.rank,
                                                                                generation=self.generation, serving_listener=sl))
        self.state = "initialized"

    def wait_for_ready(self, timeout_s: float = 60.0, poll_s: float = 0.1) -> None:
        deadline = self.clock() + timeout_s
        while not self.client.ready().system_ready:
            if self.clock() >= deadline:
                raise InstanceStartupError(f"system not ready after {timeout_s:.0f} s")
            self.sleep(poll_s)
        self.state = "ready"

    # ------------------------------------------------------------------ serving
    def _on_failure(self, f: InstanceFailure) -> None:
        self.state = "failed"
        self.failure = f

    failure: InstanceFailure | None = None

    def start_failure_monitor(self) -> None:
        if self.monitor is not None:
            self.monitor.start()

    # ------------------------------------------------------------------ retirement
    def detach(self) -> bool:
        """Ordered retirement of this rank: stop watching, unbind the transport, give the lease back, stop the
        heartbeat. Returns False when a step could not be confirmed (the owner then retains what it holds)."""
        ok = True
        if self.monitor is not None:
            self.monitor.stop()
        close = getattr(self.transport, "close", None)
        if close is not None:
            try:
                close()
            except Exception:
                ok = False
        self.transport = None
        try:
            if self.generation is not None:
                self.client.deregister_instance(self.model_id, TransportArenaAcquire(owner=self.owner, rank=self.rank,
                                                                                    generation=self.generation))
        except Exception:
            ok = False
        if self._heartbeat is not None:
            ok = self._heartbeat.stop() and ok
            self._heartbeat = None
        self.state = "detached" if ok else "retained"
        return ok


def _as_failure(f) -> InstanceFailure | None:
    if f is None:
        return None
    return InstanceFailure(f.result_code, f.origin_pe, f.invocation_sequence, f.layer_ordinal)
