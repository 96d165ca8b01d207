"""Long-running role processes: register, heartbeat, follow the daemon's generation plan.

An agent is a small state machine driven by the phase the daemon publishes
(reference: src/xpool/runtime/agent.py:270-367, 511-620):

    PREPARING_JOIN       prepare_join()      -> report JOIN_READY   (load shards / allocate arenas,
                                                                      publish arena handles)
    JOINING              join()              -> report JOINED        (map the peers' arenas)
    PREPARING_EXECUTION  prepare_execution() -> report EXECUTION_READY (install Lanes / build engines)
    ACTIVATING           activate()          -> report ACTIVE
    EXECUTABLE           poll_health()          (report an invocation failure if one was recorded)
    QUIESCING/ABORTING   quiesce()           -> report QUIESCED
    DRAINING             drain()             -> report DRAINED
    FINALIZING           finalize()          -> report FINALIZED

Device work lives in a *backend* object so that the protocol can be exercised on CPU with a fake
backend; the GPU backends are in :mod:`crosspool_b200.runtime.backends`. If cleanup cannot be
confirmed the agent keeps ownership of its resources and exits non-zero rather than freeing memory a
peer may still be writing (the reference's "retain on unconfirmed cleanup").
"""

from __future__ import annotations

import threading
import time
from typing import Protocol

from ..native import EXPECTED_ABI
from ..service.client import XpoolClient, self_ref
from ..service.errors import ClientError, DaemonError
from ..service.wire import FabricPhase, FabricPlan, InvocationFailure, ParticipantPhase, ParticipantReport, ProcessRef

HEARTBEAT_SECONDS = 5.0  # reference: heartbeat every 5 s, stale after 15 s


class Backend(Protocol):
    def prepare_join(self, plan: FabricPlan) -> dict[str, str]: ...   # returns arena handles to publish (hex)
    def join(self, plan: FabricPlan) -> None: ...
    def prepare_execution(self, plan: FabricPlan) -> None: ...
    def activate(self, plan: FabricPlan) -> None: ...
    def poll_health(self) -> InvocationFailure | None: ...
    def quiesce(self) -> None: ...
    def drain(self) -> bool: ...       # True when everything in flight has finished
    def finalize(self) -> None: ...


_STEPS = {
    FabricPhase.PREPARING_JOIN: (ParticipantPhase.REGISTERED, ParticipantPhase.JOIN_READY),
    FabricPhase.JOINING: (ParticipantPhase.JOIN_READY, ParticipantPhase.JOINED),
    FabricPhase.PREPARING_EXECUTION: (ParticipantPhase.JOINED, ParticipantPhase.EXECUTION_READY),
    FabricPhase.ACTIVATING: (ParticipantPhase.EXECUTION_READY, ParticipantPhase.ACTIVE),
}
_ORDER = list(ParticipantPhase)


class Agent:
    role = "agent"

    def __init__(self, client: XpoolClient, device: int, backend: Backend, owner: ProcessRef | None = None,
                 sleep=time.sleep):
        self.client, self.device, self.backend = client, device, backend
        self.owner = owner or self_ref(EXPECTED_ABI)
        self.phase = ParticipantPhase.REGISTERED
        self.generation: int | None = None
        self.pe: int | None = None
        self.failed: str | None = None
        self.retained = False
        self._sleep = sleep
        self.daemon_lost_seconds = 15.0      # how long the daemon may stay unreachable before the agent retires on its own
        self._stop = threading.Event()
        self._hb: threading.Thread | None = None

    # -- to be provided by the role
    def register(self) -> None:
        raise NotImplementedError

    def heartbeat(self):
        raise NotImplementedError

    def find_pe(self, plan: FabricPlan) -> int:
        raise NotImplementedError

    # -- lifecycle
    def start_heartbeat(self, period: float = HEARTBEAT_SECONDS) -> None:
        def loop():
            while not self._stop.wait(period):
                try:
                    self.heartbeat()
                except (ClientError, DaemonError):
                    pass

        self._hb = threading.Thread(target=loop, daemon=True, name=f"{self.role}-heartbeat")
        self._hb.start()

    def _report(self, phase: ParticipantPhase, failure: InvocationFailure | None = None, control: str | None = None) -> FabricPhase:
        rep = ParticipantReport(owner=self.owner, generation=self.generation, pe=self.pe, phase=phase,
                                invocation_failure=failure, control_failure=control)
        out = self.client.report(rep)
        self.phase = phase
        return FabricPhase(out)

    def advance(self) -> FabricPhase | None:
        """One lifecycle step. Returns the fabric phase seen, or None when no plan exists yet."""
        try:
            plan = self.client.fabric_plan()
        except DaemonError as e:
            if e.code == "not_ready":
                return None
            raise
        if self.generation != plan.generation:
            if self.generation is not None and self.phase not in (ParticipantPhase.REGISTERED, ParticipantPhase.FINALIZED):
                return plan.phase  # still retiring the previous generation
            self.generation, self.pe, self.phase = plan.generation, self.find_pe(plan), ParticipantPhase.REGISTERED
        fp = plan.phase
        try:
            if fp in _STEPS:
                have, want = _STEPS[fp]
                if _ORDER.index(self.phase) < _ORDER.index(want):
                    if fp == FabricPhase.PREPARING_JOIN:
                        handles = self.backend.prepare_join(plan)
                        if handles:
                            self.client.publish_slot_handles(self.owner, plan.generation, handles)
                    elif fp == FabricPhase.JOINING:
                        self.backend.join(self.client.fabric_plan())
                    elif fp == FabricPhase.PREPARING_EXECUTION:
                        self.backend.prepare_execution(plan)
                    else:
                        self.backend.activate(plan)
                    self._report(want)
            elif fp == FabricPhase.EXECUTABLE:
                f = self.backend.poll_health()
                if f is not None:
                    self._report(ParticipantPhase.ACTIVE, failure=f)
            elif fp in (FabricPhase.QUIESCING, FabricPhase.ABORTING):
                if _ORDER.index(self.phase) < _ORDER.index(ParticipantPhase.QUIESCED):
                    self.backend.quiesce()
                    self._report(ParticipantPhase.QUIESCED)
            elif fp == FabricPhase.DRAINING:
                if _ORDER.index(self.phase) < _ORDER.index(ParticipantPhase.DRAINED):
                    if self.backend.drain():
                        self._report(ParticipantPhase.DRAINED)
            elif fp == FabricPhase.FINALIZING:
                if _ORDER.index(self.phase) < _ORDER.index(ParticipantPhase.FINALIZED):
                    self.backend.finalize()
                    self._report(ParticipantPhase.FINALIZED)
        except (DaemonError, ClientError):
            raise
        except Exception as e:  # device or loader failure: tell the daemon, then stop
            self.failed = f"{type(e).__name__}: {e}"
            try:
                self._report(self.phase, control=self.failed)
            except (DaemonError, ClientError):
                pass
        return fp

    def run(self, poll_seconds: float = 0.05, until=None) -> int:
        """Main loop. ``until(agent, phase)`` may end it (tests). Exit code 0 clean, 1 failed."""
        self.register()
        self.start_heartbeat()
        lost_since: float | None = None
        try:
            while not self._stop.is_set():
                try:
                    fp = self.advance()
                    lost_since = None
                except ClientError as e:
                    # The daemon does not answer. It is the only authority of the deployment, so after a grace period
                    # the agent stops serving on its own: quiesce, drain, finalise in order, exit non-zero.
                    now = time.monotonic()
                    lost_since = now if lost_since is None else lost_since
                    if now - lost_since < self.daemon_lost_seconds:
                        self._sleep(min(1.0, max(poll_seconds, 0.2)))
                        continue
                    self.failed = f"daemon lost for {now - lost_since:.0f} s: {e}"
                    self._retire_locally()
                    break
                if self.failed:
                    break
                if until is not None and until(self, fp):
                    break
                if fp == FabricPhase.STOPPED and self.phase == ParticipantPhase.FINALIZED:
                    break
                self._sleep(poll_seconds)
        finally:
            self._stop.set()
            hb = getattr(self, "_hb", None)
            if hb is not None:
                hb.join(2.0)       # no thread of this process is inside a request while the interpreter shuts down
        if self.failed:
            # cleanup of a failed generation cannot be confirmed: keep the resources, exit non-zero
            self.retained = True
            return 1
        return 0

    def _retire_locally(self) -> None:
        """Orderly local shutdown without the daemon's barrier (it is gone): every step is attempted, a failing one does
        not keep the later ones from running."""
        for step in (self.backend.quiesce, self.backend.drain, self.backend.finalize):
            try:
                step()
            except Exception:
                pass
        self.phase = ParticipantPhase.FINALIZED

    def stop(self) -> None:
        self._stop.set()
