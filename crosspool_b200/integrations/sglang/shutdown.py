"""Ordered, deadline-bound retirement of a serving process that hosts an Instance rank.

Steps run in the order given; each has its own deadline and must *confirm* (return True) before the next one
starts. When a step cannot be confirmed the set stops and reports ``retained``: the process keeps what it still
owns and exits non-zero rather than freeing memory another participant may still read -- the reference's "retain
owner on unconfirmed cleanup" rule (src/xpool/integrations/sglang/hooks/shutdown.py:44-555,
src/xpool/runtime/agent.py:511-593).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable


@dataclass
class ShutdownStep:
    name: str
    run: Callable[[float], bool]      # receives the seconds it may take; True = confirmed
    deadline_s: float = 10.0


@dataclass
class ShutdownReport:
    completed: list[str] = field(default_factory=list)
    failed: str | None = None
    retained: bool = False
    elapsed_s: float = 0.0


class ShutdownHookSet:
    def __init__(self, clock: Callable[[], float] = time.monotonic):
        self.steps: list[ShutdownStep] = []
        self.clock = clock
        self.report: ShutdownReport | None = None

    def add(self, name: str, run: Callable[[float], bool], deadline_s: float = 10.0) -> "ShutdownHookSet":
        self.steps.append(ShutdownStep(name, run, deadline_s))
        return self

    def run(self) -> ShutdownReport:
        """Idempotent: a second call returns the first report."""
        if self.report is not None:
            return self.report
        rep, t0 = ShutdownReport(), self.clock()
        for st in self.steps:
            started = self.clock()
            try:
                ok = bool(st.run(st.deadline_s))
            except Exception:
                ok = False
            if not ok or self.clock() - started > st.deadline_s:
                rep.failed, rep.retained = st.name, True
                break
            rep.completed.append(st.name)
        rep.elapsed_s = self.clock() - t0
        self.report = rep
        return rep


def instance_shutdown_set(*, stop_admission: Callable[[], None], drain: Callable[[float], bool], runtime, terminate_children:
                          Callable[[float], bool] | None = None, clock=time.monotonic) -> ShutdownHookSet:
    """The retirement order of an Instance rank: stop admitting requests, let the step in flight finish (no kernel of
    this rank may be waiting on the FFN tier when the arena goes away), unbind the transport and give the lease back,
    then end the engine's child processes."""
    s = ShutdownHookSet(clock)
    s.add("stop_admission", lambda _d: (stop_admission(), True)[1], 5.0)
    s.add("drain_in_flight", drain, 30.0)
    s.add("detach_instance", lambda _d: runtime.detach(), 15.0)
    if terminate_children is not None:
        s.add("terminate_children", terminate_children, 20.0)
    return s
