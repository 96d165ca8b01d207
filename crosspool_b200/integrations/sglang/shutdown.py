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


# ---------------------------------------------------------------------------------------------- process tree

import os
import signal
import threading

from ...utils.procs import ProcUniqId

CLEANUP_TIMEOUT_S = 60.0        # one budget for the whole retirement, fixed by whoever asks first
TERMINATION_TIMEOUT_S = 15.0    # the tail of that budget kept for forced termination


class OwnerRetained(RuntimeError):
    """Cleanup could not be confirmed: the owner keeps what it holds (and its process) for manual resolution."""


class ProcessTreeRetirement:
    """Keeps track of the child processes a serving engine creates for an Instance (schedulers that *import*
    peer memory, cache daemons that *export* it) and retires them in an order that is safe for shared device memory.

    Creation is sealed: every factory call runs inside :meth:`creating`, which records the children's identities
    (pid + creation time) as soon as the factory returns and marks the set ``creation_unconfirmed`` when the factory
    raises (a child may exist whose handle never reached us). A cancellation signal that arrives while a factory is
    running is remembered and turned into ``SystemExit(128 + signal)`` only after the factory has unwound.

    Retirement (:meth:`retire`) has one deadline for everything, fixed by the first call of :meth:`begin_retirement`:
    refuse if creation was never sealed; ask the engine once to shut down cooperatively; give the importing workers
    until the cooperative deadline to leave by themselves (skipped for a failed generation); have the caller's
    ``confirm_context`` confirm that their device contexts are gone; force what is left of the importers, newest
    first; only then end the exporters, with SIGTERM first so that they can clean up their sockets. Anything that
    cannot be confirmed inside the deadline raises :class:`OwnerRetained`.
    Reference: src/xpool/integrations/sglang/hooks/shutdown.py:44-555 (same rules, bound there to one engine's
    launch functions; ``hooks()`` names those seams for a registry that has them).
    """

    def __init__(self, *, request_shutdown: Callable[[float], None] | None = None,
                 confirm_context: Callable[[list[ProcUniqId], float], None] | None = None,
                 cleanup_timeout_s: float = CLEANUP_TIMEOUT_S, termination_timeout_s: float = TERMINATION_TIMEOUT_S,
                 clock: Callable[[], float] = time.monotonic, sleep: Callable[[float], None] = time.sleep):
        self._request_shutdown, self._confirm_context = request_shutdown, confirm_context
        self.cleanup_timeout_s, self.termination_timeout_s = cleanup_timeout_s, termination_timeout_s
        self.clock, self.sleep = clock, sleep
        self.deadline: float | None = None
        self.cancelled: int | None = None
        self.launching = self.creating_now = self.creation_unconfirmed = False
        self.failed = self.retiring = self.shutdown_requested = self.retained = False
        self.importers: list[ProcUniqId] = []
        self.exporters: list[ProcUniqId] = []
        self._lock = threading.Lock()

    # ------------------------------------------------------------------ creation
    def begin_retirement(self) -> float:
        with self._lock:
            if self.deadline is None:
                self.deadline = self.clock() + self.cleanup_timeout_s
            return self.deadline

    def note_signal(self, signum: int) -> None:
        """Signal handler body for the launch phase: remembers the first signal; SIGQUIT marks the generation failed."""
        if self.cancelled is None:
            self.cancelled = signum
        self.begin_retirement()
        if signum == signal.SIGQUIT:
            self.failed = True

    def _raise_if_cancelled(self) -> None:
        if self.cancelled is not None:
            raise SystemExit(128 + self.cancelled)

    def creating(self, factory: Callable[[], object], *, exporters: bool = False):
        """Runs ``factory()`` (which starts child processes and returns one handle or a sequence of handles with a
        ``pid``) as one sealed creation."""
        self._raise_if_cancelled()
        self.creating_now = True
        try:
            made = factory()
            handles = list(made) if isinstance(made, (list, tuple)) else [made]
            idents = []
            for h in handles:
                pid = getattr(h, "pid", h)
                if pid is None:
                    raise RuntimeError("the factory returned a process that was never started")
                idents.append(ProcUniqId.of(int(pid)))
            (self.exporters if exporters else self.importers).extend(idents)
        except BaseException:
            self.creation_unconfirmed = True     # a child may have started before its handle was published
            raise
        finally:
            self.creating_now = False
        self._raise_if_cancelled()
        return made

    def launch(self, fn: Callable[[], object]):
        """Runs the engine's whole launch sequence; on failure everything created so far is retired."""
        self.launching = True
        try:
            out = fn()
        except BaseException:
            self.launching = False
            self.failed = True
            self.retire()
            raise
        self.launching = False
        if self.cancelled is not None:
            self.retire()
            raise SystemExit(128 + self.cancelled)
        return out

    # ------------------------------------------------------------------ retirement
    def retire(self, wait_timeout_s: float | None = 60.0) -> None:
        deadline = self.begin_retirement()
        self.retiring = True
        try:
            if self.creating_now or self.creation_unconfirmed:
                raise RuntimeError("child creation was never sealed and confirmed")
            cooperative = deadline - self.termination_timeout_s
            if not self.shutdown_requested and self._request_shutdown is not None:
                self.shutdown_requested = True
                try:
                    self._request_shutdown(self.clock() if self.failed else cooperative)
                except Exception:
                    pass       # the notification is a courtesy; the confirmed termination below is what counts
            while not self.failed and any(p.alive() for p in self.importers) and self.clock() < cooperative:
                self.sleep(min(0.05, max(0.0, cooperative - self.clock())))
            targets = [p for p in self.importers + self.exporters if p.alive()]
            if self._confirm_context is not None and targets:
                self._confirm_context(sorted(targets, key=lambda p: p in self.exporters), deadline)   # importers first
            host_deadline = deadline if wait_timeout_s is None else min(deadline, self.clock() + wait_timeout_s)
            for p in reversed(self.importers):
                _signal(p, signal.SIGKILL)
            self._wait_gone(self.importers, host_deadline, "importing worker")
            for p in self.exporters:           # every consumer of their memory has retired by now
                _signal(p, signal.SIGTERM)
            try:
                self._wait_gone(self.exporters, host_deadline, "exporting daemon")
            except TimeoutError:
                for p in self.exporters:
                    _signal(p, signal.SIGKILL)
                self._wait_gone(self.exporters, max(host_deadline, self.clock() + 2.0), "exporting daemon")
        except Exception as e:
            self.retained = True
            raise OwnerRetained(f"serving cleanup unconfirmed; the owner is retained: {e}") from e

    def _wait_gone(self, procs: list[ProcUniqId], deadline: float, what: str) -> None:
        while any(p.alive() for p in procs):
            if self.clock() >= deadline:
                raise TimeoutError(f"{what} retirement is unconfirmed")
            self.sleep(0.02)

    def as_step(self) -> Callable[[float], bool]:
        """This retirement as the last step of a :class:`ShutdownHookSet`."""
        def run(_deadline_s: float) -> bool:
            try:
                self.retire()
                return True
            except OwnerRetained:
                return False
        return run

    def hooks(self):
        """The launch and kill seams of the serving engine this set attaches to, for a hook registry that has them."""
        from .adapter import Hook

        def around_factory(exporters):
            def handler(original, *a, **kw):
                return self.creating(lambda: original(*a, **kw), exporters=exporters)
            return handler

        def around_launch(original, *a, **kw):
            return self.launch(lambda: original(*a, **kw))

        def around_kill(original, *a, **kw):
            self.retire(kw.get("wait_timeout", 60))

        return [
            Hook("sglang.srt.entrypoints.engine.Engine._launch_subprocesses", around_launch, "around", required=False),
            Hook("sglang.srt.entrypoints.engine.Engine._launch_scheduler_processes", around_factory(False), "around", required=False),
            Hook("sglang.srt.weight_cache.daemon.spawn_weight_cache_daemon", around_factory(True), "around", required=False),
            Hook("sglang.srt.utils.common.kill_process_tree", around_kill, "around", required=False),
        ]


def _signal(p: ProcUniqId, signum: int) -> None:
    if p.alive():             # never a recycled pid: the identity includes the creation time
        try:
            os.kill(p.pid, signum)
        except ProcessLookupError:
            pass
