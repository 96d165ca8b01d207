"""Owned process groups with retirement deadlines, device leases and port reservation.

Everything a local deployment starts -- daemon, agents, load generators -- is *owned*: started in its own process
group, identified by (pid, creation time) so that a recycled PID is never signalled, and retired in reverse start
order with a deadline per process: SIGTERM to the group, wait, SIGKILL to the exact survivors. Devices are leased
so that two deployments (or two test cases) never run on the same GPU, and listening ports are reserved by binding
them first (reference: src/xpool-dev/xkit/supervisor.py, xkit/device.py, xkit/scheduler.py).
Processes are only ever signalled through PIDs this supervisor created itself, or that the kernel handed to it:
with ``adopt_orphans=True`` the supervising process becomes a *child subreaper* (``prctl(PR_SET_CHILD_SUBREAPER)``),
so a grandchild that left its process group (its own session) and lost its parent is re-parented to the supervisor
instead of to init; after a task's group is gone the supervisor drains exactly those adopted processes, by identity,
and reports them. Infrastructure children of the interpreter itself (multiprocessing's resource tracker) are protected.
"""

from __future__ import annotations

import os
import signal
import socket
import subprocess
import time
from contextlib import contextmanager
from dataclasses import dataclass
from pathlib import Path

import ctypes

import psutil

from ..utils.procs import ProcUniqId

PR_SET_CHILD_SUBREAPER = 36
LOG_TAIL_CHARS = 4000


def become_child_subreaper() -> None:
    """Linux: orphaned descendants of this process are re-parented to it (so that it can find and retire them)."""
    libc = ctypes.CDLL(None, use_errno=True)
    if libc.prctl(PR_SET_CHILD_SUBREAPER, 1, 0, 0, 0) != 0:
        e = ctypes.get_errno()
        raise OSError(e, os.strerror(e))


@dataclass(frozen=True)
class TaskCompletion:
    """How a supervised task ended: ``completed`` (exit 0), ``failed`` (non-zero exit), ``timed_out`` (retired at its
    time limit), ``cancelled`` (retired on request), with whatever it left behind."""

    name: str
    kind: str
    exit_code: int | None
    elapsed_s: float
    orphans: tuple[int, ...] = ()
    log_tail: str = ""

    @property
    def ok(self) -> bool:
        return self.kind == "completed" and not self.orphans


@dataclass
class Owned:
    name: str
    proc: subprocess.Popen
    ident: ProcUniqId
    retire_deadline_s: float
    log: Path | None = None
    exit_code: int | None = None


class Supervisor:
    def __init__(self, log_dir: str | os.PathLike | None = None, adopt_orphans: bool = False):
        self.log_dir = Path(log_dir) if log_dir else None
        self.owned: list[Owned] = []
        self.events: list[tuple[str, str]] = []
        self.adopt_orphans = adopt_orphans
        self.protected: set[ProcUniqId] = set()
        if adopt_orphans:
            become_child_subreaper()
            self.protected = set(self._direct_children())     # whatever the interpreter already runs (resource tracker)

    # ------------------------------------------------------------------ adopted descendants
    @staticmethod
    def _direct_children() -> list[ProcUniqId]:
        out = []
        for c in psutil.Process().children():
            try:
                out.append(ProcUniqId(c.pid, c.create_time()))
            except psutil.NoSuchProcess:
                pass
        return out

    def adopted(self) -> list[ProcUniqId]:
        """Direct children of this process that it neither started nor protects: orphans the kernel re-parented here."""
        mine = {o.ident for o in self.owned} | self.protected
        return [c for c in self._direct_children() if c not in mine and c.alive()]

    def drain_adopted(self, term_s: float = 2.0, kill_s: float = 3.0) -> list[int]:
        """SIGTERM, then SIGKILL, to every adopted process and its tree; returns their PIDs."""
        if not self.adopt_orphans:
            return []
        seen: list[int] = []
        deadline = time.monotonic() + term_s + kill_s
        while time.monotonic() < deadline:
            orphans = self.adopted()
            if not orphans:
                break
            for o in orphans:
                if o.pid not in seen:
                    seen.append(o.pid)
                    self.events.append(("orphan", str(o.pid)))
                sig = signal.SIGTERM if time.monotonic() < deadline - kill_s else signal.SIGKILL
                if o.alive():
                    try:
                        os.kill(o.pid, sig)
                    except ProcessLookupError:
                        pass
            time.sleep(0.05)
        for pid in seen:                          # adopted children are ours to wait for: leave no zombie behind
            try:
                os.waitpid(pid, os.WNOHANG)
            except ChildProcessError:
                pass
        return seen

    def run(self, name: str, argv: list[str], timeout_s: float, env: dict[str, str] | None = None, cwd: str | None = None,
            cancel=None) -> TaskCompletion:
        """Starts a task, waits for it up to ``timeout_s`` (or until ``cancel()`` turns true), retires its process group
        and whatever it orphaned, and says how it ended."""
        t0 = time.monotonic()
        o = self.start(name, argv, env=env, cwd=cwd)
        kind = None
        while o.proc.poll() is None:
            if time.monotonic() - t0 >= timeout_s:
                kind = "timed_out"
                break
            if cancel is not None and cancel():
                kind = "cancelled"
                break
            time.sleep(0.02)
        rc = self.retire(o)
        self.owned.remove(o)
        orphans = tuple(self.drain_adopted())
        if kind is None:
            kind = "completed" if rc == 0 else "failed"
        tail = ""
        if o.log is not None and o.log.exists():
            tail = o.log.read_text(errors="replace")[-LOG_TAIL_CHARS:]
        return TaskCompletion(name, kind, rc, time.monotonic() - t0, orphans, tail)

    def start(self, name: str, argv: list[str], env: dict[str, str] | None = None, retire_deadline_s: float = 20.0,
              cwd: str | None = None) -> Owned:
        out = None
        log = None
        if self.log_dir is not None:
            self.log_dir.mkdir(parents=True, exist_ok=True)
            log = self.log_dir / f"{name}.log"
            out = open(log, "w")
        p = subprocess.Popen(argv, env=env, cwd=cwd, stdout=out or subprocess.DEVNULL, stderr=subprocess.STDOUT if out else subprocess.DEVNULL,
                             start_new_session=True)
        o = Owned(name, p, ProcUniqId.of(p.pid), retire_deadline_s, log)
        self.owned.append(o)
        self.events.append(("start", name))
        return o

    def poll(self) -> dict[str, int | None]:
        return {o.name: o.proc.poll() for o in self.owned}

    def wait_until(self, predicate, timeout_s: float, poll_s: float = 0.05, what: str = "condition") -> None:
        """Waits for ``predicate()``; fails early when an owned process has exited with an error."""
        deadline = time.monotonic() + timeout_s
        while time.monotonic() < deadline:
            if predicate():
                return
            for o in self.owned:
                rc = o.proc.poll()
                if rc not in (None, 0):
                    raise RuntimeError(f"{o.name} exited with code {rc} while waiting for {what}")
            time.sleep(poll_s)
        raise TimeoutError(f"{what} not reached within {timeout_s:.0f} s")

    def retire(self, o: Owned) -> int | None:
        """SIGTERM to the process group, SIGKILL after the deadline; only if the PID still names the process we started."""
        if o.proc.poll() is None and o.ident.status() == "alive":
            try:
                os.killpg(o.proc.pid, signal.SIGTERM)
            except ProcessLookupError:
                pass
            try:
                o.proc.wait(o.retire_deadline_s)
            except subprocess.TimeoutExpired:
                self.events.append(("kill", o.name))
                try:
                    os.killpg(o.proc.pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
                o.proc.wait(5)
        o.exit_code = o.proc.poll()
        self.events.append(("retired", o.name))
        return o.exit_code

    def retire_all(self) -> dict[str, int | None]:
        """Reverse start order: what was started last depends on what was started first."""
        out = {}
        for o in reversed(self.owned):
            out[o.name] = self.retire(o)
        self.owned.clear()
        return out

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.retire_all()
        return False


class DeviceLeases:
    """Exclusive leases of GPU indices inside one process tree (test cases that need devices take them from here)."""

    def __init__(self, devices: list[int]):
        self.free, self.taken = sorted(devices), {}

    def acquire(self, holder: str, n: int) -> list[int] | None:
        if n > len(self.free):
            return None
        got, self.free = self.free[:n], self.free[n:]
        self.taken[holder] = got
        return got

    def release(self, holder: str) -> None:
        self.free = sorted(self.free + self.taken.pop(holder, []))

    @contextmanager
    def lease(self, holder: str, n: int):
        got = self.acquire(holder, n)
        if got is None:
            raise RuntimeError(f"{holder} needs {n} devices, {len(self.free)} free")
        try:
            yield got
        finally:
            self.release(holder)


def reserve_port(host: str = "127.0.0.1") -> int:
    """A port that was free a moment ago (bound to find it, released at once; the caller binds it next)."""
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind((host, 0))
        return s.getsockname()[1]
