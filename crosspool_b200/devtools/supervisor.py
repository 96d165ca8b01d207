"""Owned process groups with retirement deadlines, device leases and port reservation.

Everything a local deployment starts -- daemon, agents, load generators -- is *owned*: started in its own process
group, identified by (pid, creation time) so that a recycled PID is never signalled, and retired in reverse start
order with a deadline per process: SIGTERM to the group, wait, SIGKILL to the exact survivors. Devices are leased
so that two deployments (or two test cases) never run on the same GPU, and listening ports are reserved by binding
them first (reference: src/xpool-dev/xkit/supervisor.py, xkit/device.py, xkit/scheduler.py).
Processes are only ever signalled through PIDs this supervisor created itself.
"""

from __future__ import annotations

import os
import signal
import socket
import subprocess
import time
from contextlib import contextmanager
from dataclasses import dataclass, field
from pathlib import Path

from ..utils.procs import ProcUniqId


@dataclass
class Owned:
    name: str
    proc: subprocess.Popen
    ident: ProcUniqId
    retire_deadline_s: float
    log: Path | None = None
    exit_code: int | None = None


class Supervisor:
    def __init__(self, log_dir: str | os.PathLike | None = None):
        self.log_dir = Path(log_dir) if log_dir else None
        self.owned: list[Owned] = []
        self.events: list[tuple[str, str]] = []

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
