"""Process identity and process-tree control.

A PID alone is not an identity: the kernel reuses it. ``ProcUniqId`` pairs it with the process
creation time so that a restarted owner is told apart from the one that registered
(reference: src/xpool/utils/procs.py:38-64). Termination always targets exact PIDs collected from
the tree of a given root, never a name pattern.
"""

from __future__ import annotations

import os
import signal
import time
from dataclasses import dataclass

import psutil


@dataclass(frozen=True)
class ProcUniqId:
    pid: int
    create_time: float

    @classmethod
    def current(cls) -> "ProcUniqId":
        return cls.of(os.getpid())

    @classmethod
    def of(cls, pid: int) -> "ProcUniqId":
        return cls(pid, psutil.Process(pid).create_time())

    def status(self) -> str:
        """``alive`` | ``exited`` | ``replaced`` (the PID now belongs to another process)."""
        try:
            p = psutil.Process(self.pid)
            if p.status() == psutil.STATUS_ZOMBIE:
                return "exited"
            return "alive" if abs(p.create_time() - self.create_time) < 0.01 else "replaced"
        except psutil.NoSuchProcess:
            return "exited"

    def alive(self) -> bool:
        return self.status() == "alive"


def tree(root_pid: int) -> list[int]:
    """PIDs of ``root_pid`` and all of its descendants, children first."""
    try:
        root = psutil.Process(root_pid)
    except psutil.NoSuchProcess:
        return []
    kids = [c.pid for c in root.children(recursive=True)]
    return list(reversed(kids)) + [root_pid]


def kill_tree(root: ProcUniqId, grace_s: float = 5.0) -> list[int]:
    """SIGTERM to the tree of ``root`` (only if it is still the same process), SIGKILL to whatever
    is left after ``grace_s``. Returns the PIDs signalled."""
    if not root.alive():
        return []
    pids = tree(root.pid)
    procs = []
    for pid in pids:
        try:
            p = psutil.Process(pid)
            p.send_signal(signal.SIGTERM)
            procs.append(p)
        except psutil.NoSuchProcess:
            pass
    _, alive = psutil.wait_procs(procs, timeout=grace_s)
    for p in alive:
        try:
            p.kill()
        except psutil.NoSuchProcess:
            pass
    return pids


def wait_exit(ident: ProcUniqId, timeout_s: float, poll_s: float = 0.05) -> bool:
    end = time.monotonic() + timeout_s
    while time.monotonic() < end:
        if not ident.alive():
            return True
        time.sleep(poll_s)
    return not ident.alive()
