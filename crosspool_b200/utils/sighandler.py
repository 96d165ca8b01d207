"""Signal handling for long-running roles: the first SIGINT/SIGTERM asks for an orderly shutdown, a
second one while that is in progress exits at once (reference: src/xpool/utils/sighandler.py)."""

from __future__ import annotations

import os
import signal
import threading
from typing import Callable


class ShutdownSignals:
    def __init__(self, on_request: Callable[[int], None] | None = None, hard_exit_code: int = 130):
        self.requested = threading.Event()
        self.signum: int | None = None
        self._on_request, self._hard = on_request, hard_exit_code
        self._old: dict[int, object] = {}

    def _handle(self, signum, frame) -> None:
        if self.requested.is_set():
            os._exit(self._hard)
        self.signum = signum
        self.requested.set()
        if self._on_request:
            self._on_request(signum)

    def install(self, signals=(signal.SIGINT, signal.SIGTERM)) -> "ShutdownSignals":
        for s in signals:
            self._old[s] = signal.signal(s, self._handle)
        return self

    def restore(self) -> None:
        for s, h in self._old.items():
            signal.signal(s, h)
        self._old.clear()

    def __enter__(self):
        return self.install()

    def __exit__(self, *exc):
        self.restore()
