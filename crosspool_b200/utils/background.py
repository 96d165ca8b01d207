"""Periodic background work with an orderly stop (reference: src/xpool/utils/background.py)."""

from __future__ import annotations

import threading
from typing import Callable


class BackgroundThread:
    def __init__(self, target: Callable[[threading.Event], None], name: str):
        self._stop = threading.Event()
        self.error: BaseException | None = None

        def run():
            try:
                target(self._stop)
            except BaseException as e:  # surfaced to the owner through .error / .check()
                self.error = e

        self._t = threading.Thread(target=run, name=name, daemon=True)

    @classmethod
    def periodic(cls, fn: Callable[[], None], interval_s: float, name: str, run_first: bool = True) -> "BackgroundThread":
        def loop(stop: threading.Event):
            if run_first:
                fn()
            while not stop.wait(interval_s):
                fn()

        return cls(loop, name)

    def start(self) -> "BackgroundThread":
        self._t.start()
        return self

    def stop(self, timeout_s: float = 5.0) -> bool:
        self._stop.set()
        if self._t.is_alive():
            self._t.join(timeout_s)
        return not self._t.is_alive()

    def check(self) -> None:
        if self.error is not None:
            raise RuntimeError(f"background thread {self._t.name} failed") from self.error
