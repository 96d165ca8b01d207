"""Wrappers around the serving engine's worker process mains.

A scheduler (or data-parallel controller) subprocess that dies must not leave the generation guessing: the wrapper
reports the failure to the daemon, runs the ordered shutdown set and exits with a distinct code
(reference: src/xpool/integrations/sglang/worker.py:106-152).
"""

from __future__ import annotations

import os
import traceback
from typing import Any, Callable

EXIT_OK, EXIT_WORKER_FAILED, EXIT_RETAINED = 0, 30, 31


class WorkerLifecycle:
    def __init__(self, role: str, report_failure: Callable[[str], None] | None = None, shutdown=None,
                 exit_fn: Callable[[int], None] = os._exit):
        self.role, self._report, self.shutdown, self._exit = role, report_failure, shutdown, exit_fn
        self.failure: str | None = None

    def run(self, main: Callable[..., Any], *args, **kw) -> Any:
        try:
            out = main(*args, **kw)
        except BaseException as e:  # SystemExit included: a worker that leaves early fails its generation
            self.failure = f"{self.role}: {type(e).__name__}: {e}"
            if self._report is not None:
                try:
                    self._report(self.failure + "\n" + traceback.format_exc(limit=5))
                except Exception:
                    pass
            code = EXIT_WORKER_FAILED
            if self.shutdown is not None and self.shutdown.run().retained:
                code = EXIT_RETAINED
            self._exit(code)
            return None
        if self.shutdown is not None and self.shutdown.run().retained:
            self._exit(EXIT_RETAINED)
        return out


def run_scheduler_process(original: Callable[..., Any], *args, lifecycle: WorkerLifecycle | None = None, **kw):
    """AROUND handler for the engine's scheduler subprocess entry."""
    return (lifecycle or WorkerLifecycle("scheduler")).run(original, *args, **kw)


def run_data_parallel_controller_process(original: Callable[..., Any], *args, lifecycle: WorkerLifecycle | None = None, **kw):
    return (lifecycle or WorkerLifecycle("dp_controller")).run(original, *args, **kw)
