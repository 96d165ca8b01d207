"""NVTX ranges around engine iterations, off unless ``XPOOL_NVTX=1``.

A profiler that understands NVTX shows one range per prefill chunk and per decode step, named by Instance and row
count, above the kernels of that iteration. When disabled (the default) ``range`` costs one attribute read. The
reference marks its Python phases the same way through ``torch.cuda.nvtx`` (src/xpool/devkit, tracing section of its
observability design).
"""

from __future__ import annotations

import contextlib
import os

_enabled: bool | None = None
_push = _pop = None


def enabled() -> bool:
    global _enabled, _push, _pop
    if _enabled is None:
        _enabled = False
        if os.environ.get("XPOOL_NVTX", "") in ("1", "true", "on"):
            try:
                import torch

                if torch.cuda.is_available():
                    _push, _pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
                    _enabled = True
            except Exception:
                _enabled = False
    return _enabled


def set_enabled(flag: bool, push=None, pop=None) -> None:
    """Forces the state (tests pass recording ``push`` / ``pop`` callables)."""
    global _enabled, _push, _pop
    _enabled, _push, _pop = flag, push, pop


@contextlib.contextmanager
def range(name: str):  # noqa: A001 - mirrors torch.cuda.nvtx.range
    if not enabled():
        yield
        return
    _push(name)
    try:
        yield
    finally:
        _pop()


def push(name: str) -> None:
    if enabled():
        _push(name)


def pop() -> None:
    if enabled():
        _pop()
