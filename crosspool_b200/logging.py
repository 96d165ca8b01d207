"""One ``xpool`` logger per process: stderr, ``<iso-ms> <LEVEL> <Role> | key=value ...``, colour when
attached to a terminal (reference: src/xpool/logging.py:32-70)."""

from __future__ import annotations

import logging
import sys
import time

_COLORS = {"DEBUG": "\033[36m", "INFO": "\033[32m", "WARNING": "\033[33m", "ERROR": "\033[31m"}


class _Formatter(logging.Formatter):
    def __init__(self, role: str, color: bool):
        super().__init__()
        self.role, self.color = role, color

    def format(self, record: logging.LogRecord) -> str:
        t = time.strftime("%Y-%m-%dT%H:%M:%S", time.localtime(record.created)) + f".{int(record.msecs):03d}"
        lvl = record.levelname
        if self.color:
            lvl = f"{_COLORS.get(lvl, '')}{lvl}\033[0m"
        return f"{t} {lvl} {self.role} | {record.getMessage()}"


def kv(**fields) -> str:
    """``key=value`` message body in a stable order."""
    return " ".join(f"{k}={v}" for k, v in fields.items())


def init_logging(role: str, level: str = "info", color: str = "auto") -> logging.Logger:
    log = logging.getLogger("xpool")
    log.handlers.clear()
    h = logging.StreamHandler(sys.stderr)
    use_color = color == "always" or (color == "auto" and sys.stderr.isatty())
    h.setFormatter(_Formatter(role, use_color))
    log.addHandler(h)
    log.setLevel(getattr(logging, level.upper()))
    log.propagate = False
    return log


def get_logger() -> logging.Logger:
    return logging.getLogger("xpool")
