"""File helpers. Reference: src/xpool/utils/files.py (atomic text writes for persisted state)."""

from __future__ import annotations

import os
import tempfile
from pathlib import Path


def atomic_write_text(path: str | Path, text: str, *, mode: int = 0o644) -> None:
    """Replaces ``path`` with ``text`` so that a reader (or a restart after a crash) sees the old content or the new
    one, never a torn file: the text goes to a temporary file in the same directory, is flushed to the disk, and is
    renamed over the target. Calibration evidence, memory profiles and sealed benchmark manifests are read back by
    later runs, so they are written this way."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=f".{path.name}.", suffix=".tmp", dir=path.parent)
    try:
        with os.fdopen(fd, "w") as f:
            f.write(text)
            f.flush()
            os.fsync(f.fileno())
        os.chmod(tmp, mode)
        os.replace(tmp, path)
    except BaseException:
        try:
            os.unlink(tmp)
        except FileNotFoundError:
            pass
        raise
