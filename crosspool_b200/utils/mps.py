"""CUDA MPS endpoints.

The reference shares each attention GPU between an AtnAgent process and the Instance processes
through an MPS control daemon (src/xpool/utils/mps.py). This system needs no MPS -- a GPU is owned by
one process that hosts all of its Instances -- so nothing here starts, stops or reconfigures a
daemon. What remains is the description of an endpoint and the environment a client would need, for
operators who run under an existing MPS daemon.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from pathlib import Path


@dataclass(frozen=True)
class MpsEndpoint:
    device_uuid: str
    pipe_dir: Path
    log_dir: Path

    @classmethod
    def for_device(cls, device_uuid: str, root: str | os.PathLike = "/tmp/xpool-mps") -> "MpsEndpoint":
        tag = device_uuid.replace("GPU-", "")[:12]
        base = Path(root) / tag
        return cls(device_uuid, base / "pipe", base / "log")

    def client_env(self, active_thread_percentage: int | None = None) -> dict[str, str]:
        env = {"CUDA_MPS_PIPE_DIRECTORY": str(self.pipe_dir), "CUDA_MPS_LOG_DIRECTORY": str(self.log_dir),
               "CUDA_VISIBLE_DEVICES": self.device_uuid}
        if active_thread_percentage is not None:
            if not 1 <= active_thread_percentage <= 100:
                raise ValueError("active thread percentage must be within 1..100")
            env["CUDA_MPS_ACTIVE_THREAD_PERCENTAGE"] = str(active_thread_percentage)
        return env

    def daemon_running(self) -> bool:
        return (self.pipe_dir / "control").exists()


class MpsScope:
    """Applies an endpoint's client environment for the duration of a block (for child launches)."""

    def __init__(self, endpoint: MpsEndpoint, environ=os.environ, **kw):
        self.env, self.environ, self._saved = endpoint.client_env(**kw), environ, {}

    def __enter__(self):
        for k, v in self.env.items():
            self._saved[k] = self.environ.get(k)
            self.environ[k] = v
        return self

    def __exit__(self, *exc):
        for k, old in self._saved.items():
            if old is None:
                self.environ.pop(k, None)
            else:
                self.environ[k] = old
