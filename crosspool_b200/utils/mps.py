"""CUDA MPS endpoints.

The reference shares each attention GPU between an AtnAgent process and the Instance processes
through an MPS control daemon (src/xpool/utils/mps.py). With this repository's own engine a GPU is owned by
one process that hosts all of its Instances and no MPS is involved; ``MpsEndpoint`` / ``MpsScope`` describe an
endpoint and apply a client's environment. Deployments that run Instances inside another engine's processes
share the GPU between processes: ``OwnedMpsScope`` (below) is the daemon's ownership of a control daemon for
them -- start, client termination with confirmation, stop. It is never used unless a deployment asks for it.
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


# ---------------------------------------------------------------------------------------------------------------
# Owning an MPS control daemon (engine-integration deployments only).
#
# When Instances run inside another engine's processes (the plugin path), several processes share one attention GPU
# and the daemon owns an MPS control daemon per attention device, as the reference does
# (src/xpool/utils/mps.py:289-393 MpsScope.start, :514-588 client termination; directories
# /tmp/xpool-mps-<uid>/<key>/{pipe,log}). Starting an MPS control daemon changes how a GPU is shared for everybody
# who uses it afterwards, so nothing here runs unless a deployment asks for it ([atn] mps = true is NOT a default),
# and the tests drive it against a stand-in control binary.

class MpsControlError(RuntimeError):
    pass


class MpsControl:
    """Talks to ``nvidia-cuda-mps-control``: every command is one run of the binary with the command on stdin and the
    endpoint's pipe / log directories in its environment."""

    def __init__(self, endpoint: MpsEndpoint, binary: str = "nvidia-cuda-mps-control", run=None, timeout_s: float = 10.0):
        import subprocess

        self.endpoint, self.binary, self.timeout_s = endpoint, binary, timeout_s
        self._run = run or (lambda argv, **kw: subprocess.run(argv, **kw))

    def _env(self) -> dict[str, str]:
        env = dict(os.environ)
        env.update({"CUDA_MPS_PIPE_DIRECTORY": str(self.endpoint.pipe_dir), "CUDA_MPS_LOG_DIRECTORY": str(self.endpoint.log_dir),
                    "CUDA_VISIBLE_DEVICES": self.endpoint.device_uuid})
        return env

    def start_daemon(self) -> None:
        self.endpoint.pipe_dir.mkdir(parents=True, exist_ok=True, mode=0o700)
        self.endpoint.log_dir.mkdir(parents=True, exist_ok=True, mode=0o700)
        r = self._run([self.binary, "-d"], env=self._env(), capture_output=True, text=True, timeout=self.timeout_s)
        if r.returncode != 0:
            raise MpsControlError(f"MPS control daemon did not start: {r.stderr.strip() or r.stdout.strip()}")

    def command(self, text: str) -> str:
        r = self._run([self.binary], input=text + "\n", env=self._env(), capture_output=True, text=True, timeout=self.timeout_s)
        if r.returncode != 0:
            raise MpsControlError(f"MPS control command {text!r} failed: {r.stderr.strip() or r.stdout.strip()}")
        return r.stdout

    def server_pids(self) -> list[int]:
        return [int(x) for x in self.command("get_server_list").split() if x.strip().isdigit()]

    def client_pids(self, server_pid: int) -> list[int]:
        return [int(x) for x in self.command(f"get_client_list {server_pid}").split() if x.strip().isdigit()]

    def terminate_client(self, server_pid: int, client_pid: int) -> None:
        self.command(f"terminate_client {server_pid} {client_pid}")

    def quit(self) -> None:
        self.command("quit")


class OwnedMpsScope:
    """The daemon's ownership of one attention device's MPS control daemon: ``start`` brings it up (idempotent),
    ``terminate_client`` ends one client process and *confirms* that it is gone from every server's client list
    (the daemon's ``POST /serving/mps/terminate-client``), ``stop`` quits the control daemon. A scope that could not
    confirm a termination reports it instead of pretending: the caller retains ownership."""

    def __init__(self, endpoint: MpsEndpoint, control: MpsControl | None = None):
        self.endpoint, self.control = endpoint, control or MpsControl(endpoint)
        self.started = False

    def start(self) -> None:
        if self.started:
            return
        if not self.endpoint.daemon_running():
            self.control.start_daemon()
        self.started = True

    def clients(self) -> dict[int, list[int]]:
        return {s: self.control.client_pids(s) for s in self.control.server_pids()}

    def terminate_client(self, client_pid: int) -> bool:
        """True when the client was found and is confirmed gone, or was not a client at all."""
        found = False
        for server, clients in self.clients().items():
            if client_pid in clients:
                found = True
                self.control.terminate_client(server, client_pid)
        if not found:
            return True
        return all(client_pid not in c for c in self.clients().values())

    def stop(self) -> None:
        if self.started:
            self.control.quit()
            self.started = False
