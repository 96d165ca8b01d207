"""``xpool memory-profile --calibrate``: measure real device-memory peaks of a corpus of synthetic FFN
deployments, fit the overhead coefficients of the memory model and persist the profile
(reference: src/xpool/runtime/memory_calibration.py and runtime/ffnagent/memory_profile/*).

Each experiment builds an :class:`~crosspool_b200.parallel.fabric.FfnRankRuntime` with a given
number of Instances, layers, Lanes and workspace size on the current GPU, installs and starts it,
and records how much device memory the process gained (``cudaMemGetInfo`` before and after). The
measuring function is injectable so that the fit and the bookkeeping are testable without a GPU.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable

from .. import memory as M
from ..utils.files import atomic_write_text


@dataclass(frozen=True)
class Experiment:
    preset: str
    layers: int
    instances: int
    lanes: int
    ws_mb: int = 64
    capacity_rows: int = 512


DEFAULT_CORPUS = (
    Experiment("tiny-qwen3", 2, 1, 1), Experiment("tiny-qwen3", 2, 4, 2), Experiment("Qwen/Qwen3-0.6B", 4, 1, 1),
    Experiment("Qwen/Qwen3-0.6B", 8, 2, 2), Experiment("Qwen/Qwen3-0.6B", 28, 1, 4), Experiment("Qwen/Qwen3-1.7B", 8, 3, 1),
    Experiment("Qwen/Qwen3-8B", 4, 1, 2, ws_mb=128), Experiment("Qwen/Qwen3-0.6B", 2, 8, 8, ws_mb=32),
)


def features_of(exp: Experiment) -> M.DeviceMemoryFeatures:
    from ..models import config as mc
    from ..parallel import fabric as F

    cfg = mc.preset(exp.preset).with_layers(exp.layers)
    place = F.InstancePlacement("m", cfg, 0, 0, (1,), exp.capacity_rows)
    weights = sum(cfg.ffn_param_bytes_per_layer(l) for l in range(cfg.num_layers)) * exp.instances
    slot = F.ffn_slot_layout(place).total_bytes * exp.instances
    return M.DeviceMemoryFeatures(weight_bytes=weights, n_instances=exp.instances, n_layers=exp.layers * exp.instances,
                                  slot_bytes=slot, lanes=exp.lanes, ws_bytes_per_lane=exp.ws_mb << 20)


def measure_on_gpu(exp: Experiment) -> int:
    """Bytes of device memory one experiment holds at its peak (weights resident, Lanes running)."""
    import gc

    import torch

    from ..models import config as mc
    from ..parallel import fabric as F

    torch.cuda.synchronize()
    gc.collect()
    torch.cuda.empty_cache()
    free0, _ = torch.cuda.mem_get_info()
    cfg = mc.preset(exp.preset).with_layers(exp.layers)
    ffn = F.FfnRankRuntime("cuda", n_lanes=exp.lanes, ws_bytes_per_lane=exp.ws_mb << 20)
    bufs = []
    try:
        for i in range(exp.instances):
            p = F.InstancePlacement(f"m{i}", cfg, i, 0, (1,), exp.capacity_rows)
            st = ffn.add_instance(p, 0)
            buf = F.PeerBuffer(F.atn_slot_layout(p).total_bytes)  # stands in for the attention side
            st.atn_base = buf.ptr
            bufs.append(buf)
        ffn.install()
        ffn.start(lease_ms=1.0)
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        atn_side = sum(b.nbytes for b in bufs)
        return free0 - free1 - atn_side
    finally:
        ffn.close()
        for b in bufs:
            b.free()
        torch.cuda.empty_cache()


def current_environment() -> M.MemoryCalibrationEnvironment:
    import torch

    name = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    drv = ""
    try:
        import pynvml

        pynvml.nvmlInit()
        drv = pynvml.nvmlSystemGetDriverVersion()
        drv = drv.decode() if isinstance(drv, bytes) else drv
    except Exception:
        pass
    lib = Path(__file__).resolve().parents[1] / "native" / "libxpool_kernels.so"
    digest = hashlib.sha256(lib.read_bytes()).hexdigest()[:16] if lib.exists() else "nolib"
    return M.MemoryCalibrationEnvironment(name, drv, torch.version.cuda or "", f"torch {torch.__version__}", digest)


def experiment_key(exp: Experiment) -> str:
    return hashlib.sha256(repr(exp).encode()).hexdigest()[:12]


class EvidenceStore:
    """Measured peaks kept on disk, one JSON file per (environment, experiment): a calibration run that was interrupted
    -- or a corpus that grew -- only measures what is missing, and a profile can be re-fitted without a GPU
    (reference: memory_profile/evidence.py and experiment.py persist every experiment's evidence before fitting)."""

    def __init__(self, root: str | Path, environment: M.MemoryCalibrationEnvironment):
        self.dir = Path(root) / "memory-calibration" / environment.key()
        self.environment = environment

    def path(self, exp: Experiment) -> Path:
        return self.dir / f"{experiment_key(exp)}.json"

    def load(self, exp: Experiment) -> int | None:
        p = self.path(exp)
        if not p.exists():
            return None
        try:
            d = json.loads(p.read_text())
        except ValueError:
            return None
        return int(d["measured_bytes"]) if d.get("experiment") == asdict(exp) else None

    def save(self, exp: Experiment, measured_bytes: int) -> None:
        self.dir.mkdir(parents=True, exist_ok=True)
        f = features_of(exp)
        # a fit resumes from these files: an interrupted run must leave each one whole or absent
        atomic_write_text(self.path(exp), json.dumps({"experiment": asdict(exp), "measured_bytes": int(measured_bytes),
                                                      "features": asdict(f), "environment": asdict(self.environment)}, indent=1))

    def all(self) -> list[tuple[Experiment, int]]:
        out = []
        for p in sorted(self.dir.glob("*.json")) if self.dir.exists() else []:
            try:
                d = json.loads(p.read_text())
                out.append((Experiment(**d["experiment"]), int(d["measured_bytes"])))
            except (ValueError, KeyError, TypeError):
                continue
        return out


def calibrate(corpus=DEFAULT_CORPUS, measure: Callable[[Experiment], int] = measure_on_gpu,
              environment: M.MemoryCalibrationEnvironment | None = None, evidence_root: str | Path | None = None
              ) -> M.XpoolMemoryCalibrationProfile:
    """Measures the corpus (skipping experiments whose evidence is already stored under ``evidence_root``), fits the
    overhead coefficients to all stored evidence of this environment and returns the profile."""
    env = environment or current_environment()
    store = EvidenceStore(evidence_root, env) if evidence_root is not None else None
    samples = []
    for e in corpus:
        got = store.load(e) if store is not None else None
        if got is None:
            got = measure(e)
            if store is not None:
                store.save(e, got)
        samples.append((features_of(e), got))
    if store is not None:                      # evidence of earlier runs with other experiments counts too
        known = {experiment_key(e) for e in corpus}
        samples += [(features_of(e), b) for e, b in store.all() if experiment_key(e) not in known]
    coef, resid = M.fit_coefficients(samples)
    return M.XpoolMemoryCalibrationProfile(env, coef, len(samples), resid)
