"""Device-memory model of an FFN device: analytic ledger, calibration coefficients, persisted profile.

The daemon admits a placement only if every stage of bring-up fits (``service/daemon/placement.py``);
the figures it uses come from here. The analytic part counts what this system allocates by
construction -- weight shards, fabric slots, Lane state, split-K workspaces, MoE scratch, descriptor
tables -- rounded to the allocator's granularity. What cannot be derived (context size, graph
memory, allocator slack) is covered by a small linear model whose coefficients are fitted from
measured peaks and stored in a calibration profile bound to the environment it was measured in
(reference: src/xpool/memory.py, src/xpool/runtime/ffnagent/device_memory.py,
src/xpool/runtime/memory_calibration.py).
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from .utils.files import atomic_write_text

ALLOC_GRANULE = 2 << 20      # cudaMalloc hands out physical memory in 2 MiB units
SMALL_POOL = 20 << 20        # framework caching allocator: small blocks come from 2 MiB, large from >= 20 MiB segments


def round_up(n: int, q: int) -> int:
    return -(-n // q) * q


def allocator_reservation_bytes(sizes: list[int]) -> int:
    """Bytes a caching allocator reserves to serve ``sizes`` (each request rounded to 512 B; requests
    under 1 MiB share 2 MiB segments, requests up to 10 MiB come from 20 MiB segments, larger ones are
    rounded to 2 MiB)."""
    small = sum(round_up(s, 512) for s in sizes if s < (1 << 20))
    mid = sum(round_up(s, 512) for s in sizes if (1 << 20) <= s < (10 << 20))
    large = sum(round_up(s, ALLOC_GRANULE) for s in sizes if s >= (10 << 20))
    return round_up(small, ALLOC_GRANULE) + (round_up(mid, SMALL_POOL) if mid else 0) + large


@dataclass(frozen=True)
class GemmDeviceProperties:
    compute_capability: tuple[int, int] = (10, 0)
    sm_count: int = 148


@dataclass(frozen=True)
class DeviceMemoryFeatures:
    """What one FFN device hosts, in the units the ledger needs."""

    weight_bytes: int
    n_instances: int
    n_layers: int
    slot_bytes: int
    lanes: int
    ws_bytes_per_lane: int
    moe_routes: int = 0          # capacity_rows x top_k of the largest MoE instance (0: dense only)
    moe_hidden: int = 0
    moe_inter: int = 0
    moe_experts_padded: int = 0
    moe_rows: int = 0


@dataclass(frozen=True)
class FfnMemoryCalibrationCoefficients:
    context_bytes: float = 600e6       # CUDA context, module image, library workspaces
    per_lane_bytes: float = 8e6        # graph + stream resources of a Lane
    per_instance_bytes: float = 1e6
    weight_slack: float = 0.0          # fraction of weight bytes lost to allocator rounding


@dataclass(frozen=True)
class MemoryCalibrationEnvironment:
    gpu_name: str
    driver: str
    cuda: str
    framework: str
    package_digest: str

    def key(self) -> str:
        return hashlib.sha256(json.dumps(asdict(self), sort_keys=True).encode()).hexdigest()[:16]


@dataclass
class XpoolMemoryCalibrationProfile:
    environment: MemoryCalibrationEnvironment
    coefficients: FfnMemoryCalibrationCoefficients
    samples: int = 0
    max_abs_error_bytes: int = 0

    def save(self, path: str | Path) -> None:
        atomic_write_text(path, json.dumps({"environment": asdict(self.environment), "coefficients": asdict(self.coefficients),
                                            "samples": self.samples, "max_abs_error_bytes": self.max_abs_error_bytes,
                                            "key": self.environment.key()}, indent=1))

    @classmethod
    def load(cls, path: str | Path, expect: MemoryCalibrationEnvironment | None = None) -> "XpoolMemoryCalibrationProfile":
        d = json.loads(Path(path).read_text())
        env = MemoryCalibrationEnvironment(**d["environment"])
        if expect is not None and env.key() != expect.key():
            raise ValueError("memory calibration profile was measured in a different environment; run `xpool memory-profile`")
        return cls(env, FfnMemoryCalibrationCoefficients(**d["coefficients"]), d.get("samples", 0), d.get("max_abs_error_bytes", 0))


@dataclass
class DeviceMemoryEstimate:
    weights: int = 0
    slots: int = 0
    lane_state: int = 0
    workspaces: int = 0
    moe_scratch: int = 0
    tables: int = 0
    calibrated_overhead: int = 0
    detail: dict = field(default_factory=dict)

    @property
    def total(self) -> int:
        return self.weights + self.slots + self.lane_state + self.workspaces + self.moe_scratch + self.tables + self.calibrated_overhead


class DeviceMemoryEstimator:
    def __init__(self, coefficients: FfnMemoryCalibrationCoefficients | None = None,
                 device: GemmDeviceProperties | None = None):
        self.c = coefficients or FfnMemoryCalibrationCoefficients()
        self.device = device or GemmDeviceProperties()

    def analytic(self, f: DeviceMemoryFeatures) -> DeviceMemoryEstimate:
        e = DeviceMemoryEstimate()
        e.weights = round_up(f.weight_bytes, ALLOC_GRANULE)
        e.slots = round_up(f.slot_bytes, ALLOC_GRANULE) if f.slot_bytes else 0
        # LaneCtl + InstanceSlot table + LaneCur per lane + status (see csrc/include/xpool/lane.cuh)
        e.lane_state = allocator_reservation_bytes([4096 + 64 * 32, 1536 * max(1, f.n_instances), 64 * f.lanes, 64])
        counters = 4 * (1 << 14)
        e.workspaces = f.lanes * (round_up(f.ws_bytes_per_lane, ALLOC_GRANULE) + round_up(counters, 512)) if f.weight_bytes else 0
        if f.moe_routes:
            tm = max(f.moe_hidden, f.moe_inter) // 128
            max_tiles = tm * (f.moe_routes // 16 + 1024) + 8
            per_lane = [f.moe_rows * f.moe_experts_padded * 2, f.moe_routes * 4, f.moe_routes * 4, 4100, f.moe_routes * 4,
                        f.moe_routes * 4, max_tiles * 16, max_tiles * 16, 256, f.moe_routes * f.moe_hidden * 2,
                        f.moe_routes * f.moe_inter * 2, f.moe_routes * f.moe_hidden * 2]
            e.moe_scratch = f.lanes * sum(round_up(max(s, 256), 512) for s in per_lane)
            e.moe_scratch = round_up(e.moe_scratch, ALLOC_GRANULE)
        # tensor maps: two per layer (+ one router map for MoE layers), five per instance for inputs/scratch
        if self.device.compute_capability >= (9, 0):
            e.tables = allocator_reservation_bytes([f.n_layers * 512 + f.n_instances * 1536])
        return e

    def estimate(self, f: DeviceMemoryFeatures) -> DeviceMemoryEstimate:
        e = self.analytic(f)
        c = self.c
        e.calibrated_overhead = int(c.context_bytes + c.per_lane_bytes * f.lanes + c.per_instance_bytes * f.n_instances +
                                    c.weight_slack * f.weight_bytes)
        return e


def fit_coefficients(samples: list[tuple[DeviceMemoryFeatures, int]],
                     estimator: DeviceMemoryEstimator | None = None) -> tuple[FfnMemoryCalibrationCoefficients, int]:
    """Least-squares fit of the overhead model to measured peaks: ``measured - analytic ~= c0 + c1 * lanes +
    c2 * instances + c3 * weights``. Returns the coefficients and the largest absolute residual."""
    import numpy as np

    est = estimator or DeviceMemoryEstimator()
    if len(samples) < 4:
        raise ValueError("need at least four calibration samples")
    A = np.array([[1.0, f.lanes, f.n_instances, f.weight_bytes] for f, _ in samples])
    y = np.array([float(m - est.analytic(f).total) for f, m in samples])
    x, *_ = np.linalg.lstsq(A, y, rcond=None)
    coef = FfnMemoryCalibrationCoefficients(float(max(x[0], 0.0)), float(max(x[1], 0.0)), float(max(x[2], 0.0)), float(max(x[3], 0.0)))
    fitted = DeviceMemoryEstimator(coef, est.device)
    resid = max(abs(fitted.estimate(f).total - m) for f, m in samples)
    return coef, int(resid)
