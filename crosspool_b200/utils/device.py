"""Device inventory from ``nvidia-smi`` (read-only queries; nothing here changes a GPU setting).

Devices are identified by UUID so that a configuration written for one visibility mask still names
the same boards under another (reference: src/xpool/utils/device.py).
"""

from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass

QUERY = ["nvidia-smi", "--query-gpu=index,uuid,name,memory.total,memory.used", "--format=csv,noheader,nounits"]


@dataclass(frozen=True)
class DeviceInfo:
    index: int
    uuid: str
    name: str
    memory_total_mib: int
    memory_used_mib: int


def parse_inventory(text: str) -> list[DeviceInfo]:
    out = []
    for line in text.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 5:
            continue
        out.append(DeviceInfo(int(f[0]), f[1], f[2], int(float(f[3])), int(float(f[4]))))
    return out


def inventory(run=subprocess.run) -> list[DeviceInfo]:
    r = run(QUERY, capture_output=True, text=True, timeout=30)
    if r.returncode != 0:
        raise RuntimeError(f"nvidia-smi failed: {r.stderr.strip()}")
    return parse_inventory(r.stdout)


def visible_indices(n_physical: int, env=os.environ) -> list[int]:
    """Physical indices this process sees, honouring ``CUDA_VISIBLE_DEVICES`` (index form only)."""
    mask = env.get("CUDA_VISIBLE_DEVICES")
    if mask is None or mask == "":
        return list(range(n_physical))
    out = []
    for tok in mask.split(","):
        tok = tok.strip()
        if not tok.lstrip("-").isdigit() or int(tok) < 0 or int(tok) >= n_physical:
            break  # CUDA stops at the first invalid entry
        out.append(int(tok))
    return out


def resolve_uuids(devices: list[int], inv: list[DeviceInfo]) -> dict[int, str]:
    by = {d.index: d.uuid for d in inv}
    missing = [d for d in devices if d not in by]
    if missing:
        raise LookupError(f"configured devices {missing} are not present (have {sorted(by)})")
    return {d: by[d] for d in devices}
