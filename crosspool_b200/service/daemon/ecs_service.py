"""Daemon side of elastic KV in a running deployment.

For every generation the service creates the seqlock control channel (one partition per Instance rank,
one report slot per attention device), publishes its name and index maps through
``GET /ecs/control-channel/{generation}``, waits until every Instance rank has described its partition
(floor = one bundle, reservation = its whole KV address range) and every attention device has reported
its free memory, then freezes the device pools and runs the capacity policy every tick
(reference: src/xpool/service/daemon/ecs.py:150-163 budget freeze, app.py:58 10 ms policy task).
"""

from __future__ import annotations

import os
from typing import Callable

from ..wire import EcsChannelRef, FabricPhase
from .ecs import CapacityPolicy, Partition


class EcsService:
    def __init__(self, control, publish_ref: Callable[[EcsChannelRef | None], None], utilization: float = 0.95,
                 channel_factory=None):
        self.cp, self.publish_ref, self.utilization = control, publish_ref, utilization
        self._factory = channel_factory
        self.generation = 0
        self.channel = None
        self.ref: EcsChannelRef | None = None
        self.policy: CapacityPolicy | None = None
        self.frozen = False

    def _open(self, plan) -> None:
        from ...native.runtime import EcsChannel

        self.close()
        devices = {str(d): i for i, d in enumerate(plan.atn_devices)}
        parts = {f"{r.model_id}:{r.rank}": i for i, r in enumerate(plan.instance_ranks)}
        name = f"/xpool-ecs-{os.getpid()}-{plan.generation}"
        make = self._factory or EcsChannel.create
        self.channel = make(name, len(devices), len(parts), plan.generation)
        for d, i in devices.items():
            self.channel.set_device(i, int(d))
        self.generation, self.frozen, self.policy = plan.generation, False, None
        self.ref = EcsChannelRef(generation=plan.generation, name=name, partitions=parts, devices=devices)
        self._rank_device = {f"{r.model_id}:{r.rank}": r.device for r in plan.instance_ranks}
        self.publish_ref(self.ref)

    def close(self) -> None:
        if self.channel is not None:
            self.channel.close()
            self.channel = None
        self.ref = None
        self.publish_ref(None)

    def _try_freeze(self) -> bool:
        parts = []
        for key, idx in self.ref.partitions.items():
            info = self.channel.partition(idx)
            if info["reservation_bytes"] == 0:
                return False           # this Instance rank has not described its partition yet
            parts.append(Partition(idx, key, self._rank_device[key], info["floor_bytes"], info["reservation_bytes"],
                                   bundle_bytes=max(1, info["floor_bytes"]), mapped_bytes=info["floor_bytes"]))
        for d, i in self.ref.devices.items():
            free, total, seq = self.channel.read_report(i)
            if seq == 0 or total == 0:
                return False
        index = {int(d): i for d, i in self.ref.devices.items()}
        self.policy = CapacityPolicy(self.channel, parts, index, utilization=self.utilization)
        self.policy.freeze_pools()
        self.frozen = True
        return True

    def state(self) -> dict:
        """What an operator wants to see of the arbitration: pools, every partition's floor / reservation / target /
        mapped bytes and current demand, and the most recent policy events (``GET /ecs/state``)."""
        out: dict = {"generation": self.generation, "frozen": self.frozen, "pools": {}, "partitions": [], "events": []}
        pol = self.policy
        if pol is None:
            return out
        out["pools"] = {str(d): {"budget_bytes": p.budget_bytes, "unassigned_bytes": p.unassigned_bytes} for d, p in pol.pools.items()}
        out["partitions"] = [{"key": p.key, "device": p.device, "floor_bytes": p.floor_bytes, "reservation_bytes": p.reservation_bytes,
                              "target_bytes": p.target_bytes, "mapped_bytes": p.mapped_bytes, "demand_bytes": p.demand_bytes,
                              "pending": p.pending} for p in pol.parts.values()]
        out["events"] = [{"step": e.step, "kind": e.kind, "partition": e.partition, "bytes": e.bytes, "detail": e.detail}
                         for e in pol.events[-200:]]
        return out

    def tick(self):
        gen = self.cp.generation
        if gen is None or gen.phase in (FabricPhase.STOPPED, FabricPhase.ABORTING, FabricPhase.FINALIZING):
            if self.channel is not None:
                self.close()
            return None
        if self.channel is None or gen.number != self.generation:
            self._open(gen.plan)
        if not self.frozen:
            self._try_freeze()
            return None
        return self.policy.tick()
