"""SLO-aware arbitration of elastic physical KV memory between co-located Instances.

Every Instance rank owns a KV *partition* on its attention device. A partition has a floor (never
taken away), a reservation (its virtual size) and a target (bytes it may keep mapped right now).
Instances publish demand — bytes they need mapped and the SLO deadline by which they need them —
through the shared-memory control channel; the policy answers with quota commands. Policy rules
(the reference's ``CapacityPolicy``, src/xpool/service/daemon/ecs.py:124-525):

* the per-device budget is frozen once: ``free + mapped - max(total * (1 - utilization), headroom)``;
  the floors must fit in it; spare bytes are split equally as initial targets;
* each step first retires completed commands, then serves borrowers: overdue ones first, then the
  earliest deadline among devices that no overdue borrower needs;
* a borrower is funded from unassigned bytes first; otherwise exactly one donor on that device is
  shrunk — a donor without demand of its own before one with, then the latest deadline;
* at most one new command per step, and every command is validated against the exact
  ``(sequence, bytes, deadline)`` witness of the demand it answers.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol


class Channel(Protocol):
    def read_demand(self, idx: int) -> tuple[int, int, int, int]: ...
    def read_completion(self, idx: int) -> tuple[int, int]: ...
    def publish_command(self, idx: int, sequence: int, target_bytes: int) -> None: ...
    def read_report(self, idx: int) -> tuple[int, int, int]: ...


@dataclass
class Partition:
    index: int
    key: str               # "<model>:<rank>"
    device: int
    floor_bytes: int
    reservation_bytes: int
    bundle_bytes: int = 1
    target_bytes: int = 0
    mapped_bytes: int = 0
    command_seq: int = 0
    completed_seq: int = 0
    demand_seq: int = 0
    demand_bytes: int = 0
    demand_deadline_ns: int = 0

    @property
    def pending(self) -> bool:
        return self.command_seq != self.completed_seq

    @property
    def wants(self) -> int:
        """Bytes the partition still lacks for its demand (0 when satisfied or no demand)."""
        want = min(self.demand_bytes, self.reservation_bytes)
        return max(0, want - self.target_bytes)


@dataclass
class DevicePool:
    device: int
    budget_bytes: int = 0
    unassigned_bytes: int = 0
    frozen: bool = False


@dataclass
class PolicyEvent:
    step: int
    kind: str  # grow | shrink | retire | freeze | reject
    partition: str
    bytes: int
    detail: str = ""


class CapacityPolicy:
    def __init__(self, channel: Channel, partitions: list[Partition], device_index: dict[int, int],
                 utilization: float = 0.95, headroom_bytes: dict[int, int] | None = None, clock=None):
        self.ch = channel
        self.parts = {p.index: p for p in partitions}
        self.device_index = device_index
        self.utilization = utilization
        self.headroom = headroom_bytes or {}
        self.pools = {d: DevicePool(d) for d in {p.device for p in partitions}}
        self.clock = clock
        self.events: list[PolicyEvent] = []
        self.steps = 0

    # ------------------------------------------------------------------ freeze
    def freeze_pools(self) -> None:
        """Computes each device's budget from its reported free/total bytes and hands out the initial
        targets: floors plus an equal share of the spare bytes (rounded down to whole bundles)."""
        for d, pool in self.pools.items():
            free, total, _ = self.ch.read_report(self.device_index[d])
            mapped = sum(p.mapped_bytes for p in self.parts.values() if p.device == d)
            reserve = max(int(total * (1.0 - self.utilization)), self.headroom.get(d, 0))
            pool.budget_bytes = free + mapped - reserve
            on = [p for p in self.parts.values() if p.device == d]
            floors = sum(p.floor_bytes for p in on)
            if floors > pool.budget_bytes:
                raise ValueError(f"device {d}: KV floors {floors} exceed the budget {pool.budget_bytes}")
            spare = pool.budget_bytes - floors
            share = spare // max(1, len(on))
            used = 0
            for p in sorted(on, key=lambda q: q.index):
                extra = min(share, p.reservation_bytes - p.floor_bytes)
                extra -= extra % max(1, p.bundle_bytes)
                p.target_bytes = p.floor_bytes + max(0, extra)
                used += p.target_bytes
                p.command_seq += 1
                self.ch.publish_command(p.index, p.command_seq, p.target_bytes)
            pool.unassigned_bytes = pool.budget_bytes - used
            pool.frozen = True
            self.events.append(PolicyEvent(self.steps, "freeze", f"device{d}", pool.budget_bytes,
                                           f"unassigned={pool.unassigned_bytes}"))

    # ------------------------------------------------------------------ step
    def _now_ns(self) -> int:
        import time

        return int(self.clock() * 1e9) if self.clock else time.monotonic_ns()

    def _refresh(self) -> None:
        for p in self.parts.values():
            seq, need, deadline, mapped = self.ch.read_demand(p.index)
            p.demand_seq, p.demand_bytes, p.demand_deadline_ns, p.mapped_bytes = seq, need, deadline, mapped
            cseq, cmapped = self.ch.read_completion(p.index)
            if cseq > p.completed_seq and cseq <= p.command_seq:
                p.completed_seq = cseq
                p.mapped_bytes = cmapped
                self.events.append(PolicyEvent(self.steps, "retire", p.key, cmapped, f"seq={cseq}"))

    def _borrowers(self, now: int) -> list[Partition]:
        cand = [p for p in self.parts.values() if p.wants > 0 and not p.pending and self.pools[p.device].frozen]
        overdue = sorted((p for p in cand if p.demand_deadline_ns and p.demand_deadline_ns <= now),
                         key=lambda p: (p.demand_deadline_ns, p.index))
        busy = {p.device for p in overdue}
        rest = sorted((p for p in cand if p not in overdue and p.device not in busy),
                      key=lambda p: (p.demand_deadline_ns or 2**63, p.index))
        return overdue + rest

    def _donor(self, borrower: Partition) -> Partition | None:
        cands = [p for p in self.parts.values()
                 if p.device == borrower.device and p.index != borrower.index and not p.pending
                 and p.target_bytes > max(p.floor_bytes, min(p.demand_bytes, p.reservation_bytes))]
        if not cands:
            return None
        # donors without demand first, then the latest deadline
        cands.sort(key=lambda p: (p.demand_bytes > 0, -(p.demand_deadline_ns or 2**63), p.index))
        return cands[0]

    def step(self) -> PolicyEvent | None:
        """One policy tick (the daemon runs it every 10 ms). Returns the command it issued, if any."""
        self.steps += 1
        self._refresh()
        now = self._now_ns()
        for b in self._borrowers(now):
            witness = (b.demand_seq, b.demand_bytes, b.demand_deadline_ns)
            pool = self.pools[b.device]
            need = b.wants
            need += (-need) % max(1, b.bundle_bytes)
            need = min(need, b.reservation_bytes - b.target_bytes)
            if need <= 0:
                continue
            if pool.unassigned_bytes >= b.bundle_bytes:
                grant = min(need, pool.unassigned_bytes)
                grant -= grant % max(1, b.bundle_bytes)
                if grant <= 0:
                    continue
                # the demand must still be the one this decision was made for
                if witness != tuple(self.ch.read_demand(b.index)[:3]):
                    ev = PolicyEvent(self.steps, "reject", b.key, grant, "demand changed")
                    self.events.append(ev)
                    return ev
                pool.unassigned_bytes -= grant
                b.target_bytes += grant
                b.command_seq += 1
                self.ch.publish_command(b.index, b.command_seq, b.target_bytes)
                ev = PolicyEvent(self.steps, "grow", b.key, grant, f"target={b.target_bytes} seq={b.command_seq}")
                self.events.append(ev)
                return ev
            donor = self._donor(b)
            if donor is None:
                continue
            keep = max(donor.floor_bytes, min(donor.demand_bytes, donor.reservation_bytes))
            give = min(need, donor.target_bytes - keep)
            give -= give % max(1, donor.bundle_bytes)
            if give <= 0:
                continue
            donor.target_bytes -= give
            donor.command_seq += 1
            donor._giving = give  # returned to the pool when the shrink completes
            self.ch.publish_command(donor.index, donor.command_seq, donor.target_bytes)
            ev = PolicyEvent(self.steps, "shrink", donor.key, give, f"for={b.key} target={donor.target_bytes}")
            self.events.append(ev)
            return ev
        return None

    def reconcile_completions(self) -> None:
        """Moves bytes freed by completed shrinks into the device's unassigned pool."""
        for p in self.parts.values():
            give = getattr(p, "_giving", 0)
            if give and not p.pending:
                self.pools[p.device].unassigned_bytes += give
                p._giving = 0

    def tick(self) -> PolicyEvent | None:
        self._refresh()
        self.reconcile_completions()
        return self.step()
