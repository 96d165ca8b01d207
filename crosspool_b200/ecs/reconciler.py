"""Instance-rank side of elastic KV capacity: demand publication, command execution, event-gated
retirement, admission and the allocation journal.

The daemon's :class:`~crosspool_b200.service.daemon.ecs.CapacityPolicy` owns the *targets*; an
Instance rank owns its *mapped bundles*. They talk through the seqlock channel
(``native.runtime.EcsChannel``):

    rank   -> publish_report(free, total)           physical memory it can see
    rank   -> publish_demand(seq, required, deadline, mapped)   before it would stall or retract
    daemon -> publish_command(seq, target_bytes)     grow or shrink order
    rank   -> publish_completion(seq, mapped_bytes)  once the order is carried out

Growing is immediate (map bundles, publish their pages). Shrinking is *event gated*: a bundle is
first taken out of circulation when it holds no pages, and unmapped only after the retirement gate
(a CUDA event recorded behind the last step that may have read it, or any callable for tests)
reports completion -- the same discipline as the reference's ``CapacityReconciler``
(src/xpool/integrations/sglang/ecs/reconciler.py:77-139,345-436) and its admission / journal
helpers (ecs/admission.py:19-81, ecs/allocation.py:37-72).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Protocol

from ..engine.kv_cache import OutOfPages, PagedKvCache
from . import vmm


class PartitionChannel(Protocol):
    def publish_report(self, idx: int, free_bytes: int, total_bytes: int, sequence: int) -> None: ...
    def publish_demand(self, idx: int, evaluated_sequence: int, required_bytes: int, deadline_ns: int,
                       mapped_bytes: int) -> None: ...
    def read_command(self, idx: int) -> tuple[int, int]: ...
    def publish_completion(self, idx: int, sequence: int, mapped_bytes: int) -> None: ...


@dataclass
class AllocationJournal:
    """Undo log of one scheduling attempt: page allocations recorded here are rolled back together
    if the attempt cannot be completed (a request is admitted whole or not at all)."""

    cache: PagedKvCache
    entries: list[tuple[int, int]] = field(default_factory=list)  # (seq_id, table length before)

    def ensure(self, seq_id: int, new_len: int) -> None:
        before = len(self.cache.tables.get(seq_id, ()))
        self.cache.ensure(seq_id, new_len)
        self.entries.append((seq_id, before))

    def rollback(self) -> None:
        for seq_id, before in reversed(self.entries):
            t = self.cache.tables.get(seq_id)
            if t is None:
                continue
            extra = t[before:]
            del t[before:]
            self.cache.allocator.free(extra)
            if before == 0:
                self.cache.tables.pop(seq_id, None)
        self.entries.clear()

    def commit(self) -> None:
        self.entries.clear()


@dataclass
class AdmissionDecision:
    admitted: bool
    missing_pages: int = 0


def admit(cache: PagedKvCache, requests: list[tuple[int, int]], reserve_pages: int = 0) -> AdmissionDecision:
    """All-or-nothing admission of ``(seq_id, target_len)`` pairs, keeping ``reserve_pages`` free for
    the decode growth of running sequences."""
    need = sum(cache.pages_needed(s, n) for s, n in requests)
    free = cache.allocator.free_pages - reserve_pages
    if need > free:
        return AdmissionDecision(False, need - free)
    j = AllocationJournal(cache)
    try:
        for s, n in requests:
            j.ensure(s, n)
    except OutOfPages:
        j.rollback()
        return AdmissionDecision(False, need)
    j.commit()
    return AdmissionDecision(True)


@dataclass
class _Retiring:
    bundle: int
    gate: Callable[[], bool]


class CapacityReconciler:
    def __init__(self, cache: PagedKvCache, channel: PartitionChannel, index: int, *, floor_bundles: int = 1,
                 gate_factory: Callable[[], Callable[[], bool]] | None = None,
                 clock_ns: Callable[[], int] = time.monotonic_ns):
        if cache.backing is None:
            raise ValueError("the KV cache has no elastic backing")
        self.cache, self.channel, self.index = cache, channel, index
        self.floor_bundles = floor_bundles
        self.gate_factory = gate_factory or (lambda: (lambda: True))
        self.clock_ns = clock_ns
        self.bundle_bytes = cache.backing.bundle_bytes
        self._retiring: list[_Retiring] = []
        self._done_command = 0
        self._pending: tuple[int, int] | None = None  # (sequence, target bundles) of a shrink in progress
        self._demand_seq = 0
        self.events: list[tuple[str, int]] = []

    # ------------------------------------------------------------------ views
    @property
    def mapped_bundles(self) -> int:
        return len(self.cache.allocator.mapped_bundles()) + len(self._retiring)

    @property
    def mapped_bytes(self) -> int:
        return self.mapped_bundles * self.bundle_bytes

    def report(self, free_device_bytes: int, total_device_bytes: int) -> None:
        self.channel.publish_report(self.index, free_device_bytes, total_device_bytes, self._done_command)

    # ------------------------------------------------------------------ demand
    def publish_demand(self, missing_pages: int, deadline_ns: int = 0) -> int:
        """Asks for enough bundles to cover ``missing_pages`` beyond what is mapped; ``deadline_ns`` is
        the earliest SLO deadline among the waiting requests (0: none)."""
        ppb = self.cache.allocator.pages_per_bundle
        want_bundles = len(self.cache.allocator.mapped_bundles()) + (missing_pages + ppb - 1) // ppb
        want_bundles = min(want_bundles, self.cache.allocator.num_bundles)
        self._demand_seq += 1
        self.channel.publish_demand(self.index, self._demand_seq, want_bundles * self.bundle_bytes, deadline_ns, self.mapped_bytes)
        return want_bundles * self.bundle_bytes

    def withdraw_demand(self) -> None:
        self._demand_seq += 1
        self.channel.publish_demand(self.index, self._demand_seq, 0, 0, self.mapped_bytes)

    # ------------------------------------------------------------------ commands
    def poll(self) -> None:
        """Carries out the newest command as far as currently possible; call once per engine step."""
        self._finish_retirements()
        seq, target_bytes = self.channel.read_command(self.index)
        if seq != self._done_command and (self._pending is None or self._pending[0] != seq):
            target = max(self.floor_bundles, target_bytes // self.bundle_bytes)
            self._pending = (seq, target)
        if self._pending is None:
            return
        seq, target = self._pending
        live = len(self.cache.allocator.mapped_bundles())
        if target > live:
            # A bundle still waiting for its retirement gate is physically mapped: a command that grows past it takes it
            # back instead of mapping another one. (The daemon sends no command to a partition that owes an answer, so
            # this arises only when a command is superseded, e.g. by a restarted policy.)
            while self._retiring and live < target:
                r = self._retiring.pop()
                self.cache.allocator.publish_bundle(r.bundle)
                self.events.append(("reclaim", r.bundle))
                live += 1
            if target > live:
                retiring = {r.bundle for r in self._retiring}
                take = [b for b in self.cache.allocator.unmapped_bundles() if b not in retiring][: target - live]
                if take and vmm.grow(self.cache, take) == 0:
                    self.events.append(("grow", len(take)))
            if not self._retiring:
                self._complete(seq)   # partial growth is reported through mapped_bytes
            return
        # shrink: retire empty bundles (highest index first keeps low addresses dense)
        excess = live - target
        for b in sorted(self.retirable_empty(), reverse=True)[:max(0, excess)]:
            self.cache.allocator.begin_retirement(b)
            self._retiring.append(_Retiring(b, self.gate_factory()))
            self.events.append(("retire", b))
        self._finish_retirements()
        if len(self.cache.allocator.mapped_bundles()) <= target and not self._retiring:
            self._complete(seq)

    def _finish_retirements(self) -> None:
        still = []
        for r in self._retiring:
            if r.gate():
                self.cache.backing.unmap([r.bundle])
                self.events.append(("unmap", r.bundle))
            else:
                still.append(r)
        self._retiring = still

    def _complete(self, seq: int) -> None:
        self._done_command = seq
        self._pending = None
        self.channel.publish_completion(self.index, seq, self.mapped_bytes)

    def retirable_empty(self) -> list[int]:
        """Empty bundles a shrink may take: the floor bundles (lowest indices, the base of every KV
        tensor) stay mapped for the life of the cache."""
        return [b for b in self.cache.allocator.empty_bundles() if b >= self.floor_bundles]

    @property
    def shrink_in_progress(self) -> bool:
        return self._pending is not None

    def bundles_to_vacate(self) -> int:
        """How many more bundles must become empty for the pending shrink (the engine retracts or
        finishes sequences to get there)."""
        if self._pending is None:
            return 0
        return max(0, len(self.cache.allocator.mapped_bundles()) - self._pending[1])


def cuda_event_gate(stream=None) -> Callable[[], bool]:
    """A retirement gate that opens when everything enqueued on ``stream`` so far has finished."""
    import torch

    ev = torch.cuda.Event()
    ev.record(stream or torch.cuda.current_stream())
    return ev.query


class TpAgreedReconciler(CapacityReconciler):
    """Capacity reconciler of one rank of an attention tensor-parallel group.

    The ranks of a TP group run the same schedule without exchanging it, so everything the scheduler can see
    of the KV capacity (which bundles hand out pages) has to change in the same engine step on every rank,
    although each rank has its own partition, its own commands from the daemon and its own device memory.
    ``agree(values)`` is an all-gather over the group (every rank calls it once per :meth:`poll`, in step order;
    it returns every rank's list). With it the ranks act on a command only in a step in which *all* of them hold
    an unserved command and none still has bundles in retirement, on the smallest of their targets; a growth is
    kept only if every rank's mapping succeeded. What the scheduler cannot see stays local: unmapping behind
    the retirement gate and the completion message. A rank whose peers get no command for ``patience`` steps
    answers its own command without changing capacity, so that the daemon's policy never waits on it forever.

    The reference agrees the same decisions over a gloo group of the TP ranks
    (src/xpool/integrations/sglang/ecs/capacity.py:183-207).
    """

    def __init__(self, *args, agree: Callable[[list[int]], list[list[int]]], patience: int = 2000, **kw):
        super().__init__(*args, **kw)
        self.agree, self.patience = agree, patience
        self._agreed: tuple[int, int] | None = None   # (own command sequence, agreed target) once acted on
        self._waited = 0

    def poll(self) -> None:
        self._finish_retirements()
        seq, target_bytes = self.channel.read_command(self.index)
        if seq != self._done_command and (self._pending is None or self._pending[0] != seq):
            self._pending = (seq, max(self.floor_bundles, target_bytes // self.bundle_bytes))
            self._agreed = None
        unserved = self._pending is not None and self._agreed is None
        votes = self.agree([int(unserved), self._pending[1] if unserved else 0, len(self._retiring)])
        if unserved:
            if all(v[0] for v in votes) and not any(v[2] for v in votes):
                self._agreed = (self._pending[0], min(v[1] for v in votes))
                self._waited = 0
                self._act_on_agreement()
            else:
                self._waited += 1
                if self._waited > self.patience:     # the peers were given no command: answer, capacity unchanged
                    self.events.append(("unanswered", self._pending[0]))
                    self._waited = 0
                    self._complete(self._pending[0])
            return
        if self._agreed is not None:
            self._continue_shrink()

    def _act_on_agreement(self) -> None:
        seq, target = self._agreed
        live = len(self.cache.allocator.mapped_bundles())
        if target > live:
            take = self.cache.allocator.unmapped_bundles()[: target - live]   # nothing is retiring on any rank
            rc = self.cache.backing.try_map(take) if take else 0
            ok = all(v[0] for v in self.agree([int(rc == 0), 0, 0]))
            if ok:
                for b in take:
                    self.cache.allocator.publish_bundle(b)
                self.events.append(("grow", len(take)))
            elif rc == 0 and take:
                self.cache.backing.unmap(take)     # a peer could not map: nobody grows
            self._finish(seq)
            return
        self._continue_shrink()

    def _continue_shrink(self) -> None:
        seq, target = self._agreed
        excess = len(self.cache.allocator.mapped_bundles()) - target
        for b in sorted(self.retirable_empty(), reverse=True)[:max(0, excess)]:
            self.cache.allocator.begin_retirement(b)
            self._retiring.append(_Retiring(b, self.gate_factory()))
            self.events.append(("retire", b))
        self._finish_retirements()
        if len(self.cache.allocator.mapped_bundles()) <= target and not self._retiring:
            self._finish(seq)

    def _finish(self, seq: int) -> None:
        self._agreed = None
        self._complete(seq)

    def bundles_to_vacate(self) -> int:
        if self._agreed is None:
            return 0
        return max(0, len(self.cache.allocator.mapped_bundles()) - self._agreed[1])


def gloo_agreement(group=None) -> Callable[[list[int]], list[list[int]]]:
    """``agree`` for :class:`TpAgreedReconciler` over a ``torch.distributed`` CPU group (three integers per rank)."""
    import torch
    import torch.distributed as dist

    n = dist.get_world_size(group)

    def agree(values: list[int]) -> list[list[int]]:
        mine = torch.tensor(values, dtype=torch.int64)
        out = [torch.empty_like(mine) for _ in range(n)]
        dist.all_gather(out, mine, group=group)
        return [t.tolist() for t in out]

    return agree
