"""Instance-rank capacity reconciler against the daemon's policy over a real seqlock channel, with
the fake VMM driver: demand -> grow command -> mapping; shrink -> event-gated retirement; admission
is all-or-nothing and journalled."""
import os

import pytest

from crosspool_b200.ecs import reconciler as R
from crosspool_b200.ecs import vmm
from crosspool_b200.models import config as mc
from crosspool_b200.native.runtime import EcsChannel


def _cache(bundles=6, initial=1, quota=None):
    cfg = mc.preset("Qwen/Qwen3-0.6B")
    ppb, _ = vmm.bundle_geometry(cfg, 16)
    drv = vmm.Driver.fake(1 << 40)
    cache = vmm.elastic_kv_cache(cfg, max_pages=bundles * ppb, page_size=16, device="cpu", driver=drv, quota=quota,
                                 initial_bundles=initial, make_tensors=False)
    return cache, ppb, drv


@pytest.fixture
def channel():
    ch = EcsChannel.create(f"/xp-test-recon-{os.getpid()}", 1, 2, 1)
    yield ch
    ch.close()


def test_demand_then_grow_command_maps_bundles_and_reports_completion(channel):
    cache, ppb, drv = _cache()
    rec = R.CapacityReconciler(cache, channel, 0)
    bb = rec.bundle_bytes
    d = R.admit(cache, [(1, 16 * ppb), (2, 16 * 10)])            # needs ppb + 10 pages, one bundle mapped
    assert not d.admitted and d.missing_pages == 10 and cache.tables == {}
    assert rec.publish_demand(d.missing_pages, deadline_ns=123) == 2 * bb
    assert channel.read_demand(0) == (1, 2 * bb, 123, bb)
    rec.poll()                                                      # no command yet: nothing happens
    assert rec.mapped_bundles == 1
    channel.publish_command(0, 1, 3 * bb)                           # the daemon grants more than asked
    rec.poll()
    assert rec.mapped_bundles == 3 and channel.read_completion(0) == (1, 3 * bb)
    assert R.admit(cache, [(1, 16 * ppb), (2, 16 * 10)]).admitted
    rec.poll()                                                      # same command again: idempotent
    assert rec.mapped_bundles == 3 and drv.counts()["allocated_bytes"] == 3 * bb


def test_shrink_waits_for_empty_bundles_and_for_the_retirement_gate(channel):
    cache, ppb, drv = _cache(initial=4)
    gates = []

    def gate_factory():
        g = {"open": False}
        gates.append(g)
        return lambda: g["open"]

    rec = R.CapacityReconciler(cache, channel, 1, gate_factory=gate_factory)
    bb = rec.bundle_bytes
    assert R.admit(cache, [(1, 16 * ppb), (2, 16 * ppb)]).admitted  # two bundles full, two empty
    channel.publish_command(1, 5, 1 * bb)                           # shrink to one bundle
    rec.poll()
    assert [e for e in rec.events if e[0] == "retire"] == [("retire", 3), ("retire", 2)]
    assert rec.mapped_bundles == 4 and rec.shrink_in_progress      # gates closed: memory still mapped
    assert channel.read_completion(1) == (0, 0) and rec.bundles_to_vacate() == 1
    with pytest.raises(Exception):
        cache.ensure(3, 16 * ppb)                                   # retiring bundles hand out nothing
    for g in gates:
        g["open"] = True
    rec.poll()
    assert rec.mapped_bundles == 2 and drv.counts()["allocated_bytes"] == 2 * bb
    assert rec.shrink_in_progress                                   # one more bundle must drain first
    cache.release(2)                                                # the engine finished / retracted a sequence
    rec.poll()
    gates[-1]["open"] = True
    rec.poll()
    assert rec.mapped_bundles == 1 and not rec.shrink_in_progress
    assert channel.read_completion(1) == (5, 1 * bb)
    channel.publish_command(1, 6, 0)                                # never below the floor
    rec.poll()
    assert rec.mapped_bundles == 1 and channel.read_completion(1) == (6, bb)


def test_growth_stops_at_the_shared_quota_and_reports_what_was_mapped(channel):
    q = vmm.MemoryQuota(0)
    cache, ppb, drv = _cache(initial=0, quota=q)
    rec = R.CapacityReconciler(cache, channel, 0, floor_bundles=0)
    q.set_limit(2 * rec.bundle_bytes)
    channel.publish_command(0, 1, 4 * rec.bundle_bytes)
    rec.poll()
    assert rec.mapped_bundles == 0 and channel.read_completion(0) == (1, 0)   # a 4-bundle map is refused whole
    channel.publish_command(0, 2, 2 * rec.bundle_bytes)
    rec.poll()
    assert rec.mapped_bundles == 2 and q.charged == 2 * rec.bundle_bytes


def test_journal_rolls_back_partial_allocations():
    cache, ppb, _ = _cache(initial=1)
    cache.ensure(7, 16 * 4)
    j = R.AllocationJournal(cache)
    j.ensure(7, 16 * 9)
    j.ensure(8, 16 * 3)
    assert len(cache.tables[7]) == 9 and cache.allocator.free_pages == ppb - 12
    j.rollback()
    assert len(cache.tables[7]) == 4 and 8 not in cache.tables and cache.allocator.free_pages == ppb - 4
    assert not R.admit(cache, [(9, 16 * 10)], reserve_pages=ppb - 8).admitted


def test_policy_and_two_reconcilers_move_memory_from_the_idle_partition_to_the_busy_one(channel):
    """The daemon's policy and two Instance ranks on one device, all over the real channel."""
    from crosspool_b200.service.daemon.ecs import CapacityPolicy, Partition

    q = vmm.MemoryQuota(1 << 40)
    a, ppb, _ = _cache(bundles=6, initial=1, quota=q)
    b, _, _ = _cache(bundles=6, initial=1, quota=q)
    ra, rb = R.CapacityReconciler(a, channel, 0), R.CapacityReconciler(b, channel, 1)
    bb = ra.bundle_bytes
    parts = [Partition(i, f"m{i}:0", device=0, floor_bytes=bb, reservation_bytes=6 * bb, bundle_bytes=bb, mapped_bytes=bb)
             for i in (0, 1)]
    pol = CapacityPolicy(channel, parts, {0: 0}, utilization=1.0)
    channel.publish_report(0, 5 * bb, 100 * bb, 0)        # 5 free + 2 mapped = a 7-bundle budget
    pol.freeze_pools()                                     # floors 1+1, spare 5 -> 2 extra each, 1 unassigned
    for r in (ra, rb):
        r.poll()
    assert (ra.mapped_bundles, rb.mapped_bundles) == (3, 3)
    # A fills up and needs 3 more bundles; B is idle
    assert R.admit(a, [(1, 16 * ppb * 3)]).admitted
    d = R.admit(a, [(2, 16 * ppb * 3)])
    assert not d.admitted
    ra.publish_demand(d.missing_pages)
    for _ in range(12):
        pol.tick()
        ra.poll()
        rb.poll()
    assert ra.mapped_bundles == 6 and rb.mapped_bundles == 1
    assert R.admit(a, [(2, 16 * ppb * 3)]).admitted
    kinds = [e.kind for e in pol.events]
    assert "grow" in kinds and "shrink" in kinds
    assert q.charged == 7 * bb


class _LockstepAgreement:
    """All-gather between reconcilers driven from one thread each (stands in for the gloo group)."""

    def __init__(self, n):
        import threading

        self.n, self.slots, self.barrier = n, [None] * n, threading.Barrier(n)

    def for_rank(self, r):
        def agree(values):
            self.slots[r] = list(values)
            self.barrier.wait(10)
            out = [list(v) for v in self.slots]
            self.barrier.wait(10)
            return out
        return agree


def test_tp_ranks_change_capacity_in_the_same_step_on_the_smallest_target():
    import threading

    ch = EcsChannel.create(f"/xp-test-recon-tp-{os.getpid()}", 1, 2, 1)
    try:
        ag = _LockstepAgreement(2)
        caches = [_cache(initial=1) for _ in range(2)]
        recs = [R.TpAgreedReconciler(c[0], ch, i, agree=ag.for_rank(i), patience=3) for i, c in enumerate(caches)]
        bb, ppb = recs[0].bundle_bytes, caches[0][1]
        history = [[], []]

        def steps(n):
            def run(i):
                for _ in range(n):
                    recs[i].poll()
                    history[i].append(len(caches[i][0].allocator.mapped_bundles()))
            ts = [threading.Thread(target=run, args=(i,)) for i in range(2)]
            for t in ts:
                t.start()
            for t in ts:
                t.join(20)
                assert not t.is_alive()

        ch.publish_command(0, 1, 4 * bb)                 # only rank 0 has its command yet
        steps(2)
        assert history == [[1, 1], [1, 1]]
        ch.publish_command(1, 1, 3 * bb)                 # rank 1 is granted less: both grow to 3, in the same step
        steps(1)
        assert history[0][-1] == history[1][-1] == 3
        assert ch.read_completion(0) == (1, 3 * bb) and ch.read_completion(1) == (1, 3 * bb)
        for c, _, _ in caches:                            # identical allocations on both ranks
            assert R.admit(c, [(1, 16 * ppb), (2, 16 * ppb)]).admitted
        ch.publish_command(0, 2, 1 * bb)
        ch.publish_command(1, 2, 2 * bb)                 # shrink: the smaller target (1) on both, one bundle is free now
        steps(1)
        assert history[0][-1] == history[1][-1] == 2 and all(r.bundles_to_vacate() == 1 for r in recs)
        for c, _, _ in caches:
            c.release(2)
        steps(2)
        assert history[0][-1] == history[1][-1] == 1
        assert ch.read_completion(0) == (2, bb) and ch.read_completion(1) == (2, bb)
        ch.publish_command(0, 3, 2 * bb)                 # a command that the peer never receives is answered unchanged
        steps(5)
        assert history[0][-1] == history[1][-1] == 1 and ch.read_completion(0) == (3, bb)
        assert ("unanswered", 3) in recs[0].events
        assert history[0] == history[1]
    finally:
        ch.close()
