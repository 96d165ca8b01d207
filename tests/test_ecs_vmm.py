"""Elastic KV backing: ledger, rollback on out-of-memory, stable addresses, allocator coupling.
The driver is a book-keeping fake (no GPU); failures are injected on the host."""
import pytest

from crosspool_b200.ecs import vmm
from crosspool_b200.engine.kv_cache import OutOfPages
from crosspool_b200.models import config as mc

MB = 1 << 20


def _backing(budget=64 * MB, quota=None, buffers=4, bundles=8, chunk=2 * MB):
    drv = vmm.Driver.fake(budget)
    return drv, vmm.KvVmmBacking(drv, 0, buffers, bundles * chunk, chunk, quota)


def test_addresses_are_stable_and_bundles_map_all_buffers():
    drv, b = _backing()
    addrs = [b.address(i) for i in range(4)]
    assert addrs == sorted(addrs) and addrs[1] - addrs[0] == 16 * MB
    assert b.bundle_count == 8 and b.bundle_bytes == 8 * MB and b.mapped_bytes == 0
    assert b.try_map([0, 3]) == 0
    assert b.is_mapped(0) and b.is_mapped(3) and not b.is_mapped(1)
    assert b.mapped_bytes == 16 * MB and drv.counts()["creates"] == 8 and drv.counts()["maps"] == 8
    assert [b.address(i) for i in range(4)] == addrs  # mapping never moves a buffer
    assert b.try_map([3]) == 0 and drv.counts()["creates"] == 8  # idempotent
    assert b.unmap([0, 5]) == 1 and b.mapped_bytes == 8 * MB
    c = drv.counts()
    assert c["releases"] == 4 and c["unmaps"] == 4 and c["allocated_bytes"] == 8 * MB


def test_driver_out_of_memory_rolls_back_the_whole_call():
    drv, b = _backing(budget=20 * MB)  # room for two bundles of 8 MB, not three
    assert b.try_map([0, 1, 2]) == vmm.OUT_OF_MEMORY
    c = drv.counts()
    assert b.mapped_bytes == 0 and c["allocated_bytes"] == 0 and c["live"] == 0
    assert not any(b.is_mapped(i) for i in range(3))
    assert b.try_map([0, 1]) == 0 and b.mapped_bytes == 16 * MB


def test_failure_in_the_middle_of_a_bundle_releases_its_partial_allocations():
    drv, b = _backing()
    drv.inject(fail_create_after=2)  # third cuMemCreate of the bundle fails
    assert b.try_map([4]) == vmm.OUT_OF_MEMORY
    assert drv.counts()["live"] == 0 and not b.is_mapped(4)
    drv.inject(fail_map_after=1)     # second cuMemMap fails with a non-OOM driver error
    assert b.try_map([4]) == 999
    assert drv.counts()["live"] == 0 and drv.counts()["allocated_bytes"] == 0
    assert b.try_map([4]) == 0


def test_shared_quota_is_charged_refunded_and_enforced_across_instances():
    q = vmm.MemoryQuota(24 * MB)
    drv = vmm.Driver.fake(1 << 30)
    a = vmm.KvVmmBacking(drv, 0, 4, 16 * MB, 2 * MB, q)
    b = vmm.KvVmmBacking(drv, 0, 4, 16 * MB, 2 * MB, q)
    assert a.try_map([0, 1]) == 0 and q.charged == 16 * MB
    assert b.try_map([0, 1]) == vmm.QUOTA_EXCEEDED  # the second bundle does not fit: nothing stays
    assert q.charged == 16 * MB and b.mapped_bytes == 0
    assert b.try_map([0]) == 0 and q.charged == 24 * MB
    a.unmap([1])
    assert q.charged == 16 * MB
    q.set_limit(8 * MB)   # the policy lowered the limit: existing mappings stay, growth is refused
    assert b.try_map([1]) == vmm.QUOTA_EXCEEDED


def test_allocator_only_hands_out_pages_of_mapped_bundles_and_retires_empty_ones():
    cfg = mc.preset("Qwen/Qwen3-0.6B")
    ppb, chunk = vmm.bundle_geometry(cfg, 16)
    assert chunk % (2 * MB) == 0 and ppb == 64
    q = vmm.MemoryQuota(1 << 40)
    drv = vmm.Driver.fake(1 << 40)
    cache = vmm.elastic_kv_cache(cfg, max_pages=4 * ppb, page_size=16, device="cpu", driver=drv, quota=q,
                                 initial_bundles=1, make_tensors=False)
    al = cache.allocator
    assert al.free_pages == ppb and al.mapped_bundles() == [0]
    cache.ensure(1, 16 * ppb)  # exactly one bundle of tokens
    with pytest.raises(OutOfPages):
        cache.ensure(2, 16)
    assert vmm.grow(cache, [1, 2]) == 0 and al.free_pages == 2 * ppb
    cache.ensure(2, 16 * 3)
    assert all(p // ppb == 1 for p in cache.tables[2])  # the fullest non-full bundle is used first
    assert al.empty_bundles() == [2]
    al.begin_retirement(2)
    assert cache.backing.unmap([2]) == 1 and al.mapped_bundles() == [0, 1]
    with pytest.raises(ValueError):
        al.begin_retirement(1)  # still holds pages of sequence 2
    cache.release(2)
    assert al.empty_bundles() == [1]
    assert q.charged == 2 * cache.backing.bundle_bytes


def test_partition_geometry_states_floor_and_reservation_and_refuses_impossible_shapes():
    import os

    import pytest

    from crosspool_b200.ecs import vmm
    from crosspool_b200.ecs.profile import KvPartitionGeometry
    from crosspool_b200.models import config as mc
    from crosspool_b200.native.runtime import EcsChannel

    g = KvPartitionGeometry(bundle_bytes=4096, bundles=10, floor_bundles=2)
    assert (g.floor_bytes, g.reservation_bytes) == (8192, 40960)
    assert [g.whole_bundles(n) for n in (0, 4095, 12288, 12289, 1 << 30)] == [2, 2, 3, 3, 10]
    for bad in (dict(bundle_bytes=0, bundles=1), dict(bundle_bytes=1, bundles=0), dict(bundle_bytes=1, bundles=1, floor_bundles=2)):
        with pytest.raises(ValueError):
            KvPartitionGeometry(**bad)
    with pytest.raises(OverflowError):
        KvPartitionGeometry(bundle_bytes=1 << 40, bundles=1 << 40)
    cfg = mc.preset("tiny-qwen3")
    cache = vmm.elastic_kv_cache(cfg, 32, 16, "cpu", vmm.Driver.fake(1 << 30, granularity=16 << 10), None, initial_bundles=1,
                                 make_tensors=False, granularity=16 << 10)
    got = KvPartitionGeometry.of(cache)
    assert got.bundle_bytes == cache.backing.bundle_bytes == 4 * (16 << 10) and got.bundles == 8
    ch = EcsChannel.create(f"/xp-geo-{os.getpid()}", 1, 1, 1)
    try:
        got.describe(ch, 0, device=3, rank=1)
        assert ch.partition(0) == dict(device=3, group=0, rank=1, floor_bytes=got.floor_bytes, reservation_bytes=got.reservation_bytes)
    finally:
        ch.close()
        cache.backing.close()
