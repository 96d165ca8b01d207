"""Physical geometry of an Instance rank's elastic KV: what one bundle costs, how many there can be, how many stay.

A *pool* is one elastic backing (here: the K and V buffers of all layers of one KV cache, grown and shrunk together one
bundle at a time). The profile is what the rank tells the daemon when it describes its partition: the floor it never
gives up and the reservation it can never exceed. It holds no residency state; that lives in the page allocator and
the backing. Reference: src/xpool/ecs.py (``PoolProfile``, ``ElasticContextStateProfile``).
"""

from __future__ import annotations

from dataclasses import dataclass

from ..utils.integer import ensure_uint64


@dataclass(frozen=True)
class PoolProfile:
    bundle_bytes: int        # physical cost of one bundle over all buffers of the pool
    bundle_capacity: int     # bundles the address range can hold (the reservation)
    floor_bundles: int       # bundles that stay mapped for the life of the cache

    def __post_init__(self):
        ensure_uint64(self.bundle_bytes, self.bundle_capacity, self.floor_bundles)
        if self.bundle_bytes == 0 or self.floor_bundles > self.bundle_capacity:
            raise ValueError("a pool needs a positive bundle size and a floor inside its reservation")
        ensure_uint64(self.bundle_bytes * self.bundle_capacity)

    def bytes_for(self, bundles: int) -> int:
        ensure_uint64(bundles)
        if bundles > self.bundle_capacity:
            raise ValueError(f"{bundles} bundles exceed the pool's reservation of {self.bundle_capacity}")
        return bundles * self.bundle_bytes


@dataclass(frozen=True)
class ElasticKvProfile:
    pools: tuple[PoolProfile, ...]

    def __post_init__(self):
        if not isinstance(self.pools, tuple):
            raise ValueError("pools must be a tuple")
        ensure_uint64(self.floor_bytes, self.reservation_bytes)

    @property
    def floor_bytes(self) -> int:
        return sum(p.floor_bundles * p.bundle_bytes for p in self.pools)

    @property
    def reservation_bytes(self) -> int:
        return sum(p.bundle_capacity * p.bundle_bytes for p in self.pools)


def profile_of(cache, floor_bundles: int = 1) -> ElasticKvProfile:
    """The profile of an elastic ``PagedKvCache`` (``ecs/vmm.py::elastic_kv_cache``): one pool."""
    if cache.backing is None:
        raise ValueError("the KV cache has no elastic backing")
    return ElasticKvProfile((PoolProfile(cache.backing.bundle_bytes, cache.backing.bundle_count, floor_bundles),))
