"""What an Instance rank tells the daemon about its elastic KV before the capacity policy starts: how large one bundle
is, how many bundles its address range can ever hold, and how many it never gives up.

In this repository an Instance rank has exactly one elastic backing (the K and V buffers of all layers of its KV cache
grow and shrink together, one bundle at a time), so the geometry is one record; the reference describes a tuple of
pools per rank (src/xpool/ecs.py, ``ElasticContextStateProfile``). The record holds no residency state: which bundles
are mapped is the page allocator's and the backing's business.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..utils.integer import ensure_uint32, ensure_uint64


@dataclass(frozen=True)
class KvPartitionGeometry:
    bundle_bytes: int
    bundles: int
    floor_bundles: int = 1

    def __post_init__(self):
        ensure_uint64(self.bundle_bytes, self.bundles, self.floor_bundles, self.bundle_bytes * self.bundles)
        if self.bundle_bytes == 0 or self.bundles == 0:
            raise ValueError("an elastic KV partition needs at least one bundle of at least one byte")
        if self.floor_bundles > self.bundles:
            raise ValueError(f"a floor of {self.floor_bundles} bundles does not fit a range of {self.bundles}")

    @classmethod
    def of(cls, cache, floor_bundles: int = 1) -> "KvPartitionGeometry":
        """Geometry of an elastic ``PagedKvCache`` (``ecs/vmm.py::elastic_kv_cache``)."""
        if cache.backing is None:
            raise ValueError("the KV cache has no elastic backing")
        return cls(cache.backing.bundle_bytes, cache.backing.bundle_count, floor_bundles)

    @property
    def floor_bytes(self) -> int:
        return self.floor_bundles * self.bundle_bytes

    @property
    def reservation_bytes(self) -> int:
        return self.bundles * self.bundle_bytes

    def whole_bundles(self, nbytes: int) -> int:
        """Bundles a byte target pays for, kept between the floor and the range."""
        ensure_uint64(nbytes)
        return max(self.floor_bundles, min(self.bundles, nbytes // self.bundle_bytes))

    def describe(self, channel, index: int, device: int, rank: int, group: int = 0) -> None:
        """Writes the partition's description into the control channel; the policy freezes the device pools once
        every partition of the generation has one."""
        ensure_uint32(index, device, rank, group)
        channel.set_partition(index, device, group, rank, self.floor_bytes, self.reservation_bytes)
