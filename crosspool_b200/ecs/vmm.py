"""Python face of the native elastic KV backing (``csrc/include/xpool/kv_vmm.hpp``).

``KvVmmBacking`` reserves one virtual range per KV buffer and maps physical memory bundle by bundle
against a shared :class:`MemoryQuota`; ``elastic_kv_cache`` builds a :class:`PagedKvCache` whose
tensors view those ranges and whose allocator only hands out pages of mapped bundles. The driver is
injectable: ``Driver.real()`` resolves the CUDA driver, ``Driver.fake(budget)`` keeps books only
(CPU tests, including out-of-memory and rollback paths).
"""

from __future__ import annotations

import ctypes as C

import torch

from ..engine.kv_cache import KvLayout, PageAllocator, PagedKvCache
from ..models.config import ModelConfig
from ..native import runtime as rt

OUT_OF_MEMORY = 2
QUOTA_EXCEEDED = -2

u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p


def _lib():
    L = rt.lib()
    if not getattr(L, "_vmm_declared", False):
        sig = {
            "xr_vmm_fake_driver_create": (vp, [u64, u64]), "xr_vmm_fake_driver_destroy": (None, [vp]),
            "xr_vmm_fake_driver_inject": (None, [vp, C.c_int, C.c_int]),
            "xr_vmm_fake_driver_counts": (None, [vp, C.POINTER(u64)]), "xr_vmm_fake_driver_api": (None, [vp, vp]),
            "xr_vmm_driver_api_bytes": (u64, []),
            "xr_vmm_quota_create": (vp, [u64]), "xr_vmm_quota_destroy": (None, [vp]),
            "xr_vmm_quota_set_limit": (None, [vp, u64]), "xr_vmm_quota_get": (None, [vp, C.POINTER(u64)]),
            "xr_vmm_backing_create": (vp, [vp, C.c_int, u32, u64, u64, vp]), "xr_vmm_backing_destroy": (None, [vp]),
            "xr_vmm_backing_reserve": (C.c_int, [vp]), "xr_vmm_backing_address": (u64, [vp, u32]),
            "xr_vmm_backing_info": (None, [vp, C.POINTER(u64)]), "xr_vmm_backing_is_mapped": (C.c_int, [vp, u32]),
            "xr_vmm_backing_try_map": (C.c_int, [vp, C.POINTER(u32), u32]),
            "xr_vmm_backing_unmap": (u32, [vp, C.POINTER(u32), u32]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        L._vmm_declared = True
    return L


class Driver:
    """A VMM driver function table (real CUDA driver or the book-keeping fake)."""

    def __init__(self, table: C.Array, fake_handle=None):
        self.table, self._fake = table, fake_handle

    @classmethod
    def real(cls) -> "Driver":
        from .. import native

        L = _lib()
        buf = (C.c_uint8 * L.xr_vmm_driver_api_bytes())()
        k = native.kernels()
        k.xp_vmm_driver_api.restype = None
        k.xp_vmm_driver_api.argtypes = [vp]
        k.xp_vmm_driver_api(buf)
        return cls(buf)

    @classmethod
    def fake(cls, budget_bytes: int, granularity: int = 2 << 20) -> "Driver":
        L = _lib()
        h = L.xr_vmm_fake_driver_create(budget_bytes, granularity)
        buf = (C.c_uint8 * L.xr_vmm_driver_api_bytes())()
        L.xr_vmm_fake_driver_api(h, buf)
        return cls(buf, h)

    def inject(self, fail_create_after: int = -1, fail_map_after: int = -1) -> None:
        _lib().xr_vmm_fake_driver_inject(self._fake, fail_create_after, fail_map_after)

    def counts(self) -> dict:
        out = (u64 * 6)()
        _lib().xr_vmm_fake_driver_counts(self._fake, out)
        return dict(zip(("creates", "releases", "maps", "unmaps", "allocated_bytes", "live"), out))


class MemoryQuota:
    """Limit/charged ledger shared by co-located Instances (reference: src/xpool/ecs.py ``MemoryQuota``)."""

    def __init__(self, limit_bytes: int):
        self._h = _lib().xr_vmm_quota_create(limit_bytes)

    def set_limit(self, limit_bytes: int) -> None:
        _lib().xr_vmm_quota_set_limit(self._h, limit_bytes)

    @property
    def limit(self) -> int:
        return self._get()[0]

    @property
    def charged(self) -> int:
        return self._get()[1]

    def _get(self):
        out = (u64 * 2)()
        _lib().xr_vmm_quota_get(self._h, out)
        return out[0], out[1]


class KvVmmBacking:
    def __init__(self, driver: Driver, device: int, n_buffers: int, buffer_bytes: int, chunk_bytes: int,
                 quota: MemoryQuota | None):
        self.driver, self.quota = driver, quota
        self._h = _lib().xr_vmm_backing_create(driver.table, device, n_buffers, buffer_bytes, chunk_bytes,
                                               quota._h if quota else None)
        if not self._h:
            raise ValueError("invalid KV backing geometry")
        rc = _lib().xr_vmm_backing_reserve(self._h)
        if rc != 0:
            raise RuntimeError(f"address reservation failed with driver code {rc}")

    def close(self) -> None:
        if self._h:
            _lib().xr_vmm_backing_destroy(self._h)
            self._h = None

    def address(self, buffer: int) -> int:
        return _lib().xr_vmm_backing_address(self._h, buffer)

    def _info(self):
        out = (u64 * 3)()
        _lib().xr_vmm_backing_info(self._h, out)
        return out[0], out[1], out[2]

    @property
    def bundle_count(self) -> int:
        return self._info()[0]

    @property
    def bundle_bytes(self) -> int:
        return self._info()[1]

    @property
    def mapped_bytes(self) -> int:
        return self._info()[2]

    def is_mapped(self, bundle: int) -> bool:
        return bool(_lib().xr_vmm_backing_is_mapped(self._h, bundle))

    def try_map(self, bundles: list[int]) -> int:
        """0, ``OUT_OF_MEMORY``, ``QUOTA_EXCEEDED`` or another driver code; all-or-nothing."""
        arr = (u32 * len(bundles))(*bundles)
        return _lib().xr_vmm_backing_try_map(self._h, arr, len(bundles))

    def unmap(self, bundles: list[int]) -> int:
        arr = (u32 * len(bundles))(*bundles)
        return _lib().xr_vmm_backing_unmap(self._h, arr, len(bundles))


def bundle_geometry(cfg: ModelConfig, page_size: int, granularity: int = 2 << 20, elem_bytes: int = 2) -> tuple[int, int]:
    """(pages per bundle, chunk bytes per buffer): the smallest page count whose per-buffer bytes are a
    whole number of allocation granules."""
    page_bytes = page_size * cfg.num_kv_heads * cfg.head_dim * elem_bytes
    pages = 1
    while (pages * page_bytes) % granularity:
        pages += 1
    return pages, pages * page_bytes


def elastic_kv_cache(cfg: ModelConfig, max_pages: int, page_size: int, device, driver: Driver,
                     quota: MemoryQuota | None, initial_bundles: int = 0, make_tensors: bool = True,
                     granularity: int = 2 << 20) -> PagedKvCache:
    """A paged KV cache over VMM ranges. ``make_tensors=False`` (CPU tests with the fake driver) leaves
    the tensor lists empty; addresses are still reserved and mapped. ``granularity``: bytes of one physical
    allocation per buffer and bundle (a multiple of the driver's 2 MiB granule); larger values move memory with
    fewer driver calls per byte at the price of coarser lending."""
    from ..parallel.fabric import tensor_from_ptr

    dev_index = torch.device(device).index or 0
    ppb, chunk = bundle_geometry(cfg, page_size, granularity)
    n_bundles = (max_pages + ppb - 1) // ppb
    pages = n_bundles * ppb
    backing = KvVmmBacking(driver, dev_index, 2 * cfg.num_layers, n_bundles * chunk, chunk, quota)
    lay = KvLayout(page_size, pages, cfg.num_kv_heads, cfg.head_dim, cfg.num_layers)
    alloc = PageAllocator(pages, ppb, mapped_bundles=0)
    cache = PagedKvCache(lay, [], [], alloc, backing)
    if initial_bundles:
        grow(cache, list(range(initial_bundles)))
    if make_tensors:
        # views are created after the first bundles are mapped: the framework inspects the base
        # address of foreign memory when it wraps it
        if not backing.is_mapped(0):
            raise ValueError("bundle 0 must be mapped before tensors are created over the range")
        shape = (pages, page_size, cfg.num_kv_heads, cfg.head_dim)
        for l in range(cfg.num_layers):
            cache.k.append(tensor_from_ptr(backing.address(2 * l), shape, torch.bfloat16, device))
            cache.v.append(tensor_from_ptr(backing.address(2 * l + 1), shape, torch.bfloat16, device))
    return cache


def grow(cache: PagedKvCache, bundles: list[int]) -> int:
    """Maps bundles and publishes their pages to the allocator. Returns the driver/quota code."""
    rc = cache.backing.try_map(bundles)
    if rc == 0:
        for b in bundles:
            if b not in cache.allocator.mapped_bundles():
                cache.allocator.publish_bundle(b)
    return rc
