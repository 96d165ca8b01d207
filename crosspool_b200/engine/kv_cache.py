"""Paged KV cache of one Instance on one attention device.

Logical layer: fixed-size pages handed out by :class:`PageAllocator`; a sequence owns a list of
pages (its block table row). Physical layer: per-layer K and V buffers ``[pages, page_size,
kv_heads, head_dim]`` that are either ordinary device tensors (fixed capacity) or views over CUDA
VMM address ranges whose physical backing is mapped and unmapped in *bundles*
(:mod:`crosspool_b200.ecs.vmm`), so that co-located Instances can lend each other memory while the
tensors' addresses — and therefore captured CUDA graphs — stay valid. The allocator only hands out
pages whose bundle is mapped, like the reference's ``ElasticPageAllocator``
(src/xpool/integrations/sglang/ecs/allocator.py:61-104).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..models.config import ModelConfig


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    """Free-list allocator over page ids; pages become available bundle by bundle."""

    def __init__(self, total_pages: int, pages_per_bundle: int | None = None, mapped_bundles: int | None = None):
        self.total_pages = total_pages
        self.pages_per_bundle = pages_per_bundle or total_pages
        self.num_bundles = (total_pages + self.pages_per_bundle - 1) // self.pages_per_bundle
        self._free: list[list[int]] = [[] for _ in range(self.num_bundles)]
        self._mapped = [False] * self.num_bundles
        self._used_in_bundle = [0] * self.num_bundles
        n = self.num_bundles if mapped_bundles is None else mapped_bundles
        for b in range(n):
            self.publish_bundle(b)

    # -- physical backing events -------------------------------------------------------------
    def bundle_pages(self, b: int) -> range:
        return range(b * self.pages_per_bundle, min((b + 1) * self.pages_per_bundle, self.total_pages))

    def publish_bundle(self, b: int) -> None:
        """The bundle's memory is mapped: its pages may be handed out."""
        assert not self._mapped[b]
        self._mapped[b] = True
        self._free[b] = list(reversed(self.bundle_pages(b)))
        self._used_in_bundle[b] = 0

    def empty_bundles(self) -> list[int]:
        return [b for b in range(self.num_bundles) if self._mapped[b] and self._used_in_bundle[b] == 0]

    def begin_retirement(self, b: int) -> None:
        """Takes an empty bundle out of circulation (it may be unmapped once in-flight work that
        could still read it has finished)."""
        if not self._mapped[b] or self._used_in_bundle[b] != 0:
            raise ValueError(f"bundle {b} is not an empty mapped bundle")
        self._mapped[b] = False
        self._free[b] = []

    def mapped_bundles(self) -> list[int]:
        return [b for b in range(self.num_bundles) if self._mapped[b]]

    def used_in_bundle(self, b: int) -> int:
        return self._used_in_bundle[b]

    def unmapped_bundles(self) -> list[int]:
        return [b for b in range(self.num_bundles) if not self._mapped[b]]

    # -- page hand-out -----------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return sum(len(f) for f in self._free)

    @property
    def mapped_pages(self) -> int:
        return sum(len(self.bundle_pages(b)) for b in range(self.num_bundles) if self._mapped[b])

    def alloc(self, n: int) -> list[int]:
        if n > self.free_pages:
            raise OutOfPages(f"need {n} pages, {self.free_pages} free")
        out: list[int] = []
        # fill the fullest bundles first so that lightly used ones drain and can be lent away
        order = sorted((b for b in range(self.num_bundles) if self._free[b]),
                       key=lambda b: (-self._used_in_bundle[b], b))
        for b in order:
            while self._free[b] and len(out) < n:
                out.append(self._free[b].pop())
                self._used_in_bundle[b] += 1
            if len(out) == n:
                break
        return out

    def free(self, pages: list[int]) -> None:
        for p in pages:
            b = p // self.pages_per_bundle
            self._used_in_bundle[b] -= 1
            if self._mapped[b]:
                self._free[b].append(p)


@dataclass
class KvLayout:
    page_size: int
    num_pages: int
    kv_heads: int
    head_dim: int
    num_layers: int
    elem_bytes: int = 2

    @property
    def page_bytes_per_buffer(self) -> int:
        return self.page_size * self.kv_heads * self.head_dim * self.elem_bytes

    @property
    def buffer_bytes(self) -> int:
        return self.num_pages * self.page_bytes_per_buffer

    @property
    def bytes_per_page_all_layers(self) -> int:
        return 2 * self.num_layers * self.page_bytes_per_buffer


@dataclass
class PagedKvCache:
    layout: KvLayout
    k: list[torch.Tensor]
    v: list[torch.Tensor]
    allocator: PageAllocator
    backing: object | None = None  # ecs.vmm.KvVmmBacking when elastic
    tables: dict[int, list[int]] = field(default_factory=dict)

    @classmethod
    def fixed(cls, cfg: ModelConfig, num_pages: int, page_size: int = 16, device="cuda",
              dtype: torch.dtype = torch.bfloat16) -> "PagedKvCache":
        lay = KvLayout(page_size, num_pages, cfg.num_kv_heads, cfg.head_dim, cfg.num_layers, dtype.itemsize)
        shape = (num_pages, page_size, cfg.num_kv_heads, cfg.head_dim)
        k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(cfg.num_layers)]
        return cls(lay, k, v, PageAllocator(num_pages))

    # -- per-sequence page tables --------------------------------------------------------------
    def pages_needed(self, seq_id: int, new_len: int) -> int:
        have = len(self.tables.get(seq_id, ()))
        need = (new_len + self.layout.page_size - 1) // self.layout.page_size
        return max(0, need - have)

    def ensure(self, seq_id: int, new_len: int) -> list[int]:
        """Grows the sequence's table to cover ``new_len`` tokens."""
        n = self.pages_needed(seq_id, new_len)
        t = self.tables.setdefault(seq_id, [])
        if n:
            t.extend(self.allocator.alloc(n))
        return t

    def release(self, seq_id: int) -> None:
        t = self.tables.pop(seq_id, None)
        if t:
            self.allocator.free(t)

    def slot(self, seq_id: int, pos: int) -> int:
        t = self.tables[seq_id]
        return t[pos // self.layout.page_size] * self.layout.page_size + pos % self.layout.page_size
