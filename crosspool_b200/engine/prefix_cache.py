"""Page-granular prefix cache of one Instance.

Full KV pages of finished prompt prefixes stay resident and are shared, read-only, by later
requests that start with the same tokens: the request's block table begins with the cached pages and
its prefill starts behind them. The structure is a trie whose edges are the token tuples of one page
(``page_size`` tokens); a node owns one page of the paged KV cache. Pages referenced by running
sequences are pinned; unreferenced leaves are evicted least-recently-used first when the allocator
runs dry. (The reference delegates this to its serving engine's radix cache and only couples it to the
elastic pools, src/xpool/integrations/sglang/ecs/state.py; here the engine is ours, so the cache is too.)
"""

from __future__ import annotations

import itertools
from dataclasses import dataclass, field


@dataclass
class _Node:
    page: int
    parent: "_Node | None"
    key: tuple[int, ...] = ()
    children: dict[tuple[int, ...], "_Node"] = field(default_factory=dict)
    refs: int = 0
    last_used: int = 0


class PrefixCache:
    def __init__(self, page_size: int):
        self.page_size = page_size
        self.root = _Node(-1, None)
        self._clock = itertools.count(1)
        self._by_page: dict[int, _Node] = {}
        self.hits = self.lookups = self.hit_tokens = 0
        self.evicted_for_retirement = 0

    def __len__(self) -> int:
        return len(self._by_page)

    def owns(self, page: int) -> bool:
        return page in self._by_page

    def _pages(self, tokens: list[int], limit: int):
        ps = self.page_size
        for i in range(0, limit - limit % ps, ps):
            yield tuple(tokens[i:i + ps])

    def match(self, tokens: list[int]) -> list[int]:
        """Pages of the longest cached prefix, leaving at least one token to compute; every returned
        page is pinned until :meth:`release` is called with it."""
        self.lookups += 1
        node, out, now = self.root, [], next(self._clock)
        for key in self._pages(tokens, len(tokens) - 1):
            nxt = node.children.get(key)
            if nxt is None:
                break
            nxt.refs += 1
            nxt.last_used = now
            out.append(nxt.page)
            node = nxt
        if out:
            self.hits += 1
            self.hit_tokens += len(out) * self.page_size
        return out

    def insert(self, tokens: list[int], pages: list[int]) -> list[int]:
        """Registers the full pages of a computed prompt (``pages`` is the sequence's block table).
        Returns the pages the cache took ownership of (they must not be freed with the sequence);
        pages that duplicate an existing entry stay with the sequence."""
        node, taken, now = self.root, [], next(self._clock)
        for i, key in enumerate(self._pages(tokens, len(tokens))):
            if i >= len(pages):
                break
            nxt = node.children.get(key)
            if nxt is None:
                if pages[i] in self._by_page:     # the page already belongs to another path: stop here
                    break
                nxt = _Node(pages[i], node, key, refs=1, last_used=now)   # pinned by the inserting sequence
                node.children[key] = nxt
                self._by_page[pages[i]] = nxt
                taken.append(pages[i])
            elif nxt.page != pages[i]:
                break                              # same tokens cached under another page: keep ours private
            nxt.last_used = now
            node = nxt
        return taken

    def release(self, pages: list[int]) -> None:
        for p in pages:
            n = self._by_page.get(p)
            if n is not None and n.refs > 0:
                n.refs -= 1

    def evict(self, want_pages: int) -> list[int]:
        """Frees up to ``want_pages`` unpinned leaf pages, least recently used first."""
        out: list[int] = []
        while len(out) < want_pages:
            leaves = [n for n in self._by_page.values() if not n.children and n.refs == 0]
            if not leaves:
                break
            leaves.sort(key=lambda n: n.last_used)
            for n in leaves[:want_pages - len(out)]:
                del n.parent.children[n.key]
                del self._by_page[n.page]
                out.append(n.page)
        return out

    def evictable_among(self, pages) -> int:
        """How many of ``pages`` are cached and unpinned (a pin on a page pins its whole path, so an unpinned cached
        page has no pinned descendant)."""
        return sum(1 for p in pages if (n := self._by_page.get(p)) is not None and n.refs == 0)

    def evict_pages(self, pages) -> list[int]:
        """Evicts the unpinned cached pages among ``pages`` together with everything cached behind them (a prefix
        without its head is unreachable). Used to vacate the pages of a memory bundle that is about to be retired:
        the reference couples its radix tree to bundle retirement the same way (src/xpool/integrations/sglang/ecs/
        state.py:470-541, ecs/radix.py). Returns every page freed, in or outside ``pages``."""
        out: list[int] = []
        for p in list(pages):
            n = self._by_page.get(p)
            if n is None or n.refs != 0:
                continue
            del n.parent.children[n.key]
            stack = [n]
            while stack:
                cur = stack.pop()
                stack.extend(cur.children.values())
                del self._by_page[cur.page]
                out.append(cur.page)
        self.evicted_for_retirement += len(out)
        return out

    def stats(self) -> dict:
        return {"pages": len(self), "lookups": self.lookups, "hits": self.hits, "hit_tokens": self.hit_tokens,
                "evicted_for_retirement": self.evicted_for_retirement}
