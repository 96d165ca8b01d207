"""Prefix cache: longest-prefix match on page boundaries, pinning, ownership, LRU eviction of leaves."""
from crosspool_b200.engine.prefix_cache import PrefixCache


def test_match_insert_pin_and_evict():
    c = PrefixCache(page_size=4)
    a = list(range(10))                       # two full pages + 2 tokens
    assert c.match(a) == []
    assert c.insert(a, [7, 8, 9]) == [7, 8]   # only full pages; the inserting sequence pins them
    assert len(c) == 2 and c.owns(7) and not c.owns(9)
    assert c.evict(5) == []                   # pinned
    c.release([7, 8])
    b = a[:8] + [99, 98, 97, 96, 95]          # shares both pages, then diverges
    assert c.match(b) == [7, 8]
    assert c.match(a[:8]) == [7]              # at least one token is always left to compute
    c.release([7])
    assert c.insert(b, [7, 8, 20, 21]) == [20]
    assert c.evict(1) == []                   # leaf 20 pinned by its inserter, inner nodes are not leaves
    c.release([7, 8, 20])
    c.match(a)                                # touches 7, 8 (and pins them)
    assert c.evict(3) == [20]                 # 8 becomes a leaf but is pinned
    c.release([7, 8])
    assert c.evict(3) == [8, 7] and len(c) == 0
    st = c.stats()
    assert st["lookups"] == 4 and st["hits"] == 3 and st["hit_tokens"] == (2 + 1 + 2) * 4


def test_identical_prompts_prefilled_concurrently_keep_their_own_pages():
    c = PrefixCache(page_size=2)
    t = [1, 2, 3, 4, 5]
    assert c.insert(t, [10, 11, 12]) == [10, 11]
    assert c.insert(t, [30, 31, 32]) == []            # same tokens, other pages: stay private
    assert c.insert([1, 2, 9, 9, 9], [10, 40, 41]) == [40]   # shares page 10, adds its own second page
    assert len(c) == 3


def test_evicting_the_cached_pages_of_a_bundle_takes_their_subtrees_and_spares_pinned_paths():
    pc = PrefixCache(2)
    a = [1, 2, 3, 4, 5, 6, 0]
    assert pc.insert(a, [10, 11, 12]) == [10, 11, 12]
    pc.release([10, 11, 12])
    b = [1, 2, 9, 9, 8, 8, 0]
    assert pc.insert(b, [10, 20, 21]) == [20, 21]     # shares page 10, branches behind it
    pc.release([10, 20, 21])
    pinned = pc.match(b)                              # pins 10, 20, 21
    assert pinned == [10, 20, 21]
    assert pc.evictable_among(range(10, 13)) == 2     # 11 and 12; 10 is on a pinned path
    freed = pc.evict_pages([11])                      # evicting 11 takes 12 (cached behind it) too
    assert sorted(freed) == [11, 12] and not pc.owns(12) and pc.owns(10)
    assert pc.evict_pages([10, 20]) == []             # pinned: nothing happens
    pc.release(pinned)
    assert sorted(pc.evict_pages([10])) == [10, 20, 21] and len(pc) == 0
    assert pc.stats()["evicted_for_retirement"] == 5


def test_engine_vacates_a_bundle_by_eviction_before_it_retracts_running_work():
    """A pending shrink with no empty bundle: a bundle holding only unpinned cached pages is emptied by eviction; a
    bundle with a running sequence's page is not touched, and the engine then falls back to retraction."""
    from collections import deque

    from crosspool_b200.engine.atn_engine import AttentionEngine
    from crosspool_b200.engine.kv_cache import PageAllocator

    class Rec:
        floor_bundles = 1

        def __init__(self, alloc):
            self.alloc, self.polls, self.target = alloc, 0, 2

        def poll(self):
            self.polls += 1

        def bundles_to_vacate(self):
            return max(0, len(self.alloc.mapped_bundles()) - self.target)

        def retirable_empty(self):
            return [b for b in self.alloc.empty_bundles() if b >= self.floor_bundles]

    alloc = PageAllocator(12, pages_per_bundle=4)     # bundles 0, 1, 2
    first = alloc.alloc(4)                            # bundle 0 (fullest-first fill)
    cached = alloc.alloc(3)                           # bundle 1
    running_page = alloc.alloc(1)                     # bundle 1's last page
    more = alloc.alloc(2)                             # bundle 2
    assert {p // 4 for p in cached} == {1} and {p // 4 for p in more} == {2}
    pc = PrefixCache(2)
    pc.insert([1, 2, 3, 4, 0], more)                  # bundle 2 holds cached pages only
    pc.release(more)
    eng = AttentionEngine.__new__(AttentionEngine)
    eng.prefix, eng.stats, eng._inflight, eng.running, eng.waiting = pc, {}, None, [], deque()
    eng.kv = type("Kv", (), {"allocator": alloc})()
    eng.capacity = rec = Rec(alloc)
    eng._capacity_tick()
    assert alloc.used_in_bundle(2) == 0 and rec.retirable_empty() == [2] and eng.stats["evicted_for_shrink"] == 1
    assert rec.polls == 2 and len(pc) == 0
    # nothing evictable is left: with no running sequence the tick does nothing more
    alloc.begin_retirement(2)
    rec.target = 1
    eng._capacity_tick()
    assert eng.stats["evicted_for_shrink"] == 1 and alloc.used_in_bundle(1) == 4
    del first, running_page
