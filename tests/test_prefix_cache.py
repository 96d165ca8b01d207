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
