"""Elastic admission arithmetic: chunk search, TP agreement, decode memory check, retraction order."""
from crosspool_b200.ecs import admission as A


def test_whole_request_is_admitted_when_it_fits():
    p = A.largest_chunk_that_fits(cached_tokens=0, have_pages=0, want_tokens=1000, free_pages=100, page_size=16)
    assert (p.tokens, p.missing_pages) == (1000, 0)


def test_chunk_is_cut_to_the_longest_length_that_fits_and_reports_the_shortfall():
    # 10 free pages of 16 tokens, 3 kept in reserve: 7 pages = 112 tokens; the sequence already fills 5 tokens of a page
    p = A.largest_chunk_that_fits(cached_tokens=21, have_pages=2, want_tokens=500, free_pages=10, page_size=16, reserve_pages=3)
    assert p.tokens == (2 + 7) * 16 - 21 == 123
    assert A.pages_for(21 + p.tokens, 16) - 2 == 7 and A.pages_for(21 + p.tokens + 1, 16) - 2 == 8
    assert p.missing_pages == A.pages_for(521, 16) - 2 - 7
    # brute force agrees for every budget
    for free in range(0, 40):
        got = A.largest_chunk_that_fits(cached_tokens=21, have_pages=2, want_tokens=300, free_pages=free, page_size=16).tokens
        want = max([n for n in range(0, 301) if A.pages_for(21 + n, 16) - 2 <= free])
        assert got == want


def test_nothing_fits_below_the_minimum_chunk():
    p = A.largest_chunk_that_fits(cached_tokens=16, have_pages=1, want_tokens=100, free_pages=0, page_size=16, min_tokens=8)
    assert p.tokens == 0 and p.missing_pages == A.pages_for(116, 16) - 1


def test_tp_group_runs_the_smallest_proposal():
    local = A.PrefillProposal(300, 4)
    assert A.coordinate_prefill(local, agree_min=lambda v: min(v, 180)).tokens == 180
    assert A.coordinate_prefill(local).tokens == 300


def test_decode_needs_a_page_per_boundary_crossing_and_retracts_newest_first():
    lens = [31, 32, 48, 7, 64]            # 32, 48, 64 start a new page next
    assert A.check_decode_mem(lens, 3, 16) == (True, 3)
    assert A.check_decode_mem(lens, 2, 16) == (False, 3)
    pages = [2, 2, 3, 1, 4]
    assert A.retract_decode(lens, pages, 2, 16) == [4]           # dropping the newest (a crosser holding 4 pages) is enough
    assert A.retract_decode(lens, pages, 0, 16) == [4]           # its 4 pages cover the other two crossers
    assert A.retract_decode([16, 16, 16], [1, 1, 1], 0, 16) == [2, 1]
