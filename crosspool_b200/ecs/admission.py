"""Prefill and decode admission against elastic KV backing.

What the engine may run next depends on how much of its KV address range is backed by physical memory right now:
a prefill chunk is cut to the longest length whose pages fit (binary search over the chunk length, as
``ElasticPrefillAdder.coordinate_prefill`` does in src/xpool/integrations/sglang/ecs/admission.py:125-183), every
rank of an attention TP group must arrive at the same answer (the proposal is reduced with MIN over the group), a
decode step needs one free page per sequence that crosses a page boundary (``check_decode_mem``), and when even that
is missing the newest sequences are retracted until the rest fits (``retract_decode``, :315-374).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Sequence


@dataclass
class PrefillProposal:
    tokens: int              # chunk length that fits current backing (0: nothing fits)
    missing_pages: int       # pages short of the full request (demand to publish)


def pages_for(tokens: int, page_size: int) -> int:
    return (tokens + page_size - 1) // page_size


def largest_chunk_that_fits(*, cached_tokens: int, have_pages: int, want_tokens: int, free_pages: int, page_size: int,
                            reserve_pages: int = 0, min_tokens: int = 1) -> PrefillProposal:
    """The longest prefix of ``want_tokens`` new tokens (after ``cached_tokens`` already in the cache, for which the
    sequence holds ``have_pages`` pages) whose KV fits in ``free_pages - reserve_pages``. Binary search over the length;
    the page count is monotone in it."""
    def need(n: int) -> int:
        return max(0, pages_for(cached_tokens + n, page_size) - have_pages)

    budget = max(0, free_pages - reserve_pages)     # tokens that fit the pages the sequence already holds always run
    full = need(want_tokens)
    if full <= budget:
        return PrefillProposal(want_tokens, 0)
    lo, hi = 0, want_tokens          # invariant: need(lo) <= budget (0 tokens need nothing) and need(hi) > budget
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if need(mid) <= budget:
            lo = mid
        else:
            hi = mid
    return PrefillProposal(lo if lo >= min_tokens else 0, full - budget)


def coordinate_prefill(local: PrefillProposal, agree_min: Callable[[int], int] | None = None) -> PrefillProposal:
    """All ranks of an attention TP group run the same chunk: the smallest proposal wins."""
    if agree_min is None:
        return local
    return PrefillProposal(int(agree_min(local.tokens)), local.missing_pages)


def check_decode_mem(seq_lens: Sequence[int], free_pages: int, page_size: int) -> tuple[bool, int]:
    """(fits, pages needed): a sequence whose next token starts a new page needs one."""
    need = sum(1 for n in seq_lens if n % page_size == 0)
    return need <= free_pages, need


def retract_decode(seq_lens: Sequence[int], seq_pages: Sequence[int], free_pages: int, page_size: int) -> list[int]:
    """Indices of the sequences to retract (newest first, i.e. from the end) until the remaining batch's next decode
    step fits; a retracted sequence gives its pages back."""
    idx = list(range(len(seq_lens)))
    out: list[int] = []
    free = free_pages
    while idx:
        ok, _ = check_decode_mem([seq_lens[i] for i in idx], free, page_size)
        if ok:
            break
        victim = idx.pop()
        out.append(victim)
        free += seq_pages[victim]
    return out
