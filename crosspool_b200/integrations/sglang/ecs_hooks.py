"""Elastic Context State hooks: the seams of a serving engine's KV management that change when physical KV memory is
lent between co-located Instances.

The engine's token-to-KV pool becomes a view over VMM address ranges (stable addresses, backing mapped in bundles,
``ecs/vmm.py``); its allocator only hands out pages whose bundle is mapped; the prefill adder cuts a chunk to what
current backing holds and publishes demand for the rest; decode checks memory per page-boundary crossing and retracts
the newest sequences when a shrink needs their pages; every scheduling round starts by serving the daemon's quota
commands and ends by publishing demand. Targets follow the reference's table
(src/xpool/integrations/sglang/hooks/ecs.py:391-495); handlers are built on ``ecs.admission``, ``ecs.reconciler`` and
``engine.kv_cache`` and work on duck-typed engine objects.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from ...ecs import admission as adm
from .adapter import Hook

T = "sglang.srt."


@dataclass
class ElasticContextState:
    """Per-worker elastic KV state shared by the hooks (reference: ``SglangElasticContextState``, ecs/state.py)."""

    cache: Any                       # engine.kv_cache.PagedKvCache with an elastic backing
    reconciler: Any                  # ecs.reconciler.CapacityReconciler (or the TP-agreed one)
    page_size: int
    agree_min: Callable[[int], int] | None = None
    ttft_slo_s: float = 0.0
    evict: Callable[[int], list[int]] | None = None     # radix cache: free up to n pages, returns the page ids
    stats: dict = field(default_factory=lambda: {"prefill_cut": 0, "retracted": 0, "evicted_pages": 0, "demand_published": 0})

    # -- scheduling round ------------------------------------------------------------------
    def begin_scheduling(self) -> None:
        self.reconciler.poll()       # grow / shrink commands, retirement of drained bundles

    def finish_scheduling(self, missing_pages: int, head_arrival_s: float | None = None) -> None:
        if missing_pages > 0:
            deadline = int((head_arrival_s + self.ttft_slo_s) * 1e9) if head_arrival_s is not None and self.ttft_slo_s > 0 else 0
            self.reconciler.publish_demand(missing_pages, deadline)
            self.stats["demand_published"] += 1
        else:
            self.reconciler.withdraw_demand()

    # -- prefill ----------------------------------------------------------------------------
    def plan_prefill(self, seq_id: int, cached_tokens: int, want_tokens: int, reserve_pages: int = 0) -> adm.PrefillProposal:
        alloc = self.cache.allocator
        have = len(self.cache.tables.get(seq_id, ()))
        prop = adm.largest_chunk_that_fits(cached_tokens=cached_tokens, have_pages=have, want_tokens=want_tokens,
                                           free_pages=alloc.free_pages, page_size=self.page_size, reserve_pages=reserve_pages)
        if prop.tokens < want_tokens and self.evict is not None:
            freed = self.evict(prop.missing_pages)          # radix-cache nodes nobody reads any more
            if freed:
                alloc.free(freed)
                self.stats["evicted_pages"] += len(freed)
                prop = adm.largest_chunk_that_fits(cached_tokens=cached_tokens, have_pages=have, want_tokens=want_tokens,
                                                   free_pages=alloc.free_pages, page_size=self.page_size, reserve_pages=reserve_pages)
        prop = adm.coordinate_prefill(prop, self.agree_min)
        if prop.tokens < want_tokens:
            self.stats["prefill_cut"] += 1
        return prop

    # -- decode -----------------------------------------------------------------------------
    def check_decode_mem(self, seq_lens: list[int]) -> bool:
        return adm.check_decode_mem(seq_lens, self.cache.allocator.free_pages, self.page_size)[0]

    def retract_decode(self, seq_ids: list[int], seq_lens: list[int]) -> list[int]:
        pages = [len(self.cache.tables.get(s, ())) for s in seq_ids]
        victims = adm.retract_decode(seq_lens, pages, self.cache.allocator.free_pages, self.page_size)
        for i in victims:
            self.cache.release(seq_ids[i])
        self.stats["retracted"] += len(victims)
        return [seq_ids[i] for i in victims]

    def finalize_after_capture(self) -> None:
        """Post-capture sizing: report what the device has free so the daemon can freeze the pool budget."""
        rep = getattr(self.reconciler, "report_device_memory", None)
        if rep is not None:
            rep()


class ElasticHooks:
    """Handlers bound to one worker's :class:`ElasticContextState` (looked up lazily: the state exists only after
    ``alloc_memory_pool``)."""

    def __init__(self, state_of: Callable[[], ElasticContextState | None]):
        self.state_of = state_of

    def _st(self) -> ElasticContextState:
        st = self.state_of()
        if st is None:
            raise RuntimeError("elastic context state is not built yet (alloc_memory_pool has not run)")
        return st

    # replace: the engine asks "may this batch decode?" / "whom do I drop?"
    def check_decode_mem(self, batch: Any, *a, **kw) -> bool:
        return self._st().check_decode_mem([int(n) for n in batch.seq_lens])

    def retract_decode(self, batch: Any, *a, **kw):
        st = self._st()
        ids = [r.rid for r in batch.reqs]
        order = st.retract_decode(ids, [int(n) for n in batch.seq_lens])       # newest first
        dropped = set(order)
        by_id = {r.rid: r for r in batch.reqs}
        keep = [i for i, r in enumerate(batch.reqs) if r.rid not in dropped]
        batch.seq_lens = [batch.seq_lens[i] for i in keep]
        batch.reqs = [batch.reqs[i] for i in keep]
        return [by_id[rid] for rid in order]

    # around: one scheduling round
    def get_next_batch_to_run(self, original: Callable, scheduler: Any, *a, **kw):
        st = self._st()
        st.begin_scheduling()
        out = original(scheduler, *a, **kw)
        missing = int(getattr(scheduler, "xpool_missing_pages", 0))
        st.finish_scheduling(missing, getattr(scheduler, "xpool_head_arrival_s", None))
        return out

    # replace: prefill admission of one request; returns the tokens admitted
    def add_one_req(self, adder: Any, req: Any, *a, **kw) -> int:
        st = self._st()
        want = min(int(req.extend_input_len), int(adder.rem_chunk_tokens))
        prop = st.plan_prefill(req.rid, int(req.prefix_len), want, reserve_pages=int(getattr(adder, "reserve_pages", 0)))
        if prop.tokens <= 0:
            adder.scheduler.xpool_missing_pages = prop.missing_pages
            adder.scheduler.xpool_head_arrival_s = getattr(req, "arrival_s", None)
            return 0
        st.cache.ensure(req.rid, int(req.prefix_len) + prop.tokens)
        adder.rem_chunk_tokens -= prop.tokens
        adder.can_run_list.append((req, prop.tokens))
        adder.scheduler.xpool_missing_pages = prop.missing_pages
        if prop.missing_pages > 0:
            adder.scheduler.xpool_head_arrival_s = getattr(req, "arrival_s", None)
        return prop.tokens

    def hooks(self) -> list[Hook]:
        return [
            Hook(T + "managers.schedule_batch.ScheduleBatch.check_decode_mem", self.check_decode_mem, "replace"),
            Hook(T + "managers.schedule_batch.ScheduleBatch.retract_decode", self.retract_decode, "replace"),
            Hook(T + "managers.scheduler.Scheduler.get_next_batch_to_run", self.get_next_batch_to_run, "around"),
            Hook(T + "managers.schedule_policy.PrefillAdder.add_one_req", self.add_one_req, "replace"),
        ]
