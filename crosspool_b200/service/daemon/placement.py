"""Placement of FFN shards onto FFN devices with memory admission.

Input: per model its layer byte sizes, FFN TP size and slot geometry; per FFN device its free bytes.
Output: for every model a list of contiguous layer ranges, each assigned to a TP group (an ordered
tuple of devices; order = TP rank = reduction order). The search is exact for the sizes this system
is built for (a handful of models on at most eight FFN devices): depth-first over models, each model
tries every TP group and, if it does not fit whole, a split of its layers over several groups.

Objectives, lexicographic like the reference's CP-SAT formulation
(src/xpool/service/daemon/ffn_placement.py:762-767): (1) fewest (model, device) materialisations,
(2) largest minimum headroom, (3) smallest total peak. Admission checks the peak over five stages per
device — weight materialisation, fabric join, graph capture, execution installation, retained —
against ``free - margin`` (ffn_placement.py:694-700). The reference solves the same model with
OR-tools; this build has no OR-tools wheel, so the solver is native Python and deterministic.
"""

from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field


class PlacementError(Exception):
    pass


@dataclass(frozen=True)
class ModelDemand:
    model_id: str
    layer_bytes: tuple[int, ...]      # full (unsharded) FFN bytes per layer
    tp_size: int
    hidden_size: int
    max_rows: int                     # slot capacity (rows) per attention rank
    atn_ranks: int = 1
    max_intermediate: int = 0         # widest local intermediate (scratch between the two GEMMs)

    def shard_bytes(self, layer: int) -> int:
        return -(-self.layer_bytes[layer] // self.tp_size)

    def slot_bytes(self) -> int:
        """Per device: invocation record + input payload + activation scratch, per attention rank."""
        inter_local = -(-self.max_intermediate // self.tp_size) if self.max_intermediate else 4 * self.hidden_size
        return self.atn_ranks * (256 + self.max_rows * (self.hidden_size + inter_local) * 2 + 1024)


@dataclass(frozen=True)
class DeviceSupply:
    device: int
    free_bytes: int
    total_bytes: int = 0


@dataclass
class StageBytes:
    weight_materialization: int = 0
    fabric_join: int = 0
    graph_capture: int = 0
    execution_installation: int = 0
    retained: int = 0

    @property
    def peak(self) -> int:
        return max(self.weight_materialization, self.fabric_join, self.graph_capture, self.execution_installation,
                   self.retained)


@dataclass(frozen=True)
class LayerGroupPlacement:
    model_id: str
    layer_begin: int
    layer_end: int
    devices: tuple[int, ...]  # TP rank order


@dataclass
class PlacementResult:
    groups: list[LayerGroupPlacement]
    stages: dict[int, StageBytes]
    headroom: dict[int, int]
    materializations: int
    solve_seconds: float = 0.0
    explored: int = 0

    def shards(self):
        """Flat (model, layer range, tp rank, device) list."""
        for g in self.groups:
            for r, d in enumerate(g.devices):
                yield g.model_id, g.layer_begin, g.layer_end, r, len(g.devices), d


@dataclass
class _State:
    weights: dict[int, int]
    slots: dict[int, int]
    models_on: dict[int, set]
    layers_on: dict[int, int]


def stage_bytes(weights: int, slots: int, n_models: int, n_layers: int, lanes: int, ws_per_lane: int) -> StageBytes:
    """The five admission stages of one device. Staging uses one pinned-to-device copy of the largest
    layer at a time (folded into a 64 MiB allowance); joining adds the fabric slots; capture adds the
    per-Lane split-K workspaces and counters; installation adds the descriptor tables."""
    staging = 64 << 20 if weights else 0
    tables = n_models * 4096 + n_layers * 512
    lane_ws = lanes * (ws_per_lane + (64 << 10)) if weights else 0
    s = StageBytes()
    s.weight_materialization = weights + staging
    s.fabric_join = weights + slots
    s.graph_capture = s.fabric_join + lane_ws
    s.execution_installation = s.graph_capture + tables
    s.retained = s.execution_installation
    return s


def place_ffn_models(models: list[ModelDemand], devices: list[DeviceSupply], *, margin_bytes: int = 0, lanes: int = 1,
                     ws_per_lane: int = 64 << 20, timeout_seconds: float = 60.0,
                     stagnation_nodes: int | None = None) -> PlacementResult:
    """Depth-first search over whole-model placements (then greedy layer splits) with the lexicographic objective
    (fewest materialisations, largest minimum headroom, smallest total peak). Small deployments are searched
    exhaustively; the search also stops when ``stagnation_nodes`` options were explored since the incumbent last
    improved (default ``max(4000, 40 * models)``), which keeps planning of deployments with hundreds of
    co-located models to a few seconds: the first leaf already takes the most-headroom choice at every step."""
    if not devices:
        raise PlacementError("no FFN devices")
    ids = [d.device for d in devices]
    free = {d.device: d.free_bytes - margin_bytes for d in devices}
    for m in models:
        if m.tp_size < 1 or m.tp_size > len(ids):
            raise PlacementError(f"model {m.model_id}: ffn_tp_size {m.tp_size} exceeds {len(ids)} FFN devices")
    order = sorted(range(len(models)), key=lambda i: (-sum(models[i].layer_bytes), models[i].model_id))
    t0 = time.monotonic()
    best: dict = {"score": None, "groups": None, "at": 0}
    explored = 0
    stagnation = stagnation_nodes if stagnation_nodes is not None else max(4000, 40 * len(models))

    def peak(st: _State, d: int) -> int:
        return stage_bytes(st.weights[d], st.slots[d], len(st.models_on[d]), st.layers_on[d], lanes, ws_per_lane).peak

    def fits(st: _State) -> bool:
        return all(peak(st, d) <= free[d] for d in ids)

    def add(st: _State, m: ModelDemand, lo: int, hi: int, group: tuple[int, ...]) -> None:
        b = sum(m.shard_bytes(l) for l in range(lo, hi))
        for d in group:
            st.weights[d] += b
            st.layers_on[d] += hi - lo
            if m.model_id not in st.models_on[d]:
                st.models_on[d].add(m.model_id)
                st.slots[d] += m.slot_bytes()

    def clone(st: _State) -> _State:
        return _State(dict(st.weights), dict(st.slots), {d: set(s) for d, s in st.models_on.items()}, dict(st.layers_on))

    def score(st: _State):
        mats = sum(len(s) for s in st.models_on.values())
        head = min(free[d] - peak(st, d) for d in ids)
        total = sum(peak(st, d) for d in ids)
        return (mats, -head, total)

    def options(st: _State, m: ModelDemand):
        """Whole-model placements first (fewest materialisations), then greedy splits."""
        n = len(m.layer_bytes)
        combos = list(itertools.combinations(ids, m.tp_size))
        whole = []
        for g in combos:
            s2 = clone(st)
            add(s2, m, 0, n, g)
            if fits(s2):
                whole.append(([LayerGroupPlacement(m.model_id, 0, n, g)], s2))
        if whole:
            # most headroom first so that good solutions are found early
            whole.sort(key=lambda o: (score(o[1]), o[0][0].devices))
            return whole
        # split: fill groups in lexicographic order with as many contiguous layers as fit
        s2, groups, lo = clone(st), [], 0
        for g in combos:
            if lo >= n:
                break
            hi = lo
            while hi < n:
                s3 = clone(s2)
                add(s3, m, lo, hi + 1, g) if hi == lo else add(s3, m, hi, hi + 1, g)
                if not fits(s3):
                    break
                s2, hi = s3, hi + 1
            if hi > lo:
                groups.append(LayerGroupPlacement(m.model_id, lo, hi, g))
                lo = hi
        return [(groups, s2)] if lo >= n else []

    def dfs(k: int, st: _State, acc: list[LayerGroupPlacement]) -> None:
        nonlocal explored
        if best["groups"] is not None and (explored - best["at"] > stagnation or time.monotonic() - t0 > timeout_seconds):
            return
        if k == len(order):
            sc = score(st)
            if best["score"] is None or sc < best["score"]:
                best["score"], best["groups"], best["state"], best["at"] = sc, list(acc), st, explored
            return
        if best["score"] is not None and sum(len(s) for s in st.models_on.values()) > best["score"][0]:
            return  # already more materialisations than the incumbent
        for groups, s2 in options(st, models[order[k]]):
            explored += 1
            dfs(k + 1, s2, acc + groups)

    empty = _State({d: 0 for d in ids}, {d: 0 for d in ids}, {d: set() for d in ids}, {d: 0 for d in ids})
    dfs(0, empty, [])
    if best["groups"] is None:
        need = sum(sum(m.layer_bytes) for m in models)
        raise PlacementError(f"FFN shards do not fit: {need} weight bytes over {len(ids)} devices "
                             f"with {sum(free.values())} admissible bytes")
    st = best["state"]
    stages = {d: stage_bytes(st.weights[d], st.slots[d], len(st.models_on[d]), st.layers_on[d], lanes, ws_per_lane)
              for d in ids}
    groups = sorted(best["groups"], key=lambda g: (g.model_id, g.layer_begin))
    return PlacementResult(groups, stages, {d: free[d] - stages[d].peak for d in ids}, best["score"][0],
                           time.monotonic() - t0, explored)
