"""Placement of FFN shards onto FFN devices with memory admission.

Input: per model its layer byte sizes, FFN TP size and slot geometry; per FFN device its free bytes.
Output: for every model a list of contiguous layer ranges, each assigned to a TP group (an ordered
tuple of devices; order = TP rank = reduction order). The search is exact for the sizes this system
is built for (a handful of models on at most eight FFN devices): depth-first over models, each model
tries every TP group and, if it does not fit whole, a split of its layers over several groups.

Objectives, lexicographic like the reference's CP-SAT formulation
(src/xpool/service/daemon/ffn_placement.py:762-767): (1) fewest signature materialisations -- a device prepares
execution state once per distinct layer Signature it hosts (kind, hidden, local width, experts), and layers of
different models with the same Signature share it; (2) most Primary-Group reuse -- models placed on a TP group that
another model already uses; (3) largest minimum headroom; (4) smallest total peak. Admission checks the peak over
five stages per device — weight materialisation, fabric join, graph capture, execution installation, retained —
each plus an optional calibrated overhead that is linear in MiB of tensor storage, allocation count, dense / MoE
signature counts, Lanes and the joined flag (ffn_placement.py:664-700), against ``free - margin``.
Layers with identical per-rank bytes and Signature form one *class* (ffn_placement.py:207-252); a split placement
counts layers per class, and per-rank device counts are turned back into concrete TP groups by peeling
lexicographically-first perfect matchings (``decompose_into_tp_groups``, ffn_placement.py:57-148). The reference
solves the same model with OR-tools; this build has no OR-tools wheel, so the solver is native Python and
deterministic.
"""

from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field


class PlacementError(Exception):
    pass


@dataclass(frozen=True)
class LayerSignature:
    """What a device has to prepare once per distinct kind of layer it hosts."""

    kind: str            # "dense" | "moe"
    hidden: int
    local_width: int     # local intermediate size (per TP rank)
    experts: int = 0
    top_k: int = 0


@dataclass(frozen=True)
class LayerClass:
    """Layers of one model that are interchangeable for placement: same per-rank bytes, same Signature."""

    signature: LayerSignature
    shard_bytes: int
    layers: tuple[int, ...]


@dataclass(frozen=True)
class ModelDemand:
    model_id: str
    layer_bytes: tuple[int, ...]      # full (unsharded) FFN bytes per layer
    tp_size: int
    hidden_size: int
    max_rows: int                     # slot capacity (rows) per attention rank
    atn_ranks: int = 1
    max_intermediate: int = 0         # widest local intermediate (scratch between the two GEMMs)
    layer_kinds: tuple[str, ...] = () # "dense" / "moe" per layer (empty: all dense)
    experts: int = 0
    top_k: int = 0

    def signature(self, layer: int) -> LayerSignature:
        kind = self.layer_kinds[layer] if self.layer_kinds else "dense"
        inter = self.max_intermediate or 4 * self.hidden_size
        return LayerSignature(kind, self.hidden_size, -(-inter // self.tp_size), self.experts if kind == "moe" else 0,
                              self.top_k if kind == "moe" else 0)

    def layer_classes(self) -> list[LayerClass]:
        """Classes in order of first appearance."""
        seen: dict = {}
        for l in range(len(self.layer_bytes)):
            key = (self.signature(l), self.shard_bytes(l))
            seen.setdefault(key, []).append(l)
        return [LayerClass(sig, b, tuple(ls)) for (sig, b), ls in seen.items()]

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


@dataclass(frozen=True)
class StageOverheads:
    """Calibrated bytes added to every stage, linear in what the device hosts (fitted by ``xpool memory-profile``;
    all zero = the analytic ledger alone)."""

    base_bytes: float = 0.0
    per_storage_mib: float = 0.0
    per_allocation: float = 0.0
    per_dense_signature: float = 0.0
    per_moe_signature: float = 0.0
    per_lane: float = 0.0
    joined_bytes: float = 0.0

    def bytes_for(self, storage_bytes: int, allocations: int, dense_sigs: int, moe_sigs: int, lanes: int, joined: bool) -> int:
        if storage_bytes == 0:
            return 0
        return int(self.base_bytes + self.per_storage_mib * storage_bytes / (1 << 20) + self.per_allocation * allocations +
                   self.per_dense_signature * dense_sigs + self.per_moe_signature * moe_sigs + self.per_lane * lanes +
                   (self.joined_bytes if joined else 0.0))

    @classmethod
    def from_profile(cls, profile) -> "StageOverheads":
        """From a persisted ``XpoolMemoryCalibrationProfile``."""
        c = profile.coefficients
        return cls(base_bytes=c.context_bytes, per_lane=c.per_lane_bytes, per_allocation=c.per_instance_bytes,
                   per_storage_mib=c.weight_slack * (1 << 20))


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
    signature_materializations: int = 0       # distinct (device, Signature) pairs
    group_reuse: int = 0                      # models placed on a TP group another model also uses
    objectives: tuple = ()                    # (signature materialisations, -group reuse, -min headroom, total peak)

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
    sigs_on: dict[int, set] = field(default_factory=dict)      # distinct Signatures per device
    groups_used: dict = field(default_factory=dict)            # TP group -> number of models on it


def stage_bytes(weights: int, slots: int, n_models: int, n_layers: int, lanes: int, ws_per_lane: int,
                overheads: StageOverheads | None = None, dense_sigs: int = 0, moe_sigs: int = 0) -> StageBytes:
    """The five admission stages of one device. Staging uses one pinned-to-device copy of the largest
    layer at a time (folded into a 64 MiB allowance); joining adds the fabric slots; capture adds the
    per-Lane split-K workspaces and counters; installation adds the descriptor tables. ``overheads`` adds the
    calibrated part per stage (the joined flag is set from the fabric-join stage on)."""
    staging = 64 << 20 if weights else 0
    tables = n_models * 4096 + n_layers * 512
    lane_ws = lanes * (ws_per_lane + (64 << 10)) if weights else 0
    o = overheads or StageOverheads()
    allocs = 2 * n_layers + 3 * n_models

    def extra(joined: bool) -> int:
        return o.bytes_for(weights, allocs, dense_sigs, moe_sigs, lanes, joined)

    s = StageBytes()
    s.weight_materialization = weights + staging + extra(False)
    s.fabric_join = weights + slots + extra(True)
    s.graph_capture = weights + slots + lane_ws + extra(True)
    s.execution_installation = s.graph_capture + tables
    s.retained = s.execution_installation
    return s


def decompose_into_tp_groups(counts: list[dict[int, int]]) -> list[tuple[tuple[int, ...], int]]:
    """``counts[r][d]`` = layers whose TP rank ``r`` shard lives on device ``d`` (every rank holds the same total).
    Returns ``[(group, layers)]`` with ``group[r]`` the device of rank ``r``, all devices of a group distinct: the
    lexicographically first group whose removal leaves the rest decomposable is peeled off with as many layers as it
    can take, until nothing is left (the reference peels perfect matchings with max-flow feasibility checks,
    ffn_placement.py:57-148; the sizes here allow plain backtracking). Raises ``PlacementError`` when no
    decomposition exists (some device would have to host two ranks of one layer)."""
    tp = len(counts)
    totals = {sum(c.values()) for c in counts}
    if len(totals) != 1:
        raise PlacementError("every TP rank must hold the same number of layers")
    rem = [dict((d, n) for d, n in c.items() if n > 0) for c in counts]

    def feasible(r: list[dict[int, int]]) -> bool:
        left = sum(r[0].values())
        if left == 0:
            return True
        return first_group(r) is not None

    def first_group(r: list[dict[int, int]]):
        def rec(rank: int, used: tuple[int, ...]):
            if rank == tp:
                return used
            for d in sorted(r[rank]):
                if r[rank][d] > 0 and d not in used:
                    g = rec(rank + 1, used + (d,))
                    if g is not None:
                        return g
            return None
        return rec(0, ())

    out: list[tuple[tuple[int, ...], int]] = []
    guard = 0
    while sum(rem[0].values()) > 0:
        guard += 1
        if guard > 10000:
            raise PlacementError("TP group decomposition did not terminate")
        picked = None
        for g in _groups_in_order(rem):
            take = min(rem[r][g[r]] for r in range(tp))
            while take > 0:
                trial = [dict(c) for c in rem]
                for r in range(tp):
                    trial[r][g[r]] -= take
                if feasible(trial):
                    picked = (g, take, trial)
                    break
                take -= 1
            if picked:
                break
        if picked is None:
            raise PlacementError("per-rank device counts cannot be arranged into TP groups of distinct devices")
        out.append((picked[0], picked[1]))
        rem = picked[2]
    return out


def _groups_in_order(rem: list[dict[int, int]]):
    tp = len(rem)

    def rec(rank: int, used: tuple[int, ...]):
        if rank == tp:
            yield used
            return
        for d in sorted(rem[rank]):
            if rem[rank][d] > 0 and d not in used:
                yield from rec(rank + 1, used + (d,))
    yield from rec(0, ())


def place_ffn_models(models: list[ModelDemand], devices: list[DeviceSupply], *, margin_bytes: int = 0, lanes: int = 1,
                     ws_per_lane: int = 64 << 20, timeout_seconds: float = 60.0,
                     stagnation_nodes: int | None = None, overheads: StageOverheads | None = None,
                     objectives: str = "balanced") -> PlacementResult:
    """Depth-first search over whole-model placements (then greedy layer splits) with the lexicographic objective
    (fewest signature materialisations, most TP-group reuse, largest minimum headroom, smallest total peak);
    ``overheads`` adds calibrated per-stage bytes to the admission check.

    ``objectives``: ``"reference"`` orders the objectives as the reference does -- signature materialisations, TP-group
    reuse, minimum headroom, total peak -- which packs layers of equal Signature onto as few devices as memory allows
    (there every Signature costs a pair of graph captures per device). ``"balanced"`` (default) puts (model, device)
    materialisations and headroom first and uses Signature count and group reuse as tie-breakers: with one generic Lane
    graph a Signature costs nothing here, while an FFN device that hosts everything becomes the compute bottleneck of
    the whole tier. Small deployments are searched
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

    def sig_counts(st: _State, d: int) -> tuple[int, int]:
        sigs = st.sigs_on.get(d, ())
        return sum(1 for x in sigs if x.kind == "dense"), sum(1 for x in sigs if x.kind == "moe")

    def stages_of(st: _State, d: int) -> StageBytes:
        dn, mo = sig_counts(st, d)
        return stage_bytes(st.weights[d], st.slots[d], len(st.models_on[d]), st.layers_on[d], lanes, ws_per_lane, overheads, dn, mo)

    def peak(st: _State, d: int) -> int:
        return stages_of(st, d).peak

    def fits(st: _State) -> bool:
        return all(peak(st, d) <= free[d] for d in ids)

    def add(st: _State, m: ModelDemand, lo: int, hi: int, group: tuple[int, ...]) -> None:
        b = sum(m.shard_bytes(l) for l in range(lo, hi))
        sigs = {m.signature(l) for l in range(lo, hi)}
        for d in group:
            st.weights[d] += b
            st.layers_on[d] += hi - lo
            st.sigs_on.setdefault(d, set()).update(sigs)
            if m.model_id not in st.models_on[d]:
                st.models_on[d].add(m.model_id)
                st.slots[d] += m.slot_bytes()
        users = st.groups_used.setdefault(group, set())
        users.add(m.model_id)

    def clone(st: _State) -> _State:
        return _State(dict(st.weights), dict(st.slots), {d: set(s) for d, s in st.models_on.items()}, dict(st.layers_on),
                      {d: set(s) for d, s in st.sigs_on.items()}, {g: set(u) for g, u in st.groups_used.items()})

    def score(st: _State):
        mats = sum(len(s) for s in st.sigs_on.values())                       # (1) signature materialisations
        reuse = sum(len(u) - 1 for u in st.groups_used.values() if len(u) > 1)  # (2) models sharing a TP group
        head = min(free[d] - peak(st, d) for d in ids)                        # (3) minimum headroom
        total = sum(peak(st, d) for d in ids)                                 # (4) total peak
        if objectives == "reference":
            return (mats, -reuse, -head, total)
        shards = sum(len(s) for s in st.models_on.values())
        return (shards, -head, total, mats, -reuse)

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
        first = sum(len(s) for s in (st.sigs_on if objectives == "reference" else st.models_on).values())
        if best["score"] is not None and first > best["score"][0]:
            return  # the leading objective is already worse than the incumbent's
        for groups, s2 in options(st, models[order[k]]):
            explored += 1
            dfs(k + 1, s2, acc + groups)

    empty = _State({d: 0 for d in ids}, {d: 0 for d in ids}, {d: set() for d in ids}, {d: 0 for d in ids},
                   {d: set() for d in ids}, {})
    dfs(0, empty, [])
    if best["groups"] is None:
        need = sum(sum(m.layer_bytes) for m in models)
        raise PlacementError(f"FFN shards do not fit: {need} weight bytes over {len(ids)} devices "
                             f"with {sum(free.values())} admissible bytes")
    st = best["state"]
    stages = {d: stages_of(st, d) for d in ids}
    groups = sorted(best["groups"], key=lambda g: (g.model_id, g.layer_begin))
    reuse = sum(len(u) - 1 for u in st.groups_used.values() if len(u) > 1)
    mats = sum(len(x) for x in st.models_on.values())
    return PlacementResult(groups, stages, {d: free[d] - stages[d].peak for d in ids}, mats,
                           time.monotonic() - t0, explored, group_reuse=reuse, objectives=best["score"],
                           signature_materializations=sum(len(x) for x in st.sigs_on.values()))
