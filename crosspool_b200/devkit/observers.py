"""Collectors behind the four observers and the chrome-trace exporter.

The native side records fixed-size events into pre-allocated buffers (slot reservation by atomic add,
``%globaltimer`` stamps, overflow counted as ``dropped``, never wrapping:
``csrc/include/xpool/trace.hpp`` / ``trace.cuh``). The collectors here drain those buffers at shutdown
and write artifacts, like the reference's ``src/xpool/devkit/{transport,fabric,graph,ffn_routing}.py``
with role-aware discovery (``src/xpool/devkit/registry.py:17-68``):

* transport observer -- mailbox transitions of the CPU transport / the attention-side publish+wait;
* fabric observer    -- Lane admissions, completions, idle replays, rejections on an FFN device;
* graph observer     -- a snapshot of what the generic Lane graph will execute for every
  (instance, layer, row bucket): tile width and split-K per projection (the counterpart of the
  reference's graph topology + binding-site dump, ``src/cext/devkit/graph_observer.cpp``);
* routing observer   -- top-k expert ids / weights of sampled MoE invocations (safetensors).
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterable

LANE_EVENT_NAMES = {1: "admitted", 2: "completed", 3: "idle", 4: "shutdown", 5: "rejected", 6: "discovered", 7: "lock_timeout",
                    8: "failure_claimed", 9: "failure_observed"}
ATN_EVENT_NAMES = {16: "published", 17: "fold_wait_timed_out", 18: "wait_begin", 19: "wait_end", 20: "wait_timed_out",
                   21: "wait_cancelled"}
TRANSPORT_EVENT_NAMES = {1: "publish", 2: "wait_begin", 3: "wait_end", 4: "timeout", 5: "cancelled", 6: "host_submit",
                         7: "host_collect"}


@dataclass
class TraceArtifact:
    observer: str
    role: str
    pid: int
    events: list[dict]
    dropped: int = 0
    meta: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return {"observer": self.observer, "role": self.role, "pid": self.pid, "dropped": self.dropped, "meta": self.meta,
                "events": self.events}


class _Base:
    name = ""

    def __init__(self, role: str, out_dir: str | os.PathLike | None = None):
        self.role, self.out_dir = role, Path(out_dir) if out_dir else None

    def collect(self) -> TraceArtifact:  # pragma: no cover - abstract
        raise NotImplementedError

    def write(self) -> Path | None:
        art = self.collect()
        if self.out_dir is None:
            return None
        self.out_dir.mkdir(parents=True, exist_ok=True)
        p = self.out_dir / f"{self.name}-{self.role}-{art.pid}.json"
        p.write_text(json.dumps(art.to_json()))
        return p


class FabricObserver(_Base):
    """Drains the Lane event buffer of an ``FfnRankRuntime`` (``enable_trace`` must have been called)."""

    name = "fabric"

    def __init__(self, runtime, role: str = "FfnAgent", out_dir=None):
        super().__init__(role, out_dir)
        self.runtime = runtime

    def collect(self) -> TraceArtifact:
        raw, dropped = self.runtime.trace_events()
        ev = []
        for kind, a, b, ts in raw:
            e = {"name": LANE_EVENT_NAMES.get(kind, str(kind)), "ts_ns": ts}
            if kind == 1:
                e.update(instance=a, layer=b >> 16, rows=b & 0xFFFF)
            elif kind == 2:
                e.update(instance=a, sequence=b)
            elif kind in (5, 8):
                e.update(instance=a, result_code=b)
            elif kind == 6:
                e.update(instance=a, sequence=b)
            elif kind == 9:
                e.update(lane=a, origin_pe=b)
            else:
                e.update(lane=a, count=b)
            ev.append(e)
        return TraceArtifact(self.name, self.role, os.getpid(), ev, dropped)


def lane_busy_summary(events: list[dict], lanes: int) -> dict:
    """How busy the Lanes of one FFN GPU were, from its fabric observer's events: an invocation occupies a Lane from
    ``admitted`` to ``completed`` (device timestamps); the busy fraction is the sum of those spans over the observed
    interval times the number of Lanes. Also the service-time distribution and the rows served."""
    open_at: dict[int, list[int]] = {}
    spans: list[int] = []
    rows = 0
    first = last = None
    for e in events:
        ts = e["ts_ns"]
        first = ts if first is None else min(first, ts)
        last = ts if last is None else max(last, ts)
        if e["name"] == "admitted":
            open_at.setdefault(e["instance"], []).append(ts)
            rows += e.get("rows", 0)
        elif e["name"] == "completed":
            q = open_at.get(e["instance"])
            if q:
                spans.append(ts - q.pop(0))
    if not spans or first is None or last <= first:
        return {"invocations": len(spans), "busy_fraction": 0.0}
    spans.sort()
    busy = sum(spans)

    def pct(p):
        return spans[min(len(spans) - 1, int(p * (len(spans) - 1)))] / 1e3

    return {"invocations": len(spans), "rows": rows, "observed_s": round((last - first) / 1e9, 3),
            "busy_fraction": round(busy / ((last - first) * max(1, lanes)), 4),
            "service_us": {"mean": round(busy / len(spans) / 1e3, 1), "p50": round(pct(0.5), 1), "p99": round(pct(0.99), 1)}}


class AtnFabricObserver(_Base):
    """Drains the device event buffer of an attention-side Fabric port (``FabricFfnPort.enable_trace``) and groups the
    events of each invocation into a timeline: published -> wait_begin -> wait_end | wait_timed_out | wait_cancelled,
    keyed by the invocation sequence (the reference keeps a ``Timeline<Event>`` per invocation,
    src/cext/devkit/fabric_observer.cu)."""

    name = "fabric"

    def __init__(self, port, role: str = "AtnAgent", out_dir=None):
        super().__init__(role, out_dir)
        self.port = port

    def collect(self) -> TraceArtifact:
        raw, dropped = self.port.trace.read()
        ev, timelines = [], {}
        for kind, a, b, ts in raw:
            name = ATN_EVENT_NAMES.get(kind, str(kind))
            e = {"name": name, "ts_ns": ts, "sequence": b}
            if kind == 16:
                e.update(layer=a >> 16, rows=a & 0xFFFF)
            else:
                e.update(flag=a)
            ev.append(e)
            t = timelines.setdefault(b, {"sequence": b})
            t.setdefault(name, ts)
        done = [t for t in timelines.values() if "published" in t and "wait_end" in t]
        for t in done:
            t["round_trip_ns"] = t["wait_end"] - t["published"]
        return TraceArtifact(self.name, self.role, os.getpid(), ev, dropped, {"timelines": sorted(timelines.values(), key=lambda t: t["sequence"])})


class TransportObserver(_Base):
    """Host-side transport events recorded into a native ``TraceBuffer``."""

    name = "transport"

    def __init__(self, role: str = "Instance", capacity: int = 1 << 16, out_dir=None):
        super().__init__(role, out_dir)
        from ..native.runtime import TraceBuffer

        self.buffer = TraceBuffer(capacity)

    def record(self, kind: int, a: int = 0, b: int = 0) -> None:
        self.buffer.record(kind, a, b, time.monotonic_ns())

    def collect(self) -> TraceArtifact:
        _, dropped = self.buffer.counts()
        ev = [{"name": TRANSPORT_EVENT_NAMES.get(k, str(k)), "a": a, "b": b, "ts_ns": ts} for k, a, b, ts in self.buffer.events()]
        return TraceArtifact(self.name, self.role, os.getpid(), ev, dropped)


class GraphObserver(_Base):
    """What each Lane replay executes: per instance and layer, the tile plan of both projections."""

    name = "graph"

    def __init__(self, role: str = "FfnAgent", out_dir=None):
        super().__init__(role, out_dir)
        self.nodes: list[dict] = []

    def snapshot_lane_graph(self, instances: Iterable[Any], row_buckets=(1, 16, 64, 256, 1024, 4096)) -> None:
        """``instances``: objects with ``model_id``, ``cfg`` (hidden, intermediate, layers) and ``tp_size``."""
        from ..ops import gemm

        for inst in instances:
            cfg = inst.cfg
            inter = cfg.intermediate_size // max(1, getattr(inst, "tp_size", 1))
            for rows in row_buckets:
                gu = gemm.plan_shape(inter, cfg.hidden_size, rows, 1)
                dn = gemm.plan_shape(cfg.hidden_size, inter, rows, 0)
                self.nodes.append({"instance": inst.model_id, "layers": cfg.num_layers, "rows": rows,
                                   "sequence": ["lane_wait", "gemm_gateup_swiglu", "gemm_down", "lane_complete"],
                                   "gateup": gu, "down": dn})

    def collect(self) -> TraceArtifact:
        return TraceArtifact(self.name, self.role, os.getpid(), [], 0, {"nodes": self.nodes})


class RoutingObserver(_Base):
    """Keeps the top-k ids / weights of up to ``max_samples`` MoE invocations."""

    name = "ffn_routing"

    def __init__(self, role: str = "FfnAgent", max_samples: int = 64, out_dir=None):
        super().__init__(role, out_dir)
        self.max_samples, self.samples, self.dropped = max_samples, [], 0

    def capture(self, layer: int, ids, weights) -> None:
        if len(self.samples) >= self.max_samples:
            self.dropped += 1
            return
        self.samples.append((layer, ids.detach().to("cpu", copy=True), weights.detach().to("cpu", copy=True)))

    def collect(self) -> TraceArtifact:
        ev = [{"name": "routing", "layer": l, "rows": int(i.shape[0]), "top_k": int(i.shape[1])} for l, i, _ in self.samples]
        return TraceArtifact(self.name, self.role, os.getpid(), ev, self.dropped)

    def write(self) -> Path | None:
        p = super().write()
        if p is not None and self.samples:
            from safetensors.torch import save_file

            tensors = {}
            for n, (l, i, w) in enumerate(self.samples):
                tensors[f"sample{n}.layer{l}.ids"], tensors[f"sample{n}.layer{l}.weights"] = i.contiguous(), w.contiguous()
            save_file(tensors, str(p.with_suffix(".safetensors")))
        return p


@dataclass
class ObserverSet:
    observers: list[_Base] = field(default_factory=list)

    def write_all(self) -> list[Path]:
        return [p for p in (o.write() for o in self.observers) if p is not None]


# which observers make sense in which role (reference: src/xpool/devkit/registry.py:17-68)
ROLE_OBSERVERS = {"Instance": ("transport",), "AtnAgent": ("transport", "fabric"), "FfnAgent": ("fabric", "graph", "ffn_routing"),
                  "Daemon": ()}


def observers_for_role(role: str, cfg, *, lane_runtime=None) -> ObserverSet:
    """Builds the enabled observers for ``role`` from the ``debug_<name>_observer_*`` settings of the
    resolved configuration (any object with those attributes)."""
    def opt(name, key, default):
        return getattr(cfg, f"debug_{name}_observer_{key}", default)

    s = ObserverSet()
    allowed = ROLE_OBSERVERS.get(role, ())
    if "transport" in allowed and opt("transport", "enable", False):
        s.observers.append(TransportObserver(role, opt("transport", "record_capacity", 1 << 16), opt("transport", "outdir", "") or None))
    if "fabric" in allowed and opt("fabric", "enable", False) and lane_runtime is not None:
        lane_runtime.enable_trace(opt("fabric", "record_capacity", 1 << 16))
        s.observers.append(FabricObserver(lane_runtime, role, opt("fabric", "outdir", "") or None))
    if "graph" in allowed and opt("graph", "enable", False):
        s.observers.append(GraphObserver(role, opt("graph", "outdir", "") or None))
    if "ffn_routing" in allowed and opt("ffn_routing", "enable", False):
        s.observers.append(RoutingObserver(role, min(64, opt("ffn_routing", "record_capacity", 64)), opt("ffn_routing", "outdir", "") or None))
    return s


def chrome_trace(artifacts: Iterable[TraceArtifact | dict], host_spans: Iterable[dict] = ()) -> dict:
    """Merges observer artifacts (and optional host spans ``{name, ts_ns, dur_ns, pid, tid}``) into the
    chrome://tracing JSON object format. Lane admissions and completions of the same instance pair up
    into duration events; everything else becomes an instant event."""
    out = []
    for art in artifacts:
        a = art.to_json() if isinstance(art, TraceArtifact) else art
        pid, open_at = a["pid"], {}
        for e in a["events"]:
            ts = e["ts_ns"] / 1e3
            if a["observer"] == "fabric" and e["name"] == "admitted":
                open_at[e["instance"]] = e
            elif a["observer"] == "fabric" and e["name"] == "completed" and e["instance"] in open_at:
                b = open_at.pop(e["instance"])
                out.append({"name": f"inst{b['instance']} L{b['layer']} rows={b['rows']}", "ph": "X", "pid": pid,
                            "tid": f"instance {b['instance']}", "ts": b["ts_ns"] / 1e3, "dur": (e["ts_ns"] - b["ts_ns"]) / 1e3,
                            "cat": "lane"})
            else:
                out.append({"name": e["name"], "ph": "i", "s": "t", "pid": pid, "tid": a["observer"], "ts": ts,
                            "args": {k: v for k, v in e.items() if k not in ("name", "ts_ns")}})
    for h in host_spans:
        out.append({"name": h["name"], "ph": "X", "pid": h.get("pid", 0), "tid": h.get("tid", "host"), "ts": h["ts_ns"] / 1e3,
                    "dur": h["dur_ns"] / 1e3, "cat": "host"})
    out.sort(key=lambda e: e["ts"])
    return {"traceEvents": out, "displayTimeUnit": "ns"}
