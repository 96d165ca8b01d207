"""Observers: role-aware discovery, event decoding, overflow accounting, chrome-trace export."""
import json
import types

import torch

from crosspool_b200 import devkit
from crosspool_b200.devkit.observers import TraceArtifact
from crosspool_b200.models.config import PRESETS


class FakeLaneRuntime:
    def __init__(self):
        self.capacity = None

    def enable_trace(self, capacity):
        self.capacity = capacity

    def trace_events(self):
        return [(1, 0, (3 << 16) | 64, 1000), (1, 1, (0 << 16) | 8, 1500), (2, 0, 7, 9000), (3, 1, 2, 9500), (2, 1, 4, 12000),
                (5, 1, 2, 13000)], 3


def test_role_aware_discovery_and_settings():
    cfg = types.SimpleNamespace(debug_fabric_observer_enable=True, debug_fabric_observer_record_capacity=128,
                                debug_graph_observer_enable=True, debug_transport_observer_enable=True,
                                debug_ffn_routing_observer_enable=False)
    lane = FakeLaneRuntime()
    s = devkit.observers_for_role("FfnAgent", cfg, lane_runtime=lane)
    assert [o.name for o in s.observers] == ["fabric", "graph"] and lane.capacity == 128   # transport is not an FFN-side observer
    assert [o.name for o in devkit.observers_for_role("Instance", cfg).observers] == ["transport"]
    assert devkit.observers_for_role("Daemon", cfg).observers == []
    off = types.SimpleNamespace()
    assert devkit.observers_for_role("FfnAgent", off, lane_runtime=lane).observers == []


def test_fabric_events_decode_and_pair_into_spans(tmp_path):
    obs = devkit.FabricObserver(FakeLaneRuntime(), out_dir=tmp_path)
    art = obs.collect()
    assert art.dropped == 3
    assert art.events[0] == {"name": "admitted", "ts_ns": 1000, "instance": 0, "layer": 3, "rows": 64}
    assert art.events[-1]["name"] == "rejected" and art.events[-1]["result_code"] == 2
    path = obs.write()
    assert json.loads(path.read_text())["observer"] == "fabric"
    tr = devkit.chrome_trace([art], host_spans=[{"name": "step", "ts_ns": 500, "dur_ns": 20000}])
    spans = [e for e in tr["traceEvents"] if e["ph"] == "X" and e.get("cat") == "lane"]
    assert [(e["name"], e["dur"]) for e in spans] == [("inst0 L3 rows=64", 8.0), ("inst1 L0 rows=8", 10.5)]
    assert tr["traceEvents"][0]["name"] == "step"          # sorted by time
    assert sum(1 for e in tr["traceEvents"] if e["ph"] == "i") == 2


def test_transport_observer_counts_overflow_without_wrapping():
    t = devkit.TransportObserver(capacity=4)
    for i in range(6):
        t.record(1 + (i % 3), i, 0)
    art = t.collect()
    assert len(art.events) == 4 and art.dropped == 2 and [e["a"] for e in art.events] == [0, 1, 2, 3]
    assert art.events[0]["name"] == "publish"


def test_graph_observer_snapshots_the_tile_plan_per_row_bucket():
    g = devkit.GraphObserver()
    inst = types.SimpleNamespace(model_id="q", cfg=PRESETS["Qwen/Qwen3-0.6B"], tp_size=1)
    g.snapshot_lane_graph([inst], row_buckets=(1, 256))
    nodes = g.collect().meta["nodes"]
    assert [n["rows"] for n in nodes] == [1, 256]
    assert nodes[0]["gateup"]["bn"] == 16 and nodes[1]["gateup"]["bn"] >= 64
    assert nodes[0]["down"]["splits"] >= 1 and nodes[0]["sequence"][0] == "lane_wait"


def test_routing_observer_keeps_a_bounded_number_of_samples(tmp_path):
    r = devkit.RoutingObserver(max_samples=2, out_dir=tmp_path)
    for l in range(3):
        r.capture(l, torch.randint(0, 8, (5, 2), dtype=torch.int32), torch.rand(5, 2))
    art = r.collect()
    assert len(art.events) == 2 and art.dropped == 1 and art.events[1]["top_k"] == 2
    p = r.write()
    from safetensors.torch import load_file

    t = load_file(str(p.with_suffix(".safetensors")))
    assert set(t) == {"sample0.layer0.ids", "sample0.layer0.weights", "sample1.layer1.ids", "sample1.layer1.weights"}


def test_lane_busy_summary_pairs_admissions_with_completions_per_instance():
    from crosspool_b200.devkit.observers import lane_busy_summary

    ev = [{"name": "discovered", "ts_ns": 1000, "instance": 0, "sequence": 1},
          {"name": "admitted", "ts_ns": 2000, "instance": 0, "layer": 0, "rows": 8},
          {"name": "admitted", "ts_ns": 2500, "instance": 1, "layer": 3, "rows": 4},
          {"name": "completed", "ts_ns": 42000, "instance": 0, "sequence": 1},
          {"name": "completed", "ts_ns": 62500, "instance": 1, "sequence": 1},
          {"name": "idle", "ts_ns": 101000, "lane": 0, "count": 1}]
    s = lane_busy_summary(ev, lanes=2)
    assert s["invocations"] == 2 and s["rows"] == 12
    assert s["busy_fraction"] == round((40000 + 60000) / (100000 * 2), 4)
    assert s["service_us"] == {"mean": 50.0, "p50": 40.0, "p99": 40.0}
    assert lane_busy_summary([], 2) == {"invocations": 0, "busy_fraction": 0.0}
