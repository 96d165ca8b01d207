"""Executor-Lane kernels on one GPU. The invocation is published *before* the Lane iteration is
enqueued, so nothing on the GPU waits for another launch: lane_wait finds the work at once, the two
GEMMs run from the descriptor table, lane_complete publishes the completion record."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(cfgs, n_lanes=1, policy=0, tile=False, cap=128):
    from crosspool_b200.models import config as mc
    from crosspool_b200.parallel import fabric as F

    ffn = F.FfnRankRuntime("cuda", n_lanes=n_lanes, policy=policy, tile_weights=tile)
    places, atn = [], []
    for i, (preset, layers) in enumerate(cfgs):
        cfg = mc.preset(preset).with_layers(layers)
        p = F.InstancePlacement(f"m{i}", cfg, seed=i + 1, atn_rank=0, ffn_ranks=(1,), capacity_rows=cap)
        st = ffn.add_instance(p, 0)
        buf = F.PeerBuffer(F.atn_slot_layout(p).total_bytes)  # stands in for the attention device's arena
        st.atn_base = buf.ptr
        places.append(p)
        atn.append(buf)
    ffn.install()
    return ffn, places, atn


def _publish(F, st, place, x, layer, seq, mode=2, deadline=0):
    flay = F.ffn_slot_layout(place)
    rows = x.shape[0]
    st.slot.tensor(flay.input_offset, (place.capacity_rows, place.cfg.hidden_size), torch.bfloat16, "cuda")[:rows] = x
    rec = st.slot.tensor(flay.record_offset, (64,), torch.int32, "cuda")
    rec[0], rec[1], rec[2], rec[3] = rows, layer, mode, deadline
    rec[8] = seq  # InvocationRecord.sequence
    torch.cuda.synchronize()


def _result(F, buf, place, rows):
    alay = F.atn_slot_layout(place)
    out = buf.tensor(alay.output_offset, (place.capacity_rows, place.cfg.hidden_size), torch.bfloat16, "cuda")[:rows]
    done = buf.tensor(alay.completion_offset, (64,), torch.int32, "cuda")
    return out.clone(), int(done[0]), int(done[1]), int(done[4])


def _ref(x, w):
    inter = w.gate_up.shape[0] // 2
    gu = (x.float() @ w.gate_up.float().t()).bfloat16().float()
    act = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).bfloat16().float()
    return act @ w.down.float().t()


@pytest.mark.parametrize("tile", [False, True])
@pytest.mark.parametrize("rows", [1, 7, 64, 128])
def test_lane_iteration_computes_the_layer_from_the_descriptor_table(rows, tile):
    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 3)], tile=tile)
    try:
        st, place = ffn.instances[0], places[0]
        for seq, layer in enumerate([2, 0, 1], start=1):
            x = (torch.randn(rows, place.cfg.hidden_size, device="cuda") * 0.5).bfloat16()
            _publish(F, st, place, x, layer, seq)
            ffn.launch_once(0, lease_ms=50)
            torch.cuda.synchronize()
            out, rc, nrows, done_seq = _result(F, atn[0], place, rows)
            assert (rc, nrows, done_seq) == (0, rows, seq)
            torch.testing.assert_close(out.float(), _ref(x, st.weights[layer]), atol=2e-2, rtol=2e-2)
        s = ffn.stats()
        assert s["served"] == [3] and s["status"] == 0
        gemm.check_status(torch.device("cuda"))
    finally:
        ffn.close()


def test_idle_lane_iteration_gives_up_after_its_lease_and_serves_later_work():
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 1)])
    try:
        ffn.launch_once(0, lease_ms=5)  # nothing published: the bounded wait runs out, GEMMs are no-ops
        torch.cuda.synchronize()
        s = ffn.stats()
        assert s["served"] == [0] and s["idle_replays"] == [1] and s["status"] == 0
        st, place = ffn.instances[0], places[0]
        x = (torch.randn(4, place.cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        _publish(F, st, place, x, 0, 1)
        ffn.launch_once(0, lease_ms=5)
        torch.cuda.synchronize()
        out, rc, nrows, seq = _result(F, atn[0], place, 4)
        assert (rc, nrows, seq) == (0, 4, 1)
        torch.testing.assert_close(out.float(), _ref(x, st.weights[0]), atol=2e-2, rtol=2e-2)
    finally:
        ffn.close()


def test_two_models_share_one_lane_in_fifo_order_and_bad_records_are_refused():
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 2), ("Qwen/Qwen3-1.7B", 1)])
    try:
        xs = []
        for i, (st, place) in enumerate(zip(ffn.instances, places)):
            x = (torch.randn(5 + i, place.cfg.hidden_size, device="cuda") * 0.5).bfloat16()
            xs.append(x)
            _publish(F, st, place, x, 0, 1)
        ffn.launch_once(0, lease_ms=20)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        for i, (st, place) in enumerate(zip(ffn.instances, places)):
            out, rc, nrows, seq = _result(F, atn[i], place, 5 + i)
            assert (rc, nrows, seq) == (0, 5 + i, 1)
            torch.testing.assert_close(out.float(), _ref(xs[i], st.weights[0]), atol=2e-2, rtol=2e-2)
        assert ffn.stats()["served"] == [1, 1]
        # a record naming a layer that does not exist is answered with ProtocolMismatch, not executed
        _publish(F, ffn.instances[0], places[0], xs[0], 99, 2)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        _, rc, nrows, seq = _result(F, atn[0], places[0], 5)
        assert (rc, nrows, seq) == (2, 0, 2)
    finally:
        ffn.close()


def test_fabric_observer_records_lane_events_in_order_and_counts_overflow():
    from crosspool_b200 import devkit
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 1)])
    try:
        ffn.enable_trace(6)
        st, place = ffn.instances[0], places[0]
        ffn.launch_once(0, lease_ms=2)                      # idle
        x = (torch.randn(3, place.cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        for seq in (1, 2):
            _publish(F, st, place, x, 0, seq)
            ffn.launch_once(0, lease_ms=20)
            torch.cuda.synchronize()
        art = devkit.FabricObserver(ffn).collect()
        names = [e["name"] for e in art.events]
        # capacity 6, never wraps: the second invocation's completion does not fit
        assert names == ["idle", "discovered", "admitted", "completed", "discovered", "admitted"] and art.dropped == 1
        assert art.events[2]["rows"] == 3 and art.events[2]["layer"] == 0 and art.events[3]["sequence"] == 1
        ts = [e["ts_ns"] for e in art.events]
        assert ts == sorted(ts)
    finally:
        ffn.close()


def _moe_cfg(E=8, k=2, hidden=256, inter=128, layers=1, shared=0, **kw):
    from crosspool_b200.models.config import ModelConfig

    return ModelConfig(name="tmoe", architecture="Qwen3MoeForCausalLM", hidden_size=hidden, num_layers=layers, num_q_heads=4,
                       num_kv_heads=2, head_dim=64, intermediate_size=inter, vocab_size=128, num_experts=E,
                       num_experts_per_tok=k, moe_intermediate_size=inter, num_shared_experts=shared, **kw)


@pytest.mark.parametrize("precision,scoring", [("fp32_logits", "softmax"), ("fp32", "sigmoid")])
def test_lane_routes_with_an_fp32_router_projection(precision, scoring):
    """A layer whose router asks for fp32 logits is served by the Lane's SIMT projection node; a payload-precision
    layer of a second model keeps the tensor-core projection in the same graph."""
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.parallel import fabric as F

    rows = 37
    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    cfgs = [_moe_cfg(64, 4, 1024, 256, router_precision=precision, router_scoring=scoring), _moe_cfg(8, 2, 256, 128)]
    places, atn = [], []
    for i, cfg in enumerate(cfgs):
        p = F.InstancePlacement(f"m{i}", cfg, seed=i + 11, atn_rank=0, ffn_ranks=(1,), capacity_rows=128)
        st = ffn.add_instance(p, 0)
        buf = F.PeerBuffer(F.atn_slot_layout(p).total_bytes)
        st.atn_base = buf.ptr
        places.append(p)
        atn.append(buf)
    ffn.install()
    try:
        g = torch.Generator(device="cuda").manual_seed(rows)
        xs = [(torch.randn(rows, c.hidden_size, device="cuda", generator=g) * 0.5).bfloat16() for c in cfgs]
        for i in (0, 1):
            _publish(F, ffn.instances[i], places[i], xs[i], 0, 1)
        ffn.launch_once(0, lease_ms=20)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        assert ffn.stats()["status"] == 0 and ffn.stats()["served"] == [1, 1]
        for i in (0, 1):
            out, rc, nrows, _ = _result(F, atn[i], places[i], rows)
            assert (rc, nrows) == (0, rows)
            ref = moe_ffn(xs[i], ffn.instances[i].weights[0], cfgs[i]).float()
            err = (out.float() - ref).abs()
            assert (err.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-9)).item() < 0.03, i
    finally:
        ffn.close()


@pytest.mark.parametrize("E,k,hidden,inter,rows", [(8, 2, 256, 128, 7), (128, 8, 2048, 768, 64), (128, 8, 2048, 768, 1)])
def test_lane_serves_a_moe_layer_and_a_dense_model_from_one_graph(E, k, hidden, inter, rows):
    from crosspool_b200.models import config as mc
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.parallel import fabric as F

    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    cfgs = [_moe_cfg(E, k, hidden, inter), mc.preset("Qwen/Qwen3-0.6B").with_layers(1)]
    places, atn = [], []
    for i, cfg in enumerate(cfgs):
        p = F.InstancePlacement(f"m{i}", cfg, seed=i + 3, atn_rank=0, ffn_ranks=(1,), capacity_rows=128)
        st = ffn.add_instance(p, 0)
        buf = F.PeerBuffer(F.atn_slot_layout(p).total_bytes)
        st.atn_base = buf.ptr
        places.append(p)
        atn.append(buf)
    ffn.install()
    try:
        g = torch.Generator(device="cuda").manual_seed(rows)
        xs = [(torch.randn(rows, c.hidden_size, device="cuda", generator=g) * 0.5).bfloat16() for c in cfgs]
        for i in (0, 1):
            _publish(F, ffn.instances[i], places[i], xs[i], 0, 1)
        ffn.launch_once(0, lease_ms=20)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        assert ffn.stats()["status"] == 0 and ffn.stats()["served"] == [1, 1]
        out, rc, nrows, seq = _result(F, atn[0], places[0], rows)
        assert (rc, nrows, seq) == (0, rows, 1)
        ref = moe_ffn(xs[0], ffn.instances[0].weights[0], cfgs[0]).float()
        err = (out.float() - ref).abs()
        assert (err.max() / ref.abs().max().clamp_min(1e-6)).item() < 0.05
        assert (err.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-9)).item() < 0.02
        out1, rc1, _, _ = _result(F, atn[1], places[1], rows)
        assert rc1 == 0
        torch.testing.assert_close(out1.float(), _ref(xs[1], ffn.instances[1].weights[0]), atol=2e-2, rtol=2e-2)
    finally:
        ffn.close()


def test_lane_moe_layer_with_expert_biases_and_gate_transform():
    """A GPT-OSS shaped expert layer in a Lane: per-expert biases on both grouped projections, router bias,
    clamped activation with offset and sigmoid slope."""
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.parallel import fabric as F
    from crosspool_b200.testing import assert_ffn_close

    E, k, hidden, inter, rows = 8, 2, 256, 128, 21
    cfg = _moe_cfg(E, k, hidden, inter)
    place = F.InstancePlacement("m", cfg, seed=4, atn_rank=0, ffn_ranks=(1,), capacity_rows=64)
    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    st = ffn.add_instance(place, 0)
    w = st.weights[0]
    g = torch.Generator(device="cuda").manual_seed(2)
    w.gate_up_bias = torch.randn(E, 2 * inter, device="cuda", generator=g) * 0.3
    w.down_bias = torch.randn(E, hidden, device="cuda", generator=g) * 0.3
    w.extra["router_bias"] = torch.randn(E, device="cuda", generator=g) * 0.5
    w.extra["gate_transform"] = (1.5, 1.0, 1.702)
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    st.atn_base = buf.ptr
    ffn.install()
    try:
        x = (torch.randn(rows, hidden, device="cuda", generator=g) * 0.5).bfloat16()
        _publish(F, st, place, x, 0, 1)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        out, rc, nrows, seq = _result(F, buf, place, rows)
        assert (rc, nrows, seq) == (0, rows, 1) and ffn.stats()["status"] == 0
        assert_ffn_close(out.float(), moe_ffn(x, w, cfg).float())
    finally:
        ffn.close()


def test_expert_parallel_lane_partials_fold_to_the_full_moe_output():
    """Two FFN ranks' runtimes (run one after the other here; they never wait on each other) each own
    half of the experts; the rank-order fp32 fold of their partials equals the full layer."""
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.models.weights import random_ffn_layer
    from crosspool_b200.parallel import fabric as F

    cfg = _moe_cfg(16, 4, 512, 256)
    place = F.InstancePlacement("m", cfg, seed=9, atn_rank=0, ffn_ranks=(1, 2), capacity_rows=64)
    assert place.expert_parallel and place.expert_range(1) == (8, 16)
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    x = (torch.randn(33, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
    rts = []
    try:
        for r in (0, 1):
            ffn = F.FfnRankRuntime("cuda", n_lanes=1)
            rts.append(ffn)
            st = ffn.add_instance(place, r)
            st.atn_base = buf.ptr
            ffn.install()
            _publish(F, st, place, x, 0, 1)
            ffn.launch_once(0, lease_ms=20)
            torch.cuda.synchronize()
            assert ffn.stats()["status"] == 0
        alay = F.atn_slot_layout(place)
        parts = [buf.tensor(alay.output_offset + r * alay.output_stride, (64, cfg.hidden_size), torch.bfloat16, "cuda")[:33]
                 for r in (0, 1)]
        full = random_ffn_layer(cfg, 0, 9, "cuda", torch.bfloat16)
        ref = moe_ffn(x, full, cfg).float()
        got = parts[0].float() + parts[1].float()
        err = (got - ref).abs()
        assert (err.max() / ref.abs().max()).item() < 0.05
    finally:
        for ffn in rts:
            ffn.close()
        buf.free()


def test_slo_policy_serves_the_earliest_deadline_first():
    from crosspool_b200 import devkit
    from crosspool_b200.native import runtime as rt
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 1)] * 3, policy=rt.POLICY_SLO)
    try:
        ffn.enable_trace(64)
        for i, dl in enumerate((9000, 0, 100)):          # instance 1 carries no deadline: it goes last
            x = (torch.randn(2, places[i].cfg.hidden_size, device="cuda") * 0.5).bfloat16()
            _publish(F, ffn.instances[i], places[i], x, 0, 1, deadline=dl)
        for _ in range(3):
            ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        ev = devkit.FabricObserver(ffn).collect().events
        assert [e["instance"] for e in ev if e["name"] == "admitted"] == [2, 0, 1]
        assert ffn.stats()["served"] == [1, 1, 1] and ffn.stats()["status"] == 0
    finally:
        ffn.close()


def test_a_rank_refuses_layers_of_another_layer_group():
    from crosspool_b200.models import config as mc
    from crosspool_b200.parallel import fabric as F

    cfg = mc.preset("Qwen/Qwen3-0.6B").with_layers(2)
    place = F.InstancePlacement("m", cfg, seed=2, atn_rank=0, ffn_ranks=(1, 2), capacity_rows=64,
                                layer_groups=((0, 1, (1,)), (1, 2, (2,))))
    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    st = ffn.add_instance(place, *place.locate(2)[:1], place.locate(2)[1:])      # this rank holds layer 1 only
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    st.atn_base = buf.ptr
    ffn.install()
    try:
        assert st.weights[0] is None and st.weights[1] is not None
        x = (torch.randn(4, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        _publish(F, st, place, x, 1, 4)                           # sequence numbers may jump: other groups served 1..3
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        out, rc, nrows, seq = _result(F, buf, place, 4)
        assert (rc, nrows, seq) == (0, 4, 4)
        torch.testing.assert_close(out.float(), _ref(x, st.weights[1]), atol=2e-2, rtol=2e-2)
        _publish(F, st, place, x, 0, 5)                           # a layer of the other group
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        _, rc, nrows, seq = _result(F, buf, place, 4)
        assert (rc, nrows, seq) == (2, 0, 5)                      # ProtocolMismatch, nothing computed
        f = ffn.failure()                                         # ... and the generation's canonical failure
        assert f is not None and (f.result_code, f.invocation_sequence, f.layer_ordinal) == (2, 5, 0)
    finally:
        ffn.close()
        buf.free()


@pytest.mark.parametrize("rows", [5, 70])
def test_lane_adds_shared_experts_to_the_routed_output(rows):
    from crosspool_b200.models.reference import moe_ffn
    from crosspool_b200.parallel import fabric as F

    cfg = _moe_cfg(16, 4, 512, 256, shared=2)
    place = F.InstancePlacement("m", cfg, seed=11, atn_rank=0, ffn_ranks=(1,), capacity_rows=128)
    ffn = F.FfnRankRuntime("cuda", n_lanes=1)
    st = ffn.add_instance(place, 0)
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    st.atn_base = buf.ptr
    ffn.install()
    try:
        assert st.weights[0].shared_gate_up.shape == (2 * 2 * 256, 512)
        x = (torch.randn(rows, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        _publish(F, st, place, x, 0, 1)
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        assert ffn.stats()["status"] == 0
        out, rc, nrows, seq = _result(F, buf, place, rows)
        assert (rc, nrows, seq) == (0, rows, 1)
        ref = moe_ffn(x, st.weights[0], cfg).float()
        err = (out.float() - ref).abs()
        assert (err.max() / ref.abs().max().clamp_min(1e-6)).item() < 0.05
        assert (err.pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()).item() < 0.02
    finally:
        ffn.close()
        buf.free()


def test_native_replay_threads_serve_invocations_without_a_python_thread():
    """The library's own replay threads keep Lane iterations enqueued (2 ms leases, so no iteration outlives the test
    step); the host publishes invocations with plain copies and polls the completion record. No kernel here needs
    another launch to run at the same time: an idle iteration simply ends with its lease."""
    import time

    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 2)], n_lanes=2)
    try:
        st, place = ffn.instances[0], places[0]
        flay, alay = F.ffn_slot_layout(place), F.atn_slot_layout(place)
        ffn.start(lease_ms=2.0, depth=3)
        side = torch.cuda.Stream()
        inp = st.slot.tensor(flay.input_offset, (place.capacity_rows, place.cfg.hidden_size), torch.bfloat16, "cuda")
        rec = st.slot.tensor(flay.record_offset, (64,), torch.int32, "cuda")
        done = atn[0].tensor(alay.completion_offset, (64,), torch.int32, "cuda")
        out = atn[0].tensor(alay.output_offset, (place.capacity_rows, place.cfg.hidden_size), torch.bfloat16, "cuda")
        done_host = torch.zeros(64, dtype=torch.int32).pin_memory()
        for seq, (layer, rows) in enumerate([(0, 5), (1, 64), (0, 1)], start=1):
            x = (torch.randn(rows, place.cfg.hidden_size) * 0.5).bfloat16().pin_memory()
            rec_host = torch.zeros(64, dtype=torch.int32).pin_memory()
            rec_host[0], rec_host[1], rec_host[2], rec_host[8] = rows, layer, 2, seq
            with torch.cuda.stream(side):
                inp[:rows].copy_(x, non_blocking=True)      # payload first, then the record that names it
                side.synchronize()
                rec.copy_(rec_host, non_blocking=True)
                side.synchronize()
                t0 = time.monotonic()
                while True:
                    done_host.copy_(done, non_blocking=True)
                    side.synchronize()
                    if int(done_host[4]) == seq or time.monotonic() - t0 > 10:
                        break
                    time.sleep(0.001)
                assert (int(done_host[0]), int(done_host[1]), int(done_host[4])) == (0, rows, seq)
                got = out[:rows].float().cpu()
            torch.testing.assert_close(got, _ref(x.cuda(), st.weights[layer]).cpu(), atol=2e-2, rtol=2e-2)
        s = ffn.stats()
        assert s["served"] == [3] and s["status"] == 0 and s["replays"] >= 3
        ffn.stop()
        assert not ffn.errors
        gemm.check_status(torch.device("cuda"))
    finally:
        ffn.close()


def test_a_rejected_invocation_becomes_the_canonical_failure_and_cancels_waits_at_once():
    """First failure wins: the Lane that refuses a bad record claims the device's failure slot and copies it into the
    attention-side slot; a wait that polls that slot as its cancel word returns at once instead of running into its
    limit, the hook points record both sides, and later Lane iterations serve nothing more."""
    import time

    from crosspool_b200 import devkit, native
    from crosspool_b200.ops import gemm
    from crosspool_b200.parallel import fabric as F

    ffn, places, atn = _make([("Qwen/Qwen3-0.6B", 2)])
    try:
        ffn.enable_trace(64)
        st, place = ffn.instances[0], places[0]
        alay = F.atn_slot_layout(place)
        assert ffn.failure() is None
        x = (torch.randn(3, place.cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        _publish(F, st, place, x, 77, 1)                      # no such layer
        ffn.launch_once(0, lease_ms=20)
        torch.cuda.synchronize()
        f = ffn.failure()
        assert f is not None and (f.result_code, f.origin_pe, f.instance_index, f.invocation_sequence, f.layer_ordinal) == (2, 0, 0, 1, 77)
        words = atn[0].tensor(alay.completion_offset + F.FAILURE_SLOT_OFFSET, (8,), torch.int32, "cuda").cpu().tolist()
        assert F.FabricFailure.from_words(words) == f         # the attention side holds the same payload
        # a wait for a completion that will never come: cancelled by the failure word, far inside its 2 s limit
        w = native.WaitArgs()
        w.flags[0] = atn[0].ptr + alay.completion_offset + F.COMPLETION_SEQ_OFFSET
        w.n, w.want, w.wait_ns = 1, 9, 2_000_000_000
        w.cancel = atn[0].ptr + alay.completion_offset + F.FAILURE_SLOT_OFFSET
        status = gemm.status_words(torch.device("cuda"))
        status.zero_()
        w.status = status.data_ptr()
        trace = F.DeviceTrace(16)
        w.trace_events, w.trace_state, w.trace_capacity = trace.args()
        t0 = time.monotonic()
        native.check(native.kernels().xp_wait_flags(C.byref(w), torch.cuda.current_stream().cuda_stream), "xp_wait_flags")
        torch.cuda.synchronize()
        assert time.monotonic() - t0 < 0.5 and int(status[0]) == 5
        status.zero_()
        kinds = [k for k, _, _, _ in trace.read()[0]]
        assert kinds == [18, 21]                              # wait_begin, wait_cancelled
        trace.close()
        # the generation is failed: a valid invocation published afterwards is not served
        _publish(F, st, place, x, 0, 2)
        ffn.launch_once(0, lease_ms=5)
        torch.cuda.synchronize()
        assert ffn.stats()["served"] == [1]
        names = [e["name"] for e in devkit.FabricObserver(ffn).collect().events]
        assert names[:4] == ["discovered", "rejected", "failure_claimed", "admitted"] and "failure_observed" in names
    finally:
        ffn.close()
