"""The engine integration driven end to end against a stand-in engine: ``plugin.install`` registers its hooks with a
registry that really patches the (fake) engine classes; constructing the engine's scheduler then runs the whole Instance
start-up (adapter, filtered load, shims, registration, Fabric wait, arena lease, bound operator), a forward goes through
``torch.ops.xpool.ffn_shim``, and retirement happens in order."""
import types

import pytest
import torch

from crosspool_b200.integrations.sglang import plugin, shim
from crosspool_b200.integrations.sglang.shutdown import ShutdownHookSet
from crosspool_b200.integrations.sglang.topology import AttentionTopology, ModelShape, TopologyError
from crosspool_b200.integrations.sglang.worker import EXIT_RETAINED, EXIT_WORKER_FAILED, WorkerLifecycle
from crosspool_b200.native import runtime as rt
from crosspool_b200.runtime.instance import InstanceFailure, InstanceRankFailureMonitor, InstanceRankRuntime, InstanceStartupError
from tests.sglang_fakes import FakeDaemonClient, PatchingHookRegistry, install_fake_engine


def _config(tp=1, dp=1):
    m = types.SimpleNamespace(id="Qwen/Qwen3-0.6B", path="/models/qwen3", atn_tp_size=tp, atn_dp_size=dp)
    return types.SimpleNamespace(models=(m,), model=lambda _id: m)


def _server_args(**kw):
    d = dict(model_path="/models/qwen3", tp_size=1, dp_size=1, tp_rank=0, chunked_prefill_size=2048, cuda_graph_max_bs=64,
             max_running_requests=48, cuda_graph_bs=[1, 2, 4, 8, 16, 32, 64],
             cuda_graph_backend_decode="full", cuda_graph_backend_prefill="breakable", host="127.0.0.1", port=30000)
    d.update(kw)
    return types.SimpleNamespace(**d)


@pytest.fixture()
def engine():
    fake = install_fake_engine()
    reg = PatchingHookRegistry()
    yield fake, reg
    reg.restore()
    shim.bind_submit(None)


def test_install_drives_the_whole_instance_startup_and_a_forward_reaches_the_ffn_boundary(engine):
    fake, reg = engine
    client = FakeDaemonClient("Qwen/Qwen3-0.6B")
    ffn_calls, made = [], {}

    def attach(arena, plan):
        def submit(h, rows, out, layer, mode, req, layout):      # stands in for the FFN tier
            ffn_calls.append((layer, mode, req, layout, tuple(h.shape)))
            out.copy_(h * 0.5)
        shim.bind_submit(submit)
        made["transport"] = types.SimpleNamespace(failure=lambda: None, close=lambda: made.__setitem__("closed", True))
        return made["transport"]

    def runtime_factory(binding, rank, profile, device):
        made["runtime"] = InstanceRankRuntime(client, binding.model_id, rank, device, profile, attach=attach, sleep=lambda s: None)
        return made["runtime"]

    hooks = plugin.install(reg, environ={}, config=_config(), runtime_factory=runtime_factory)
    assert {h.target for h in hooks} >= reg.applied_targets() >= {
        "sglang.srt.models.qwen3.Qwen3MLP", "sglang.srt.models.qwen3.Qwen3ForCausalLM.load_weights",
        "sglang.srt.model_executor.model_runner.ModelRunner.load_model", "sglang.srt.managers.scheduler.Scheduler.__init__"}

    sched = fake.sched.Scheduler(_server_args())
    model = sched.model_runner.model
    # every decoder MLP is a shim, the attention side holds and loaded no FFN tensor
    assert [type(l.mlp).__name__ for l in model.model.layers] == ["FfnShimModule"] * 3
    assert [l.mlp.layer_ordinal for l in model.model.layers] == [0, 1, 2]
    assert not any(".mlp." in n for n in model.loaded) and "model.layers.1.self_attn.weight" in model.loaded
    assert not any(".mlp." in n for n, _ in model.named_parameters())
    # the Instance rank registered with the row capacities derived from the launch arguments, waited, leased its arena
    kinds = [c[0] for c in client.calls]
    assert kinds[:2] == ["register", "acquire"] and client.calls[0][3:] == (2048, 64) and client.calls[1][3] == 7
    scope = plugin.install.lifecycle.scope
    assert scope.events == ["scheduler_init", "load_model", "alloc_memory_pool"] and made["runtime"].state == "attached"
    assert sched.get_init_info() == {"status": "ready"}
    assert ("initialized", "Qwen/Qwen3-0.6B", 0, 7) in client.calls and made["runtime"].state == "ready"
    # a forward pass: three layers, three FFN invocations in layer order through the operator
    fb = types.SimpleNamespace(forward_mode=types.SimpleNamespace(name="DECODE"), dp_padding_mode=None)
    y = model(torch.ones(4, 8), fb)
    assert torch.isfinite(y).all()
    assert [c[0] for c in ffn_calls] == [0, 1, 2] and all(c[1:] == (rt.MODE_DECODE, rt.OUT_PER_RANK_COMPLETE, rt.DP_NONE, (4, 8)) for c in ffn_calls)
    # the failure monitor lives for the life of the event loop
    assert sched.run_event_loop() == "loop-done" and made["runtime"].monitor is not None
    # ordered retirement: admission closed, drained, detached (lease returned, heartbeat stopped), then the engine's own release
    assert sched.release_host_resources() == "released"
    assert scope.shutdown.report.completed == ["stop_admission", "drain_in_flight", "detach_instance"]
    assert made.get("closed") and client.calls[-1][0] == "deregister" and made["runtime"].state == "detached"


def test_unconfirmed_cleanup_retains_the_owner_and_skips_the_engines_release(engine):
    fake, reg = engine
    client = FakeDaemonClient("Qwen/Qwen3-0.6B", warm=0)
    plugin.install(reg, environ={}, config=_config(),
                   runtime_factory=lambda b, r, p, d: InstanceRankRuntime(client, b.model_id, r, d, p, sleep=lambda s: None))
    sched = fake.sched.Scheduler(_server_args())
    sched.xpool_drain = lambda deadline: False          # a step in flight never finished
    assert sched.release_host_resources() is None
    assert sched.xpool_retained == "drain_in_flight" and "released" not in sched.log
    assert plugin.install.lifecycle.scope.shutdown.report.retained


def test_launch_arguments_and_topology_are_checked_before_anything_is_loaded(engine):
    fake, reg = engine
    plugin.install(reg, environ={}, config=_config(tp=2), runtime_factory=lambda *a: pytest.fail("must not start"))
    with pytest.raises(Exception, match="tensor-parallel-size"):
        fake.sched.Scheduler(_server_args(tp_size=1))
    shape = ModelShape.load({"architectures": ["X"], "hidden_size": 64, "num_attention_heads": 6, "num_key_value_heads": 2})
    with pytest.raises(TopologyError, match="query heads"):
        shape.validate_attention_tp(4)
    shape.validate_attention_tp(2)
    with pytest.raises(TopologyError, match="combined"):
        AttentionTopology.from_runtime(_server_args(tp_size=4), shape, atn_tp_size=2, atn_dp_size=2, supports_dp_attention=True)
    t = AttentionTopology.from_runtime(_server_args(tp_size=2, tp_rank=1), shape, atn_tp_size=2, atn_dp_size=1, supports_dp_attention=False)
    assert (t.tp_rank, t.dp_rank, t.instance_rank) == (1, 0, 1)
    mla = ModelShape.load({"hidden_size": 64, "num_attention_heads": 8, "kv_lora_rank": 512})
    assert mla.latent_attention and mla.kv_heads_per_rank(4) == 1


def test_instance_runtime_times_out_and_reports_generation_failures():
    t = [0.0]
    client = FakeDaemonClient("m", warm=10 ** 9)
    prof = types.SimpleNamespace(max_prefill_rows=1, max_decode_rows=1)
    r = InstanceRankRuntime(client, "m", 0, 0, prof, owner=types.SimpleNamespace(), clock=lambda: t[0],
                            sleep=lambda s: t.__setitem__(0, t[0] + s))
    with pytest.raises(InstanceStartupError, match="not executable after 5 s"):
        r.wait_for_fabric_executable(timeout_s=5.0, poll_s=1.0)
    failing = FakeDaemonClient("m", warm=0, fail="ffnagent 1 exited")
    r2 = InstanceRankRuntime(failing, "m", 0, 0, prof, owner=types.SimpleNamespace())
    with pytest.raises(InstanceStartupError, match="exited"):
        r2.wait_for_fabric_executable(timeout_s=5.0)


def test_failure_monitor_fires_once_and_worker_lifecycle_maps_outcomes_to_exit_codes():
    seen, state = [], {"f": None}
    mon = InstanceRankFailureMonitor(lambda: state["f"], seen.append)
    assert mon.poll_once() is None
    state["f"] = InstanceFailure(3, 2, 41, 7)
    assert mon.poll_once().origin_pe == 2 and mon.poll_once() is not None and len(seen) == 1
    codes, reports = [], []
    shut = ShutdownHookSet().add("a", lambda d: True)
    assert WorkerLifecycle("scheduler", reports.append, shut, codes.append).run(lambda: "ok") == "ok" and codes == []

    def boom():
        raise RuntimeError("cuda error")
    WorkerLifecycle("scheduler", reports.append, ShutdownHookSet().add("a", lambda d: True), codes.append).run(boom)
    WorkerLifecycle("scheduler", reports.append, ShutdownHookSet().add("a", lambda d: False), codes.append).run(boom)
    assert codes == [EXIT_WORKER_FAILED, EXIT_RETAINED] and "cuda error" in reports[0]


def test_elastic_hooks_cut_prefill_to_backing_publish_demand_and_retract_newest_first(engine):
    from crosspool_b200.engine.kv_cache import PageAllocator, PagedKvCache, KvLayout
    from crosspool_b200.integrations.sglang.ecs_hooks import ElasticContextState, ElasticHooks

    class Rec:
        def __init__(self):
            self.log = []

        def poll(self):
            self.log.append("poll")

        def publish_demand(self, pages, deadline_ns=0):
            self.log.append(("demand", pages, deadline_ns))

        def withdraw_demand(self):
            self.log.append("withdraw")

    cache = PagedKvCache(KvLayout(16, 8, 2, 64, 1), [], [], PageAllocator(8))
    rec = Rec()
    st = ElasticContextState(cache, rec, page_size=16, ttft_slo_s=2.0)
    hooks = ElasticHooks(lambda: st)
    sched = types.SimpleNamespace()
    adder = types.SimpleNamespace(rem_chunk_tokens=4096, can_run_list=[], scheduler=sched, reserve_pages=2)
    req = types.SimpleNamespace(rid=1, extend_input_len=500, prefix_len=0, arrival_s=10.0)
    assert hooks.add_one_req(adder, req) == 6 * 16            # 8 pages free, 2 reserved
    assert adder.can_run_list == [(req, 96)] and sched.xpool_missing_pages == 32 - 6 and st.stats["prefill_cut"] == 1
    out = hooks.get_next_batch_to_run(lambda s: "batch", sched)
    assert out == "batch" and rec.log == ["poll", ("demand", 26, int(12.0 * 1e9))]
    # decode: 2 pages left; three sequences cross a page boundary -> the newest is retracted
    for rid, n in ((2, 16), (3, 16)):
        cache.ensure(rid, n)
    assert cache.allocator.free_pages == 0
    batch = types.SimpleNamespace(reqs=[types.SimpleNamespace(rid=1), types.SimpleNamespace(rid=2), types.SimpleNamespace(rid=3)],
                                  seq_lens=[96, 16, 16])
    assert not hooks.check_decode_mem(batch)
    gone = hooks.retract_decode(batch)
    assert [r.rid for r in gone] == [3, 2] and [r.rid for r in batch.reqs] == [1] and st.stats["retracted"] == 2


def test_ffn_profile_is_derived_strictly_from_the_resolved_serving_state():
    import torch

    from crosspool_b200.integrations.sglang import lifecycle as L
    from crosspool_b200.integrations.sglang.adapter import InstanceRankBinding

    def runner(**sa):
        args = dict(chunked_prefill_size=2048, max_running_requests=48, cuda_graph_bs=[1, 8, 64], cuda_graph_max_bs=64)
        args.update(sa)
        return types.SimpleNamespace(server_args=types.SimpleNamespace(**args), model_config=types.SimpleNamespace(dtype=torch.bfloat16))

    shims = [types.SimpleNamespace(layer_ordinal=1, hidden_size=64, layer_kind="moe"),
             types.SimpleNamespace(layer_ordinal=0, hidden_size=64, layer_kind="dense")]
    p = L.derive_instance_ffn_profile(runner(), 64, shims)
    assert (p.max_prefill_rows, p.max_decode_rows, p.payload_dtype, p.layer_kinds) == (2048, 64, "bfloat16", ["dense", "moe"])
    assert not p.group_sum_complete_admitted
    # graphs off: the eager limit alone; attention DP: one invocation carries every rank's rows and may ask for the sum
    assert L.derive_instance_ffn_profile(runner(disable_cuda_graph=True), 64, shims).max_decode_rows == 48
    dp = L.derive_instance_ffn_profile(runner(enable_dp_attention=True, dp_size=4), 64, shims, dp_size=4)
    assert (dp.max_prefill_rows, dp.max_decode_rows, dp.group_sum_complete_admitted) == (8192, 256, True)
    for bad, match in ((dict(cuda_graph_bs=[8, 0]), "bucket"), (dict(cuda_graph_max_bs=-1), "maximum"),
                       (dict(max_running_requests=True), "eager decode")):
        with pytest.raises(L.ProfileError, match=match):
            L.derive_instance_ffn_profile(runner(**bad), 64, shims)
    with pytest.raises(L.ProfileError, match="no FFN shim"):
        L.derive_instance_ffn_profile(runner(), 64, [])
    with pytest.raises(L.ProfileError, match="hidden size"):
        L.derive_instance_ffn_profile(runner(), 64, [types.SimpleNamespace(layer_ordinal=0, hidden_size=128)])
    for other in (torch.float32, torch.float16, "float16"):      # the operator carries bf16 rows only: refused at registration
        wide = runner()
        wide.model_config.dtype = other
        with pytest.raises(L.ProfileError, match="bfloat16 only"):
            L.derive_instance_ffn_profile(wide, 64, shims)
    b = InstanceRankBinding("m", rank=5, tp_size=2, dp_size=4)
    t = L.InstanceRankTransportProfile.derive(b, dp)
    assert (t.payload_row_capacity, t.atn_tp_rank, t.atn_tp_size, t.atn_dp_rank, t.atn_dp_size) == (8192, 1, 2, 2, 4)


def test_topology_checks_cover_kinds_context_parallelism_and_both_directions_of_the_dp_switch():
    mk = lambda **kw: ModelShape.load({"hidden_size": 64, "num_attention_heads": 8, **kw})
    assert mk().attention_kind == "mha" and mk(num_key_value_heads=2).attention_kind == "gqa"
    assert mk(num_key_value_heads=1).attention_kind == "mqa" and mk(kv_lora_rank=16).attention_kind == "mla"
    assert mk(num_key_value_heads="2", hidden_size=64.0).num_kv_heads == 2
    for bad in ({"num_key_value_heads": 2.5}, {"num_attention_heads": True}, {"num_key_value_heads": 16}):
        with pytest.raises(TopologyError):
            mk(**bad)
    with pytest.raises(TopologyError, match="lacks hidden_size"):
        ModelShape.load({"num_attention_heads": 8})
    shape = mk(num_key_value_heads=2)
    ok = dict(atn_tp_size=1, atn_dp_size=2, supports_dp_attention=True)
    t = AttentionTopology.from_runtime(_server_args(tp_size=2, dp_size=2, enable_dp_attention=True, tp_rank=1), shape, **ok)
    assert (t.tp_rank, t.dp_rank, t.instance_rank) == (0, 1, 1)
    with pytest.raises(TopologyError, match="context parallel"):
        AttentionTopology.from_runtime(_server_args(tp_size=2, dp_size=2, enable_dp_attention=True, attn_cp_size=2), shape, **ok)
    with pytest.raises(TopologyError, match="must be set"):
        AttentionTopology.from_runtime(_server_args(tp_size=2, dp_size=2), shape, **ok)
    with pytest.raises(TopologyError, match="must be unset"):
        AttentionTopology.from_runtime(_server_args(tp_size=2, enable_dp_attention=True), shape, atn_tp_size=2, atn_dp_size=1,
                                       supports_dp_attention=True)
    with pytest.raises(TopologyError, match="data-parallel-size must be 2"):
        AttentionTopology.from_runtime(_server_args(tp_size=2, dp_size=1, enable_dp_attention=True), shape, **ok)
    with pytest.raises(TopologyError, match="positive integer"):
        AttentionTopology.from_runtime(_server_args(), shape, atn_tp_size=0, atn_dp_size=1, supports_dp_attention=False)
