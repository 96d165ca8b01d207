"""Graph observer and static request limits of the serving-engine integration, on fakes (no engine, no GPU)."""
import json

import pytest

from crosspool_b200.integrations.sglang import devkit


class _Backend:
    pass


class FakeDecodeRunner:
    def __init__(self, model_id):
        self.model_id, self.backend, self.calls = model_id, _Backend(), []

    def capture(self):
        self.calls.append("capture")
        return "captured"

    def execute(self, batch, fail=False):
        if fail:
            raise RuntimeError("replay failed")
        self.calls.append(("execute", batch))
        return batch * 2


class FakePrefillRunner(FakeDecodeRunner):
    pass


def test_graph_observer_records_begin_end_and_error_per_process_file(tmp_path):
    clock = iter(range(1000, 2000))
    obs = devkit.GraphObserver(tmp_path / "obs", clock=lambda: next(clock))
    obs.install({"decode": FakeDecodeRunner, "prefill": FakePrefillRunner})
    obs.install({"decode": FakeDecodeRunner})          # a second install wraps nothing twice
    try:
        d, p = FakeDecodeRunner("m0"), FakePrefillRunner("m1")
        assert d.capture() == "captured" and d.execute(3) == 6 and p.execute(4) == 8
        with pytest.raises(RuntimeError, match="replay failed"):
            d.execute(1, fail=True)
        events = devkit.read_graph_events(tmp_path / "obs")
        assert [(e["forward_phase"], e["event"], e["model_id"]) for e in events] == [
            ("decode", "capture_begin", "m0"), ("decode", "capture_end", "m0"),
            ("decode", "execute_begin", "m0"), ("decode", "execute_end", "m0"),
            ("prefill", "execute_begin", "m1"), ("prefill", "execute_end", "m1"),
            ("decode", "execute_begin", "m0"), ("decode", "execute_error", "m0")]
        assert all(set(e) == set(devkit.GRAPH_EVENT_FIELDS) and e["backend_class"] == "_Backend" for e in events)
        assert obs.path.name.startswith("xpool.graph-observer.") and obs.path.suffix == ".jsonl"
    finally:
        obs.uninstall()
    assert FakeDecodeRunner("x").execute(2) == 4 and not hasattr(FakeDecodeRunner.execute, "__xpool_graph_observer__")


def test_a_failing_recorder_never_disturbs_the_engine(tmp_path):
    def broken(_runner):
        raise KeyError("no such model path")

    obs = devkit.GraphObserver(tmp_path, model_id_of=broken)
    obs.install({"decode": FakeDecodeRunner})
    try:
        assert FakeDecodeRunner("m").execute(5) == 10 and obs.dropped == 2
    finally:
        obs.uninstall()
    with pytest.raises(RuntimeError, match="outdir"):
        devkit.GraphObserver("")
    with pytest.raises(ValueError, match="forward phase"):
        devkit.GraphObserver(tmp_path).install({"verify": FakeDecodeRunner})


def test_observer_follows_the_config_switch_and_wraps_the_own_engine(tmp_path):
    from crosspool_b200.config import load_config

    toml = '[atn]\ndevices = [0]\n[ffn]\ndevices = [1]\n'
    off = load_config(env={}, toml_text=toml, require=False)
    assert devkit.install_from_config(off, {"decode": FakeDecodeRunner}) is None
    on = load_config(env={"XPOOL_DEBUG_GRAPH_OBSERVER_ENABLE": "1", "XPOOL_DEBUG_GRAPH_OBSERVER_OUTDIR": str(tmp_path)},
                     toml_text=toml, require=False)
    obs = devkit.install_from_config(on, {"decode": FakeDecodeRunner})
    try:
        class Engine:
            model_id = "own"

            def _capture_decode(self, B):
                return B

            def _replay_decode(self, B):
                return -B

        devkit.observe_engine(obs, Engine)
        e = Engine()
        assert e._capture_decode(8) == 8 and e._replay_decode(8) == -8
        assert [x["event"] for x in devkit.read_graph_events(tmp_path)] == ["capture_begin", "capture_end", "execute_begin",
                                                                           "execute_end"]
    finally:
        obs.uninstall()


def test_request_limits_match_the_engines_acceptance_rules():
    lim = devkit.RequestLimits.from_context(4096)
    assert lim.max_req_input_len == 4090
    assert lim.input_budget(100) == min(4089, 3996, 3994) and lim.output_budget(1000) == min(3096, 3094)
    lim.validate_request(3000, 1000)
    with pytest.raises(ValueError, match="exceeds the static service limits"):
        lim.validate_request(3990, 200)
    info = json.dumps({"max_req_input_len": 4090, "max_total_num_tokens": 2048, "page_size": 64, "dcp_size": 1, "other": 1})
    paged = devkit.RequestLimits.from_server_info(info, context_length=4096)
    # 1000 input tokens occupy 16 pages (1024 tokens); one more page and one token stay free
    assert paged.output_budget(1000) == 2048 - 1024 - 64 - 1
    assert paged.clamp(4000, 500) == (1472, 500) and paged.output_budget(1472) == 2048 - 1472 - 64 - 1 >= 500
    assert devkit.RequestLimits.from_context(4096).clamp(4000, 500) == (3594, 500)
    with pytest.raises(ValueError, match="lacks 'page_size'"):
        devkit.RequestLimits.from_server_info(json.dumps({"max_req_input_len": 1, "max_total_num_tokens": 1}), context_length=8)
    with pytest.raises(ValueError):
        devkit.RequestLimits(context_length=0, max_req_input_len=1)


def test_local_model_metadata_from_a_checkpoint_directory_without_tokenizer(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"vocab_size": 50, "max_position_embeddings": 128, "hidden_size": 8}))
    meta = devkit.LocalModelMetadata.from_checkpoint(tmp_path)
    assert meta.vocab_size == 50 and meta.limits.context_length == 128 and meta.admissible_ids == tuple(range(50))
    with pytest.raises(ValueError, match="tokenizer"):
        devkit.LocalModelMetadata.from_checkpoint(tmp_path, text_prompts={"a": "hello"})
    m2 = devkit.LocalModelMetadata.from_config({"vocab_size": 10, "max_position_embeddings": 32}, special_ids=[0, 9],
                                               vocab=[0, 1, 2, 9, 11], text_lengths={"p": 5})
    assert m2.admissible_ids == (1, 2) and m2.text_lengths == {"p": 5}
    with pytest.raises(ValueError, match="input limit"):
        devkit.LocalModelMetadata.from_config({"vocab_size": 10, "max_position_embeddings": 32}, text_lengths={"p": 32})
    with pytest.raises(ValueError, match="vocabulary"):
        devkit.LocalModelMetadata(10, devkit.RequestLimits.from_context(32), (10,))


def test_nvtx_ranges_are_off_by_default_and_balanced_when_on():
    from crosspool_b200.utils import nvtx

    calls = []
    nvtx.set_enabled(False)
    with nvtx.range("idle"):
        pass
    nvtx.set_enabled(True, push=lambda n: calls.append(("push", n)), pop=lambda: calls.append(("pop",)))
    try:
        with pytest.raises(RuntimeError):
            with nvtx.range("step"):
                raise RuntimeError("x")
        assert calls == [("push", "step"), ("pop",)]
    finally:
        nvtx.set_enabled(False)
