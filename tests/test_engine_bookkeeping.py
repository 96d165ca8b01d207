"""Host-side bookkeeping of the attention engine that needs no GPU: request validation, the prefill
stream of a retracted sequence, and an engine loop that keeps serving after a bad request."""
import time
from collections import deque

import pytest

from crosspool_b200.engine.atn_engine import AttentionEngine, EngineConfig, Sequence
from crosspool_b200.models import config as mc
from crosspool_b200.runtime.serving import EngineLoop


class _Kv:
    def __init__(self):
        self.released = []
        self.tables = {}

    def release(self, seq_id):
        self.released.append(seq_id)


def bare_engine() -> AttentionEngine:
    """An engine object with the host-side state only (no device buffers)."""
    eng = AttentionEngine.__new__(AttentionEngine)
    eng.cfg = mc.preset("Qwen/Qwen3-0.6B").with_layers(1)
    eng.ecfg = EngineConfig(max_batch=4, prefill_chunk=64, max_seq_len=128)
    eng.waiting, eng.running, eng.prefilling = deque(), [], []
    eng._next_id, eng._b_key, eng.prefix, eng.kv = 0, None, None, _Kv()
    return eng


@pytest.mark.parametrize("prompt,new,match", [([], 4, "empty prompt"), ([1, 2], 0, "max_new_tokens"),
                                              ([1, -3], 4, "token id"), ([1, 10 ** 9], 4, "token id"),
                                              (list(range(100)), 64, "max_seq_len")])
def test_add_request_rejects_bad_requests(prompt, new, match):
    eng = bare_engine()
    with pytest.raises(ValueError, match=match):
        eng.add_request(prompt, new)
    assert not eng.waiting


def test_retraction_keeps_emitted_tokens_and_recomputes_them():
    eng = bare_engine()
    s = eng.add_request([5, 6, 7], 8)
    eng.waiting.clear()
    s.generated, s.computed, s.first_token_time = [11, 12, 13], 5, 1.0
    eng.running.append(s)
    eng._retract(s)
    assert s.generated == [11, 12, 13] and s.max_new_tokens == 8 and s.prompt == [5, 6, 7]
    assert s.computed == 0 and not s.prefill_done and s.fill_len == 6
    assert s.fill_tokens(0, 6) == [5, 6, 7, 11, 12, 13] and s.fill_tokens(2, 3) == [7, 11, 12]
    assert list(eng.waiting) == [s] and eng.kv.released == [s.seq_id]
    # the token sampled by the re-prefill continues the same stream; the request is not finished early
    s.computed = 6
    s.generated.append(14)
    assert s.prefill_done and s.total_len == 7 and not s.finished


def test_fill_stream_of_a_fresh_sequence_is_its_prompt():
    s = Sequence(0, [1, 2, 3, 4], 2)
    assert s.fill_len == 4 and s.fill_tokens(1, 2) == [2, 3]


class _Dep:
    """Deployment whose add_request is the real engine's (validation included) and whose step emits one token."""

    def __init__(self):
        self.eng = bare_engine()

    def add_request(self, model_id, prompt, max_new_tokens, arrival=None):
        return self.eng.add_request(prompt, max_new_tokens, arrival)

    @property
    def has_work(self):
        return bool(self.eng.waiting)

    def step(self):
        class R:
            tokens = {}
        out = []
        for s in list(self.eng.waiting):
            s.generated.append(1)
            out.append((s, 1))
            if s.finished:
                self.eng.waiting.remove(s)
        R.tokens = {"m": out}
        return R


def test_engine_loop_survives_an_empty_prompt():
    loop = EngineLoop(_Dep())
    loop.start()
    try:
        bad = loop.submit("m", [], 4)
        item = bad.out.get(timeout=5)
        assert isinstance(item, ValueError)
        good = loop.submit("m", [3, 4], 2)
        assert good.out.get(timeout=5) == (1, False) and good.out.get(timeout=5) == (1, True)
        assert loop.error is None
    finally:
        loop.stop()


class _FakeEngine:
    """Engine whose steps finish after a set number of readiness polls."""

    def __init__(self, name, work, polls_per_step):
        self.name, self.work, self.polls_per_step = name, work, polls_per_step
        self.step_in_flight, self._polls, self.launched, self.collected, self.blocking_collects = False, 0, 0, 0, 0

    @property
    def has_work(self):
        return self.work > 0

    def launch_step(self):
        assert not self.step_in_flight
        self.step_in_flight, self._polls = True, 0
        self.launched += 1

    def step_ready(self):
        self._polls += 1
        return self._polls > self.polls_per_step

    def collect_step(self):
        if self._polls <= self.polls_per_step:
            self.blocking_collects += 1
        self.step_in_flight = False
        self.work -= 1
        self.collected += 1
        return [(self.name, self.collected)]


def test_event_driven_stepping_lets_a_fast_instance_run_while_a_slow_step_is_in_flight():
    from crosspool_b200.deployment import Deployment, InstanceHandle

    slow, fast = _FakeEngine("slow", 2, polls_per_step=6), _FakeEngine("fast", 10, polls_per_step=0)
    dep = Deployment([InstanceHandle("slow", None, slow), InstanceHandle("fast", None, fast)])
    tokens = {"slow": [], "fast": []}
    calls = 0
    while dep.has_work and calls < 200:
        for m, pairs in dep.step_async(poll_s=0.0).tokens.items():
            tokens[m] += pairs
        calls += 1
    assert slow.collected == 2 and fast.collected == 10 and not dep.has_work
    # the fast Instance finished several steps before the slow one's first step came back
    first_slow = 6
    assert fast.launched >= 5 and calls < 40
    assert [n for _, n in tokens["fast"]] == list(range(1, 11)) and [n for _, n in tokens["slow"]] == [1, 2]
    # once only the slow Instance is left, the driver waits for it instead of polling
    assert slow.blocking_collects >= 1 and fast.blocking_collects == 0
    del first_slow


def test_lockstep_step_still_runs_every_instance_once_per_call():
    from crosspool_b200.deployment import Deployment, InstanceHandle

    a, b = _FakeEngine("a", 3, 0), _FakeEngine("b", 1, 0)
    dep = Deployment([InstanceHandle("a", None, a), InstanceHandle("b", None, b)])
    assert set(dep.step().tokens) == {"a", "b"} and set(dep.step().tokens) == {"a"}


def test_vectorised_chunk_metadata_equals_the_per_token_definition():
    import numpy as np

    rnd = __import__("random").Random(4)
    for ps in (16, 64):
        for _ in range(20):
            P = 512
            prompt = [rnd.randrange(1000) for _ in range(rnd.randrange(1, 400))]
            s = Sequence(0, prompt, 8)
            s.generated = [rnd.randrange(1000) for _ in range(rnd.randrange(0, 5))]
            s.refill_len = s.total_len if s.generated else 0
            fill = s.fill_len
            s.computed = rnd.randrange(0, fill)
            n = rnd.randrange(1, min(P, fill - s.computed) + 1)
            r = rnd.randrange(0, P - n + 1)
            table = rnd.sample(range(5000), (fill + ps) // ps + 1)
            hv = np.full(3 * P, -7, dtype=np.int32)
            AttentionEngine._fill_chunk_rows(hv, P, r, s, n, table, ps)
            want = np.full(3 * P, -7, dtype=np.int32)
            toks = s.fill_tokens(s.computed, n)
            for j in range(n):
                p = s.computed + j
                want[r + j], want[P + r + j], want[2 * P + r + j] = toks[j], p, table[p // ps] * ps + p % ps
            assert np.array_equal(hv, want)


def test_event_driven_stepping_sleeps_while_every_instance_waits_on_the_host():
    """An Instance that cannot admit anything (no KV capacity yet) produces empty steps; the driver must not spin."""
    from crosspool_b200 import deployment as D

    class Starved(_FakeEngine):
        step_is_device_work = False

        def collect_step(self):
            self.step_in_flight = False
            self.collected += 1
            return []

    e = Starved("starved", 1, polls_per_step=0)
    dep = D.Deployment([D.InstanceHandle("starved", None, e)])
    slept = []
    real_sleep = D.time.sleep
    D.time.sleep = slept.append
    try:
        for _ in range(5):
            assert dep.step_async(poll_s=0.123).tokens.get("starved", []) == []
    finally:
        D.time.sleep = real_sleep
    assert slept == [0.123] * 5 and e.launched == 5


def test_the_gpu_attention_engine_refuses_attention_forms_it_does_not_compute():
    """Before anything touches a device: a model with latent attention, sinks, windows, learned positions or scaled
    rotary embeddings is refused by name instead of being run as plain rotary GQA."""
    import pytest

    from crosspool_b200.engine.atn_engine import AttentionEngine, UnsupportedAttention
    from crosspool_b200.models import config as mc

    base = {"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256,
            "intermediate_size": 128}
    refused = [
        {**base, "architectures": ["OPTForCausalLM"], "ffn_dim": 128},
        {**base, "architectures": ["GptOssForCausalLM"], "sliding_window": 128, "num_local_experts": 4, "num_experts_per_tok": 2},
        {**base, "architectures": ["DeepseekV2ForCausalLM"], "kv_lora_rank": 32, "qk_nope_head_dim": 16, "qk_rope_head_dim": 8,
         "v_head_dim": 16},
        {**base, "architectures": ["Qwen3ForCausalLM"], "rope_scaling": {"rope_type": "yarn", "factor": 4.0,
                                                                          "original_max_position_embeddings": 32768}},
    ]
    for hf in refused:
        cfg = mc.from_hf_config(hf)
        assert not cfg.gpu_attention_supported
        with pytest.raises(UnsupportedAttention, match=cfg.architecture):
            AttentionEngine(cfg, None, None, device="cpu")
    # a Qwen2 config.json carries a sliding_window it does not use: still plain GQA
    plain = mc.from_hf_config({**base, "architectures": ["Qwen2ForCausalLM"], "sliding_window": 4096, "use_sliding_window": False,
                               "layer_types": ["full_attention", "full_attention"]})
    assert plain.gpu_attention_supported and plain.sliding_window == 0
    assert all(mc.preset(n).gpu_attention_supported for n in mc.PRESETS)
