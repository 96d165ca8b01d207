"""A stand-in serving engine for the integration tests: module tree, classes and a hook registry with the shapes the
plugin targets (``sglang.srt...``), carrying just enough state to observe what the hooks did. The reference tests its
hooks the same way, against lightweight fakes of the engine's types
(src/xpool-dev/xtest/harness/support/sglang/fakes.py)."""
import importlib
import sys
import types

import torch


def _module(name):
    if name in sys.modules:
        return sys.modules[name]
    m = types.ModuleType(name)
    sys.modules[name] = m
    if "." in name:
        parent, child = name.rsplit(".", 1)
        setattr(_module(parent), child, m)
    return m


def install_fake_engine():
    """Creates the fake ``sglang.srt`` tree (idempotent) and returns its interesting modules."""
    models = _module("sglang.srt.models.qwen3")
    sched = _module("sglang.srt.managers.scheduler")
    runner = _module("sglang.srt.model_executor.model_runner")
    batch = _module("sglang.srt.managers.schedule_batch")
    policy = _module("sglang.srt.managers.schedule_policy")

    class Qwen3MLP(torch.nn.Module):
        def __init__(self, hidden=8, inter=16, prefix=""):
            super().__init__()
            self.gate_up_proj = torch.nn.Linear(hidden, 2 * inter, bias=False)
            self.down_proj = torch.nn.Linear(inter, hidden, bias=False)

        def forward(self, x, forward_batch=None):
            g, u = self.gate_up_proj(x).chunk(2, -1)
            return self.down_proj(torch.nn.functional.silu(g) * u)

    class Layer(torch.nn.Module):
        def __init__(self, i, hidden):
            super().__init__()
            self.self_attn = torch.nn.Linear(hidden, hidden, bias=False)
            # looked up in the module at construction time, so a REPLACE hook takes effect
            self.mlp = models.Qwen3MLP(hidden=hidden, inter=2 * hidden, prefix=f"model.layers.{i}.mlp")

    class Qwen3ForCausalLM(torch.nn.Module):
        def __init__(self, layers=3, hidden=8):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList(Layer(i, hidden) for i in range(layers))
            self.loaded = []

        def load_weights(self, weights):
            self.loaded = [n for n, _ in weights]

        def forward(self, x, forward_batch):
            for l in self.model.layers:
                x = x + l.self_attn(x)
                x = x + l.mlp(x, forward_batch)
            return x

    class ModelRunner:
        def __init__(self, server_args, layers=3, hidden=8):
            self.server_args, self.gpu_id = server_args, 0
            self.model_config = types.SimpleNamespace(
                architecture="Qwen3ForCausalLM", hidden_size=hidden,
                hf_config={"architectures": ["Qwen3ForCausalLM"], "hidden_size": hidden, "num_attention_heads": 4,
                           "num_key_value_heads": 2, "num_hidden_layers": layers})
            self.layers, self.hidden, self.model, self.pool = layers, hidden, None, None

        def checkpoint(self):
            names = ["model.embed_tokens.weight", "lm_head.weight"]
            for i in range(self.layers):
                names += [f"model.layers.{i}.self_attn.weight", f"model.layers.{i}.mlp.gate_up_proj.weight",
                          f"model.layers.{i}.mlp.down_proj.weight", f"model.layers.{i}.post_attention_layernorm.weight"]
            return [(n, None) for n in names]

        def load_model(self):
            self.model = models.Qwen3ForCausalLM(self.layers, self.hidden)
            self.model.load_weights(iter(self.checkpoint()))

        def alloc_memory_pool(self):
            self.pool = "kv-pool"
            return self.pool

    class Scheduler:
        def __init__(self, server_args):
            self.server_args, self.log = server_args, []
            self.model_runner = runner.ModelRunner(server_args)
            self.model_runner.load_model()
            self.model_runner.alloc_memory_pool()

        def get_init_info(self):
            return {"status": "ready"}

        def run_event_loop(self):
            self.log.append("loop")
            return "loop-done"

        def release_host_resources(self):
            self.log.append("released")
            return "released"

    models.Qwen3MLP, models.Qwen3ForCausalLM = Qwen3MLP, Qwen3ForCausalLM
    runner.ModelRunner, sched.Scheduler = ModelRunner, Scheduler
    batch.ScheduleBatch = type("ScheduleBatch", (), {"check_decode_mem": lambda self: True, "retract_decode": lambda self: []})
    policy.PrefillAdder = type("PrefillAdder", (), {"add_one_req": lambda self, req: 0})
    return types.SimpleNamespace(models=models, sched=sched, runner=runner, batch=batch, policy=policy)


class PatchingHookRegistry:
    """Applies hooks the way the engine's registry does: ``replace`` swaps the symbol, ``around`` passes the original as
    the first argument, ``after`` passes the original's result. Targets that do not resolve are skipped (and therefore
    missing from ``applied_targets``)."""

    def __init__(self):
        self.applied, self._undo = [], []

    def register(self, target, handler, kind):
        mod_path, _, attr = target.rpartition(".")
        try:
            owner = importlib.import_module(mod_path)
        except ModuleNotFoundError:
            owner_mod, _, cls = mod_path.rpartition(".")
            try:
                owner = getattr(importlib.import_module(owner_mod), cls)
            except (ModuleNotFoundError, AttributeError):
                return
        if not hasattr(owner, attr):
            return
        original = getattr(owner, attr)
        if kind == "replace":
            new = handler
        elif kind == "around":
            def new(*a, _o=original, _h=handler, **kw):
                return _h(_o, *a, **kw)
        else:
            def new(*a, _o=original, _h=handler, **kw):
                return _h(_o(*a, **kw), *a, **kw)
        setattr(owner, attr, new)
        self._undo.append((owner, attr, original))
        self.applied.append(target)

    def applied_targets(self):
        return set(self.applied)

    def restore(self):
        for owner, attr, original in reversed(self._undo):
            setattr(owner, attr, original)
        self._undo.clear()


class FakeDaemonClient:
    """Answers like the daemon for one Instance rank: not executable for the first ``warm`` polls, then executable."""

    def __init__(self, model_id, warm=2, fail=None):
        from crosspool_b200.service.wire import FabricPhase, ReadinessSnapshot

        self.model_id, self.polls, self.warm, self.fail = model_id, 0, warm, fail
        self.calls, self.FabricPhase, self.ReadinessSnapshot = [], FabricPhase, ReadinessSnapshot

    def register_instance(self, r):
        self.calls.append(("register", r.model_id, r.rank, r.ffn_profile.max_prefill_rows, r.ffn_profile.max_decode_rows))

    def heartbeat_instance(self, model_id, rank, owner):
        self.calls.append(("heartbeat", model_id, rank))

    def ready(self):
        self.polls += 1
        ok = self.polls > self.warm
        return self.ReadinessSnapshot(fabric_executable=ok, system_ready=ok, serving_healthy=ok, generation=7 if ok else None,
                                      phase=self.FabricPhase.EXECUTABLE if ok else self.FabricPhase.ACTIVATING, failure=self.fail)

    def fabric_plan(self):
        return types.SimpleNamespace(generation=7, instance_ranks=[types.SimpleNamespace(model_id=self.model_id, rank=0)])

    def acquire_arena(self, model_id, req):
        self.calls.append(("acquire", model_id, req.rank, req.generation))
        return types.SimpleNamespace(model_id=model_id, rank=req.rank, handle_hex="00", nbytes=0)

    def instance_initialized(self, model_id, req):
        self.calls.append(("initialized", model_id, req.rank, req.generation))

    def deregister_instance(self, model_id, req):
        self.calls.append(("deregister", model_id, req.rank))
