"""Lifecycle hooks: what happens around the serving engine's own start-up and shutdown so that an Instance rank
exists, reaches the FFN tier and leaves in order.

Hook targets and kinds follow the reference (src/xpool/integrations/sglang/hooks/lifecycle.py:57-100):

* ``Scheduler.__init__`` (around)          validate launch arguments against the deployment, resolve the binding;
* ``ModelRunner.load_model`` (around)      pick the architecture adapter, load without decoder-FFN tensors, check that
                                           every decoder MLP became a shim and no FFN parameter is left, derive the
                                           FFN profile, register the Instance rank, wait until the Fabric is
                                           executable, acquire the transport arena and bind the native submit path
                                           (:161-238);
* ``ModelRunner.alloc_memory_pool`` (after) build the elastic context state when elastic KV is on (:240-332);
* ``Scheduler.get_init_info`` (after)      publish "initialized" once graphs are captured, wait for System Ready (:334-377);
* ``Scheduler.run_event_loop`` (around)    run the failure monitor for the life of the loop (:118-135);
* ``Scheduler.release_host_resources`` (around) ordered retirement (hooks/shutdown.py).

The engine's own classes are never imported here: handlers work on whatever object the engine passes, which is what
lets the test suite drive them with lightweight fakes.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

from ...service.wire import InstanceFfnProfile
from .adapter import Hook, InstanceRankBinding, ShimAdapter, find_adapter, weight_filter_scope
from .server_args import validate_server_args
from .shim import FfnShimModule
from .shutdown import ShutdownHookSet, instance_shutdown_set
from .topology import AttentionTopology, ModelShape

T = "sglang.srt."
LIFECYCLE_TARGETS = [
    (T + "managers.scheduler.Scheduler.__init__", "around", "scheduler_init"),
    (T + "managers.scheduler.Scheduler.run_event_loop", "around", "run_event_loop"),
    (T + "model_executor.model_runner.ModelRunner.load_model", "around", "load_model"),
    (T + "model_executor.model_runner.ModelRunner.alloc_memory_pool", "after", "alloc_memory_pool"),
    (T + "managers.scheduler.Scheduler.get_init_info", "after", "get_init_info"),
    (T + "managers.scheduler.Scheduler.release_host_resources", "around", "release_host_resources"),
]


def derive_instance_ffn_profile(model_runner: Any, hidden_size: int) -> InstanceFfnProfile:
    """Row capacities the Instance will ever submit: a prefill invocation carries at most one chunk, a decode
    invocation at most the largest captured batch (src/xpool/integrations/sglang/hooks/lifecycle.py:402-467)."""
    sa = getattr(model_runner, "server_args", None)
    chunk = int(getattr(sa, "chunked_prefill_size", 0) or 0)
    if chunk <= 0:
        chunk = int(getattr(sa, "max_prefill_tokens", 0) or 8192)
    decode = int(getattr(sa, "cuda_graph_max_bs", 0) or getattr(sa, "max_running_requests", 0) or 256)
    dp = max(1, int(getattr(sa, "dp_size", 1) or 1))
    if getattr(sa, "enable_dp_attention", False) and dp > 1:
        chunk, decode = chunk * dp, decode * dp      # one invocation carries every data-parallel rank's rows
    return InstanceFfnProfile(max_prefill_rows=chunk, max_decode_rows=decode, hidden_size=hidden_size)


@dataclass
class InstanceScope:
    """What the hooks of one worker process share."""

    binding: InstanceRankBinding | None = None
    adapter: ShimAdapter | None = None
    topology: AttentionTopology | None = None
    runtime: Any = None                      # runtime.instance.InstanceRankRuntime
    shims: list[FfnShimModule] = field(default_factory=list)
    context_state: Any = None
    shutdown: ShutdownHookSet | None = None
    events: list[str] = field(default_factory=list)


class LifecycleHooks:
    """``runtime_factory(binding, profile, device) -> InstanceRankRuntime``; ``context_state_factory(model_runner, scope)``
    builds the elastic KV state (None: fixed KV). ``config`` is the resolved deployment configuration."""

    def __init__(self, config: Any, runtime_factory: Callable, context_state_factory: Callable | None = None,
                 hf_config_of: Callable[[Any], dict] | None = None):
        self.config, self.runtime_factory, self.context_state_factory = config, runtime_factory, context_state_factory
        self.hf_config_of = hf_config_of or (lambda mr: dict(getattr(getattr(mr, "model_config", None), "hf_config", {}) or {}))
        self.scope = InstanceScope()

    # ------------------------------------------------------------------ registration
    def hooks(self) -> list[Hook]:
        return [Hook(target, getattr(self, name), kind) for target, kind, name in LIFECYCLE_TARGETS]

    # ------------------------------------------------------------------ handlers
    def scheduler_init(self, original: Callable, scheduler: Any, server_args: Any, *a, **kw):
        b = InstanceRankBinding.resolve(server_args, self.config)
        validate_server_args(server_args, atn_tp_size=b.tp_size, atn_dp_size=b.dp_size)
        self.scope.binding = b
        self.scope.events.append("scheduler_init")
        out = original(scheduler, server_args, *a, **kw)
        scheduler.xpool_scope = self.scope
        return out

    def load_model(self, original: Callable, model_runner: Any, *a, **kw):
        s = self.scope
        s.adapter = find_adapter(model_runner)
        if s.binding is None:
            s.binding = InstanceRankBinding.resolve(model_runner.server_args, self.config)
        hf = self.hf_config_of(model_runner)
        shape = ModelShape.load(hf) if hf else None
        if shape is not None:
            s.topology = AttentionTopology.from_runtime(model_runner.server_args, shape, atn_tp_size=s.binding.tp_size,
                                                        atn_dp_size=s.binding.dp_size,
                                                        supports_dp_attention=s.adapter.supports_dp_attention)
        s.adapter.validate_before_load(model_runner, s.binding)
        with weight_filter_scope():
            out = original(model_runner, *a, **kw)        # adapter hooks build shims and skip the FFN tensors
        layers = len(s.adapter.decoder_layers(model_runner.model))
        s.shims = s.adapter.validate_after_load(model_runner.model, layers)
        hidden = shape.hidden_size if shape is not None else int(getattr(model_runner.model_config, "hidden_size"))
        profile = derive_instance_ffn_profile(model_runner, hidden)
        device = int(getattr(model_runner, "gpu_id", 0))
        rank = s.topology.instance_rank if s.topology is not None else s.binding.rank
        s.runtime = self.runtime_factory(s.binding, rank, profile, device)
        s.runtime.start()
        plan = s.runtime.wait_for_fabric_executable()
        s.runtime.attach_arena_from_daemon(plan)
        s.events.append("load_model")
        return out

    def alloc_memory_pool(self, result: Any, model_runner: Any, *a, **kw):
        if self.context_state_factory is not None:
            self.scope.context_state = self.context_state_factory(model_runner, self.scope)
        self.scope.events.append("alloc_memory_pool")
        return result

    def get_init_info(self, result: Any, scheduler: Any, *a, **kw):
        rt = self.scope.runtime
        if rt is not None:
            sa = getattr(scheduler, "server_args", None)
            listener = (getattr(sa, "host", "127.0.0.1"), int(getattr(sa, "port", 0))) if sa is not None and self.scope.binding.rank == 0 else None
            finalize = getattr(self.scope.context_state, "finalize_after_capture", None)
            if finalize is not None:
                finalize()                      # post-capture KV sizing: report free memory, take the initial quota
            rt.publish_initialized(listener)
            rt.wait_for_ready()
        self.scope.events.append("get_init_info")
        return result

    def run_event_loop(self, original: Callable, scheduler: Any, *a, **kw):
        rt = self.scope.runtime
        if rt is not None:
            rt.start_failure_monitor()
        self.scope.events.append("run_event_loop")
        try:
            return original(scheduler, *a, **kw)
        finally:
            if rt is not None and rt.monitor is not None:
                rt.monitor.stop()

    def release_host_resources(self, original: Callable, scheduler: Any, *a, **kw):
        s = self.scope
        if s.shutdown is None and s.runtime is not None:
            s.shutdown = instance_shutdown_set(
                stop_admission=lambda: setattr(scheduler, "xpool_admission_closed", True),
                drain=lambda deadline: bool(getattr(scheduler, "xpool_drain", lambda d: True)(deadline)),
                runtime=s.runtime)
        rep = s.shutdown.run() if s.shutdown is not None else None
        s.events.append("release_host_resources")
        if rep is not None and rep.retained:
            # cleanup could not be confirmed: keep what this process still owns, let the caller exit non-zero
            scheduler.xpool_retained = rep.failed
            return None
        return original(scheduler, *a, **kw)
