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


class ProfileError(RuntimeError):
    pass


def _positive_int(v: Any, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ProfileError(f"cannot derive {what}: got {v!r}")
    return v


def resolved_graph_capacity(eager_capacity: int, *, enabled: bool, buckets: Any = None, max_bs: Any = None, label: str) -> int:
    """Rows one invocation of a phase may carry: the eager capacity, or the largest captured bucket if graphs are on
    and capture more (a disabled graph path contributes nothing).
    Reference: src/xpool/integrations/sglang/hooks/lifecycle.py:470-505."""
    if not enabled:
        return eager_capacity
    candidates = [eager_capacity]
    if buckets is not None:
        if not isinstance(buckets, (list, tuple)):
            raise ProfileError(f"cannot derive {label} buckets from {buckets!r}")
        candidates += [_positive_int(b, f"a {label} bucket") for b in buckets]
    if max_bs is not None:
        candidates.append(_positive_int(max_bs, f"the {label} maximum"))
    return max(candidates)


def derive_instance_ffn_profile(model_runner: Any, hidden_size: int, shims: list | None = None, dp_size: int = 1
                                ) -> InstanceFfnProfile:
    """The profile registered with the daemon, from the *resolved* state of the serving process: payload dtype bf16
    (fp16 is refused here, before the first operator call would refuse it); at least one installed FFN shim, all of
    one hidden size; row capacities from the eager limits
    (``max_running_requests`` for decode, the prefill chunk for prefill) widened by the captured graph buckets; with
    attention DP one invocation carries every data-parallel rank's rows and may ask for the group sum.
    Reference: src/xpool/integrations/sglang/hooks/lifecycle.py:402-467."""
    import torch

    dtype = getattr(getattr(model_runner, "model_config", None), "dtype", torch.bfloat16)
    from ...utils.dtype import encode_dtype

    try:
        payload = encode_dtype(dtype)
    except (TypeError, ValueError):
        payload = None
    if payload != "bfloat16":       # the FFN kernels and the ffn_shim operator of this build carry bf16 rows only
        raise ProfileError(f"the FFN payload does not support the serving dtype {dtype!r} (bfloat16 only)")
    kinds: list[str] = []
    if shims is not None:
        if not shims:
            raise ProfileError("no FFN shim is installed in the loaded model")
        widths = {int(getattr(s, "hidden_size", hidden_size) or hidden_size) for s in shims}
        if len(widths) != 1 or widths != {hidden_size}:
            raise ProfileError(f"FFN shims disagree on the hidden size: {sorted(widths)} against {hidden_size}")
        kinds = [str(getattr(s, "layer_kind", "dense")) for s in sorted(shims, key=lambda s: s.layer_ordinal)]
    sa = getattr(model_runner, "server_args", None)
    eager_decode = getattr(model_runner, "max_running_requests", None) or getattr(sa, "max_running_requests", None) or 256
    chunk = getattr(sa, "chunked_prefill_size", None)
    eager_prefill = chunk if isinstance(chunk, int) and chunk > 0 else (getattr(sa, "max_prefill_tokens", None) or 8192)
    graphs_off = bool(getattr(sa, "disable_cuda_graph", False))
    decode = resolved_graph_capacity(_positive_int(eager_decode, "eager decode rows"), enabled=not graphs_off,
                                     buckets=getattr(sa, "cuda_graph_bs", None), max_bs=getattr(sa, "cuda_graph_max_bs", None),
                                     label="decode graph")
    prefill = resolved_graph_capacity(_positive_int(eager_prefill, "eager prefill rows"),
                                      enabled=bool(getattr(sa, "enable_prefill_cuda_graph", False)),
                                      buckets=getattr(sa, "prefill_cuda_graph_bs", None), label="prefill graph")
    dp = max(1, int(dp_size or getattr(sa, "dp_size", 1) or 1)) if getattr(sa, "enable_dp_attention", False) else 1
    return InstanceFfnProfile(max_prefill_rows=prefill * dp, max_decode_rows=decode * dp, hidden_size=hidden_size,
                              payload_dtype=payload, layer_kinds=kinds, group_sum_complete_admitted=dp > 1)


@dataclass(frozen=True)
class InstanceRankTransportProfile:
    """Geometry of the transport arena one Instance rank needs: rows of the widest invocation, hidden size, and the
    rank's place in the attention TP x DP grid (src/xpool/integrations/sglang/hooks/lifecycle.py:507-530)."""

    hidden_size: int
    payload_row_capacity: int
    atn_tp_rank: int
    atn_tp_size: int
    atn_dp_rank: int
    atn_dp_size: int

    @classmethod
    def derive(cls, binding: InstanceRankBinding, profile: InstanceFfnProfile) -> "InstanceRankTransportProfile":
        tp, dp = max(1, binding.tp_size), max(1, binding.dp_size)
        return cls(profile.hidden_size, max(profile.max_decode_rows, profile.max_prefill_rows), binding.rank % tp, tp,
                   (binding.rank // tp) % dp, dp)


@dataclass
class InstanceScope:
    """What the hooks of one worker process share."""

    binding: InstanceRankBinding | None = None
    adapter: ShimAdapter | None = None
    topology: AttentionTopology | None = None
    runtime: Any = None                      # runtime.instance.InstanceRankRuntime
    shims: list[FfnShimModule] = field(default_factory=list)
    transport_profile: Any = None
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
        profile = derive_instance_ffn_profile(model_runner, hidden, s.shims, s.binding.dp_size)
        s.transport_profile = InstanceRankTransportProfile.derive(s.binding, profile)
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
