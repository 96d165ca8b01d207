"""Plugin entry point for a serving engine (``sglang.srt.plugins`` group, name ``xpool``).

``install()`` sets the engine environment switches the split needs, proves to the daemon that this
process resolved the same configuration, discovers the architecture adapters and registers their
hooks with the engine's hook registry; it fails loudly when a required hook could not be applied
(reference: src/xpool/integrations/sglang/plugin.py:19-66).
"""

from __future__ import annotations

import os
from typing import Any, Callable

from .adapter import ADAPTERS, Hook

ENGINE_ENV = {
    "SGLANG_ENABLE_POST_CAPTURE_KV_SIZING": "True",
    "SGLANG_ONE_VISIBLE_DEVICE_PER_PROCESS": "False",
    "SGLANG_KILLPG_ON_SCHEDULER_EXCEPTION": "False",
}

_applied: list[Hook] = []


def install(registry: Any = None, check_config: Callable[[], None] | None = None, environ=os.environ, *, config: Any = None,
            runtime_factory: Callable | None = None, context_state_factory: Callable | None = None,
            hf_config_of: Callable | None = None, graph_runners: dict[str, type] | None = None) -> list[Hook]:
    """Registers every hook of the integration with the engine's hook registry and returns them.

    ``registry`` must offer ``register(target, handler, kind)``; without one the engine's own registry is imported.
    ``config`` is the resolved deployment configuration and ``runtime_factory(binding, rank, profile, device)`` builds the
    worker's :class:`~crosspool_b200.runtime.instance.InstanceRankRuntime` (default: one that talks to the configured
    daemon and binds the native transport); ``context_state_factory`` turns elastic KV on. ``graph_runners`` (forward
    phase -> graph runner class; default: the engine's decode and prefill runners when importable) are observed when
    ``debug.graph_observer.enable`` is set."""
    from .ecs_hooks import ElasticHooks
    from .lifecycle import LifecycleHooks

    for k, v in ENGINE_ENV.items():
        environ.setdefault(k, v)
    if check_config is not None:
        check_config()
    if registry is None:
        try:
            from sglang.srt.plugins import HookRegistry  # type: ignore

            registry = HookRegistry
        except Exception as e:
            raise RuntimeError("no serving engine hook registry available; pass one explicitly") from e
    if config is None:
        try:
            from ...config import init_global_config

            config = init_global_config()
        except Exception:          # no deployment configuration in this process: hooks still register, binding fails later
            import types

            config = types.SimpleNamespace(models=())
    life = LifecycleHooks(config, runtime_factory or default_runtime_factory(config), context_state_factory, hf_config_of)
    hooks = life.hooks()
    for a in ADAPTERS:
        hooks.extend(a.hooks())
    if context_state_factory is not None:
        hooks.extend(ElasticHooks(lambda: life.scope.context_state).hooks())
    from .shutdown import ProcessTreeRetirement

    retirement = ProcessTreeRetirement()      # sealed creation and ordered retirement of the engine's child processes
    hooks.extend(retirement.hooks())
    _applied.clear()
    for h in hooks:
        registry.register(h.target, h.handler, h.kind)
        _applied.append(h)
    verify_required_hooks_applied(registry, hooks)
    install.lifecycle = life
    install.retirement = retirement
    install.graph_observer = _install_graph_observer(config, graph_runners)
    return list(_applied)


def _install_graph_observer(config: Any, runners: dict[str, type] | None):
    if not getattr(config, "debug_graph_observer_enable", False):
        return None
    from . import devkit

    if runners is None:
        try:
            from sglang.srt.model_executor.runner.decode_cuda_graph_runner import DecodeCudaGraphRunner  # type: ignore
            from sglang.srt.model_executor.runner.prefill_cuda_graph_runner import PrefillCudaGraphRunner  # type: ignore

            runners = {"decode": DecodeCudaGraphRunner, "prefill": PrefillCudaGraphRunner}
        except Exception:
            return None

    def model_id_of(runner):
        path = getattr(getattr(getattr(runner, "model_runner", None), "model_config", None), "model_path", None)
        for m in getattr(config, "models", ()):
            if path is not None and str(getattr(m, "path", "")) == str(path):
                return m.id
        return str(getattr(runner, "model_id", path or ""))

    return devkit.install_from_config(config, runners, model_id_of)


def default_runtime_factory(config: Any) -> Callable:
    """Instance runtimes that reach the daemon named in ``config`` and bind the native transport from the handles
    the daemon brokers (the attention-side arena through the lease, the FFN slots through the plan)."""
    def make(binding, rank, profile, device):
        from ...runtime.backends import placement_for
        from ...runtime.instance import InstanceRankRuntime
        from ...service.client import XpoolClient
        from .transport import FabricInstanceTransport

        client = XpoolClient(getattr(config, "daemon_host", "127.0.0.1"), getattr(config, "daemon_port", 9810))

        def attach(arena, plan):
            place = placement_for(config, plan, binding.model_id, rank, max(profile.max_prefill_rows, profile.max_decode_rows))
            ffn = [plan.slot_handles[f"ffn:{binding.model_id}:{rank}:{pe}"] for pe in place.ffn_ranks]
            tr = FabricInstanceTransport.from_handles(place, arena.handle_hex, ffn, f"cuda:{device}")
            tr.make_current()
            return tr

        return InstanceRankRuntime(client, binding.model_id, rank, device, profile, attach=attach)

    return make


def verify_required_hooks_applied(registry: Any, hooks: list[Hook]) -> None:
    applied = getattr(registry, "applied_targets", None)
    if applied is None:
        return
    missing = [h.target for h in hooks if h.required and h.target not in applied()]
    if missing:
        raise RuntimeError(f"required hooks were not applied: {missing[:3]}")
