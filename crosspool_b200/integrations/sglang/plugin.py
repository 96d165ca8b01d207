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


def lifecycle_hooks() -> list[Hook]:
    """Engine lifecycle seams the Instance runtime attaches to."""
    names = [("sglang.srt.managers.scheduler.Scheduler.__init__", "around"),
             ("sglang.srt.managers.scheduler.Scheduler.run_event_loop", "around"),
             ("sglang.srt.model_executor.model_runner.ModelRunner.load_model", "around"),
             ("sglang.srt.model_executor.model_runner.ModelRunner.alloc_memory_pool", "after"),
             ("sglang.srt.managers.scheduler.Scheduler.get_init_info", "after"),
             ("sglang.srt.managers.scheduler.Scheduler.release_host_resources", "around")]
    return [Hook(t, _passthrough, k) for t, k in names]


def _passthrough(original: Callable | None = None, *a, **kw):
    return original(*a, **kw) if callable(original) else None


def install(registry: Any = None, check_config: Callable[[], None] | None = None, environ=os.environ) -> list[Hook]:
    """``registry`` must offer ``register(target, handler, kind)``; without one the engine's own
    registry is imported. Returns the hooks that were applied."""
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
    hooks = lifecycle_hooks()
    for a in ADAPTERS:
        hooks.extend(a.hooks())
    _applied.clear()
    for h in hooks:
        registry.register(h.target, h.handler, h.kind)
        _applied.append(h)
    verify_required_hooks_applied(registry, hooks)
    return list(_applied)


def verify_required_hooks_applied(registry: Any, hooks: list[Hook]) -> None:
    applied = getattr(registry, "applied_targets", None)
    if applied is None:
        return
    missing = [h.target for h in hooks if h.target not in applied()]
    if missing:
        raise RuntimeError(f"required hooks were not applied: {missing[:3]}")
