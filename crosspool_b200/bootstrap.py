"""Process bootstrap: resolve the configuration, set up logging, check the native ABI, pick the device
and install the observers the role is entitled to (reference: src/xpool/bootstrap.py)."""

from __future__ import annotations

from dataclasses import dataclass

ROLES = ("Daemon", "Instance", "AtnAgent", "FfnAgent")
_state: "RuntimeState | None" = None


@dataclass
class RuntimeState:
    role: str
    device: int | None
    config: object
    observers: object


def init(role: str, device: int | None = None, config=None, argv_overrides: dict | None = None) -> RuntimeState:
    global _state
    if role not in ROLES:
        raise ValueError(f"unknown role {role!r}")
    if _state is not None:
        if (_state.role, _state.device) != (role, device):
            raise RuntimeError(f"process already initialised as {_state.role} on device {_state.device}")
        return _state
    from . import config as cfgmod
    from . import devkit, logging as xlog, native

    from .native import runtime as native_runtime

    cfg = config if config is not None else cfgmod.init_global_config(argv_overrides or {})
    xlog.init_logging(role, getattr(cfg, "logging_level", "info"), getattr(cfg, "logging_color", "auto"))
    options = {n: bool(getattr(cfg, f"debug_{n}_enable", False)) for n in native_runtime.DEBUG_OPTION_NAMES}
    if role != "Daemon":
        native_runtime.lib()  # loads the host library and checks its ABI number
        native_runtime.runtime_initialize(role, device, options)   # the native library's own record of role / device / options
        if device is not None:
            import torch

            if torch.cuda.is_available():
                torch.cuda.set_device(device)
                native.set_debug_options(options)                   # ... and their mirror in device constant memory
    obs = devkit.observers_for_role(role, cfg)
    _state = RuntimeState(role, device, cfg, obs)
    return _state


def get_runtime_role() -> str | None:
    return _state.role if _state else None


def reset_for_tests() -> None:
    global _state
    _state = None
    try:
        from .native import runtime as native_runtime

        native_runtime.runtime_reset_for_tests()
    except Exception:
        pass
