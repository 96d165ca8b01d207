"""Deployment configuration: one declarative registry, four sources.

Every setting names its TOML path, optional environment variable, optional CLI flag, parser and
default; the effective value is resolved with the precedence **CLI > environment > TOML > default**.
``XPOOL_CONFIG`` (or ``--config``) points at the TOML file. The key set and the precedence are the
reference's (src/xpool/config.py:86-402, docs/designs/control-plane.md:10-20) so that an existing
deployment TOML loads unchanged; ``digest()`` lets every joining process prove to the daemon that it
resolved the same effective configuration (``POST /config/check``).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Mapping, Sequence

from .model import ModelId

_MISSING = object()


class ConfigError(ValueError):
    pass


def _bool(v: Any) -> bool:
    if isinstance(v, bool):
        return v
    s = str(v).strip().lower()
    if s in ("1", "true", "yes", "on"):
        return True
    if s in ("0", "false", "no", "off"):
        return False
    raise ConfigError(f"not a boolean: {v!r}")


def _int(lo: int | None = None, hi: int | None = None) -> Callable[[Any], int]:
    def parse(v: Any) -> int:
        if isinstance(v, bool):
            raise ConfigError(f"not an integer: {v!r}")
        try:
            i = int(v)
        except (TypeError, ValueError):
            raise ConfigError(f"not an integer: {v!r}") from None
        if (lo is not None and i < lo) or (hi is not None and i > hi):
            raise ConfigError(f"{i} outside [{lo}, {hi}]")
        return i

    return parse


def _float(lo: float | None = None, hi: float | None = None) -> Callable[[Any], float]:
    def parse(v: Any) -> float:
        try:
            f = float(v)
        except (TypeError, ValueError):
            raise ConfigError(f"not a number: {v!r}") from None
        if (lo is not None and f < lo) or (hi is not None and f > hi):
            raise ConfigError(f"{f} outside [{lo}, {hi}]")
        return f

    return parse


def _choice(*allowed: str) -> Callable[[Any], str]:
    def parse(v: Any) -> str:
        s = str(v).lower()
        if s not in allowed:
            raise ConfigError(f"{v!r} not one of {allowed}")
        return s

    return parse


def _int_choice(*allowed: int) -> Callable[[Any], int]:
    def parse(v: Any) -> int:
        try:
            n = int(v)
        except (TypeError, ValueError):
            raise ConfigError(f"{v!r} is not an integer") from None
        if n not in allowed:
            raise ConfigError(f"{v!r} not one of {allowed}")
        return n

    return parse


def _devices(v: Any) -> tuple[int, ...]:
    if isinstance(v, str):
        v = [p for p in v.replace(",", " ").split() if p]
    try:
        out = tuple(int(x) for x in v)
    except (TypeError, ValueError):
        raise ConfigError(f"not a device list: {v!r}") from None
    if len(set(out)) != len(out) or any(d < 0 for d in out):
        raise ConfigError(f"device list has duplicates or negatives: {out}")
    return out


def _slo(v: Any) -> "Slo":
    if isinstance(v, Slo):
        return v
    if not isinstance(v, Mapping) or set(v) - {"ttft_ms", "tbt_ms"}:
        raise ConfigError(f"slo must be a table with ttft_ms and tbt_ms, got {v!r}")
    try:
        return Slo(float(v["ttft_ms"]), float(v["tbt_ms"]))
    except KeyError as e:
        raise ConfigError(f"slo misses {e.args[0]}") from None


@dataclass(frozen=True)
class Slo:
    ttft_ms: float
    tbt_ms: float

    def __post_init__(self):
        if self.ttft_ms <= 0 or self.tbt_ms <= 0:
            raise ConfigError("slo values must be positive")


@dataclass(frozen=True)
class ModelEntry:
    id: str
    path: str
    atn_tp_size: int = 1
    atn_dp_size: int = 1
    ffn_tp_size: int | None = None  # None: all FFN devices
    ffn_ep_size: int = 1            # expert parallelism (not in the reference, which rejects EP)
    slo: Slo | None = None
    # The Instance ranks run in other processes (an external serving engine with the plugin, or a transformers model):
    # the attention agent of their device only brokers their Transport arenas instead of hosting an engine for them.
    external: bool = False

    @property
    def atn_world_size(self) -> int:
        return self.atn_tp_size * self.atn_dp_size


@dataclass(frozen=True)
class ConfigSetting:
    name: str
    path: tuple[str, ...] | None          # TOML path; None = bootstrap-only (no TOML source)
    parser: Callable[[Any], Any]
    default: Any = _MISSING
    cli: str | None = None
    env_var: str | None = None
    required: bool = False
    description: str = ""


def _observer(name: str) -> list[ConfigSetting]:
    up = name.upper()
    return [
        ConfigSetting(f"debug_{name}_observer_enable", ("debug", f"{name}_observer", "enable"), _bool, False,
                      env_var=f"XPOOL_DEBUG_{up}_OBSERVER_ENABLE", description=f"record {name} events"),
        ConfigSetting(f"debug_{name}_observer_outdir", ("debug", f"{name}_observer", "outdir"), str, "",
                      env_var=f"XPOOL_DEBUG_{up}_OBSERVER_OUTDIR", description="artifact directory"),
        ConfigSetting(f"debug_{name}_observer_record_capacity", ("debug", f"{name}_observer", "record_capacity"),
                      _int(1), 65536, env_var=f"XPOOL_DEBUG_{up}_OBSERVER_RECORD_CAPACITY",
                      description="events kept before dropping"),
    ]


CONFIG_REGISTRY: tuple[ConfigSetting, ...] = (
    ConfigSetting("cache_root", ("cache_root",), str, ".xpool-cache", cli="--cache-root", env_var="XPOOL_CACHE_ROOT",
                  description="directory for calibration profiles and caches"),
    ConfigSetting("config", None, str, "", cli="--config", env_var="XPOOL_CONFIG",
                  description="path of the deployment TOML"),
    ConfigSetting("logging_level", ("logging", "level"), _choice("debug", "info", "warning", "error"), "info",
                  cli="--log-level", env_var="XPOOL_LOG_LEVEL", description="log level of every process of the deployment"),
    ConfigSetting("logging_color", ("logging", "color"), _choice("auto", "always", "never"), "auto",
                  description="coloured log lines: when attached to a terminal, always or never"),
    *_observer("graph"), *_observer("transport"), *_observer("fabric"), *_observer("ffn_routing"),
    ConfigSetting("vendor_model_base_uri", ("vendor", "model_base_uri"), str, "",
                  description="directory that relative model paths are resolved against"),
    ConfigSetting("atn_devices", ("atn", "devices"), _devices, required=True,
                  description="GPUs that run attention Instances (indices; disjoint from [ffn].devices)"),
    ConfigSetting("atn_device_memory_utilization", ("atn", "device_memory_utilization"), _float(0.05, 1.0), 0.95,
                  description="fraction of an attention GPU's memory the KV budget may use"),
    ConfigSetting("atn_elastic_kv", ("atn", "elastic_kv"), _bool, False, env_var="XPOOL_ATN_ELASTIC_KV",
                  description="back the KV caches with VMM bundles lent between co-located Instances"),
    ConfigSetting("ffn_devices", ("ffn", "devices"), _devices, required=True,
                  description="GPUs of the shared FFN tier"),
    ConfigSetting("ffn_device_memory_calibration", ("ffn", "device_memory_calibration"), _bool, False,
                  env_var="XPOOL_FFN_DEVICE_MEMORY_CALIBRATION",
                  description="admit placements with the persisted calibration profile (xpool memory-profile) instead of the analytic ledger alone"),
    ConfigSetting("ffn_device_memory_extra_margin_bytes", ("ffn", "device_memory_extra_margin_bytes"), _int(0), 0,
                  description="bytes kept free on every FFN GPU on top of the admitted peak"),
    ConfigSetting("ffn_loader_parallelism", ("ffn", "loader", "parallelism"), _int(1, 256), 4,
                  cli="--ffn-loader-parallelism", env_var="XPOOL_FFN_LOADER_PARALLELISM",
                  description="checkpoint reader threads (and pinned staging slots) per FFN rank"),
    ConfigSetting("ffn_placement_parallelism", ("ffn", "placement", "parallelism"), _int(1, 256), 1,
                  cli="--ffn-placement-parallelism", env_var="XPOOL_FFN_PLACEMENT_PARALLELISM",
                  description="worker threads of the placement search"),
    ConfigSetting("ffn_placement_timeout_seconds", ("ffn", "placement", "timeout_seconds"), _float(0.001), 60.0,
                  description="time limit of the placement search; the best placement found so far is used"),
    ConfigSetting("daemon_host", ("daemon", "host"), str, "127.0.0.1", cli="--daemon-host",
                  description="address the daemon listens on and agents connect to"),
    ConfigSetting("daemon_port", ("daemon", "port"), _int(1, 65535), 9810, cli="--daemon-port",
                  description="daemon HTTP port"),
    ConfigSetting("scheduler_ffn_concurrency", ("scheduler", "ffn_concurrency"), _int(1, 64), 1,
                  cli="--ffn-concurrency", description="Executor Lanes per FFN device"),
    ConfigSetting("scheduler_ffn_policy", ("scheduler", "ffn_policy"), _choice("fifo", "random", "slo"), "fifo",
                  cli="--ffn-policy", description="order in which waiting Instances get a free Lane: arrival, seeded random, or earliest SLO deadline"),
    ConfigSetting("scheduler_ffn_random_seed", ("scheduler", "ffn_random_seed"), _int(0), 0,
                  description="seed of the random Lane policy"),
    ConfigSetting("scheduler_slo", ("scheduler", "slo"), _slo, required=True,
                  description="default service-level objective {ttft_ms, tbt_ms} (time to first token, time between tokens); a [[models]] entry may override it"),
    # engine sizing of the attention ranks this repository hosts itself (covered by the configuration digest: every
    # process of a deployment must agree on the row capacities the slots are sized for)
    ConfigSetting("engine_max_rows", ("engine", "max_rows"), _int(1, 1 << 20), 4096, env_var="XPOOL_MAX_ROWS",
                  description="row capacity of an FFN invocation (prefill chunk and decode batch fit in it)"),
    ConfigSetting("engine_max_batch", ("engine", "max_batch"), _int(1, 1 << 16), 256, env_var="XPOOL_MAX_BATCH",
                  description="running requests per Instance"),
    ConfigSetting("engine_prefill_chunk", ("engine", "prefill_chunk"), _int(16, 1 << 20), 4096, env_var="XPOOL_PREFILL_CHUNK",
                  description="tokens per prefill step"),
    ConfigSetting("engine_max_seq_len", ("engine", "max_seq_len"), _int(16, 1 << 22), 4096, env_var="XPOOL_MAX_SEQ_LEN",
                  description="longest prompt plus output of a request"),
    ConfigSetting("engine_page_size", ("engine", "page_size"), _int_choice(16, 32, 64, 128), 16, env_var="XPOOL_PAGE_SIZE",
                  description="tokens per KV page"),
    ConfigSetting("serving_base_port", ("serving", "base_port"), _int(1, 65535), 30000, env_var="XPOOL_SERVING_BASE_PORT",
                  description="HTTP port of the first attention device's Instances; device i listens on base + i"),
    ConfigSetting("serving_tp_rendezvous_base_port", ("serving", "tp_rendezvous_base_port"), _int(1, 65535), 30500,
                  env_var="XPOOL_TP_RENDEZVOUS_BASE_PORT",
                  description="loopback port at which the ranks of an attention TP group meet (+ first rank of the group)"),
)

_BY_NAME = {s.name: s for s in CONFIG_REGISTRY}


def _toml_get(doc: Mapping[str, Any], path: Sequence[str]) -> Any:
    cur: Any = doc
    for p in path:
        if not isinstance(cur, Mapping) or p not in cur:
            return _MISSING
        cur = cur[p]
    return cur


def _parse_models(doc: Mapping[str, Any], ffn_devices: tuple[int, ...]) -> tuple[ModelEntry, ...]:
    out = []
    seen = set()
    for i, m in enumerate(doc.get("models", []) or []):
        if not isinstance(m, Mapping):
            raise ConfigError(f"models[{i}] is not a table")
        extra = set(m) - {"id", "path", "atn_tp_size", "atn_dp_size", "ffn_tp_size", "ffn_ep_size", "slo", "external"}
        if extra:
            raise ConfigError(f"models[{i}] has unknown keys {sorted(extra)}")
        if "id" not in m:
            raise ConfigError(f"models[{i}] misses id")
        mid = str(m["id"])
        try:
            ModelId.parse(mid)
        except ValueError as e:
            raise ConfigError(f"models[{i}]: {e}") from None
        if mid in seen:
            raise ConfigError(f"duplicate model id {mid}")
        seen.add(mid)
        tp = _int(1)(m.get("atn_tp_size", 1))
        dp = _int(1)(m.get("atn_dp_size", 1))
        if tp > 1 and dp > 1:
            # same restriction as the reference (src/cext/fabric/projection.cpp:27-28)
            raise ConfigError(f"model {mid}: combined attention TP-by-DP is not supported")
        ftp = m.get("ffn_tp_size")
        ftp = _int(1, max(1, len(ffn_devices)))(ftp) if ftp is not None else None
        ep = _int(1, max(1, len(ffn_devices)))(m.get("ffn_ep_size", 1))
        out.append(ModelEntry(mid, str(m.get("path", mid)), tp, dp, ftp, ep, _slo(m["slo"]) if "slo" in m else None,
                              external=_bool(m.get("external", False))))
    return tuple(out)


@dataclass(frozen=True)
class XpoolConfig:
    values: Mapping[str, Any]
    models: tuple[ModelEntry, ...] = ()
    sources: Mapping[str, str] = field(default_factory=dict, compare=False)

    def __getattr__(self, name: str) -> Any:
        try:
            return self.__dict__["values"][name]
        except KeyError:
            raise AttributeError(name) from None

    def model(self, model_id: str) -> ModelEntry:
        for m in self.models:
            if m.id == model_id:
                return m
        raise KeyError(model_id)

    def model_shape(self, model_id: str):
        """The model's shape (``models.config.ModelConfig``): the preset named by ``path`` or ``id``, else the
        ``config.json`` of the checkpoint directory ``path``. Daemon, agents and tools all resolve it here."""
        from .models import config as mc

        m = self.model(model_id)
        for name in (m.path, m.id):
            if name and name in mc.PRESETS:
                return mc.PRESETS[name]
        try:
            return mc.load(str(self.model_path(model_id)))
        except FileNotFoundError as e:
            raise ConfigError(f"model {model_id!r}: {e}") from None

    def model_path(self, model_id: str) -> Path | None:
        """Where the model's checkpoint is looked for: ``path`` (default: the id written as a relative path), taken
        relative to ``vendor.model_base_uri`` unless absolute. None for a preset, which has no files."""
        from .models import config as mc

        m = self.model(model_id)
        if m.path in mc.PRESETS or (m.path == m.id and m.id in mc.PRESETS):
            return None
        p = Path(m.path)
        base = self.values.get("vendor_model_base_uri") or ""
        return p if p.is_absolute() or not base else Path(base) / p

    def slo_for(self, model_id: str) -> Slo:
        m = self.model(model_id)
        return m.slo or self.values["scheduler_slo"]

    def ffn_tp_for(self, model_id: str) -> int:
        m = self.model(model_id)
        return m.ffn_tp_size or max(1, len(self.values["ffn_devices"]))

    def as_dict(self) -> dict[str, Any]:
        def enc(v):
            if isinstance(v, Slo):
                return {"ttft_ms": v.ttft_ms, "tbt_ms": v.tbt_ms}
            if isinstance(v, tuple):
                return list(v)
            return v

        d = {k: enc(v) for k, v in sorted(self.values.items()) if k != "config"}
        d["models"] = [{"id": m.id, "path": m.path, "atn_tp_size": m.atn_tp_size, "atn_dp_size": m.atn_dp_size,
                        "ffn_tp_size": m.ffn_tp_size, "ffn_ep_size": m.ffn_ep_size, "slo": enc(m.slo) if m.slo else None,
                        **({"external": True} if m.external else {})}
                       for m in self.models]
        return d

    def digest(self) -> str:
        return hashlib.sha256(json.dumps(self.as_dict(), sort_keys=True).encode()).hexdigest()


def reference_markdown() -> str:
    """The settings table of the user documentation (``xpool config reference``), generated from the registry so the
    two cannot drift apart."""
    def cell(v) -> str:
        return str(v).replace("|", "\\|")

    lines = ["| TOML key | environment | command line | default | meaning |", "| --- | --- | --- | --- | --- |"]
    for s in CONFIG_REGISTRY:
        key = ".".join(s.path) if s.path else "(bootstrap only)"
        default = "required" if s.required else ("" if s.default is _MISSING else repr(s.default))
        lines.append(f"| `{key}` | {f'`{s.env_var}`' if s.env_var else ''} | {f'`{s.cli}`' if s.cli else ''} | {cell(default)} | "
                     f"{cell(s.description or s.name)} |")
    return "\n".join(lines) + "\n"


def add_cli_arguments(parser: argparse.ArgumentParser) -> None:
    for s in CONFIG_REGISTRY:
        if s.cli:
            parser.add_argument(s.cli, dest=f"cfg_{s.name}", default=None, metavar="VALUE", help=s.description or s.name)


def cli_overrides(ns: argparse.Namespace) -> dict[str, Any]:
    return {s.name: getattr(ns, f"cfg_{s.name}") for s in CONFIG_REGISTRY
            if s.cli and getattr(ns, f"cfg_{s.name}", None) is not None}


def load_config(cli: Mapping[str, Any] | None = None, env: Mapping[str, str] | None = None,
                toml_text: str | None = None, require: bool = True) -> XpoolConfig:
    """Resolves the effective configuration. ``toml_text`` overrides reading the file named by
    ``--config`` / ``XPOOL_CONFIG``."""
    cli = dict(cli or {})
    env = os.environ if env is None else env
    path = cli.get("config") or env.get("XPOOL_CONFIG") or ""
    doc: Mapping[str, Any] = {}
    if toml_text is not None:
        doc = tomllib.loads(toml_text)
    elif path:
        p = Path(path)
        if not p.exists():
            raise ConfigError(f"config file {path} does not exist")
        doc = tomllib.loads(p.read_text())
    values: dict[str, Any] = {}
    sources: dict[str, str] = {}
    for s in CONFIG_REGISTRY:
        raw, src = _MISSING, "default"
        if s.name in cli and cli[s.name] is not None:
            raw, src = cli[s.name], "cli"
        elif s.env_var and s.env_var in env:
            raw, src = env[s.env_var], "env"
        elif s.path is not None and (v := _toml_get(doc, s.path)) is not _MISSING:
            raw, src = v, "toml"
        elif s.default is not _MISSING:
            raw = s.default
        if raw is _MISSING:
            if s.required and require:
                raise ConfigError(f"required setting {'.'.join(s.path or (s.name,))} is missing")
            values[s.name] = None
            sources[s.name] = "missing"
            continue
        try:
            values[s.name] = s.parser(raw)
        except ConfigError as e:
            raise ConfigError(f"{'.'.join(s.path or (s.name,))} ({src}): {e}") from None
        sources[s.name] = src
    values["config"] = str(path)
    atn, ffn = values.get("atn_devices") or (), values.get("ffn_devices") or ()
    if set(atn) & set(ffn):
        raise ConfigError(f"devices {sorted(set(atn) & set(ffn))} are listed under both [atn] and [ffn]")
    models = _parse_models(doc, ffn)
    for m in models:
        if m.atn_world_size > max(1, len(atn)) and require:
            raise ConfigError(f"model {m.id} needs {m.atn_world_size} attention devices, {len(atn)} configured")
    return XpoolConfig(values, models, sources)


_GLOBAL: XpoolConfig | None = None


def init_global_config(cli: Mapping[str, Any] | None = None, **kw) -> XpoolConfig:
    global _GLOBAL
    _GLOBAL = load_config(cli, **kw)
    return _GLOBAL


def global_config() -> XpoolConfig:
    if _GLOBAL is None:
        raise ConfigError("configuration not initialised")
    return _GLOBAL
