"""``xpool`` command line (reference: src/xpool/cli/main.py, subcommands/*).

    xpool daemon serve | check     control plane (exit 20 if a failure was recorded, else 0)
    xpool atnagent --device N      attention role for one GPU (hosts the Instances placed on it)
    xpool ffnagent --device N      FFN role for one GPU
    xpool exec -- <cmd ...>        normalise device visibility, export daemon endpoint, exec the command
    xpool config dump              print the effective configuration
    xpool memory-profile           print the analytic device memory estimate per FFN device
    xpool bench ...                serving benchmark (load generator + metrics)
"""

from __future__ import annotations

import argparse
import json
import os
import sys

from .. import config as C


def _parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="xpool", description="multi-model co-location serving for B200")
    C.add_cli_arguments(p)
    sub = p.add_subparsers(dest="command", required=True)
    d = sub.add_parser("daemon", help="control plane")
    ds = d.add_subparsers(dest="daemon_command", required=True)
    ds.add_parser("serve", help="run the daemon")
    ds.add_parser("check", help="print a running daemon's readiness snapshot; exit code 0 when the system is ready")
    for name, what in (("atnagent", "attention agent of one device: hosts its Instances (engine, KV, POST /generate) or brokers "
                                    "the arenas of external ones"),
                       ("ffnagent", "FFN agent of one device: loads the FFN shards the plan assigns to it and serves them")):
        a = sub.add_parser(name, help=what)
        a.add_argument("--device", type=int, required=True)
        a.add_argument("--backend", choices=("gpu", "cpu"), default="gpu",
                       help="cpu: the same control plane with the shared-memory data plane and the PyTorch oracle (no GPU needed)")
    r = sub.add_parser("router", help="one POST /generate endpoint in front of the data-parallel ranks the daemon lists")
    r.add_argument("--host", default="127.0.0.1")
    r.add_argument("--port", type=int, required=True)
    r.add_argument("--model", action="append", default=None, help="restrict to these models (default: every model with a listener)")
    e = sub.add_parser("exec", help="run a command in the deployment's environment")
    e.add_argument("argv", nargs=argparse.REMAINDER)
    c = sub.add_parser("config", help="dump the resolved configuration; print the settings and supported-model references")
    cs = c.add_subparsers(dest="config_command", required=True)
    cs.add_parser("dump", help="the resolved configuration with the source of every value")
    cs.add_parser("reference", help="every setting with its TOML key, environment variable, flag and default (markdown)")
    cs.add_parser("models", help="supported architectures and what runs where (markdown)")
    mp = sub.add_parser("memory-profile", help="placement and memory admission of the configured models; --calibrate fits the overhead model")
    mp.add_argument("--calibrate", action="store_true", help="measure a corpus of synthetic deployments on this GPU and fit the model")
    mp.add_argument("--out", default="xpool-memory-profile.json")
    b = sub.add_parser("bench", help="open-loop load generator against running Instances (--targets MODEL=URL ...)")
    b.add_argument("rest", nargs=argparse.REMAINDER)
    q = sub.add_parser("qualify", help="check an architecture's FFN path against its checkpoint description")
    q.add_argument("rest", nargs=argparse.REMAINDER)
    return p


def _load(ns, require=True) -> C.XpoolConfig:
    return C.init_global_config(C.cli_overrides(ns), require=require)


def cmd_config_dump(ns) -> int:
    cfg = _load(ns, require=False)
    print(json.dumps({"digest": cfg.digest(), "config": cfg.as_dict(), "sources": dict(cfg.sources)}, indent=2))
    return 0


def cmd_config_reference(ns) -> int:
    print(C.reference_markdown(), end="")
    return 0


def cmd_config_models(ns) -> int:
    from ..models.support import support_markdown

    print(support_markdown(), end="")
    return 0


def cmd_daemon_serve(ns) -> int:
    import uvicorn

    from ..logging import init_logging
    from ..service.daemon.app import create_app
    from ..service.daemon.control import ControlPlane

    cfg = _load(ns)
    init_logging("Daemon", cfg.logging_level, cfg.logging_color)
    cp = ControlPlane(cfg)
    factory = None
    if cfg.atn_elastic_kv:
        from ..service.daemon.ecs_service import EcsService

        holder = {}

        def factory(control):
            return EcsService(control, lambda ref: setattr(holder["app"].state, "ecs_channel_ref", ref) if "app" in holder else None,
                              utilization=cfg.atn_device_memory_utilization)

        app = create_app(cfg, cp, ecs_factory=factory)
        holder["app"] = app
    else:
        app = create_app(cfg, cp)
    uvicorn.run(app, host=cfg.daemon_host, port=cfg.daemon_port, log_level="warning")
    return cp.exit_code


def cmd_daemon_check(ns) -> int:
    from ..service.client import XpoolClient
    from ..service.errors import ClientError, DaemonError

    cfg = _load(ns, require=False)
    cl = XpoolClient(cfg.daemon_host, cfg.daemon_port)
    try:
        snap = cl.ready()
    except (ClientError, DaemonError) as e:
        print(json.dumps({"reachable": False, "error": str(e)}))
        return 1
    print(snap.model_dump_json(indent=2))
    return 0 if snap.system_ready else 1


def exec_environment(cfg: C.XpoolConfig, environ: dict[str, str]) -> dict[str, str]:
    """Environment for ``xpool exec``: all configured devices visible in configuration order, the
    daemon endpoint and the config path exported. (The reference additionally exports its MPS pipe
    directory, src/xpool/cli/subcommands/exec.py:29-48; this system runs one process per GPU and
    needs no MPS.)"""
    env = dict(environ)
    devs = list(cfg.atn_devices or ()) + list(cfg.ffn_devices or ())
    if devs:
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(d) for d in devs)
    env["XPOOL_DAEMON_HOST"] = str(cfg.daemon_host)
    env["XPOOL_DAEMON_PORT"] = str(cfg.daemon_port)
    if cfg.config:
        env["XPOOL_CONFIG"] = str(cfg.config)
    env.setdefault("SGLANG_PLUGINS", "xpool")
    return env


def cmd_exec(ns) -> int:
    argv = [a for a in ns.argv if a != "--"] if ns.argv and ns.argv[0] == "--" else list(ns.argv)
    if not argv:
        print("xpool exec: no command given", file=sys.stderr)
        return 2
    cfg = _load(ns, require=False)
    os.execvpe(argv[0], argv, exec_environment(cfg, dict(os.environ)))
    return 127  # not reached


def cmd_memory_profile(ns) -> int:
    if getattr(ns, "calibrate", False):
        from ..runtime import memory_calibration as mcal

        cfg = _load(ns, require=False)
        prof = mcal.calibrate(evidence_root=cfg.cache_root)     # evidence persists under the cache root; re-runs resume
        prof.save(ns.out)
        print(json.dumps({"saved": ns.out, "samples": prof.samples, "max_abs_error_bytes": prof.max_abs_error_bytes,
                          "coefficients": vars(prof.coefficients)}, indent=2))
        return 0
    from ..service.daemon.placement import DeviceSupply, ModelDemand, place_ffn_models

    cfg = _load(ns)
    demands = []
    for m in cfg.models:
        c = cfg.model_shape(m.id)
        inter = c.moe_intermediate_size * max(1, c.num_experts_per_tok) if c.is_moe else c.intermediate_size
        demands.append(ModelDemand(m.id, tuple(c.ffn_param_bytes_per_layer(l) for l in range(c.num_layers)),
                                   cfg.ffn_tp_for(m.id), c.hidden_size, 4096, m.atn_world_size, inter))
    devs = [DeviceSupply(d, 170 << 30, 180 << 30) for d in cfg.ffn_devices]
    r = place_ffn_models(demands, devs, margin_bytes=cfg.ffn_device_memory_extra_margin_bytes,
                         lanes=cfg.scheduler_ffn_concurrency)
    out = {str(d): {"stages": vars(s), "peak": s.peak, "headroom": r.headroom[d]} for d, s in r.stages.items()}
    print(json.dumps({"devices": out, "groups": [vars(g) for g in r.groups]}, indent=2, default=list))
    return 0


def cmd_agent(ns, role: str) -> int:
    from ..runtime.launch import run_agent

    cfg = _load(ns)
    return run_agent(cfg, role, ns.device, backend=ns.backend)


def cmd_bench(ns) -> int:
    from ..bench import serving

    return serving.main(ns.rest)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    # `bench` and `qualify` hand everything behind them to their own parsers (option-like words included, which
    # argparse's REMAINDER does not accept as the first word)
    passthrough = None
    for i, word in enumerate(argv):
        if word in ("bench", "qualify"):
            argv, passthrough = argv[: i + 1], argv[i + 1:]
            break
    ns = _parser().parse_args(argv)
    if passthrough is not None:
        ns.rest = passthrough
    try:
        if ns.command == "config":
            return {"dump": cmd_config_dump, "reference": cmd_config_reference, "models": cmd_config_models}[ns.config_command](ns)
        if ns.command == "daemon":
            return cmd_daemon_serve(ns) if ns.daemon_command == "serve" else cmd_daemon_check(ns)
        if ns.command == "exec":
            return cmd_exec(ns)
        if ns.command == "router":
            from ..runtime.dp_router import serve_router

            cfg = _load(ns, require=False)
            return serve_router(f"http://{cfg.daemon_host}:{cfg.daemon_port}", ns.host, ns.port, ns.model)
        if ns.command == "memory-profile":
            return cmd_memory_profile(ns)
        if ns.command in ("atnagent", "ffnagent"):
            return cmd_agent(ns, ns.command)
        if ns.command == "bench":
            return cmd_bench(ns)
        if ns.command == "qualify":
            from ..devtools import qualification

            return qualification.main(ns.rest)
    except C.ConfigError as e:
        print(f"xpool: configuration error: {e}", file=sys.stderr)
        return 2
    return 2


if __name__ == "__main__":
    sys.exit(main())
