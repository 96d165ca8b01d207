"""Process entry points of ``xpool atnagent`` / ``xpool ffnagent``."""

from __future__ import annotations

import os

from ..config import XpoolConfig
from ..logging import get_logger, init_logging, kv
from ..service.client import XpoolClient
from ..service.wire import InstanceFfnProfile, Role



def hosted_instances(cfg: XpoolConfig, device: int) -> list[tuple[str, int]]:
    """Instance ranks hosted on an attention device: rank r of every model lives on the r-th
    attention device."""
    out = []
    for m in cfg.models:
        for r in range(m.atn_world_size):
            if cfg.atn_devices[r] == device:
                out.append((m.id, r))
    return out


def run_cpu_agent(cfg: XpoolConfig, role: str, device: int) -> int:
    """The agent of ``role`` for "device" ``device`` on the CPU data plane (``runtime/cpu_backends.py``): device numbers
    are only names here; memory admission sees the host's free memory."""
    import psutil

    from ..native import EXPECTED_ABI
    from ..service.client import self_ref
    from .backends import model_config_for
    from .cpu_backends import CpuAtnBackend, CpuFfnBackend, cpu_capacity_rows
    from .roles import AtnAgent, FfnAgent

    log = init_logging("AtnAgent" if role == "atnagent" else "FfnAgent", cfg.logging_level, cfg.logging_color)
    client = XpoolClient(cfg.daemon_host, cfg.daemon_port)
    owner = self_ref(EXPECTED_ABI)
    client.check_config(owner, cfg.digest())
    client.startup_agent(owner, Role.ATNAGENT if role == "atnagent" else Role.FFNAGENT, device)
    rows = cpu_capacity_rows(cfg)
    if role == "ffnagent":
        vm = psutil.virtual_memory()
        agent = FfnAgent(client, device, CpuFfnBackend(cfg, device, capacity_rows=rows), int(vm.available), int(vm.total), owner=owner)
    else:
        from ..service.wire import TransportArenaUpsert

        here = hosted_instances(cfg, device)
        insts = [(m, r) for m, r in here if not cfg.model(m).external]
        outside = [(m, r) for m, r in here if cfg.model(m).external]
        port = cfg.serving_base_port + cfg.atn_devices.index(device)
        backend = CpuAtnBackend(cfg, device, insts, listen=("127.0.0.1", port), capacity_rows=rows,
                                max_batch=min(cfg.engine_max_batch, 16), max_seq_len=min(cfg.engine_max_seq_len, rows),
                                external=outside,
                                publish_arenas=lambda gen, arenas: client.upsert_arenas(device, TransportArenaUpsert(
                                    owner=owner, generation=gen, arenas=arenas)))
        if cfg.atn_elastic_kv:
            backend.ecs_ref = client.ecs_channel
            backend.kv_budget_bytes = int(os.environ.get("XPOOL_CPU_KV_BYTES", backend.kv_budget_bytes))
        profs = [(m, r, InstanceFfnProfile(max_prefill_rows=rows, max_decode_rows=rows,
                                           hidden_size=model_config_for(cfg, m).hidden_size)) for m, r in insts]
        agent = AtnAgent(client, device, backend, profs, owner=owner)
    log.info(kv(event="start", role=role, device=device, pid=os.getpid(), backend="cpu"))
    rc = agent.run()
    if agent.failed:
        get_logger().error(kv(event="failed", reason=agent.failed, retained=agent.retained))
    return rc


def run_agent(cfg: XpoolConfig, role: str, device: int, backend: str = "gpu") -> int:
    if backend == "cpu":
        return run_cpu_agent(cfg, role, device)
    import torch

    from ..engine.atn_engine import EngineConfig
    from ..native import EXPECTED_ABI
    from ..service.client import self_ref
    from .backends import AtnBackend, FfnBackend, model_config_for
    from .roles import AtnAgent, FfnAgent

    log = init_logging("AtnAgent" if role == "atnagent" else "FfnAgent", cfg.logging_level, cfg.logging_color)
    client = XpoolClient(cfg.daemon_host, cfg.daemon_port)
    owner = self_ref(EXPECTED_ABI)
    client.check_config(owner, cfg.digest())
    client.startup_agent(owner, Role.ATNAGENT if role == "atnagent" else Role.FFNAGENT, device)
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    local = [int(x) for x in visible.split(",")].index(device) if visible else device
    torch.cuda.set_device(local)
    max_rows = cfg.engine_max_rows
    if role == "ffnagent":
        free, total = torch.cuda.mem_get_info(local)
        agent = FfnAgent(client, device, FfnBackend(cfg, device, capacity_rows=max_rows, local_index=local), free, total,
                         owner=owner)
    else:
        from ..service.wire import TransportArenaUpsert

        here = hosted_instances(cfg, device)
        insts = [(m, r) for m, r in here if not cfg.model(m).external]
        outside = [(m, r) for m, r in here if cfg.model(m).external]     # ranks that run in processes of their own
        chunk = min(max_rows, cfg.engine_prefill_chunk)   # tokens per prefill step
        ecfg = EngineConfig(max_batch=cfg.engine_max_batch, prefill_chunk=chunk, max_seq_len=cfg.engine_max_seq_len,
                            page_size=cfg.engine_page_size)
        port = cfg.serving_base_port + cfg.atn_devices.index(device)
        backend = AtnBackend(cfg, device, insts, ecfg, capacity_rows=max_rows, local_index=local, listen=("127.0.0.1", port),
                             external=outside,
                             publish_arenas=lambda gen, arenas: client.upsert_arenas(device, TransportArenaUpsert(
                                 owner=owner, generation=gen, arenas=arenas)))
        if cfg.atn_elastic_kv:
            backend.ecs_ref = client.ecs_channel
        profs = [(m, r, InstanceFfnProfile(max_prefill_rows=ecfg.prefill_chunk, max_decode_rows=ecfg.max_batch,
                                           hidden_size=model_config_for(cfg, m).hidden_size)) for m, r in insts]
        agent = AtnAgent(client, device, backend, profs, owner=owner)
    log.info(kv(event="start", role=role, device=device, pid=os.getpid()))
    rc = agent.run()
    if agent.failed:
        get_logger().error(kv(event="failed", reason=agent.failed, retained=agent.retained))
    return rc
