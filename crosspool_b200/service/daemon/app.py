"""HTTP face of the daemon: FastAPI routes over :class:`ControlPlane`.

Route set and background tasks follow the reference's app (src/xpool/service/daemon/app.py):
``/health``, ``/ready``, ``/config``, ``/fabric/plan``, ``/fabric/quiesce``,
``/fabric/participant-reports``, ``/config/check``, ``/startup/agent``, registration and heartbeat
routes per role, Transport arena routes, ``/ecs/control-channel/{generation}``; a watchdog task every
second and the ECS capacity policy every 10 ms.
"""

from __future__ import annotations

import asyncio
import contextlib
import os

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse

from ...config import XpoolConfig
from ..errors import DaemonError
from ..wire import (AgentStartupAdmission, AtnAgentRegistration, ConfigCheckRequest, EcsChannelRef, FfnAgentRegistration,
                    HeartbeatRequest, InstanceRankInitialized, InstanceRankRegistration, ParticipantReport,
                    QuiesceRequest, SlotHandlePublication, TransportArenaAcquire, TransportArenaUpsert,
                    TransportLeaseQuiesceResponse)
from ..wire import ProcessRef
from .control import ControlPlane

WATCHDOG_SECONDS = 1.0
CAPACITY_POLICY_SECONDS = 0.010


def create_app(config: XpoolConfig, control: ControlPlane | None = None, *, background: bool = True,
               ecs_factory=None) -> FastAPI:
    cp = control or ControlPlane(config)

    @contextlib.asynccontextmanager
    async def lifespan(app: FastAPI):
        tasks = []
        if background:
            tasks.append(asyncio.create_task(_periodic(WATCHDOG_SECONDS, cp.watchdog)))
            if app.state.ecs is not None:
                tasks.append(asyncio.create_task(_periodic(CAPACITY_POLICY_SECONDS, app.state.ecs.tick)))
        try:
            yield
        finally:
            cp.begin_close()
            for t in tasks:
                t.cancel()
            for t in tasks:
                with contextlib.suppress(asyncio.CancelledError, Exception):
                    await t

    app = FastAPI(title="xpool daemon", lifespan=lifespan)
    app.state.control = cp
    app.state.ecs = ecs_factory(cp) if ecs_factory else None
    app.state.ecs_channel_ref = None

    @app.exception_handler(DaemonError)
    async def _daemon_error(_: Request, e: DaemonError):
        return JSONResponse(status_code=e.http_status, content={"detail": {"code": e.code, "message": e.message}})

    @app.get("/health")
    def health():
        return {"status": "ok", "pid": os.getpid(), "failure": cp.failure}

    @app.get("/ready")
    def ready():
        return cp.readiness()

    @app.get("/config")
    def get_config():
        return {"digest": config.digest(), "config": config.as_dict()}

    @app.post("/config/check")
    def config_check(req: ConfigCheckRequest):
        cp.check_config(req.owner, req.digest)
        return {"ok": True}

    @app.post("/startup/agent")
    def startup_agent(req: AgentStartupAdmission):
        cp.admit_agent(req)
        return {"ok": True}

    @app.get("/fabric/plan")
    def fabric_plan():
        return cp.fabric_plan()

    @app.post("/fabric/quiesce")
    def fabric_quiesce(req: QuiesceRequest):
        return {"phase": cp.quiesce(req.reason)}

    @app.post("/fabric/participant-reports")
    def participant_reports(rep: ParticipantReport):
        return {"phase": cp.report_participant(rep)}

    @app.post("/fabric/slot-handles")
    def slot_handles(pub: SlotHandlePublication):
        cp.publish_slot_handles(pub.owner, pub.generation, pub.handles)
        return {"ok": True}

    @app.get("/atnagents")
    def atnagents():
        return {str(d): {"pid": r.owner.pid, "phase": r.phase, "pe": r.pe} for d, r in cp.atnagents.items()}

    @app.get("/ffnagents")
    def ffnagents():
        return {str(d): {"pid": r.owner.pid, "phase": r.phase, "pe": r.pe, "free_bytes": r.payload.device_free_memory_bytes,
                         "total_bytes": r.payload.device_total_memory_bytes} for d, r in cp.ffnagents.items()}

    @app.get("/instances")
    def instances():
        return {f"{k[0]}:{k[1]}": {"pid": r.owner.pid, "initialized": r.initialized, "device": r.payload.device,
                                   "listener": f"{r.listener[0]}:{r.listener[1]}" if r.listener else None,
                                   "max_prefill_rows": r.payload.ffn_profile.max_prefill_rows,
                                   "max_decode_rows": r.payload.ffn_profile.max_decode_rows}
                for k, r in cp.instances.items()}

    @app.post("/atnagent/register")
    def atn_register(r: AtnAgentRegistration):
        cp.register_atnagent(r)
        return {"ok": True}

    @app.post("/atnagent/{device}/heartbeat")
    def atn_heartbeat(device: int, req: HeartbeatRequest):
        return cp.heartbeat("atnagent", device, req.owner)

    @app.post("/ffnagent/register")
    def ffn_register(r: FfnAgentRegistration):
        cp.register_ffnagent(r)
        return {"ok": True}

    @app.post("/ffnagent/{device}/heartbeat")
    def ffn_heartbeat(device: int, req: HeartbeatRequest):
        return cp.heartbeat("ffnagent", device, req.owner)

    @app.post("/atnagent/{device}/transport-arenas")
    def transport_arenas(device: int, req: TransportArenaUpsert):
        cp.upsert_arenas(device, req.owner, req.generation, req.arenas)
        return {"ok": True}

    @app.post("/atnagent/{device}/transport-leases/quiesce")
    def transport_quiesce(device: int, req: HeartbeatRequest):
        return TransportLeaseQuiesceResponse(in_use=cp.quiesce_leases(device, req.owner))

    @app.post("/instance/register")
    def instance_register(r: InstanceRankRegistration):
        cp.register_instance(r)
        return {"ok": True}

    @app.post("/instance/{model_id:path}/deregister")
    def instance_deregister(model_id: str, req: TransportArenaAcquire):
        cp.deregister_instance(model_id, req.rank, req.owner)
        return {"ok": True}

    @app.post("/instance/{model_id:path}/initialized")
    def instance_initialized(model_id: str, req: InstanceRankInitialized):
        cp.instance_initialized(model_id, req)
        return {"ok": True}

    @app.post("/instance/{model_id:path}/heartbeat/{rank}")
    def instance_heartbeat(model_id: str, rank: int, req: HeartbeatRequest):
        return cp.heartbeat("instance", (model_id, rank), req.owner)

    @app.post("/instance/{model_id:path}/transport-arena/acquire")
    def instance_acquire(model_id: str, req: TransportArenaAcquire):
        return cp.acquire_arena(model_id, req.rank, req.owner, req.generation)

    @app.post("/serving/terminate-owner")
    @app.post("/serving/mps/terminate-client")   # the reference's route name, kept for its clients
    def terminate_owner(owner: ProcessRef):
        return {"signalled": cp.terminate_owner(owner)}

    @app.get("/metrics")
    def metrics():
        from fastapi.responses import PlainTextResponse

        from ...runtime.metrics import render_daemon

        return PlainTextResponse(render_daemon(cp, app.state.ecs))

    @app.get("/ecs/state")
    def ecs_state():
        if app.state.ecs is None:
            raise DaemonError("not_ready", "elastic KV is not enabled in this deployment")
        return app.state.ecs.state()

    @app.get("/ecs/control-channel/{generation}")
    def ecs_channel(generation: int):
        ref: EcsChannelRef | None = app.state.ecs_channel_ref
        if ref is None or ref.generation != generation:
            raise DaemonError("not_ready", "no ECS control channel for this generation")
        return ref

    return app


async def _periodic(seconds: float, fn) -> None:
    while True:
        try:
            fn()
        except Exception:  # a failing tick must not kill the daemon; the next one retries
            pass
        await asyncio.sleep(seconds)
