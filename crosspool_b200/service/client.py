"""Client of the daemon's HTTP API (methods map 1:1 to routes; default timeout 5 s like the
reference's ``XpoolClient``, src/xpool/service/client.py)."""

from __future__ import annotations

import os
from typing import Any
from urllib.parse import quote

import httpx
import psutil

from .errors import ClientError, DaemonError
from .wire import (AgentStartupAdmission, AtnAgentRegistration, ConfigCheckRequest, EcsChannelRef, FabricPlan,
                   FfnAgentRegistration, HeartbeatRequest, HeartbeatResponse, InstanceRankInitialized,
                   InstanceRankRegistration, ParticipantReport, ProcessRef, QuiesceRequest, ReadinessSnapshot, Role,
                   SlotHandlePublication, TransportArenaAcquire, TransportArenaBinding, TransportArenaUpsert)


def self_ref(abi_version: int) -> ProcessRef:
    p = psutil.Process(os.getpid())
    return ProcessRef(abi_version=abi_version, pid=p.pid, create_time=p.create_time())


class XpoolClient:
    def __init__(self, host: str = "127.0.0.1", port: int = 9810, timeout: float = 5.0, transport=None):
        self._http = httpx.Client(base_url=f"http://{host}:{port}", timeout=timeout, transport=transport)

    def close(self) -> None:
        self._http.close()

    def _call(self, method: str, path: str, body: Any = None) -> Any:
        try:
            r = self._http.request(method, path, json=body.model_dump(mode="json") if body is not None else None)
        except httpx.HTTPError as e:
            raise ClientError(f"daemon unreachable: {e}") from None
        if r.status_code >= 400:
            try:
                d = r.json()["detail"]
                raise DaemonError(d["code"], d["message"])
            except (KeyError, TypeError, ValueError):
                raise ClientError(f"HTTP {r.status_code}: {r.text[:200]}") from None
        return r.json()

    # -- general
    def health(self) -> dict:
        return self._call("GET", "/health")

    def ready(self) -> ReadinessSnapshot:
        return ReadinessSnapshot.model_validate(self._call("GET", "/ready"))

    def config(self) -> dict:
        return self._call("GET", "/config")

    def check_config(self, owner: ProcessRef, digest: str) -> None:
        self._call("POST", "/config/check", ConfigCheckRequest(owner=owner, digest=digest))

    def startup_agent(self, owner: ProcessRef, role: Role, device: int) -> None:
        self._call("POST", "/startup/agent", AgentStartupAdmission(owner=owner, role=role, device=device))

    # -- fabric
    def fabric_plan(self) -> FabricPlan:
        return FabricPlan.model_validate(self._call("GET", "/fabric/plan"))

    def quiesce(self, reason: str = "operator") -> str:
        return self._call("POST", "/fabric/quiesce", QuiesceRequest(reason=reason))["phase"]

    def report(self, rep: ParticipantReport) -> str:
        return self._call("POST", "/fabric/participant-reports", rep)["phase"]

    def publish_slot_handles(self, owner: ProcessRef, generation: int, handles: dict[str, str]) -> None:
        self._call("POST", "/fabric/slot-handles", SlotHandlePublication(owner=owner, generation=generation, handles=handles))

    # -- agents
    def register_atnagent(self, r: AtnAgentRegistration) -> None:
        self._call("POST", "/atnagent/register", r)

    def register_ffnagent(self, r: FfnAgentRegistration) -> None:
        self._call("POST", "/ffnagent/register", r)

    def heartbeat_atnagent(self, device: int, owner: ProcessRef) -> HeartbeatResponse:
        return HeartbeatResponse.model_validate(self._call("POST", f"/atnagent/{device}/heartbeat", HeartbeatRequest(owner=owner)))

    def heartbeat_ffnagent(self, device: int, owner: ProcessRef) -> HeartbeatResponse:
        return HeartbeatResponse.model_validate(self._call("POST", f"/ffnagent/{device}/heartbeat", HeartbeatRequest(owner=owner)))

    def upsert_arenas(self, device: int, req: TransportArenaUpsert) -> None:
        self._call("POST", f"/atnagent/{device}/transport-arenas", req)

    def quiesce_leases(self, device: int, owner: ProcessRef) -> list:
        return self._call("POST", f"/atnagent/{device}/transport-leases/quiesce", HeartbeatRequest(owner=owner))["in_use"]

    # -- instances
    def register_instance(self, r: InstanceRankRegistration) -> None:
        self._call("POST", "/instance/register", r)

    def instance_initialized(self, model_id: str, req: InstanceRankInitialized) -> None:
        self._call("POST", f"/instance/{quote(model_id, safe='/')}/initialized", req)

    def heartbeat_instance(self, model_id: str, rank: int, owner: ProcessRef) -> HeartbeatResponse:
        return HeartbeatResponse.model_validate(
            self._call("POST", f"/instance/{quote(model_id, safe='/')}/heartbeat/{rank}", HeartbeatRequest(owner=owner)))

    def acquire_arena(self, model_id: str, req: TransportArenaAcquire) -> TransportArenaBinding:
        return TransportArenaBinding.model_validate(
            self._call("POST", f"/instance/{quote(model_id, safe='/')}/transport-arena/acquire", req))

    def deregister_instance(self, model_id: str, req: TransportArenaAcquire) -> None:
        self._call("POST", f"/instance/{quote(model_id, safe='/')}/deregister", req)

    def ecs_channel(self, generation: int) -> EcsChannelRef:
        return EcsChannelRef.model_validate(self._call("GET", f"/ecs/control-channel/{generation}"))
