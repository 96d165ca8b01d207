"""Wire models of the control plane (HTTP/JSON between the daemon and every other process).

All models forbid unknown fields. The shapes follow the reference's wire module
(src/xpool/service/wire.py): process identity is ``(pid, create_time)`` so that PID reuse is
detected, every joining process states its native ABI number, agents register by device, Instance
ranks by ``(model id, rank)``, and Fabric participants report their phase per generation.
"""

from __future__ import annotations

from enum import Enum
from typing import Any

from pydantic import BaseModel, ConfigDict, Field


class WireModel(BaseModel):
    model_config = ConfigDict(extra="forbid")


class Role(str, Enum):
    DAEMON = "daemon"
    INSTANCE = "instance"
    ATNAGENT = "atnagent"
    FFNAGENT = "ffnagent"


class ProcessRef(WireModel):
    abi_version: int
    pid: int
    create_time: float = 0.0


class ErrorDetail(WireModel):
    code: str  # conflict | not_ready | not_found | invalid | mismatch | gone
    message: str


class ConfigCheckRequest(WireModel):
    owner: ProcessRef
    digest: str


class AgentStartupAdmission(WireModel):
    owner: ProcessRef
    role: Role
    device: int


class AtnAgentRegistration(WireModel):
    owner: ProcessRef
    device: int
    device_free_memory_bytes: int = 0
    device_total_memory_bytes: int = 0


class GemmDeviceProperties(WireModel):
    compute_capability: tuple[int, int] = (10, 0)
    sm_count: int = 148


class FfnAgentRegistration(WireModel):
    owner: ProcessRef
    device: int
    device_free_memory_bytes: int
    device_total_memory_bytes: int
    model_specs: list[dict[str, Any]] = Field(default_factory=list)  # FfnModelSpec digests and byte sizes
    device_properties: GemmDeviceProperties = GemmDeviceProperties()


class InstanceFfnProfile(WireModel):
    """Row capacities the Instance will ever submit, per forward mode."""

    max_prefill_rows: int
    max_decode_rows: int
    payload_dtype: str = "bfloat16"
    hidden_size: int
    layer_kinds: list[str] = []               # "dense" | "moe" per decoder layer, as installed in the serving process
    group_sum_complete_admitted: bool = False  # attention DP > 1: the Instance may ask for the group sum


class ContextStateProfile(WireModel):
    floor_bytes: int = 0
    reservation_bytes: int = 0
    bundle_bytes: int = 0


class InstanceRankRegistration(WireModel):
    owner: ProcessRef
    model_id: str
    rank: int
    device: int
    ffn_profile: InstanceFfnProfile
    context_state_profile: ContextStateProfile = ContextStateProfile()
    atn_runtime_headroom_bytes: int = 0


class ServingListener(WireModel):
    host: str
    port: int


class InstanceRankInitialized(WireModel):
    owner: ProcessRef
    rank: int
    generation: int
    serving_listener: ServingListener | None = None


class FabricPhase(str, Enum):
    """Generation phases, advanced by the daemon only when every participant reported the matching
    participant phase (src/xpool/fabric.py:50-114)."""

    IDLE = "idle"
    PREPARING_JOIN = "preparing_join"
    JOINING = "joining"
    PREPARING_EXECUTION = "preparing_execution"
    ACTIVATING = "activating"
    EXECUTABLE = "executable"
    QUIESCING = "quiescing"
    DRAINING = "draining"
    FINALIZING = "finalizing"
    STOPPED = "stopped"
    ABORTING = "aborting"


class ParticipantPhase(str, Enum):
    REGISTERED = "registered"
    JOIN_READY = "join_ready"
    JOINED = "joined"
    EXECUTION_READY = "execution_ready"
    ACTIVE = "active"
    QUIESCED = "quiesced"
    DRAINED = "drained"
    FINALIZED = "finalized"


class InvocationFailure(WireModel):
    result_code: int
    origin_pe: int
    instance_index: int
    invocation_sequence: int
    layer_ordinal: int


class OwnerFailureReason(str, Enum):
    EXITED = "exited"
    STALE = "stale"
    REPLACED = "replaced"


class ParticipantReport(WireModel):
    owner: ProcessRef
    generation: int
    pe: int
    phase: ParticipantPhase
    invocation_failure: InvocationFailure | None = None
    control_failure: str | None = None


class HeartbeatRequest(WireModel):
    owner: ProcessRef


class HeartbeatResponse(WireModel):
    warnings: list[str] = Field(default_factory=list)
    generation: int | None = None
    fabric_phase: FabricPhase | None = None


class TransportArenaBinding(WireModel):
    model_id: str
    rank: int
    handle_hex: str
    nbytes: int


class TransportArenaUpsert(WireModel):
    owner: ProcessRef
    generation: int
    arenas: list[TransportArenaBinding]


class TransportArenaAcquire(WireModel):
    owner: ProcessRef
    rank: int
    generation: int


class TransportLeaseQuiesceResponse(WireModel):
    in_use: list[tuple[str, int]] = Field(default_factory=list)


class QuiesceRequest(WireModel):
    reason: str = "operator"


class ShardPlacement(WireModel):
    model_id: str
    layer_begin: int
    layer_end: int
    tp_rank: int
    tp_size: int
    device: int
    pe: int
    bytes: int


class InstanceRankTopology(WireModel):
    model_id: str
    rank: int
    device: int
    pe: int
    instance_index: int


class FabricPlan(WireModel):
    generation: int
    uid: str
    phase: FabricPhase
    atn_devices: list[int]
    ffn_devices: list[int]
    lanes_per_ffn_device: int
    policy: str
    shards: list[ShardPlacement]
    instance_ranks: list[InstanceRankTopology]
    slot_handles: dict[str, str] = Field(default_factory=dict)  # "ffn:<model>:<pe>" / "atn:<model>:<rank>" -> hex


class SlotHandlePublication(WireModel):
    owner: ProcessRef
    generation: int
    handles: dict[str, str]


class EcsChannelRef(WireModel):
    generation: int
    name: str
    partitions: dict[str, int] = Field(default_factory=dict)  # "<model>:<rank>" -> partition index
    devices: dict[str, int] = Field(default_factory=dict)     # "<device>" -> device index


class ReadinessEntry(WireModel):
    key: str
    state: str
    detail: str = ""


class ReadinessSnapshot(WireModel):
    fabric_executable: bool
    system_ready: bool
    serving_healthy: bool
    generation: int | None
    phase: FabricPhase
    atnagents: list[ReadinessEntry] = Field(default_factory=list)
    ffnagents: list[ReadinessEntry] = Field(default_factory=list)
    instance_ranks: list[ReadinessEntry] = Field(default_factory=list)
    warnings: list[str] = Field(default_factory=list)
    failure: str | None = None
