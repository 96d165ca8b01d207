"""Python bindings of the host-only C++ runtime (``libxpool_runtime.so``).

Objects here are thin owners of native handles: :class:`LaneScheduler` (FIFO / Random / SLO Lane
scheduling, the host twin of the device scheduler), :class:`SharedMemory`, :class:`EcsChannel`
(seqlock control channel of Elastic Context State), :class:`CpuMailbox` (Transport mailbox over
POSIX shm for CPU roles) and :class:`TraceBuffer`.
"""

from __future__ import annotations

import ctypes as C
import functools
from dataclasses import dataclass

from ..utils.integer import ensure_uint32, ensure_uint64
from . import EXPECTED_ABI, NativeLibraryError, _load

u32, u64, vp = C.c_uint32, C.c_uint64, C.c_void_p


@functools.lru_cache(maxsize=None)
def lib() -> C.CDLL:
    L = _load("libxpool_runtime.so")
    L.xr_abi_version.restype = C.c_int
    if L.xr_abi_version() != EXPECTED_ABI:
        raise NativeLibraryError(f"libxpool_runtime.so has ABI {L.xr_abi_version()}, expected {EXPECTED_ABI}")
    sig = {
        "xr_plan_ffn_slot": (C.c_int, [u64, u64, u64, u64, C.POINTER(u64)]),
        "xr_plan_atn_slot": (C.c_int, [u64, u64, u64, u64, C.POINTER(u64)]),
        "xr_runtime_initialize": (C.c_int, [C.c_uint32, C.c_int32, C.POINTER(C.c_uint32)]),
        "xr_runtime_state": (None, [C.POINTER(C.c_uint32)]),
        "xr_runtime_reset_for_tests": (None, []),
        "xr_dp_inspect_rows": (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                            C.POINTER(C.c_uint32)]),
        "xr_validate_invocation": (C.c_uint32, [C.c_uint32] * 9),
        "xr_validate_completion": (C.c_uint32, [C.c_uint32] * 5),
        "xr_record_bytes": (u64, [C.c_int]),
        "xr_mailbox_transition_allowed": (C.c_int, [u32, u32]),
        "xr_sched_create": (vp, [u32, u32, u32, u64]),
        "xr_sched_destroy": (None, [vp]),
        "xr_sched_enqueue": (C.c_int, [vp, u32, u64, u64]),
        "xr_sched_try": (C.c_int, [vp, C.POINTER(u32), C.POINTER(u32), C.POINTER(u64)]),
        "xr_sched_active": (C.c_int, [vp, u32, C.POINTER(u32), C.POINTER(u64)]),
        "xr_sched_release": (C.c_int, [vp, u32, u64]),
        "xr_splitmix64": (u64, [u64]),
        "xr_shm_create": (vp, [C.c_char_p, u64, C.POINTER(C.c_int)]),
        "xr_shm_attach": (vp, [C.c_char_p, C.POINTER(C.c_int)]),
        "xr_shm_data": (vp, [vp]),
        "xr_shm_size": (u64, [vp]),
        "xr_shm_close": (None, [vp]),
        "xr_ecs_create": (vp, [C.c_char_p, u32, u32, u32, C.POINTER(C.c_int)]),
        "xr_ecs_attach": (vp, [C.c_char_p, C.POINTER(C.c_int)]),
        "xr_ecs_close": (None, [vp]),
        "xr_ecs_counts": (u32, [vp, C.POINTER(u32), C.POINTER(u32)]),
        "xr_ecs_set_device": (C.c_int, [vp, u32, u32]),
        "xr_ecs_set_partition": (C.c_int, [vp, u32, u32, u32, u32, u64, u64]),
        "xr_ecs_get_partition": (C.c_int, [vp, u32, C.POINTER(u64)]),
        "xr_ecs_publish_report": (C.c_int, [vp, u32, u64, u64, u64]),
        "xr_ecs_read_report": (C.c_int, [vp, u32, C.POINTER(u64)]),
        "xr_ecs_publish_command": (C.c_int, [vp, u32, u64, u64]),
        "xr_ecs_read_command": (C.c_int, [vp, u32, C.POINTER(u64)]),
        "xr_ecs_publish_demand": (C.c_int, [vp, u32, u64, u64, u64, u64]),
        "xr_ecs_read_demand": (C.c_int, [vp, u32, C.POINTER(u64)]),
        "xr_ecs_publish_completion": (C.c_int, [vp, u32, u64, u64]),
        "xr_ecs_read_completion": (C.c_int, [vp, u32, C.POINTER(u64)]),
        "xr_mbox_bytes": (u64, [u64, u64]),
        "xr_mbox_create": (vp, [C.c_char_p, u64, u64, C.POINTER(C.c_int)]),
        "xr_mbox_attach": (vp, [C.c_char_p, u64, u64, C.POINTER(C.c_int)]),
        "xr_mbox_close": (None, [vp]),
        "xr_mbox_status": (u32, [vp]),
        "xr_mbox_failure": (u32, [vp]),
        "xr_mbox_activate": (C.c_int, [vp]),
        "xr_mbox_shutdown": (None, [vp]),
        "xr_mbox_wait_status": (C.c_int, [vp, u32, u64]),
        "xr_mbox_submit": (u32, [vp, vp, vp, u32, u32, u32, u32, u32, u64]),
        "xr_mbox_take": (C.c_int, [vp, u64, C.POINTER(u32)]),
        "xr_mbox_input": (vp, [vp]),
        "xr_mbox_output": (vp, [vp]),
        "xr_mbox_complete": (C.c_int, [vp, u32]),
        "xr_trace_create": (vp, [u32]),
        "xr_trace_destroy": (None, [vp]),
        "xr_trace_record": (C.c_int, [vp, u32, u32, u32, u64]),
        "xr_trace_counts": (u64, [vp, C.POINTER(u64)]),
        "xr_trace_read": (u64, [vp, u64, u64, C.POINTER(u64)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


# ------------------------------------------------------------------ enums (mirror xpool/protocol.hpp)

ROLE_DAEMON, ROLE_INSTANCE, ROLE_ATNAGENT, ROLE_FFNAGENT = 1, 2, 3, 4
MODE_PREFILL, MODE_DECODE, MODE_IDLE = 1, 2, 4
OUT_PER_RANK_COMPLETE, OUT_GROUP_SUM_COMPLETE = 1, 2
DP_NONE, DP_UNIFORM_BY_RANK, DP_PACKED_BY_RANK = 0, 1, 2
RESULT_OK, RESULT_SHUTDOWN, RESULT_PROTOCOL_MISMATCH, RESULT_TIMEOUT = 0, 1, 2, 3
MBOX_DORMANT, MBOX_IDLE, MBOX_STAGING, MBOX_PUBLISHED, MBOX_EVALUATED, MBOX_CLOSED = range(6)
POLICY_FIFO, POLICY_RANDOM, POLICY_SLO = 0, 1, 2
WAIT_READY, WAIT_TIMED_OUT, WAIT_CANCELLED = 0, 1, 2


@dataclass(frozen=True)
class FfnSlotLayout:
    record_offset: int
    input_offset: int
    act_offset: int
    total_bytes: int


@dataclass(frozen=True)
class AtnSlotLayout:
    completion_offset: int
    output_offset: int
    output_stride: int
    total_bytes: int


def plan_ffn_slot(capacity_rows: int, hidden: int, local_inter: int, elem_bytes: int = 2) -> FfnSlotLayout:
    out = (u64 * 4)()
    if lib().xr_plan_ffn_slot(capacity_rows, hidden, local_inter, elem_bytes, out) != 0:
        raise ValueError("ffn slot layout overflows")
    return FfnSlotLayout(*out)


def plan_atn_slot(capacity_rows: int, hidden: int, tp: int, elem_bytes: int = 2) -> AtnSlotLayout:
    out = (u64 * 4)()
    if lib().xr_plan_atn_slot(capacity_rows, hidden, tp, elem_bytes, out) != 0:
        raise ValueError("atn slot layout overflows")
    return AtnSlotLayout(*out)


ROLE_IDS = {"Daemon": 1, "Instance": 2, "AtnAgent": 3, "FfnAgent": 4}
DEBUG_OPTION_NAMES = ("transport_observer", "fabric_observer", "graph_observer", "ffn_routing_observer")


@dataclass(frozen=True)
class NativeRuntimeState:
    initialized: bool
    role: str | None
    device: int | None
    options: dict


def runtime_initialize(role: str, device: int | None, options: dict | None = None) -> None:
    """Records the process's role, device and debug options in the native library (one per process: the same role and
    device again only replaces the options, anything else is refused). Reference: ``native.initialize(role, device,
    debug_options)``, src/cext/runtime.cpp."""
    if role not in ROLE_IDS:
        raise ValueError(f"unknown role {role!r}")
    opts = (C.c_uint32 * 4)(*[int(bool((options or {}).get(n, False))) for n in DEBUG_OPTION_NAMES])
    rc = lib().xr_runtime_initialize(ROLE_IDS[role], -1 if device is None else int(device), opts)
    if rc == -1:
        st = runtime_state()
        raise RuntimeError(f"process already initialised as {st.role} on device {st.device}")
    if rc != 0:
        raise ValueError(f"xr_runtime_initialize failed ({rc})")


def runtime_state() -> NativeRuntimeState:
    out = (C.c_uint32 * 7)()
    lib().xr_runtime_state(out)
    names = {v: k for k, v in ROLE_IDS.items()}
    dev = C.c_int32(out[2]).value
    return NativeRuntimeState(bool(out[0]), names.get(out[1]), None if dev < 0 else dev,
                              {n: bool(out[3 + i]) for i, n in enumerate(DEBUG_OPTION_NAMES)})


def runtime_reset_for_tests() -> None:
    lib().xr_runtime_reset_for_tests()


def dp_inspect_rows(layout: int, payload_rows: int, modes: list[int], rank_rows: list[int]) -> tuple[int, list[int]] | None:
    """Checks the row table of an Instance's data-parallel attention ranks for one merged invocation (the native
    ``dp_inspect_rows``, also compiled for the device). Returns ``(merged forward mode, first row of every rank)`` or
    ``None`` when the table is inconsistent. Reference: src/cext/fabric/coordinator.cu:55-117."""
    n = len(modes)
    if n == 0 or n != len(rank_rows):
        return None
    m, r, off = (C.c_uint32 * n)(*modes), (C.c_uint32 * n)(*rank_rows), (C.c_uint32 * n)()
    merged = lib().xr_dp_inspect_rows(layout, n, payload_rows, m, r, off)
    return (int(merged), list(off)) if merged else None


def validate_invocation(rows: int, layer: int, mode: int, sequence: int, *, completed: int, capacity_rows: int, num_layers: int,
                        requirement: int = 1, dp_layout: int = 0) -> int:
    """ResultCode (0 ok, 2 protocol mismatch) of an invocation record against what its consumer expects."""
    return int(lib().xr_validate_invocation(rows, layer, mode, requirement, dp_layout, sequence, completed, capacity_rows, num_layers))


def validate_completion(result_code: int, rows: int, sequence: int, *, want_sequence: int, want_rows: int) -> int:
    return int(lib().xr_validate_completion(result_code, rows, sequence, want_sequence, want_rows))


class LaneScheduler:
    """Host instance of the Lane scheduler (same code the device coordinator runs)."""

    def __init__(self, instances: int, lanes: int, policy: int = POLICY_FIFO, seed: int = 0):
        self._h = lib().xr_sched_create(instances, lanes, policy, seed)
        if not self._h:
            raise MemoryError

    def close(self) -> None:
        if self._h:
            lib().xr_sched_destroy(self._h)
            self._h = None

    __del__ = close

    def enqueue(self, instance: int, sequence: int, deadline: int = 0) -> bool:
        return bool(lib().xr_sched_enqueue(self._h, instance, sequence, deadline))

    def try_schedule(self) -> tuple[int, int, int] | None:
        i, l, s = u32(), u32(), u64()
        if lib().xr_sched_try(self._h, C.byref(i), C.byref(l), C.byref(s)):
            return i.value, l.value, s.value
        return None

    def active(self, instance: int) -> tuple[int, int] | None:
        l, s = u32(), u64()
        if lib().xr_sched_active(self._h, instance, C.byref(l), C.byref(s)):
            return l.value, s.value
        return None

    def release(self, instance: int, lease: int) -> bool:
        return bool(lib().xr_sched_release(self._h, instance, lease))


class SharedMemory:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def create(cls, name: str, nbytes: int) -> "SharedMemory":
        ensure_uint64(nbytes)
        err = C.c_int()
        h = lib().xr_shm_create(name.encode(), nbytes, C.byref(err))
        if not h:
            raise OSError(-err.value, f"shm create {name}")
        return cls(h)

    @classmethod
    def attach(cls, name: str) -> "SharedMemory":
        err = C.c_int()
        h = lib().xr_shm_attach(name.encode(), C.byref(err))
        if not h:
            raise OSError(-err.value, f"shm attach {name}")
        return cls(h)

    @property
    def size(self) -> int:
        return lib().xr_shm_size(self._h)

    @property
    def address(self) -> int:
        return lib().xr_shm_data(self._h)

    def buffer(self):
        return (C.c_uint8 * self.size).from_address(self.address)

    def close(self) -> None:
        if self._h:
            lib().xr_shm_close(self._h)
            self._h = None

    __del__ = close


class EcsChannel:
    """Seqlock control channel shared by daemon, AtnAgents and Instance ranks."""

    def __init__(self, handle, name: str):
        self._h, self.name = handle, name

    @classmethod
    def create(cls, name: str, devices: int, partitions: int, generation: int = 0) -> "EcsChannel":
        err = C.c_int()
        h = lib().xr_ecs_create(name.encode(), devices, partitions, generation, C.byref(err))
        if not h:
            raise OSError(-err.value, f"ecs channel create {name}")
        return cls(h, name)

    @classmethod
    def attach(cls, name: str) -> "EcsChannel":
        err = C.c_int()
        h = lib().xr_ecs_attach(name.encode(), C.byref(err))
        if not h:
            raise OSError(-err.value, f"ecs channel attach {name}")
        return cls(h, name)

    def close(self) -> None:
        if self._h:
            lib().xr_ecs_close(self._h)
            self._h = None

    __del__ = close

    def counts(self) -> tuple[int, int, int]:
        d, p = u32(), u32()
        gen = lib().xr_ecs_counts(self._h, C.byref(d), C.byref(p))
        return d.value, p.value, gen

    def set_device(self, idx: int, device: int) -> None:
        _ok(lib().xr_ecs_set_device(self._h, idx, device))

    def set_partition(self, idx: int, device: int, group: int, rank: int, floor_bytes: int,
                      reservation_bytes: int) -> None:
        ensure_uint32(idx, device, group, rank)
        ensure_uint64(floor_bytes, reservation_bytes)
        _ok(lib().xr_ecs_set_partition(self._h, idx, device, group, rank, floor_bytes, reservation_bytes))

    def partition(self, idx: int) -> dict:
        out = (u64 * 5)()
        _ok(lib().xr_ecs_get_partition(self._h, idx, out))
        return dict(device=out[0], group=out[1], rank=out[2], floor_bytes=out[3], reservation_bytes=out[4])

    def publish_report(self, idx: int, free_bytes: int, total_bytes: int, sequence: int) -> None:
        ensure_uint64(free_bytes, total_bytes, sequence)      # a negative byte count must not wrap into a huge quota
        _ok(lib().xr_ecs_publish_report(self._h, idx, free_bytes, total_bytes, sequence))

    def read_report(self, idx: int) -> tuple[int, int, int]:
        out = (u64 * 3)()
        _ok(lib().xr_ecs_read_report(self._h, idx, out))
        return tuple(out)

    def publish_command(self, idx: int, sequence: int, target_bytes: int) -> None:
        ensure_uint64(sequence, target_bytes)
        _ok(lib().xr_ecs_publish_command(self._h, idx, sequence, target_bytes))

    def read_command(self, idx: int) -> tuple[int, int]:
        out = (u64 * 2)()
        _ok(lib().xr_ecs_read_command(self._h, idx, out))
        return tuple(out)

    def publish_demand(self, idx: int, evaluated_sequence: int, required_bytes: int, deadline_ns: int,
                       mapped_bytes: int) -> None:
        ensure_uint64(evaluated_sequence, required_bytes, deadline_ns, mapped_bytes)
        _ok(lib().xr_ecs_publish_demand(self._h, idx, evaluated_sequence, required_bytes, deadline_ns, mapped_bytes))

    def read_demand(self, idx: int) -> tuple[int, int, int, int]:
        out = (u64 * 4)()
        _ok(lib().xr_ecs_read_demand(self._h, idx, out))
        return tuple(out)

    def publish_completion(self, idx: int, sequence: int, mapped_bytes: int) -> None:
        ensure_uint64(sequence, mapped_bytes)
        _ok(lib().xr_ecs_publish_completion(self._h, idx, sequence, mapped_bytes))

    def read_completion(self, idx: int) -> tuple[int, int]:
        out = (u64 * 2)()
        _ok(lib().xr_ecs_read_completion(self._h, idx, out))
        return tuple(out)


class CpuMailbox:
    """Transport arena in POSIX shm with the mailbox protocol run by CPU threads."""

    def __init__(self, handle, max_rows: int, row_bytes: int):
        self._h, self.max_rows, self.row_bytes = handle, max_rows, row_bytes

    @classmethod
    def create(cls, name: str, max_rows: int, row_bytes: int) -> "CpuMailbox":
        ensure_uint32(max_rows, row_bytes)
        err = C.c_int()
        h = lib().xr_mbox_create(name.encode(), max_rows, row_bytes, C.byref(err))
        if not h:
            raise OSError(-err.value, f"mailbox create {name}")
        return cls(h, max_rows, row_bytes)

    @classmethod
    def attach(cls, name: str, max_rows: int, row_bytes: int) -> "CpuMailbox":
        err = C.c_int()
        h = lib().xr_mbox_attach(name.encode(), max_rows, row_bytes, C.byref(err))
        if not h:
            raise OSError(-err.value, f"mailbox attach {name}")
        return cls(h, max_rows, row_bytes)

    def close(self) -> None:
        if self._h:
            lib().xr_mbox_close(self._h)
            self._h = None

    __del__ = close

    @property
    def status(self) -> int:
        return lib().xr_mbox_status(self._h)

    @property
    def failure(self) -> int:
        return lib().xr_mbox_failure(self._h)

    def activate(self) -> None:
        _ok(lib().xr_mbox_activate(self._h))

    def shutdown(self) -> None:
        lib().xr_mbox_shutdown(self._h)

    def wait_status(self, want: int, timeout_s: float) -> int:
        return lib().xr_mbox_wait_status(self._h, want, int(timeout_s * 1e9))

    def submit(self, in_ptr: int, out_ptr: int, rows: int, layer: int, mode: int, requirement: int = 1,
               dp_layout: int = 0, timeout_s: float = 5.0) -> int:
        ensure_uint64(in_ptr, out_ptr)
        ensure_uint32(rows, layer, mode, requirement, dp_layout)
        return lib().xr_mbox_submit(self._h, in_ptr, out_ptr, rows, layer, mode, requirement, dp_layout,
                                    int(timeout_s * 1e9))

    def take(self, timeout_s: float) -> tuple[int, tuple[int, int, int, int] | None]:
        out = (u32 * 4)()
        rc = lib().xr_mbox_take(self._h, int(timeout_s * 1e9), out)
        return rc, (tuple(out) if rc == 0 else None)

    @property
    def input_address(self) -> int:
        return lib().xr_mbox_input(self._h)

    @property
    def output_address(self) -> int:
        return lib().xr_mbox_output(self._h)

    def complete(self, result_code: int = 0) -> None:
        _ok(lib().xr_mbox_complete(self._h, result_code))


class TraceBuffer:
    def __init__(self, capacity: int):
        self._h = lib().xr_trace_create(capacity)

    def close(self) -> None:
        if self._h:
            lib().xr_trace_destroy(self._h)
            self._h = None

    __del__ = close

    def record(self, kind: int, a: int, b: int, timestamp_ns: int) -> bool:
        return bool(lib().xr_trace_record(self._h, kind, a, b, timestamp_ns))

    def counts(self) -> tuple[int, int]:
        d = u64()
        n = lib().xr_trace_counts(self._h, C.byref(d))
        return n, d.value

    def events(self) -> list[tuple[int, int, int, int]]:
        n, _ = self.counts()
        out = (u64 * (3 * max(n, 1)))()
        k = lib().xr_trace_read(self._h, 0, n, out)
        return [(out[3 * i] >> 32, out[3 * i] & 0xFFFFFFFF, out[3 * i + 1], out[3 * i + 2]) for i in range(k)]


def _ok(rc: int) -> None:
    if rc != 0:
        raise NativeLibraryError(f"runtime call failed with code {rc}")
