"""Binds ``torch.ops.xpool.ffn_shim`` of this process to one Instance rank's slots.

The operator's CUDA implementation (``csrc/bindings/torch_ops.cpp`` -> ``csrc/kernels/instance.cu``) needs to know
where the Instance's slots live: the input buffer, invocation record and failure slot on every FFN rank of its TP
group (peer memory), and its own partial-output buffers, completion words and failure slot. This module assembles
that binding either from a Fabric port built in the same process, or -- the plugin path -- from the IPC handles the
daemon brokers: the attention-side arena through ``POST /instance/.../transport-arena/acquire`` and the FFN ranks'
slots through the plan's ``slot_handles`` (reference: attach_arena_from_daemon, src/xpool/runtime/instance.py;
``InstanceRankRuntime::attach``, src/cext/transport/instance.cpp).
"""

from __future__ import annotations

import ctypes as C

import torch

from ... import native
from ...parallel import fabric as F


class InstanceBinding(C.Structure):
    _fields_ = [("peer_inputs", C.c_void_p * 8), ("peer_records", C.c_void_p * 8), ("peer_flags", C.c_void_p * 8),
                ("peer_failures", C.c_void_p * 8), ("parts", C.c_void_p * 8), ("done_flags", C.c_void_p * 8),
                ("failure", C.c_void_p), ("status", C.c_void_p), ("wait_ns", C.c_uint64), ("n_peers", C.c_int),
                ("n_parts", C.c_int), ("hidden", C.c_int), ("capacity_rows", C.c_int), ("origin_pe", C.c_uint32),
                ("reserved", C.c_uint32)]


def _lib():
    lib = native.kernels()
    if not getattr(lib, "_xp_instance_declared", False):
        lib.xp_instance_create.restype = C.c_int
        lib.xp_instance_create.argtypes = [C.POINTER(InstanceBinding)]
        lib.xp_instance_set_current.restype = C.c_int
        lib.xp_instance_set_current.argtypes = [C.c_int]
        lib.xp_instance_current.restype = C.c_int
        lib.xp_instance_submit.restype = C.c_int
        lib.xp_instance_submit.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_int, C.c_void_p]
        lib.xp_instance_destroy.restype = None
        lib.xp_instance_destroy.argtypes = [C.c_int]
        lib._xp_instance_declared = True
    return lib


class FabricInstanceTransport:
    """One Instance rank's native transport binding; ``make_current`` points ``xpool::ffn_shim`` at it."""

    def __init__(self, place: F.InstancePlacement, atn_base: int, ffn_bases: list[int], device, wait_ns: int = 5_000_000_000,
                 keep=()):
        from ...ops.gemm import status_words

        self.place, self.device, self._keep = place, torch.device(device), list(keep)
        alay, flay = F.atn_slot_layout(place), F.ffn_slot_layout(place)
        b = InstanceBinding()
        for i, base in enumerate(ffn_bases):
            b.peer_inputs[i] = base + flay.input_offset
            b.peer_records[i] = base + flay.record_offset
            b.peer_flags[i] = base + flay.record_offset + F.RECORD_SEQ_OFFSET
            b.peer_failures[i] = base + flay.record_offset + F.FAILURE_SLOT_OFFSET
        for r in range(place.tp):
            b.parts[r] = atn_base + alay.output_offset + r * alay.output_stride
            b.done_flags[r] = atn_base + alay.completion_offset + r * F.RECORD_BYTES + F.COMPLETION_SEQ_OFFSET
        b.failure = atn_base + alay.completion_offset + F.FAILURE_SLOT_OFFSET
        self.status = status_words(self.device)
        b.status, b.wait_ns = self.status.data_ptr(), wait_ns
        b.n_peers, b.n_parts, b.hidden, b.capacity_rows = len(ffn_bases), place.tp, place.cfg.hidden_size, place.capacity_rows
        b.origin_pe = place.atn_rank
        self._failure_words = F.tensor_from_ptr(atn_base + alay.completion_offset + F.FAILURE_SLOT_OFFSET, (8,), torch.int32, self.device)
        self.handle = _lib().xp_instance_create(C.byref(b))
        if self.handle < 0:
            raise RuntimeError(f"xp_instance_create failed with {self.handle}")

    @classmethod
    def from_port(cls, port: F.FabricFfnPort, **kw) -> "FabricInstanceTransport":
        """Shares the slots of a Fabric port built in this process (its own sequence counter is not used: do not mix
        submissions of the port and of the operator on one Instance)."""
        return cls(port.place, port.local.ptr, port.ffn_bases, port.device, **kw)

    @classmethod
    def from_handles(cls, place: F.InstancePlacement, atn_handle_hex: str, ffn_handles_hex: list[str], device, **kw):
        """The plugin path: map the brokered attention-side arena and the FFN ranks' slots by their IPC handles."""
        atn_base = F.PeerBuffer.open(bytes.fromhex(atn_handle_hex))
        ffn_bases = [F.PeerBuffer.open(bytes.fromhex(h)) for h in ffn_handles_hex]
        return cls(place, atn_base, ffn_bases, device, **kw)

    def make_current(self) -> None:
        native.check(_lib().xp_instance_set_current(self.handle), "xp_instance_set_current", 0)

    def submit(self, hidden: torch.Tensor, out: torch.Tensor, layer: int, mode: int, requirement: int = 1, dp_layout: int = 0) -> None:
        """The operator's body without the dispatcher (same checks as the C++ side)."""
        rc = _lib().xp_instance_submit(self.handle, hidden.data_ptr(), hidden.shape[0], hidden.stride(0), out.data_ptr(), out.stride(0),
                                       layer, mode, requirement, dp_layout, torch.cuda.current_stream(self.device).cuda_stream)
        native.check(rc, "xp_instance_submit", 0)

    def failure(self):
        return F.FabricFailure.from_words(self._failure_words.cpu().tolist())

    def close(self) -> None:
        if self.handle >= 0:
            _lib().xp_instance_destroy(self.handle)
            self.handle = -1
