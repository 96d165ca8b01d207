"""RMSNorm family on the fused norm/publish kernel (``csrc/kernels/norm.cu``).

``add_rmsnorm`` is the attention-side workhorse: it folds one or more bf16 partial tensors in a
fixed order with fp32 accumulation (the TP reduction of FFN outputs, deterministic like the
reference's owner reduction, src/cext/ffnagent/delivery.cu:85-127), adds the residual stream in
place, normalises, and can push the normalised rows to several destinations followed by a
system-scope release of a sequence word (the transport producer).
"""

from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch

from .. import native
from .gemm import status_words

_counters: dict[int, torch.Tensor] = {}


def _done_counter(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _counters.get(idx)
    if t is None:
        t = torch.zeros(64, dtype=torch.int32, device=device)
        _counters[idx] = t
    return t


def add_rmsnorm(parts: Sequence[torch.Tensor] | torch.Tensor, weight: torch.Tensor | None, eps: float = 1e-6, *,
                resid: torch.Tensor | None = None, out: torch.Tensor | None = None,
                peer_ptrs: Sequence[int] = (), peer_flag_ptrs: Sequence[int] = (), peer_meta_ptrs: Sequence[int] = (),
                publish_seq: int = 0, wait_flag_ptrs: Sequence[int] = (), wait_seq: int = 0,
                wait_ns: int = 5_000_000_000, meta: tuple[int, int, int] = (0, 0, 0),
                want_local: bool = True, seq_counter_ptr: int = 0,
                part_ptrs: Sequence[int] | None = None, part_shape: tuple[int, int, int] | None = None,
                deadline_ptr: int = 0, cancel_ptr: int = 0, trace: tuple[int, int, int] | None = None) -> torch.Tensor | None:
    """``y = rmsnorm(sum(parts) + resid) * weight``; ``resid`` is updated in place.

    ``parts`` are bf16 ``[rows, hidden]`` tensors summed in list order. Parts that live in another
    GPU's memory are given as raw mapped pointers instead: ``part_ptrs`` with
    ``part_shape = (rows, hidden, leading dimension)``; the device then comes from ``resid``/``out``.
    With ``weight=None`` only the residual add happens. ``cancel_ptr``: a device word that ends the waits when it
    turns non-zero (the claim word of the Instance's failure slot). ``trace``: (events, state, capacity) of a device
    event buffer the kernel's hook points record into.
    """
    if isinstance(parts, torch.Tensor):
        parts = [parts]
    a = native.NormArgs()
    if part_ptrs is not None:
        rows, hidden, ld_parts = part_shape
        dev = (resid if resid is not None else out).device
        for i, ptr in enumerate(part_ptrs):
            a.parts[i] = ptr
        parts = list(part_ptrs)
    else:
        first = parts[0]
        rows, hidden = first.shape
        dev, ld_parts = first.device, first.stride(0)
        for i, p in enumerate(parts):
            assert p.dtype == torch.bfloat16 and p.stride(1) == 1 and p.stride(0) == first.stride(0)
            a.parts[i] = p.data_ptr()
    if want_local and out is None and weight is not None:
        out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
    for i, f in enumerate(wait_flag_ptrs):
        a.wait_flags[i] = f
    for i, p in enumerate(peer_ptrs):
        a.out_peers[i] = p
        a.peer_flags[i] = peer_flag_ptrs[i]
        a.peer_meta[i] = peer_meta_ptrs[i] if peer_meta_ptrs else None
    a.resid = resid.data_ptr() if resid is not None else None
    a.weight = weight.data_ptr() if weight is not None else None
    a.out_local = out.data_ptr() if (out is not None and want_local) else None
    a.done_counter = _done_counter(dev).data_ptr()
    a.status = status_words(dev).data_ptr()
    a.cancel = cancel_ptr or None
    if trace is not None:
        a.trace_events, a.trace_state, a.trace_capacity = trace
    a.wait_ns = wait_ns
    a.rows, a.hidden = rows, hidden
    a.ld_parts = ld_parts
    a.ld_out = out.stride(0) if out is not None else hidden
    a.nparts, a.npeers = len(parts), len(peer_ptrs)
    a.wait_seq, a.publish_seq = wait_seq, publish_seq
    a.meta_layer, a.meta_mode, a.meta_deadline_us = meta
    a.eps = eps
    a.seq_counter = seq_counter_ptr or None
    a.meta_deadline_ptr = deadline_ptr or None
    native.check(native.kernels().xp_norm_publish(C.byref(a), torch.cuda.current_stream(dev).cuda_stream),
                 "xp_norm_publish")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    shp = x.shape
    return add_rmsnorm(x.reshape(-1, shp[-1]), weight, eps).reshape(shp)


def swiglu(gate_up: torch.Tensor, *, limit: float = 0.0, up_add: float = 0.0, alpha: float = 0.0) -> torch.Tensor:
    """Unfused ``silu(gate) * up`` over ``[rows, 2*I]`` (baseline path only)."""
    rows, two_i = gate_up.shape
    out = torch.empty(rows, two_i // 2, dtype=torch.bfloat16, device=gate_up.device)
    native.check(native.kernels().xp_swiglu(gate_up.data_ptr(), out.data_ptr(), rows, two_i // 2, limit, up_add,
                                            alpha, torch.cuda.current_stream(gate_up.device).cuda_stream), "xp_swiglu")
    return out
