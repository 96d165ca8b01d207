"""The Fabric: attention ranks and FFN ranks connected by peer memory over NVLink.

One process per GPU. Every rank allocates its arena with ``cudaMalloc`` and publishes a CUDA IPC
handle; peers map it once and from then on all traffic is issued by kernels:

* the attention side's norm kernel stores the post-attention hidden states straight into each FFN
  rank's input buffer, writes the invocation record and releases the slot's sequence word
  (``ops.norm.add_rmsnorm(peer_ptrs=...)``);
* an FFN rank's Lane picks the invocation up, runs the two tcgen05 GEMMs, and the down-projection
  epilogue stores the rank's partial into the attention rank's partial buffer, followed by the
  completion record (``csrc/kernels/lane.cu``);
* the attention side waits for the completion words of all TP ranks and the next add-RMSNorm folds
  the partials in rank order with fp32 accumulation.

Handles travel through ``torch.distributed`` object collectives here (bench, tests); a deployed
system brokers the same hex handles through the daemon (``service.daemon``), as the reference does
for Transport arenas (src/xpool/service/daemon/transport.py).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch

from .. import native
from ..engine.atn_engine import AttentionEngine, EngineConfig, FfnPort
from ..models.config import ModelConfig
from ..models.weights import FfnLayerWeights, random_attention_weights, random_ffn_layer
from ..native import runtime as rt

RECORD_SEQ_OFFSET = 32      # InvocationRecord.sequence
COMPLETION_SEQ_OFFSET = 16  # CompletionRecord.sequence
RECORD_BYTES = 256
FAILURE_SLOT_OFFSET = 64    # failure slot inside the first 256-byte record block of a slot (protocol.hpp)
RESULT_NAMES = {0: "ok", 1: "shutdown", 2: "protocol_mismatch", 3: "timeout"}


@dataclass
class FabricFailure:
    """The canonical failure of a generation as one slot recorded it (first failure wins)."""

    result_code: int
    origin_pe: int
    instance_index: int
    invocation_sequence: int
    layer_ordinal: int

    @classmethod
    def from_words(cls, w) -> "FabricFailure | None":
        return cls(int(w[1]), int(w[2]), int(w[3]), int(w[4]), int(w[5])) if int(w[0]) == 1 else None


class DeviceTrace:
    """A device event buffer for the attention-side hook points (publish, wait begin / end)."""

    def __init__(self, capacity: int = 1 << 16):
        ev, st = C.c_void_p(), C.c_void_p()
        native.check(native.kernels().xp_trace_create(capacity, C.byref(ev), C.byref(st)), "xp_trace_create", 0)
        self.events, self.state, self.capacity = ev.value, st.value, capacity

    def args(self) -> tuple[int, int, int]:
        return self.events, self.state, self.capacity

    def read(self, stream: int = 0) -> tuple[list[tuple[int, int, int, int]], int]:
        out, dropped = (C.c_uint64 * (3 * self.capacity))(), C.c_uint64()
        n = native.kernels().xp_trace_read(self.events, self.state, self.capacity, out, self.capacity, C.byref(dropped), stream)
        if n < 0:
            raise RuntimeError(f"xp_trace_read failed with {n}")
        return [(out[3 * i] >> 32, out[3 * i] & 0xFFFFFFFF, out[3 * i + 1], out[3 * i + 2]) for i in range(n)], dropped.value

    def close(self) -> None:
        if self.events:
            native.kernels().xp_trace_destroy(self.events, self.state)
            self.events = self.state = 0


class PeerBuffer:
    """A raw device allocation that other processes can map."""

    def __init__(self, nbytes: int):
        p = C.c_void_p()
        native.check(native.kernels().xp_dev_alloc(C.byref(p), nbytes), "xp_dev_alloc", 0)
        self.ptr, self.nbytes, self.owned = p.value, nbytes, True

    def handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        native.check(native.kernels().xp_ipc_get_handle(self.ptr, buf), "xp_ipc_get_handle", 0)
        return bytes(buf.raw)

    @staticmethod
    def open(handle: bytes) -> int:
        p = C.c_void_p()
        native.check(native.kernels().xp_ipc_open(handle, C.byref(p)), "xp_ipc_open", 0)
        return p.value

    def tensor(self, offset: int, shape: tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
        return tensor_from_ptr(self.ptr + offset, shape, dtype, device)

    def free(self) -> None:
        if self.owned and self.ptr:
            native.kernels().xp_dev_free(self.ptr)
            self.ptr = 0


class _CudaArray:
    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}


def tensor_from_ptr(ptr: int, shape: tuple[int, ...], dtype: torch.dtype, device) -> torch.Tensor:
    """A tensor view over raw device memory (bf16 goes through a 16-bit integer view)."""
    if dtype == torch.bfloat16:
        return torch.as_tensor(_CudaArray(ptr, shape, "<i2"), device=device).view(torch.bfloat16)
    typestr = {torch.int32: "<i4", torch.float32: "<f4", torch.uint8: "|u1", torch.int64: "<i8"}[dtype]
    return torch.as_tensor(_CudaArray(ptr, shape, typestr), device=device)


# ------------------------------------------------------------------ topology

@dataclass(frozen=True)
class InstancePlacement:
    """Where one Instance runs: one attention rank, and the FFN ranks of its TP group (rank order =
    TP rank order = reduction order)."""

    model_id: str
    cfg: ModelConfig
    seed: int
    atn_rank: int
    ffn_ranks: tuple[int, ...]
    capacity_rows: int
    moe_parallel: str = "ep"  # how MoE layers use the FFN ranks: "ep" (experts split) or "tp" (every expert split)
    atn_tp_followers: tuple[int, ...] = ()  # further ranks of the Instance's attention TP group (atn_rank is rank 0)
    # Layer-split placement: ((first layer, end layer, FFN ranks in TP order), ...) covering all layers, every
    # group of the same TP size; ``ffn_ranks`` is then the union of the groups. Empty: one group of all layers.
    layer_groups: tuple[tuple[int, int, tuple[int, ...]], ...] = ()
    # Directory of a Hugging Face checkpoint (config.json + safetensors) to load the weights from; None: random
    # init from ``seed`` (benchmarks and tests).
    checkpoint: str | None = None
    # Instances that carry the same key (and seed / checkpoint) are ranks or replicas of one model: an FFN rank keeps
    # one copy of the FFN shard for all of them. None: private weights.
    weights_key: str | None = None

    def __post_init__(self):
        if self.layer_groups:
            sizes = {len(g[2]) for g in self.layer_groups}
            covered = sorted((g[0], g[1]) for g in self.layer_groups)
            ok = len(sizes) == 1 and covered[0][0] == 0 and covered[-1][1] == self.cfg.num_layers and \
                all(a[1] == b[0] for a, b in zip(covered, covered[1:]))
            union = tuple(dict.fromkeys(r for g in self.layer_groups for r in g[2]))
            if not ok or union != tuple(self.ffn_ranks) or len(union) != sum(len(g[2]) for g in self.layer_groups):
                raise ValueError("layer groups must tile the layers, share one TP size, use every FFN rank once, "
                                 "and ffn_ranks must list their ranks in group order")

    @property
    def atn_tp_ranks(self) -> tuple[int, ...]:
        return (self.atn_rank,) + tuple(self.atn_tp_followers)

    def groups(self) -> tuple[tuple[int, int, tuple[int, ...]], ...]:
        return self.layer_groups or ((0, self.cfg.num_layers, tuple(self.ffn_ranks)),)

    @property
    def tp(self) -> int:
        return len(self.groups()[0][2])

    def locate(self, ffn_rank: int) -> tuple[int, int, int]:
        """(TP rank, first layer, end layer) of an FFN rank of this Instance."""
        for lo, hi, ranks in self.groups():
            if ffn_rank in ranks:
                return ranks.index(ffn_rank), lo, hi
        raise LookupError(f"rank {ffn_rank} holds no shard of {self.model_id}")

    @property
    def expert_parallel(self) -> bool:
        return self.cfg.is_moe and self.moe_parallel == "ep" and self.tp > 1

    def expert_range(self, group_rank: int) -> tuple[int, int]:
        """Experts owned by the ``group_rank``-th FFN rank (all of them unless expert parallel)."""
        e = self.cfg.num_experts
        if not self.expert_parallel:
            return 0, e
        if e % self.tp:
            raise ValueError(f"{e} experts do not split evenly over {self.tp} ranks")
        per = e // self.tp
        return group_rank * per, (group_rank + 1) * per

    def dense_inter_local(self) -> int:
        """Widest dense projection of this instance on one FFN rank: dense layers and the shared experts of
        MoE layers (0 if there is neither)."""
        cfg = self.cfg
        has_dense = not cfg.is_moe or cfg.first_k_dense > 0
        dense = cfg.intermediate_size // self.tp if has_dense else 0
        shared = cfg.num_shared_experts * cfg.moe_intermediate_size if cfg.is_moe else 0
        if shared and not self.expert_parallel:
            shared //= self.tp
        return max(dense, shared)


@dataclass
class Topology:
    world_size: int
    instances: list[InstancePlacement]

    def atn_ranks(self) -> list[int]:
        return sorted({r for i in self.instances for r in i.atn_tp_ranks})

    def ffn_ranks(self) -> list[int]:
        return sorted({r for i in self.instances for r in i.ffn_ranks})

    def role(self, rank: int) -> str:
        a, f = rank in self.atn_ranks(), rank in self.ffn_ranks()
        if a and f:
            raise ValueError(f"rank {rank} has both roles; kernels that wait on one another must not share a GPU")
        return "atn" if a else "ffn" if f else "idle"


def ffn_slot_layout(p: InstancePlacement) -> rt.FfnSlotLayout:
    # the slot's activation scratch serves dense layers; MoE layers use the Lane's own scratch
    return rt.plan_ffn_slot(p.capacity_rows, p.cfg.hidden_size, max(p.dense_inter_local(), 128))


def atn_slot_layout(p: InstancePlacement) -> rt.AtnSlotLayout:
    return rt.plan_atn_slot(p.capacity_rows, p.cfg.hidden_size, p.tp)


# ------------------------------------------------------------------ attention side

class FabricFfnPort(FfnPort):
    """FFN port of an Instance whose FFN lives on other GPUs."""

    def __init__(self, place: InstancePlacement, local: PeerBuffer, ffn_bases: list[int], device):
        self.place, self.local, self.device = place, local, torch.device(device)
        self.alay, self.flay = atn_slot_layout(place), ffn_slot_layout(place)
        self.ffn_bases = ffn_bases  # mapped base pointer of this instance's slot on every rank of place.ffn_ranks
        base_of = dict(zip(place.ffn_ranks, ffn_bases))
        self._group_bases = [(lo, hi, [base_of[r] for r in ranks]) for lo, hi, ranks in place.groups()]
        tp = place.tp
        self.parts = [local.tensor(self.alay.output_offset + r * self.alay.output_stride,
                                   (place.capacity_rows, place.cfg.hidden_size), torch.bfloat16, self.device)
                      for r in range(tp)]
        self.done_flags = [local.ptr + self.alay.completion_offset + r * RECORD_BYTES + COMPLETION_SEQ_OFFSET
                           for r in range(tp)]
        self.seq = torch.zeros(4, dtype=torch.int32, device=self.device)
        # SLO deadline of the step in flight (microseconds of the monotonic host clock mod 2^32, 0 = none);
        # the norm kernel copies it into every invocation record, the FFN Lanes' SLO policy orders by it
        self.slo_tbt_ms = 0.0
        self.deadline = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._deadline_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.wait_ns = 5_000_000_000  # the reference's device wait limit (utils/wait.cuh:17-19)
        self._wait = native.WaitArgs()
        for r, f in enumerate(self.done_flags):
            self._wait.flags[r] = f
        self._wait.n = tp
        self._wait.want_ptr = self.seq.data_ptr()
        self._wait.wait_ns = self.wait_ns
        # canonical failure: this Instance's slot lives behind the first completion record; its claim word cancels
        # every wait of the Instance, and a wait of ours that runs out claims it and tells the FFN ranks
        self.failure_ptr = local.ptr + self.alay.completion_offset + FAILURE_SLOT_OFFSET
        self._failure_words = local.tensor(self.alay.completion_offset + FAILURE_SLOT_OFFSET, (8,), torch.int32, self.device)
        self._wait.cancel = self.failure_ptr
        self._wait.failure = self.failure_ptr
        for i, b in enumerate(ffn_bases[:8]):
            self._wait.peer_failures[i] = b + self.flay.record_offset + FAILURE_SLOT_OFFSET
        self._wait.n_peer_failures = min(8, len(ffn_bases))
        self._wait.origin_pe, self._wait.instance = place.atn_rank, 0
        self.trace: DeviceTrace | None = None

    def attach(self, engine: AttentionEngine) -> None:
        from ..ops.gemm import status_words

        if engine.cap > self.place.capacity_rows:
            raise ValueError("engine row capacity exceeds the fabric slot capacity")
        self._wait.status = status_words(self.device).data_ptr()

    def set_wait_limit(self, wait_ns: int) -> None:
        self.wait_ns = self._wait.wait_ns = int(wait_ns)

    def wait_args(self) -> dict:
        return dict(cancel_ptr=self.failure_ptr)

    def enable_trace(self, capacity: int = 1 << 16) -> DeviceTrace:
        """Attaches a device event buffer to this port's publish and wait kernels (the transport observer of the
        attention side)."""
        self.trace = DeviceTrace(capacity)
        self._wait.trace_events, self._wait.trace_state, self._wait.trace_capacity = self.trace.args()
        return self.trace

    def failure(self) -> FabricFailure | None:
        """The failure recorded in this Instance's slot, if any (reads six words from the device)."""
        return FabricFailure.from_words(self._failure_words.cpu().tolist())

    def begin_step(self, now_s: float | None = None) -> None:
        """Stamps the step's deadline (call before launching the step; a 16-byte pinned copy)."""
        if self.slo_tbt_ms <= 0:
            return
        import time

        now = time.monotonic() if now_s is None else now_s
        us = int((now + self.slo_tbt_ms / 1e3) * 1e6) & 0xFFFFFFFF
        self._deadline_host[0] = (us or 1) - (1 << 32) if (us or 1) >= (1 << 31) else (us or 1)
        self.deadline.copy_(self._deadline_host, non_blocking=True)

    def publish_targets(self, layer: int, rows: int, mode: int) -> dict:
        bases = next(b for lo, hi, b in self._group_bases if lo <= layer < hi)   # the TP group that holds this layer
        return dict(deadline_ptr=self.deadline.data_ptr(), trace=self.trace.args() if self.trace is not None else None,
                    peer_ptrs=[b + self.flay.input_offset for b in bases],
                    peer_flag_ptrs=[b + self.flay.record_offset + RECORD_SEQ_OFFSET for b in bases],
                    peer_meta_ptrs=[b + self.flay.record_offset for b in bases],
                    seq_counter_ptr=self.seq.data_ptr(), meta=(layer, mode, 0))

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> list[torch.Tensor]:
        native.check(native.kernels().xp_wait_flags(C.byref(self._wait), torch.cuda.current_stream(self.device).cuda_stream),
                     "xp_wait_flags")
        return [p[:rows] for p in self.parts]


class FabricFfnFollowerPort(FfnPort):
    """FFN port of an attention TP rank other than the first. Rank 0 of the TP group publishes the
    hidden states (all ranks hold identical copies) and owns the completion records and partial
    buffers; a follower keeps its own invocation counter in step, waits on rank 0's completion words
    over NVLink and lets its add-RMSNorm read the partials from rank 0's memory."""

    def __init__(self, place: InstancePlacement, atn0_base: int, device):
        self.place, self.device = place, torch.device(device)
        self.alay = atn_slot_layout(place)
        tp = place.tp
        self.part_ptrs = [atn0_base + self.alay.output_offset + r * self.alay.output_stride for r in range(tp)]
        self.seq = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._bump = native.SignalArgs()
        self._bump.n, self._bump.seq_counter = 0, self.seq.data_ptr()
        self._wait = native.WaitArgs()
        for r in range(tp):
            self._wait.flags[r] = atn0_base + self.alay.completion_offset + r * RECORD_BYTES + COMPLETION_SEQ_OFFSET
        self._wait.n, self._wait.want_ptr, self._wait.wait_ns = tp, self.seq.data_ptr(), 5_000_000_000

    def attach(self, engine: AttentionEngine) -> None:
        from ..ops.gemm import status_words

        if engine.cap > self.place.capacity_rows:
            raise ValueError("engine row capacity exceeds the fabric slot capacity")
        self._wait.status = status_words(self.device).data_ptr()

    def publish_targets(self, layer: int, rows: int, mode: int) -> dict | None:
        return None

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> dict:
        s = torch.cuda.current_stream(self.device).cuda_stream
        k = native.kernels()
        native.check(k.xp_signal_flags(C.byref(self._bump), s), "xp_signal_flags")
        native.check(k.xp_wait_flags(C.byref(self._wait), s), "xp_wait_flags")
        h = self.place.cfg.hidden_size
        return dict(parts=[], part_ptrs=self.part_ptrs, part_shape=(rows, h, h))


# ------------------------------------------------------------------ FFN side

@dataclass
class FfnInstanceState:
    place: InstancePlacement
    tp_rank: int
    slot: PeerBuffer
    weights: list[FfnLayerWeights]
    atn_base: int = 0


class CheckpointFfnSource:
    """FFN weights of one model read from its safetensors checkpoint: the architecture adapter compiles the
    FFN description from ``config.json`` and the checkpoint's key list, coverage is validated once, and each
    layer's local shard (TP rows/columns, or an expert range) goes through the pinned staging loader. The
    reference prepares FFN shards the same way, src/xpool/runtime/ffnagent/preparation.py:164-334."""

    def __init__(self, model_id: str, model_dir: str):
        import json
        from pathlib import Path

        from ..engine import checkpoint as ck
        from ..models import adapters

        self.view = ck.read_checkpoint_key_view(model_dir)
        hf = json.loads((Path(model_dir) / "config.json").read_text())
        self.spec = adapters.compile_ffn_spec(model_id, hf, self.view.keys())
        ck.validate_ffn_coverage(self.spec, self.view)

    def layer(self, layer: int, device, *, tp_rank: int = 0, tp_size: int = 1,
              expert_range: tuple[int, int] | None = None) -> FfnLayerWeights:
        from ..engine import loader

        w = loader.materialize_layer_weights(self.spec, self.view, layer, tp_rank=tp_rank, tp_size=tp_size, device=device,
                                             dtype=torch.bfloat16,
                                             experts=range(*expert_range) if expert_range is not None else None)
        if expert_range is not None and expert_range[0] != 0:
            w.shared_gate_up = w.shared_down = None   # the rank owning expert 0 adds the shared experts
        return w


class FfnRankRuntime:
    """Everything an FFN rank owns: shards, slots, the native Lane runtime and the Lane threads."""

    def __init__(self, device, n_lanes: int = 1, policy: int = rt.POLICY_FIFO, seed: int = 0,
                 ws_bytes_per_lane: int = 64 << 20, tile_weights: bool = False, pe: int = 0):
        self.device = torch.device(device)
        self.pe = pe   # this device's PE number: the origin written into failures it claims
        self.n_lanes, self.policy, self.seed, self.ws_bytes = n_lanes, policy, seed, ws_bytes_per_lane
        self.tile_weights = tile_weights
        self.instances: list[FfnInstanceState] = []
        self.handle = None
        self._running = False
        self._shared_weights: dict = {}
        self.errors: list[str] = []

    def add_instance(self, place: InstancePlacement, tp_rank: int, layers: tuple[int, int] | None = None) -> FfnInstanceState:
        """``layers``: the half-open layer range this rank holds (layer-split placements); other layers get no
        weights and an invocation naming them is refused."""
        lay = ffn_slot_layout(place)
        slot = PeerBuffer(lay.total_bytes)
        cfg = place.cfg
        lo, hi = layers or (0, cfg.num_layers)
        # The attention data-parallel ranks of one model (and replicas that name the same weights) are separate
        # Instances with their own slots, but they execute the same FFN: one copy of the shard serves them all.
        share_key = (place.weights_key, cfg.name, place.checkpoint, place.seed, tp_rank, place.tp, lo, hi, place.moe_parallel)
        if place.weights_key is not None and share_key in self._shared_weights:
            st = FfnInstanceState(place, tp_rank, slot, self._shared_weights[share_key])
            self.instances.append(st)
            return st
        weights = []
        source = CheckpointFfnSource(place.model_id, place.checkpoint) if place.checkpoint else None
        for l in range(cfg.num_layers):
            if not lo <= l < hi:
                weights.append(None)
                continue
            if source is not None:
                ep = cfg.layer_is_moe(l) and place.expert_parallel
                w = source.layer(l, self.device, tp_rank=0 if ep else tp_rank, tp_size=1 if ep else place.tp,
                                 expert_range=place.expert_range(tp_rank) if ep else None)
            elif cfg.layer_is_moe(l) and place.expert_parallel:
                w = random_ffn_layer(cfg, l, place.seed, self.device, torch.bfloat16, expert_range=place.expert_range(tp_rank))
            else:
                w = random_ffn_layer(cfg, l, place.seed, self.device, torch.bfloat16, tp_rank, place.tp)
            weights.append(w)
        if place.weights_key is not None:
            self._shared_weights[share_key] = weights
        st = FfnInstanceState(place, tp_rank, slot, weights)
        self.instances.append(st)
        return st

    def install(self) -> None:
        """Builds the native Lane runtime once every instance knows its attention-side arena."""
        from ..ops import gemm

        lib = native.kernels()
        self.handle = lib.xp_lane_create(len(self.instances), self.n_lanes, self.policy, self.seed, self.ws_bytes)
        if not self.handle:
            raise RuntimeError("xp_lane_create failed")
        self._keep = []
        for i, st in enumerate(self.instances):
            p, flay, alay = st.place, ffn_slot_layout(st.place), atn_slot_layout(st.place)
            act_ld = max(p.dense_inter_local(), 128)
            d = native.LaneInstanceDesc()
            d.input = st.slot.ptr + flay.input_offset
            d.act = st.slot.ptr + flay.act_offset
            d.in_flag = st.slot.ptr + flay.record_offset + RECORD_SEQ_OFFSET
            d.record = st.slot.ptr + flay.record_offset
            d.out_peer = st.atn_base + alay.output_offset + st.tp_rank * alay.output_stride
            d.done_record_peer = st.atn_base + alay.completion_offset + st.tp_rank * RECORD_BYTES
            d.failure_peer = st.atn_base + alay.completion_offset + FAILURE_SLOT_OFFSET
            d.pe = self.pe
            d.capacity_rows, d.hidden, d.num_layers, d.act_ld = p.capacity_rows, p.cfg.hidden_size, p.cfg.num_layers, act_ld
            native.check(lib.xp_lane_set_instance(self.handle, i, C.byref(d)), "xp_lane_set_instance", 0)
            for l, w in enumerate(st.weights):
                if w is None:
                    continue   # held by another layer group: the table entry stays empty
                gu, dn = w.gate_up, w.down
                ld = native.LaneLayerDesc()
                if w.is_moe:
                    from ..ops.moe import padded_router, router_precision_code

                    if w.shared_gate_up is not None:
                        ld.shared_inter_local = w.shared_gate_up.shape[0] // 2
                        ld.w_shared_gateup, ld.w_shared_down = w.shared_gate_up.data_ptr(), w.shared_down.data_ptr()
                    cfg = p.cfg
                    router = padded_router(w)
                    lo, hi = p.expert_range(st.tp_rank)
                    ld.router = router.data_ptr()
                    ld.router_precision = router_precision_code(w)
                    if ld.router_precision:
                        raw = w.extra["router_fp32"] if ld.router_precision == 2 else w.router
                        assert raw.is_contiguous()
                        ld.router_raw = raw.data_ptr()
                    cb, rb = w.extra.get("correction_bias"), w.extra.get("router_bias")
                    ld.correction_bias = cb.data_ptr() if cb is not None else None
                    ld.router_bias = rb.data_ptr() if rb is not None else None
                    ld.num_experts, ld.top_k, ld.expert_lo, ld.expert_hi = cfg.num_experts, cfg.num_experts_per_tok, lo, hi
                    ld.sigmoid, ld.renormalize = int(cfg.router_scoring == "sigmoid"), int(cfg.norm_topk_prob)
                    ld.scale = cfg.routed_scaling_factor
                    inter = gu.shape[1] // 2
                    ld.w_tiled = 0
                else:
                    inter = gu.shape[0] // 2
                    if self.tile_weights:
                        gu, dn = gemm.tile_weight(gu), gemm.tile_weight(dn)
                        self._keep.append((gu, dn))
                    ld.w_tiled = int(self.tile_weights)
                ld.w_gateup, ld.w_down = gu.data_ptr(), dn.data_ptr()
                ld.bias_gateup = w.gate_up_bias.data_ptr() if w.gate_up_bias is not None else None
                ld.bias_down = w.down_bias.data_ptr() if w.down_bias is not None else None
                ld.gate_limit, ld.up_add, ld.act_alpha = w.extra.get("gate_transform", (0.0, 0.0, 0.0))
                ld.inter_local, ld.gated = inter, 1
                native.check(lib.xp_lane_set_layer(self.handle, i, l, C.byref(ld)), "xp_lane_set_layer", 0)
        native.check(lib.xp_lane_commit(self.handle), "xp_lane_commit", 0)

    def launch_once(self, lane: int = 0, lease_ms: float = 20.0, stream: torch.cuda.Stream | None = None) -> None:
        s = stream or torch.cuda.current_stream(self.device)
        native.check(native.kernels().xp_lane_launch(self.handle, lane, int(lease_ms * 1e6), s.cuda_stream),
                     "xp_lane_launch", 4)

    # -- serving threads ---------------------------------------------------------------------
    def start(self, lease_ms: float = 20.0, depth: int = 3) -> None:
        """Starts one replay thread per Lane inside the native library: each captures nothing itself (the graphs
        are captured here, on the calling thread, one Lane after the other) and keeps ``depth`` replays of its
        Lane's graph enqueued. No Python thread and no interpreter lock is on the path between two Lane iterations."""
        if self.device.index is not None:
            torch.cuda.set_device(self.device)
        native.check(native.kernels().xp_lane_threads_start(self.handle, int(lease_ms * 1e6), depth),
                     "xp_lane_threads_start", 0)
        self._running = True

    def _thread_state(self) -> tuple[int, int]:
        n = C.c_uint64()
        err = native.kernels().xp_lane_threads_state(self.handle, C.byref(n))
        return n.value, err

    def stop(self) -> None:
        if self.handle and getattr(self, "_running", False):
            side = torch.cuda.Stream(self.device)
            native.kernels().xp_lane_shutdown(self.handle, side.cuda_stream)   # leases in flight end at once
            side.synchronize()
            rc = native.kernels().xp_lane_threads_stop(self.handle)
            self._running = False
            if rc != 0:
                self.errors.append(f"lane replay thread failed with CUDA error {-100 - rc}")

    def stats(self) -> dict:
        served = (C.c_uint64 * len(self.instances))()
        idle = (C.c_uint32 * self.n_lanes)()
        status = C.c_uint32()
        side = torch.cuda.Stream(self.device)
        native.check(native.kernels().xp_lane_stats(self.handle, served, idle, C.byref(status), side.cuda_stream),
                     "xp_lane_stats", 0)
        replays, err = self._thread_state()
        if err and not self.errors:
            self.errors.append(f"lane replay thread failed with CUDA error {err}")
        return {"served": list(served), "idle_replays": list(idle), "status": status.value, "replays": replays}

    def failure(self) -> FabricFailure | None:
        """The first failure this device met (claimed here, or written into a slot by an attention rank)."""
        w = (C.c_uint32 * 6)()
        side = torch.cuda.Stream(self.device)
        native.check(native.kernels().xp_lane_failure(self.handle, w, side.cuda_stream), "xp_lane_failure", 0)
        return FabricFailure.from_words(list(w))

    def enable_trace(self, capacity: int = 1 << 16) -> None:
        """Turns the fabric observer on (after ``install``, before ``start``)."""
        native.check(native.kernels().xp_lane_trace_enable(self.handle, capacity), "xp_lane_trace_enable", 0)
        self._trace_capacity = capacity

    def trace_events(self) -> tuple[list[tuple[int, int, int, int]], int]:
        """(kind, a, b, timestamp_ns) per recorded Lane event, and the count of dropped events."""
        cap = getattr(self, "_trace_capacity", 0)
        if not cap:
            return [], 0
        out, dropped = (C.c_uint64 * (3 * cap))(), C.c_uint64()
        side = torch.cuda.Stream(self.device)
        n = native.kernels().xp_lane_trace_read(self.handle, out, cap, C.byref(dropped), side.cuda_stream)
        if n < 0:
            raise RuntimeError(f"xp_lane_trace_read failed with {n}")
        return [(out[3 * i] >> 32, out[3 * i] & 0xFFFFFFFF, out[3 * i + 1], out[3 * i + 2]) for i in range(n)], dropped.value

    def close(self) -> None:
        self.stop()
        if self.handle:
            native.kernels().xp_lane_destroy(self.handle)
            self.handle = None
        for st in self.instances:
            st.slot.free()


# ------------------------------------------------------------------ bring-up over torch.distributed

@dataclass
class RankContext:
    rank: int
    role: str
    engines: dict[str, AttentionEngine] = field(default_factory=dict)
    ffn: FfnRankRuntime | None = None
    buffers: list[PeerBuffer] = field(default_factory=list)


def build_rank(topo: Topology, rank: int, device, ecfg_for: dict[str, EngineConfig], group=None, n_lanes: int = 1,
               policy: int = rt.POLICY_FIFO, tile_weights: bool = False, kv_for=None) -> RankContext:
    """Creates this rank's side of every Instance and exchanges arena handles with its peers.
    Collective over ``group`` (any backend that supports object collectives). ``kv_for(placement)`` may return
    the KV cache an attention engine should use (an elastic one, say); None keeps the engine's fixed cache."""
    import torch.distributed as dist

    role = topo.role(rank)
    ctx = RankContext(rank, role)
    mine: dict[str, bytes] = {}
    atn_local: dict[str, PeerBuffer] = {}
    tp_groups: dict = {}
    if role == "ffn":
        ctx.ffn = FfnRankRuntime(device, n_lanes=n_lanes, policy=policy, tile_weights=tile_weights, pe=rank)
        for p in topo.instances:
            if rank in p.ffn_ranks:
                tp_rank, lo, hi = p.locate(rank)
                st = ctx.ffn.add_instance(p, tp_rank, (lo, hi))
                mine[f"ffn:{p.model_id}:{rank}"] = st.slot.handle()
    elif role == "atn":
        from . import atn_tp

        for p in topo.instances:
            if p.atn_rank == rank:
                buf = PeerBuffer(atn_slot_layout(p).total_bytes)
                atn_local[p.model_id] = buf
                ctx.buffers.append(buf)
                mine[f"atn:{p.model_id}"] = buf.handle()
            if rank in p.atn_tp_ranks and len(p.atn_tp_ranks) > 1:
                e = ecfg_for[p.model_id]
                g = atn_tp.TpGroup(p.atn_tp_ranks.index(rank), len(p.atn_tp_ranks), max(e.max_batch, e.prefill_chunk),
                                   p.cfg.hidden_size, device)
                tp_groups[p.model_id] = g
                mine[f"tp:{p.model_id}:{g.rank}"] = g.handle()
    gathered: list[dict] = [None] * topo.world_size
    dist.all_gather_object(gathered, mine, group=group)
    handles = {k: v for d in gathered for k, v in d.items()}
    if role == "ffn":
        for st in ctx.ffn.instances:
            st.atn_base = PeerBuffer.open(handles[f"atn:{st.place.model_id}"])
        ctx.ffn.install()
    elif role == "atn":
        from . import atn_tp

        for p in topo.instances:
            if rank not in p.atn_tp_ranks:
                continue
            if p.atn_rank == rank:
                bases = [PeerBuffer.open(handles[f"ffn:{p.model_id}:{r}"]) for r in p.ffn_ranks]
                port = FabricFfnPort(p, atn_local[p.model_id], bases, device)
            else:
                port = FabricFfnFollowerPort(p, PeerBuffer.open(handles[f"atn:{p.model_id}"]), device)
            aw = random_attention_weights(p.cfg, p.seed, device, torch.bfloat16)
            cfg_local, tp = p.cfg, tp_groups.get(p.model_id)
            if tp is not None:
                tp.connect([handles[f"tp:{p.model_id}:{r}"] for r in range(tp.size)])
                aw = atn_tp.shard_attention_weights(aw, p.cfg, tp.rank, tp.size)
                cfg_local = atn_tp.local_config(p.cfg, tp.size)
            kv = kv_for(p) if kv_for is not None else None
            ctx.engines[p.model_id] = AttentionEngine(cfg_local, aw, port, ecfg_for[p.model_id], device, kv=kv, tp=tp)
    dist.barrier(group=group)
    return ctx
