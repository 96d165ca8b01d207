"""FFN weight loader: reads only the local tensor-parallel shard of every projection.

For each layer the loader turns the :class:`FfnModelSpec` into read descriptors (which rows or
columns of which checkpoint tensor), reader threads stage the slices through a bounded set of pinned
host slots, and the slices are copied to the device and assembled into the layout the kernels want:
gate rows followed by up rows (``CONCATENATED``) for ``i_proj`` and the column shard for ``o_proj``.
True TP as in the reference (src/xpool/runtime/ffnagent/preparation.py:164-334, loader.py:148-286):
gate/up split by output rows, down by input columns, every expert alike; the output bias lives on TP
rank 0 only so that the reduction adds it once.
"""

from __future__ import annotations

import threading
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import torch

from ..ffn import DenseFfnSpec, FfnModelSpec, GateUpOrder, MoeFfnSpec, RouterProjectionPrecision, TopKWeightRounding
from ..models.weights import FfnLayerWeights
from .checkpoint import CheckpointKeyView


@dataclass(frozen=True)
class TensorRead:
    key: str
    rows: slice | None = None   # slice of dim -2
    cols: slice | None = None   # slice of dim -1
    expert: int | None = None   # leading index of a stacked tensor
    deinterleave: int | None = None  # 0: even rows (gate), 1: odd rows (up) of an interleaved tensor
    transposed: bool = False    # stored [.., in, out]: rows / cols / deinterleave name the [out, in] view that is returned


def _local(n: int, rank: int, size: int, quantum: int = 1) -> slice:
    if n % (size * quantum):
        raise ValueError(f"dimension {n} is not divisible into {size} shards of multiples of {quantum}")
    w = n // size
    return slice(rank * w, (rank + 1) * w)


class _Reader:
    """Opens each safetensors file once per thread and reads slices without loading whole tensors."""

    def __init__(self, view: CheckpointKeyView):
        self.view = view
        self._tls = threading.local()

    def _file(self, name: str):
        from safetensors import safe_open

        cache = getattr(self._tls, "files", None)
        if cache is None:
            cache = self._tls.files = {}
        if name not in cache:
            cache[name] = safe_open(str(self.view.root / name), framework="pt")
        return cache[name]

    def read(self, r: TensorRead) -> torch.Tensor:
        sl = self._file(self.view.key_to_file[r.key]).get_slice(r.key)
        nd = len(sl.get_shape())
        idx: list = [slice(None)] * nd
        if r.expert is not None:
            idx[0] = r.expert
        row_dim, col_dim = (-1, -2) if r.transposed else (-2, -1)
        if r.deinterleave is not None:
            n = sl.get_shape()[row_dim]
            rows = r.rows or slice(0, n // 2)
            idx[row_dim] = slice(2 * rows.start + r.deinterleave, 2 * rows.stop, 2)
        elif r.rows is not None:
            idx[row_dim if nd >= 2 else -1] = r.rows
        if r.cols is not None:
            idx[col_dim] = r.cols
        if r.transposed:
            return self._sliced(sl, idx).transpose(-1, -2).contiguous()
        return self._sliced(sl, idx)

    @staticmethod
    def _sliced(sl, idx: list) -> torch.Tensor:
        strided = [i for i, v in enumerate(idx) if isinstance(v, slice) and v.step not in (None, 1)]
        if strided:   # safetensors slices take unit steps only: read the span, stride in memory
            steps = {i: idx[i].step for i in strided}
            for i in strided:
                idx[i] = slice(idx[i].start, idx[i].stop)
            t = sl[tuple(idx)]
            lead = sum(1 for v in idx[:min(strided)] if isinstance(v, int))   # dims dropped by integer indices
            for i, st in steps.items():
                t = t[(slice(None),) * (i - lead) + (slice(None, None, st),)]
            return t
        return sl[tuple(idx)]


class PinnedStager:
    """A bounded pool of pinned host slots: readers fill them, the copier drains them to the device,
    so host memory stays bounded however large the model is ([ffn.loader] parallelism slots)."""

    def __init__(self, slots: int, device):
        self.device = torch.device(device)
        self._sem = threading.Semaphore(max(1, slots))
        self.pinned = self.device.type == "cuda"

    def to_device(self, t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        with self._sem:
            t = t.to(dtype).contiguous()
            if self.pinned:
                t = t.pin_memory()
                out = t.to(self.device, non_blocking=True)
                torch.cuda.current_stream(self.device).synchronize()
                return out
            return t.to(self.device)


def _dense_reads(l: DenseFfnSpec, rank: int, size: int):
    rows = _local(l.intermediate_size, rank, size)
    ip = l.i_proj
    reads = {}
    if ip.packed is not None:
        if ip.source_order == GateUpOrder.INTERLEAVED:
            reads["gate"] = TensorRead(ip.packed.weight_key, rows=rows, deinterleave=0)
            reads["up"] = TensorRead(ip.packed.weight_key, rows=rows, deinterleave=1)
        else:
            reads["gate"] = TensorRead(ip.packed.weight_key, rows=rows)
            reads["up"] = TensorRead(ip.packed.weight_key, rows=slice(l.intermediate_size + rows.start, l.intermediate_size + rows.stop))
    else:
        if ip.gate is not None:
            reads["gate"] = TensorRead(ip.gate.weight_key, rows=rows)
            if ip.gate.bias_key:
                reads["gate_bias"] = TensorRead(ip.gate.bias_key, rows=rows)
        reads["up"] = TensorRead(ip.up.weight_key, rows=rows)
        if ip.up.bias_key:
            reads["up_bias"] = TensorRead(ip.up.bias_key, rows=rows)
    reads["down"] = TensorRead(l.o_proj.weight_key, cols=rows)
    if l.o_proj.bias_key and rank == 0:
        reads["down_bias"] = TensorRead(l.o_proj.bias_key)
    return reads


def _dense_fp8_block(l: DenseFfnSpec, reader: "_Reader", rank: int, size: int, stager: "PinnedStager", dtype: torch.dtype
                     ) -> FfnLayerWeights:
    """One gated dense layer of a block-scaled fp8 checkpoint: e4m3 ``weight`` plus ``weight_scale_inv`` (fp32, one per
    128 x 128 block; the weight is ``code * scale``). The local tensor-parallel shard is cut on block boundaries. The
    layer is returned expanded to ``dtype`` (what the Lanes compute in) and, under ``extra["fp8"]``, as the stored
    codes and scales in the layout of the fp8 GEMM path (``ops/gemm.py::linear_fp8``), so nothing is re-quantised."""
    from ..quantization import Fp8Block

    inter = l.intermediate_size
    if inter % (size * 128):
        raise ValueError(f"intermediate size {inter} does not split into {size} shards of whole 128-wide blocks")
    rows = _local(inter, rank, size, 128)
    blocks = slice(rows.start // 128, rows.stop // 128)
    fmt = Fp8Block()

    def part(p, **cut):
        blk = {k: (blocks if v is rows else v) for k, v in cut.items()}
        return {"weight": reader.read(TensorRead(p.weight_key, **cut)), "scale": reader.read(TensorRead(p.scales_key, **blk)).float()}

    gate, up, down = part(l.i_proj.gate, rows=rows), part(l.i_proj.up, rows=rows), part(l.o_proj, cols=rows)
    for name, t in (("gate", gate), ("up", up), ("down", down)):
        if t["weight"].dtype != torch.float8_e4m3fn:
            raise ValueError(f"{name} projection of layer {l.layer}: expected e4m3 codes, found {t['weight'].dtype}")
    gu = {"weight": torch.cat([gate["weight"].view(torch.uint8), up["weight"].view(torch.uint8)], 0).view(torch.float8_e4m3fn),
          "scale": torch.cat([gate["scale"], up["scale"]], 0)}
    w = FfnLayerWeights(stager.to_device(fmt.dequantize(gu, dtype), dtype), stager.to_device(fmt.dequantize(down, dtype), dtype))
    w.extra["gated"] = True
    dev = stager.device
    w.extra["fp8"] = {"gate_up": gu["weight"].to(dev), "gate_up_scale": gu["scale"].contiguous().to(dev),
                      "down": down["weight"].contiguous().to(dev), "down_scale": down["scale"].contiguous().to(dev)}
    return w


def _mxfp4_expert(reader: "_Reader", blocks_key: str, suffix: str, expert: int) -> torch.Tensor:
    """One expert's projection of a stacked MXFP4 tensor, dequantised to bf16 ``[rows, k]``. The checkpoint holds
    ``*_blocks`` ``[experts, rows, k / 32, 16]`` (two e2m1 codes per byte, low nibble first) and ``*_scales``
    ``[experts, rows, k / 32]`` (e8m0). The reference keeps such weights packed for its GEMM library
    (src/xpool/quantization/mxfp4.py); this build expands them once at load time and runs the bf16 kernels."""
    from ..quantization import Mxfp4

    blocks = reader.read(TensorRead(blocks_key, expert=expert))
    scales = reader.read(TensorRead(blocks_key.removesuffix("_blocks") + suffix, expert=expert))
    rows = blocks.shape[0]
    return Mxfp4().dequantize({"blocks": blocks.reshape(rows, -1), "scales": scales.reshape(rows, -1)}, torch.bfloat16)


def _moe_mxfp4(l: MoeFfnSpec, reader: "_Reader", rank: int, size: int, experts: range) -> dict[str, torch.Tensor]:
    """Host tensors ``gate{e}``/``up{e}``/``down{e}`` of the local shard, from packed MXFP4 expert tensors."""
    rows = _local(l.moe_intermediate_size, rank, size, 32)
    ex, inter, out = l.experts, l.moe_intermediate_size, {}
    for e in experts:
        gu = _mxfp4_expert(reader, ex.packed_key, ex.scales_suffix, e)             # [2 * inter, hidden]
        if l.source_order == GateUpOrder.INTERLEAVED:
            g, u = gu[0::2], gu[1::2]
        else:
            g, u = gu[:inter], gu[inter:]
        out[f"gate{e}"], out[f"up{e}"] = g[rows].contiguous(), u[rows].contiguous()
        out[f"down{e}"] = _mxfp4_expert(reader, ex.down_key, ex.scales_suffix, e)[:, rows].contiguous()
    return out


def _moe_reads(l: MoeFfnSpec, rank: int, size: int, experts: range, packed_weights: bool = True):
    rows = _local(l.moe_intermediate_size, rank, size)
    ex = l.experts
    reads = {"router": TensorRead(l.router_weight_key)}
    if l.router_precision == RouterProjectionPrecision.FP32:
        reads["router_fp32"] = TensorRead(l.router_weight_key)     # kept at fp32 for the exact projection
    if l.router_bias_key:
        reads["router_bias"] = TensorRead(l.router_bias_key)
    if l.correction_bias_key:
        reads["correction_bias"] = TensorRead(l.correction_bias_key)
    for e in experts:
        if ex.gate_bias_key:
            # per-expert biases: [experts, 2 * inter] in the source order of the packed projection, [experts, hidden]
            inter = l.moe_intermediate_size
            if ex.per_expert:
                raise NotImplementedError("biases of per-expert checkpoints")
            if l.source_order == GateUpOrder.INTERLEAVED:
                reads[f"gate_bias{e}"] = TensorRead(ex.gate_bias_key, expert=e, cols=slice(2 * rows.start, 2 * rows.stop, 2))
                reads[f"up_bias{e}"] = TensorRead(ex.gate_bias_key, expert=e, cols=slice(2 * rows.start + 1, 2 * rows.stop, 2))
            else:
                reads[f"gate_bias{e}"] = TensorRead(ex.gate_bias_key, expert=e, cols=rows)
                reads[f"up_bias{e}"] = TensorRead(ex.gate_bias_key, expert=e, cols=slice(inter + rows.start, inter + rows.stop))
        if ex.down_bias_key and rank == 0:
            reads[f"down_bias{e}"] = TensorRead(ex.down_bias_key, expert=e)     # added once: TP rank 0 only
        if not packed_weights:
            continue
        if ex.per_expert:
            reads[f"gate{e}"] = TensorRead(ex.gate_key.format(expert=e), rows=rows)
            reads[f"up{e}"] = TensorRead(ex.up_key.format(expert=e), rows=rows)
            reads[f"down{e}"] = TensorRead(ex.down_key.format(expert=e), cols=rows)
        else:
            inter = l.moe_intermediate_size
            if l.source_order == GateUpOrder.INTERLEAVED:
                reads[f"gate{e}"] = TensorRead(ex.packed_key, rows=rows, expert=e, deinterleave=0, transposed=ex.input_major)
                reads[f"up{e}"] = TensorRead(ex.packed_key, rows=rows, expert=e, deinterleave=1, transposed=ex.input_major)
            else:
                reads[f"gate{e}"] = TensorRead(ex.packed_key, rows=rows, expert=e, transposed=ex.input_major)
                reads[f"up{e}"] = TensorRead(ex.packed_key, rows=slice(inter + rows.start, inter + rows.stop), expert=e,
                                             transposed=ex.input_major)
            reads[f"down{e}"] = TensorRead(ex.down_key, cols=rows, expert=e, transposed=ex.input_major)
    if l.num_shared_experts:
        srows = _local(l.shared_intermediate_size, rank, size)
        reads["shared_gate"] = TensorRead(l.shared_gate_key, rows=srows)
        reads["shared_up"] = TensorRead(l.shared_up_key, rows=srows)
        reads["shared_down"] = TensorRead(l.shared_down_key, cols=srows)
    return reads


def materialize_layer_weights(spec: FfnModelSpec, view: CheckpointKeyView, layer: int, *, tp_rank: int = 0, tp_size: int = 1,
                              device="cpu", dtype: torch.dtype = torch.bfloat16, parallelism: int = 4,
                              experts: range | None = None) -> FfnLayerWeights:
    """Loads one layer's local shard. ``experts`` restricts a MoE layer to a range (expert parallelism)."""
    if spec.quantization not in ("none", "mxfp4", "fp8_block"):
        raise NotImplementedError(f"checkpoints quantised with {spec.quantization} are not loadable")
    l = spec.layers[layer]
    if spec.quantization == "fp8_block":
        if not isinstance(l, DenseFfnSpec) or l.i_proj.gate is None or l.i_proj.gate.scales_key is None:
            raise NotImplementedError("block-scaled fp8 checkpoints are loadable for gated dense layers only")
        return _dense_fp8_block(l, _Reader(view), tp_rank, tp_size, PinnedStager(parallelism, device), dtype)
    mx = spec.quantization == "mxfp4" and isinstance(l, MoeFfnSpec) and l.experts.scales_suffix is not None
    stager, reader = PinnedStager(parallelism, device), _Reader(view)
    if isinstance(l, DenseFfnSpec):
        reads = _dense_reads(l, tp_rank, tp_size)
    else:
        experts = experts if experts is not None else range(l.num_experts)
        reads = _moe_reads(l, tp_rank, tp_size, experts, packed_weights=not mx)

    def fetch(item):
        name, r = item
        wide = "bias" in name or name == "router_fp32"   # biases stay fp32: the GEMM epilogue adds them to the fp32 accumulator
        return name, stager.to_device(reader.read(r), torch.float32 if wide else dtype)

    with ThreadPoolExecutor(max_workers=max(1, parallelism)) as pool:
        got = dict(pool.map(fetch, reads.items()))
    if mx:
        got.update({k: stager.to_device(v, dtype) for k, v in _moe_mxfp4(l, reader, tp_rank, tp_size, experts).items()})
    if isinstance(l, DenseFfnSpec):
        gated = "gate" in got
        gate_up = torch.cat([got["gate"], got["up"]], 0) if gated else got["up"]
        gub = None
        if "up_bias" in got:
            gub = torch.cat([got["gate_bias"], got["up_bias"]], 0) if "gate_bias" in got else got["up_bias"]
        w = FfnLayerWeights(gate_up, got["down"], gate_up_bias=gub, down_bias=got.get("down_bias"))
        w.extra["gated"] = gated
        t = l.gate_transform
        if t is not None and (t.limit > 0 or t.up_offset != 0 or t.alpha != 1.0):
            w.extra["gate_transform"] = (float(t.limit), float(t.up_offset), float(t.alpha))
        return w
    gate_up = torch.stack([torch.cat([got[f"gate{e}"], got[f"up{e}"]], 0) for e in experts])
    down = torch.stack([got[f"down{e}"] for e in experts])
    w = FfnLayerWeights(gate_up, down, router=got["router"])
    if f"gate_bias{experts[0]}" in got:
        w.gate_up_bias = torch.stack([torch.cat([got[f"gate_bias{e}"], got[f"up_bias{e}"]]) for e in experts]).contiguous()
    if f"down_bias{experts[0]}" in got:
        w.down_bias = torch.stack([got[f"down_bias{e}"] for e in experts]).contiguous()
    t = l.gate_transform
    if t is not None and (t.limit > 0 or t.up_offset != 0 or t.alpha != 1.0):
        w.extra["gate_transform"] = (float(t.limit), float(t.up_offset), float(t.alpha))
    if "shared_gate" in got:
        w.shared_gate_up = torch.cat([got["shared_gate"], got["shared_up"]], 0)
        w.shared_down = got["shared_down"]
    for k in ("router_bias", "correction_bias"):
        if k in got:
            w.extra[k] = got[k]
    w.extra["experts"] = (experts.start, experts.stop)
    w.extra["router_precision"] = l.router_precision.value
    if l.topk_weight_rounding == TopKWeightRounding.LOGITS_DTYPE:
        w.extra["round_topk_weights"] = True      # combine weights rounded to the logits' dtype (GPT-OSS)
    if "router_fp32" in got:
        w.extra["router_fp32"] = got["router_fp32"].contiguous()
    return w


def materialize_model_weights(spec: FfnModelSpec, view: CheckpointKeyView, layers: range, **kw) -> list[FfnLayerWeights]:
    return [materialize_layer_weights(spec, view, l, **kw) for l in layers]
