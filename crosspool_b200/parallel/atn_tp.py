"""Attention tensor parallelism inside one Instance: query and KV heads are split over the attention
ranks of the Instance; the output projection produces one partial per rank and the following
add-RMSNorm folds all partials.

The all-reduce is not a library collective. Every rank keeps its partial in a peer-mapped buffer;
after the projection a one-CTA kernel releases a sequence number into a flag word on every peer, a
wait kernel holds the stream until all peers' flags carry the same number, and the add-RMSNorm kernel
then reads its own partial and the peers' partials (plain loads over NVLink) and sums them in rank
order with fp32 accumulation -- the same order on every rank, so all ranks compute bit-identical
hidden states and keep making identical scheduling and sampling decisions without exchanging them.
Two partial buffers alternate by layer parity; the flag handshake of layer ``l + 1`` orders a rank's
rewrite of a buffer after every peer's read of layer ``l - 1``.

The reference gets attention TP from its serving engine (SGLang NCCL groups; ``atn_tp_size`` in
src/xpool/config.py and src/xpool/integrations/sglang/topology.py).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import replace

import torch

from .. import native
from ..models.config import ModelConfig
from ..models.weights import AttentionWeights, AttnLayerWeights
from .fabric import PeerBuffer

FLAG_BYTES = 256


def local_config(cfg: ModelConfig, tp_size: int) -> ModelConfig:
    if cfg.num_q_heads % tp_size or cfg.num_kv_heads % tp_size:
        raise ValueError(f"{cfg.num_q_heads} query / {cfg.num_kv_heads} KV heads do not split over {tp_size} ranks")
    return replace(cfg, num_q_heads=cfg.num_q_heads // tp_size, num_kv_heads=cfg.num_kv_heads // tp_size)


def shard_attention_weights(w: AttentionWeights, cfg: ModelConfig, tp_rank: int, tp_size: int) -> AttentionWeights:
    """Rank ``tp_rank``'s heads: rows of q, k and v, the matching columns of the output projection."""
    d, hq, hkv = cfg.head_dim, cfg.num_q_heads // tp_size, cfg.num_kv_heads // tp_size
    q0, k0, v0 = 0, cfg.q_size, cfg.q_size + cfg.kv_size
    layers = []
    for lw in w.layers:
        rows = torch.cat([torch.arange(q0 + tp_rank * hq * d, q0 + (tp_rank + 1) * hq * d),
                          torch.arange(k0 + tp_rank * hkv * d, k0 + (tp_rank + 1) * hkv * d),
                          torch.arange(v0 + tp_rank * hkv * d, v0 + (tp_rank + 1) * hkv * d)]).to(lw.qkv.device)
        layers.append(AttnLayerWeights(
            input_norm=lw.input_norm, post_attn_norm=lw.post_attn_norm, qkv=lw.qkv.index_select(0, rows).contiguous(),
            o=lw.o[:, tp_rank * hq * d:(tp_rank + 1) * hq * d].contiguous(), q_norm=lw.q_norm, k_norm=lw.k_norm,
            qkv_bias=lw.qkv_bias.index_select(0, rows).contiguous() if lw.qkv_bias is not None else None))
    return AttentionWeights(w.embed, layers, w.final_norm, w.lm_head)


class TpGroup:
    """One rank's view of the Instance's attention TP group."""

    def __init__(self, tp_rank: int, tp_size: int, cap_rows: int, hidden: int, device):
        if not 2 <= tp_size <= 8:
            raise ValueError("attention TP size must be within 2..8")
        self.rank, self.size, self.cap, self.hidden = tp_rank, tp_size, cap_rows, hidden
        self.device = torch.device(device)
        self.part_bytes = cap_rows * hidden * 2
        self.buf = PeerBuffer(FLAG_BYTES + 2 * self.part_bytes)
        native.check(native.kernels().xp_memset_async(self.buf.ptr, 0, FLAG_BYTES, torch.cuda.current_stream(self.device).cuda_stream),
                     "xp_memset_async", 0)
        torch.cuda.synchronize(self.device)
        self.bases: list[int] = [0] * tp_size      # mapped base address of every rank's buffer (own included)
        self.bases[tp_rank] = self.buf.ptr
        self.local_parts = [self.buf.tensor(FLAG_BYTES + p * self.part_bytes, (cap_rows, hidden), torch.bfloat16, self.device)
                            for p in (0, 1)]
        self.seq = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._sig = self._wait = None

    def handle(self) -> bytes:
        return self.buf.handle()

    def connect(self, handles: list[bytes]) -> None:
        """``handles[r]`` is rank r's buffer handle (this rank's own entry is ignored)."""
        for r, h in enumerate(handles):
            if r != self.rank:
                self.bases[r] = PeerBuffer.open(h)
        from ..ops.gemm import status_words

        sig = native.SignalArgs()
        peers = [r for r in range(self.size) if r != self.rank]
        for i, r in enumerate(peers):
            sig.flags[i] = self.bases[r] + 4 * self.rank     # my word in the peer's flag block
        sig.n, sig.seq_counter = len(peers), self.seq.data_ptr()
        w = native.WaitArgs()
        for i, r in enumerate(peers):
            w.flags[i] = self.buf.ptr + 4 * r                # the peer's word in my flag block
        w.n, w.want_ptr, w.wait_ns = len(peers), self.seq.data_ptr(), 5_000_000_000
        w.status = status_words(self.device).data_ptr()
        self._sig, self._wait = sig, w

    def part(self, layer: int) -> torch.Tensor:
        """Where this rank's output projection of ``layer`` writes its partial."""
        return self.local_parts[layer & 1]

    def exchange(self) -> None:
        """Announces this rank's partial and waits for every peer's (both on the current stream)."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        k = native.kernels()
        native.check(k.xp_signal_flags(C.byref(self._sig), s), "xp_signal_flags")
        native.check(k.xp_wait_flags(C.byref(self._wait), s), "xp_wait_flags")

    def part_ptrs(self, layer: int) -> list[int]:
        off = FLAG_BYTES + (layer & 1) * self.part_bytes
        return [b + off for b in self.bases]

    def close(self) -> None:
        self.buf.free()
