"""Attention-side engine of one Instance on one attention device.

Owns embedding, attention (paged KV), norms, LM head, greedy sampling and a continuous-batching
scheduler with chunked prefill; every decoder FFN goes through an :class:`FfnPort` — in-stream on
the same GPU (loopback), or published to the FFN tier over peer memory. The reference borrows all of
this from SGLang and only swaps the MLP for a shim (src/xpool/integrations/sglang/shim.py:94-192);
here the engine is native so that the kernel which produces the post-attention hidden states is
itself the transport producer.

Per decode step the host does one pinned H2D copy of the step's metadata (token ids, positions, KV
slots, sequence lengths, block table), replays one CUDA graph for the batch-size bucket, and reads
the sampled token ids back with one D2H copy.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

import torch

from ..models.config import ModelConfig
from ..models.weights import AttentionWeights
from ..ops import attention as A
from ..ops import gemm, norm
from ..utils import nvtx
from .kv_cache import OutOfPages, PagedKvCache

MODE_PREFILL, MODE_DECODE = 1, 2


def capacity_buckets(max_rows: int) -> list[int]:
    """Powers of two up to the maximum plus the exact maximum — the reference's Capacity rule
    (src/xpool/runtime/ffnagent/execution.py:166-177)."""
    out, c = [], 1
    while c < max_rows:
        out.append(c)
        c *= 2
    out.append(max_rows)
    return out


FIRST_CONTACT_WAIT_NS = 30_000_000_000   # wait limit of an Instance's very first FFN invocation (warm-up)


@dataclass
class EngineConfig:
    max_batch: int = 256
    prefill_chunk: int = 2048
    max_seq_len: int = 4096
    page_size: int = 16
    num_pages: int = 0  # 0: sized for max_batch sequences of max_seq_len
    max_prefill_seqs: int = 64
    use_cuda_graph: bool = True
    decode_buckets: list[int] | None = None
    prefix_cache: bool = False  # keep full prompt pages and share them with later requests
    sampling: bool = False      # per-request temperature sampling (Gumbel-max kernel) instead of greedy argmax


@dataclass
class Sequence:
    seq_id: int
    prompt: list[int]
    max_new_tokens: int
    arrival: float = 0.0
    deadline: float = 0.0
    computed: int = 0                # tokens whose KV is cached
    generated: list[int] = field(default_factory=list)
    first_token_time: float | None = None
    finish_time: float | None = None
    token_times: list[float] = field(default_factory=list)
    temperature: float = 0.0         # 0: greedy (needs EngineConfig.sampling for anything else)
    seed: int = 0
    refill_len: int = 0              # > 0 after a retraction: prompt + generated tokens to recompute before decoding on

    @property
    def fill_len(self) -> int:
        """Tokens the prefill phase has to cache: the prompt, or after a retraction everything emitted so far."""
        return self.refill_len or len(self.prompt)

    def fill_tokens(self, start: int, n: int) -> list[int]:
        """Tokens ``start .. start + n`` of the prefill stream (prompt, then already generated tokens)."""
        if start + n <= len(self.prompt):
            return self.prompt[start:start + n]
        return (self.prompt + self.generated)[start:start + n]

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.generated)

    @property
    def prefill_done(self) -> bool:
        return self.computed >= self.fill_len

    @property
    def finished(self) -> bool:
        return len(self.generated) >= self.max_new_tokens


class UnsupportedAttention(NotImplementedError):
    """The model's attention form is not one the GPU attention engine computes."""


class FfnPort:
    """Where a layer's FFN runs. ``run`` receives the normalised hidden states of ``rows`` tokens
    and returns the tensors whose fixed-order sum is the FFN output (one per FFN TP rank)."""

    def attach(self, engine: "AttentionEngine") -> None:  # pragma: no cover - interface
        pass

    def run(self, layer: int, x: torch.Tensor, rows: int, mode: int) -> list[torch.Tensor]:
        raise NotImplementedError

    # Ports that receive the hidden states straight from the norm kernel return publish targets.
    def publish_targets(self, layer: int, rows: int, mode: int) -> dict | None:
        return None

    def wait_args(self) -> dict:
        return {}

    # Optional: ``announce_forward(rows, mode)`` is called on the host right before a forward pass of ``rows`` rows is
    # enqueued (eagerly or as a graph replay; not while a graph is being captured). A port whose FFN side must be
    # told on the host that work is coming (the library-collective arm) implements it.


def _parts_kw(parts) -> dict:
    """FFN outputs as add-RMSNorm arguments: a list of local tensors, or (for a port whose result lives
    in another GPU's memory) a dict with ``part_ptrs`` and ``part_shape``."""
    return parts if isinstance(parts, dict) else dict(parts=parts)


class AttentionEngine:
    def __init__(self, cfg: ModelConfig, weights: AttentionWeights, port: FfnPort, ecfg: EngineConfig | None = None,
                 device: str | torch.device = "cuda", kv: PagedKvCache | None = None, tp=None):
        """``tp``: a connected ``parallel.atn_tp.TpGroup`` when this engine is one attention TP rank;
        ``cfg`` and ``weights`` are then the rank-local ones (``atn_tp.local_config`` /
        ``shard_attention_weights``)."""
        if not cfg.gpu_attention_supported:
            raise UnsupportedAttention(
                f"{cfg.architecture}: this engine runs rotary grouped-query attention with RMSNorm; LayerNorm with learned "
                "positions, sliding windows, attention sinks, scaled rotary embeddings and latent attention run in the "
                "PyTorch oracle and the CPU deployment only (engine/cpu_plumbing.py). The FFN tier serves this architecture.")
        self.cfg, self.w, self.port = cfg, weights, port
        self.tp = tp
        self.ecfg = ecfg or EngineConfig()
        self.device = torch.device(device)
        e = self.ecfg
        self.max_blocks = (e.max_seq_len + e.page_size - 1) // e.page_size
        if kv is None:
            pages = e.num_pages or e.max_batch * self.max_blocks
            kv = PagedKvCache.fixed(cfg, pages, e.page_size, self.device)
        self.kv = kv
        self.cap = max(e.max_batch, e.prefill_chunk)
        self._alloc_buffers()
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.prefilling: list[Sequence] = []
        self._graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self._buckets = e.decode_buckets or capacity_buckets(e.max_batch)
        self._next_id = 0
        self._last_was_prefill = False
        self.stats = {"prefill_steps": 0, "decode_steps": 0, "h2d_bytes": 0, "d2h_bytes": 0, "launches": 0}
        self.stream = torch.cuda.Stream(self.device)
        self._b_key = None
        self._b_pos = None
        self._b_last = None
        self._inflight = None
        self._pending: list[tuple[Sequence, int]] | None = None
        self._pre_inflight: list[tuple[Sequence, int]] | None = None
        self._step_event = torch.cuda.Event() if torch.cuda.is_available() else None
        self._graph_launches: dict[int, int] = {}
        self.prefix = None
        if e.prefix_cache:
            from .prefix_cache import PrefixCache

            self.prefix = PrefixCache(e.page_size)
        self.capacity = None          # ecs.reconciler.CapacityReconciler when the KV cache is elastic
        self._demand_pages = 0
        self.ttft_slo_s = 0.0
        port.attach(self)

    # ------------------------------------------------------------------ elastic KV capacity
    def attach_capacity(self, reconciler, ttft_slo_s: float = 0.0) -> None:
        """Couples the engine to the capacity channel: it publishes demand when admission stalls,
        executes grow/shrink commands once per step, and retracts sequences when a shrink needs
        bundles that would not drain on their own."""
        self.capacity, self.ttft_slo_s = reconciler, ttft_slo_s

    def _capacity_tick(self) -> None:
        rec = self.capacity
        rec.poll()
        if rec.bundles_to_vacate() > 0 and not rec.retirable_empty() and self._inflight is None:
            if self._vacate_by_eviction(rec):        # cached prefixes go before running work does
                rec.poll()
            elif self.running:
                self._retract(self.running[-1])  # newest first: the least work is lost
                self.stats["retracted_for_shrink"] = self.stats.get("retracted_for_shrink", 0) + 1
                rec.poll()

    def _vacate_by_eviction(self, rec) -> bool:
        """Empties one memory bundle by evicting cached prefix pages, if some bundle above the floor holds nothing but
        unpinned cached pages. Returns whether a bundle became empty."""
        if self.prefix is None or len(self.prefix) == 0:
            return False
        alloc = self.kv.allocator
        cands = [b for b in alloc.mapped_bundles() if b >= rec.floor_bundles and alloc.used_in_bundle(b) > 0]
        for b in sorted(cands, key=lambda b: (alloc.used_in_bundle(b), -b)):
            pages = alloc.bundle_pages(b)
            if self.prefix.evictable_among(pages) == alloc.used_in_bundle(b):
                alloc.free(self.prefix.evict_pages(pages))
                self.stats["evicted_for_shrink"] = self.stats.get("evicted_for_shrink", 0) + 1
                return True
        return False

    def idle_tick(self) -> None:
        """Serves capacity commands while there is nothing to run: an idle Instance is the usual donor of a
        shrink, and nothing else would look at its command."""
        if self.capacity is not None and not self.has_work:
            self._capacity_tick()

    def _publish_demand(self, missing_pages: int, head: "Sequence | None") -> None:
        if self.capacity is None or missing_pages == self._demand_pages:
            return
        self._demand_pages = missing_pages
        if missing_pages <= 0:
            self.capacity.withdraw_demand()
            return
        deadline = int((head.arrival + self.ttft_slo_s) * 1e9) if head is not None and self.ttft_slo_s > 0 else 0
        self.capacity.publish_demand(missing_pages, deadline)

    # ------------------------------------------------------------------ buffers
    def _alloc_buffers(self) -> None:
        cfg, e, dev = self.cfg, self.ecfg, self.device
        bf = torch.bfloat16
        cap, B = self.cap, e.max_batch
        self.resid = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
        self.x = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
        self.x2 = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
        self.qkv = torch.zeros(cap, cfg.q_size + 2 * cfg.kv_size, dtype=bf, device=dev)
        self.q = torch.zeros(cap, cfg.num_q_heads, cfg.head_dim, dtype=bf, device=dev)
        self.attn_out = torch.zeros(cap, cfg.num_q_heads, cfg.head_dim, dtype=bf, device=dev)
        self.o = torch.zeros(cap, cfg.hidden_size, dtype=bf, device=dev)
        self.sel = torch.zeros(max(B, e.max_prefill_seqs), cfg.hidden_size, dtype=bf, device=dev)
        self.logits = torch.zeros(max(B, e.max_prefill_seqs), cfg.vocab_size, dtype=bf, device=dev)
        self.tokens = torch.zeros(max(B, e.max_prefill_seqs), dtype=torch.int32, device=dev)
        if e.sampling:
            n = max(B, e.max_prefill_seqs)
            self.samp_temps = torch.zeros(n, dtype=torch.float32, device=dev)
            self.samp_seeds = torch.zeros(n, 2, dtype=torch.int32, device=dev)
            self._samp_host = torch.zeros(n, 3, dtype=torch.float32).pin_memory()   # temperature | seed, step as int bits
        self.tokens_host = torch.zeros(max(B, e.max_prefill_seqs), dtype=torch.int32).pin_memory()
        # decode metadata: ids | positions | slots | seq_lens | block_table, one pinned mirror
        self._dec_words = 4 * B + B * self.max_blocks
        self.dec_meta = torch.zeros(self._dec_words, dtype=torch.int32, device=dev)
        self.dec_meta_host = torch.zeros(self._dec_words, dtype=torch.int32).pin_memory()
        # prefill metadata: ids | positions | slots (chunk) + q_starts | q_lens | ctx_lens | last_idx + table
        P, S = e.prefill_chunk, e.max_prefill_seqs
        self._pre_words = 3 * P + 4 * S + S * self.max_blocks
        self.pre_meta = torch.zeros(self._pre_words, dtype=torch.int32, device=dev)
        self.pre_meta_host = torch.zeros(self._pre_words, dtype=torch.int32).pin_memory()
        buckets = e.decode_buckets or capacity_buckets(B)
        ws_rows = max(b * A.decode_plan(b, cfg.num_kv_heads, e.max_seq_len)[0] for b in buckets)
        self.attn_ws = torch.zeros(ws_rows * cfg.num_q_heads * (cfg.head_dim + 2), dtype=torch.float32, device=dev)

    def _dec_views(self, B: int):
        m, cap = self.dec_meta, self.ecfg.max_batch
        return (m[0:B], m[cap:cap + B], m[2 * cap:2 * cap + B], m[3 * cap:3 * cap + B],
                m[4 * cap:4 * cap + B * self.max_blocks].view(B, self.max_blocks))

    # ------------------------------------------------------------------ request API
    def add_request(self, prompt: list[int], max_new_tokens: int, arrival: float | None = None,
                    deadline: float = 0.0, temperature: float = 0.0, seed: int = 0) -> Sequence:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        if len(prompt) + max_new_tokens > self.ecfg.max_seq_len:
            raise ValueError("request exceeds max_seq_len")
        if min(prompt) < 0 or max(prompt) >= self.cfg.vocab_size:
            raise ValueError(f"token id outside [0, {self.cfg.vocab_size})")
        if temperature > 0 and not self.ecfg.sampling:
            raise ValueError("temperature sampling needs EngineConfig(sampling=True)")
        s = Sequence(self._next_id, list(prompt), max_new_tokens, arrival if arrival is not None else time.monotonic(),
                     deadline, temperature=float(temperature), seed=int(seed) & 0x7FFFFFFF)
        self._next_id += 1
        self.waiting.append(s)
        return s

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self.prefilling)

    def _stage_sampling(self, seqs: list["Sequence"]) -> None:
        """Copies the rows' temperatures and (seed, step) pairs to the device (on the engine stream, before the
        forward that samples them)."""
        if not self.ecfg.sampling:
            return
        h = self._samp_host
        hi = h.view(torch.int32)
        for i, s in enumerate(seqs):
            h[i, 0] = s.temperature
            hi[i, 1] = s.seed
            hi[i, 2] = len(s.generated)
        n = len(seqs)
        self.samp_temps[:n].copy_(h[:n, 0], non_blocking=True)
        self.samp_seeds[:n].copy_(hi[:n, 1:3], non_blocking=True)

    # ------------------------------------------------------------------ model forward
    def _layers(self, rows: int, mode: int, attn_fn) -> None:
        """Runs all decoder layers over the first ``rows`` rows of the static buffers. ``resid``
        holds the embeddings on entry and the final residual stream (before the last FFN add) on
        exit; the last FFN output parts are left in ``self._parts``."""
        cfg, w = self.cfg, self.w
        resid, x, x2 = self.resid[:rows], self.x[:rows], self.x2[:rows]
        parts: list[torch.Tensor] | None = None
        for l, lw in enumerate(w.layers):
            if parts is None:
                norm.add_rmsnorm([resid], lw.input_norm, cfg.rms_norm_eps, out=x)
            else:
                norm.add_rmsnorm(weight=lw.input_norm, eps=cfg.rms_norm_eps, resid=resid, out=x, **_parts_kw(parts),
                                 **self.port.wait_args())
            gemm.linear(x, lw.qkv, out=self.qkv[:rows], bias=lw.qkv_bias)
            attn_fn(l, lw, rows)
            tgt = self.port.publish_targets(l, rows, mode)
            if self.tp is None:
                gemm.linear(self.attn_out[:rows].view(rows, cfg.q_size), lw.o, out=self.o[:rows])
                o_parts = dict(parts=[self.o[:rows]])
            else:
                # this rank's heads give a partial; all ranks' partials are folded by the norm below
                gemm.linear(self.attn_out[:rows].view(rows, cfg.q_size), lw.o, out=self.tp.part(l)[:rows])
                self.tp.exchange()
                o_parts = dict(parts=[], part_ptrs=self.tp.part_ptrs(l), part_shape=(rows, cfg.hidden_size, cfg.hidden_size))
            if tgt is None:
                norm.add_rmsnorm(weight=lw.post_attn_norm, eps=cfg.rms_norm_eps, resid=resid, out=x2, **o_parts)
            else:
                norm.add_rmsnorm(weight=lw.post_attn_norm, eps=cfg.rms_norm_eps, resid=resid, out=x2,
                                 want_local=False, **tgt, **o_parts)
            parts = self.port.run(l, x2, rows, mode)
        self._parts = parts

    def _head(self, rows: int, n_sel: int, sel_idx: torch.Tensor | None) -> None:
        """Final norm, row selection, LM head, greedy sampling into ``self.tokens[:n_sel]``."""
        cfg = self.cfg
        norm.add_rmsnorm(weight=self.w.final_norm, eps=cfg.rms_norm_eps, resid=self.resid[:rows], out=self.x[:rows],
                         **_parts_kw(self._parts),
                         **self.port.wait_args())
        if sel_idx is None:
            hsel = self.x[:n_sel]
        else:
            hsel = A.embedding(sel_idx, self.x[:rows], out=self.sel[:n_sel])
        gemm.linear(hsel, self.w.lm_head, out=self.logits[:n_sel])
        if self.ecfg.sampling:
            A.sample(self.logits[:n_sel], self.samp_temps[:n_sel], self.samp_seeds[:n_sel], out=self.tokens[:n_sel])
        else:
            A.argmax(self.logits[:n_sel], out=self.tokens[:n_sel])

    def _decode_forward(self, B: int) -> None:
        cfg = self.cfg
        ids, pos, slots, lens, table = self._dec_views(B)
        A.embedding(ids, self.w.embed, out=self.resid[:B])
        splits, chunk = A.decode_plan(B, cfg.num_kv_heads, self.ecfg.max_seq_len)

        def attn(l, lw, rows):
            A.rope_kv_write(self.qkv[:rows], self.q[:rows], self.kv.k[l], self.kv.v[l], pos, slots,
                            q_heads=cfg.num_q_heads, kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            theta=cfg.rope_theta, q_norm=lw.q_norm, k_norm=lw.k_norm, eps=cfg.rms_norm_eps)
            A.paged_decode(self.q[:rows], self.kv.k[l], self.kv.v[l], table, lens, out=self.attn_out[:rows],
                           num_splits=splits, ws=self.attn_ws, chunk_tokens=chunk)

        self._layers(B, MODE_DECODE, attn)
        self._head(B, B, None)

    def _prefill_forward(self, rows: int, n_seqs: int, max_q: int) -> None:
        cfg, P, S = self.cfg, self.ecfg.prefill_chunk, self.ecfg.max_prefill_seqs
        m = self.pre_meta
        ids, pos, slots = m[0:rows], m[P:P + rows], m[2 * P:2 * P + rows]
        b = 3 * P
        q_starts, q_lens, ctx_lens, last_idx = (m[b:b + n_seqs], m[b + S:b + S + n_seqs],
                                                m[b + 2 * S:b + 2 * S + n_seqs], m[b + 3 * S:b + 3 * S + n_seqs])
        table = m[b + 4 * S:b + 4 * S + n_seqs * self.max_blocks].view(n_seqs, self.max_blocks)
        A.embedding(ids, self.w.embed, out=self.resid[:rows])

        def attn(l, lw, r):
            A.rope_kv_write(self.qkv[:r], self.q[:r], self.kv.k[l], self.kv.v[l], pos, slots,
                            q_heads=cfg.num_q_heads, kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                            theta=cfg.rope_theta, q_norm=lw.q_norm, k_norm=lw.k_norm, eps=cfg.rms_norm_eps)
            A.paged_prefill(self.q[:r], self.kv.k[l], self.kv.v[l], table, q_starts, q_lens, ctx_lens, max_q,
                            out=self.attn_out[:r])

        self._layers(rows, MODE_PREFILL, attn)
        self._head(rows, n_seqs, last_idx)

    # ------------------------------------------------------------------ stepping
    def _bucket(self, n: int) -> int:
        for b in self._buckets:
            if b >= n:
                return b
        return self._buckets[-1]

    def warmup(self) -> None:
        """Runs every decode bucket once eagerly (allocates scratch) and captures its CUDA graph."""
        with torch.cuda.stream(self.stream):
            self.dec_meta_host.zero_()
            hv = self.dec_meta_host.numpy()
            hv[2 * self.ecfg.max_batch:3 * self.ecfg.max_batch] = -1  # no KV writes for padding rows
            self.dec_meta.copy_(self.dec_meta_host, non_blocking=True)
            # First contact with the FFN ranks (kernel loading on both sides, first touch of peer mappings, Lane
            # threads reaching their first replay) gets a generous wait limit; every later wait keeps the normal one.
            relax = getattr(self.port, "set_wait_limit", None)
            normal = getattr(self.port, "wait_ns", None)
            if relax is not None and normal is not None:
                relax(max(normal, FIRST_CONTACT_WAIT_NS))
            self._announce(self._buckets[0], MODE_DECODE)
            self._decode_forward(self._buckets[0])
            self.stream.synchronize()
            if relax is not None and normal is not None:
                relax(normal)
            for B in self._buckets:
                self._announce(B, MODE_DECODE)
                self._decode_forward(B)
            self.stream.synchronize()
            gemm.check_status(self.device)
            if self.ecfg.use_cuda_graph:
                for B in self._buckets:
                    self._capture_decode(B)
            self.stream.synchronize()

    def _announce(self, rows: int, mode: int) -> None:
        hook = getattr(self.port, "announce_forward", None)
        if hook is not None:
            hook(rows, mode)

    def _capture_decode(self, B: int) -> None:
        """Captures the decode step of one row bucket (on ``self.stream``, which is current)."""
        from .. import native

        g = torch.cuda.CUDAGraph()
        before = native.launch_count()
        with torch.cuda.graph(g, stream=self.stream):
            self._decode_forward(B)
        self._graph_launches[B] = native.launch_count() - before
        self._graphs[B] = g

    def _replay_decode(self, B: int) -> None:
        """One decode step of bucket ``B``: the captured graph, or the eager launches when graphs are off."""
        self._announce(B, MODE_DECODE)
        g = self._graphs.get(B)
        if g is not None:
            g.replay()
        else:
            self._decode_forward(B)

    def _admit_prefill(self) -> tuple[list[tuple[Sequence, int]], int]:
        """Chooses the sequences (and token counts) of the next prefill chunk."""
        e = self.ecfg
        budget, chosen = e.prefill_chunk, []
        for s in list(self.prefilling):
            if budget <= 0 or len(chosen) >= e.max_prefill_seqs:
                break
            n = min(s.fill_len - s.computed, budget)
            if n <= 0:
                continue
            chosen.append((s, n))
            budget -= n
        while self.waiting and budget > 0 and len(chosen) < e.max_prefill_seqs:
            if len(self.running) + len(self.prefilling) >= e.max_batch:
                break
            s = self.waiting[0]
            shared = self.prefix.match(s.prompt) if self.prefix is not None else []
            need = (s.fill_len + 1 + e.page_size - 1) // e.page_size - len(shared)
            if need > self.kv.allocator.free_pages and self.prefix is not None:
                freed = self.prefix.evict(need - self.kv.allocator.free_pages)
                self.kv.allocator.free(freed)
            if need > self.kv.allocator.free_pages:
                if self.prefix is not None:
                    self.prefix.release(shared)
                self._publish_demand(need - self.kv.allocator.free_pages, s)
                break
            self._publish_demand(0, None)
            self.waiting.popleft()
            if shared:
                self.kv.tables[s.seq_id] = list(shared)   # read-only prefix pages come first
                s.computed = len(shared) * e.page_size
                s.shared_pages = list(shared)
            self.kv.ensure(s.seq_id, s.fill_len + 1)
            self.prefilling.append(s)
            n = min(s.fill_len - s.computed, budget)
            chosen.append((s, n))
            budget -= n
        return chosen, e.prefill_chunk - budget

    def _step_prefill(self, chosen: list[tuple[Sequence, int]], rows: int) -> list[tuple[Sequence, int]]:
        self._launch_prefill(chosen, rows)
        return self._collect_prefill()

    @staticmethod
    def _fill_chunk_rows(hv, P: int, r: int, s: Sequence, n: int, table: list[int], ps: int) -> None:
        """Token ids, positions and KV slots of ``n`` chunk rows of sequence ``s`` starting at row ``r`` of the pinned
        prefill metadata (three regions of ``P`` words). Vectorised: a 4096-token chunk is three array operations, not
        8192 interpreter iterations."""
        import numpy as np

        hv[r:r + n] = s.fill_tokens(s.computed, n)
        pos = np.arange(s.computed, s.computed + n, dtype=np.int64)
        hv[P + r:P + r + n] = pos
        first, last = s.computed // ps, (s.computed + n - 1) // ps
        pages = np.asarray(table[first:last + 1], dtype=np.int64)
        hv[2 * P + r:2 * P + r + n] = pages[pos // ps - first] * ps + pos % ps

    def _launch_prefill(self, chosen: list[tuple[Sequence, int]], rows: int) -> None:
        """Fills the chunk's pinned metadata and enqueues the chunk; ``_collect_prefill`` finishes it."""
        e, P, S = self.ecfg, self.ecfg.prefill_chunk, self.ecfg.max_prefill_seqs
        hv = self.pre_meta_host.numpy()
        b = 3 * P
        r = 0
        ps = e.page_size
        for i, (s, n) in enumerate(chosen):
            self._fill_chunk_rows(hv, P, r, s, n, self.kv.tables[s.seq_id], ps)
            t = self.kv.tables[s.seq_id]
            hv[b + i] = r
            hv[b + S + i] = n
            hv[b + 2 * S + i] = s.computed
            hv[b + 3 * S + i] = r + n - 1
            tb = b + 4 * S + i * self.max_blocks
            hv[tb:tb + len(t)] = t
            r += n
        with torch.cuda.stream(self.stream):
            self.pre_meta.copy_(self.pre_meta_host, non_blocking=True)
            self._stage_sampling([s for s, _ in chosen])
            self._announce(rows, MODE_PREFILL)
            self._prefill_forward(rows, len(chosen), max(n for _, n in chosen))
            self.tokens_host[:len(chosen)].copy_(self.tokens[:len(chosen)], non_blocking=True)
            self._step_event.record(self.stream)
        self._pre_inflight = chosen
        self.stats["prefill_steps"] += 1
        self.stats["h2d_bytes"] += self._pre_words * 4
        self.stats["d2h_bytes"] += len(chosen) * 4

    def _collect_prefill(self) -> list[tuple[Sequence, int]]:
        """Finishes the prefill chunk in flight: waits for its sampled tokens and does the bookkeeping."""
        chosen, self._pre_inflight = self._pre_inflight, None
        self._step_event.synchronize()
        now = time.monotonic()
        out = []
        th = self.tokens_host.numpy()
        for i, (s, n) in enumerate(chosen):
            s.computed += n
            if s.prefill_done:
                if self.prefix is not None:
                    # full prompt pages become shareable; the sequence keeps them pinned while it runs
                    taken = self.prefix.insert(s.prompt, self.kv.tables[s.seq_id])
                    s.shared_pages = list(getattr(s, "shared_pages", [])) + taken
                tok = int(th[i])
                s.generated.append(tok)
                if s.first_token_time is None:
                    s.first_token_time = now   # a re-prefill after a retraction is not a first token
                s.token_times.append(now)
                self.prefilling.remove(s)
                out.append((s, tok))
                if s.finished:
                    self._finish(s, now)
                else:
                    self.running.append(s)
        return out

    def _release_pages(self, s: Sequence) -> None:
        """Returns the sequence's private pages to the allocator; pages of the prefix cache are only unpinned."""
        shared = getattr(s, "shared_pages", None)
        if self.prefix is not None and shared:
            keep = set(shared)
            t = self.kv.tables.pop(s.seq_id, [])
            self.kv.allocator.free([p for p in t if p not in keep])
            self.prefix.release(shared)
            s.shared_pages = []
        else:
            self.kv.release(s.seq_id)

    def _finish(self, s: Sequence, now: float) -> None:
        s.finish_time = now
        self._release_pages(s)

    def _decode_prepare(self) -> tuple[list[Sequence], int] | None:
        """Fills the pinned decode metadata for the next step. When the batch membership did not
        change since the previous step only the per-token fields advance (vectorised); the block
        table gets a new entry only for sequences that cross into a fresh page."""
        import numpy as np

        e = self.ecfg
        cap, ps = e.max_batch, e.page_size
        hv = self.dec_meta_host.numpy()
        batch = self.running[:e.max_batch]
        key = tuple(s.seq_id for s in batch)
        if key and key == self._b_key:
            n = len(batch)
            pos = self._b_pos
            pos += 1
            for i in np.nonzero(pos % ps == 0)[0]:
                s = batch[int(i)]
                try:
                    t = self.kv.ensure(s.seq_id, int(pos[i]) + 1)
                except OutOfPages:
                    self._b_key = None
                    self._retract(s)
                    return self._decode_prepare()
                hv[4 * cap + int(i) * self.max_blocks + int(pos[i]) // ps] = t[-1]
            B = self._bucket(n)
            table = hv[4 * cap:4 * cap + n * self.max_blocks].reshape(n, self.max_blocks)
            hv[0:n] = self._b_last
            hv[cap:cap + n] = pos
            hv[2 * cap:2 * cap + n] = table[np.arange(n), pos // ps] * ps + pos % ps
            hv[3 * cap:3 * cap + n] = pos + 1
            return batch, B
        # slow path: membership changed
        kept = []
        for s in batch:
            try:
                self.kv.ensure(s.seq_id, s.total_len)
                kept.append(s)
            except OutOfPages:
                self._retract(s)
        batch = kept
        n = len(batch)
        if n == 0:
            self._b_key = None
            return None
        B = self._bucket(n)
        hv[0:B] = 0
        hv[cap:cap + B] = 0
        hv[2 * cap:2 * cap + B] = -1
        hv[3 * cap:3 * cap + B] = 0
        pos = np.empty(n, dtype=np.int32)
        for i, s in enumerate(batch):
            p = s.total_len - 1  # position of the token fed in
            t = self.kv.tables[s.seq_id]
            pos[i] = p
            hv[i] = s.generated[-1]
            hv[cap + i] = p
            hv[2 * cap + i] = t[p // ps] * ps + p % ps
            hv[3 * cap + i] = p + 1
            tb = 4 * cap + i * self.max_blocks
            hv[tb:tb + len(t)] = t
        self._b_key = tuple(s.seq_id for s in batch)
        self._b_pos = pos
        return batch, B

    def _decode_launch(self) -> bool:
        prep = self._decode_prepare()
        if prep is None:
            return False
        batch, B = prep
        n = len(batch)
        with torch.cuda.stream(self.stream):
            self.dec_meta.copy_(self.dec_meta_host, non_blocking=True)
            self._stage_sampling(batch)
            self._replay_decode(B)
            self.tokens_host[:n].copy_(self.tokens[:n], non_blocking=True)
            self._step_event.record(self.stream)
        self._inflight = (batch, n)
        self.stats["decode_steps"] += 1
        self.stats["h2d_bytes"] += self._dec_words * 4
        self.stats["d2h_bytes"] += n * 4
        self.stats["launches"] += self._graph_launches.get(B, 0)
        return True

    def _decode_collect(self) -> list[tuple[Sequence, int]]:
        batch, n = self._inflight
        self._inflight = None
        self.stream.synchronize()
        now = time.monotonic()
        toks = self.tokens_host[:n].numpy().copy()
        self._b_last = toks
        out = []
        changed = False
        for s, tok in zip(batch, toks.tolist()):
            s.computed = s.total_len
            s.generated.append(tok)
            s.token_times.append(now)
            out.append((s, tok))
            if len(s.generated) >= s.max_new_tokens:
                self.running.remove(s)
                self._finish(s, now)
                changed = True
        if changed:
            self._b_key = None
        return out

    def _step_decode(self) -> list[tuple[Sequence, int]]:
        return self._decode_collect() if self._decode_launch() else []

    def _retract(self, s: Sequence) -> None:
        """Gives the sequence's pages back and queues it for recomputation. The emitted tokens stay in
        ``generated`` (readers of the sequence keep seeing all of them); the prefill phase recomputes the KV of
        prompt + generated and its sampled token continues the same output stream."""
        self.running.remove(s)
        self._b_key = None  # the cached decode batch no longer matches
        self._release_pages(s)
        s.refill_len = s.total_len
        s.computed = 0
        self.waiting.appendleft(s)

    def launch_step(self) -> None:
        """Starts one engine iteration (a prefill chunk or a decode step) without waiting for the
        GPU, so that a driver of several co-located Instances can overlap them; ``collect_step``
        finishes it and ``step_ready`` tells whether it would block."""
        self._pending: list[tuple[Sequence, int]] | None = None
        if self.capacity is not None:
            self._capacity_tick()
        begin = getattr(self.port, "begin_step", None)
        if begin is not None:
            with torch.cuda.stream(self.stream):
                begin()
        want_prefill = bool(self.waiting or self.prefilling)
        if want_prefill and (not self.running or not self._last_was_prefill):
            chosen, rows = self._admit_prefill()
            if chosen:
                self._last_was_prefill = True
                self._b_key = None
                with nvtx.range(f"{self.cfg.name} prefill {rows}"):
                    self._launch_prefill(chosen, rows)
                return
        self._last_was_prefill = False
        if self.running:
            with nvtx.range(f"{self.cfg.name} decode {len(self.running)}"):
                if not self._decode_launch():
                    self._pending = []

    @property
    def step_in_flight(self) -> bool:
        return self._pending is not None or self._pre_inflight is not None or self._inflight is not None

    @property
    def step_is_device_work(self) -> bool:
        """False when the step in flight put nothing on the GPU (nothing could be admitted, e.g. while the Instance
        waits for KV capacity): a driver should not spin on such steps."""
        return self._pre_inflight is not None or self._inflight is not None or bool(self._pending)

    def step_ready(self) -> bool:
        """Whether ``collect_step`` would return without waiting for the GPU (a driver of several co-located
        Instances polls this so that a long prefill chunk of one does not hold back the steps of the others)."""
        if self._pending is not None:
            return True
        if self._pre_inflight is not None or self._inflight is not None:
            return self._step_event.query()
        return True

    def collect_step(self) -> list[tuple[Sequence, int]]:
        if self._pending is not None:
            out, self._pending = self._pending, None
            return out
        if self._pre_inflight is not None:
            return self._collect_prefill()
        if self._inflight is not None:
            return self._decode_collect()
        return []

    def step(self) -> list[tuple[Sequence, int]]:
        """One engine iteration. Returns the (sequence, token) pairs it produced."""
        self.launch_step()
        return self.collect_step()

    def generate(self, prompts: list[list[int]], max_new_tokens: int) -> list[list[int]]:
        """Convenience: run the given prompts to completion, return generated ids per prompt."""
        seqs = [self.add_request(p, max_new_tokens) for p in prompts]
        while self.has_work:
            self.step()
        return [s.generated for s in seqs]
