"""CPU plumbing deployment: attention role and FFN role(s) as separate processes.

The attention process owns embedding, attention, norms, KV and the LM head; every decoder FFN runs
in another process that only ever loaded the FFN tensors. Hidden states cross through a Transport
arena in POSIX shared memory driven by the native mailbox state machine (claim → stage → publish →
evaluate → acknowledge), exactly the protocol the GPU data plane speaks, with CPU threads in place of
kernels. It exists to prove the plumbing: the logits must equal the monolithic forward.

``run_topology`` is the same with an FFN *tier*: one process per FFN rank, each holding only its tensor-parallel
shard or its range of experts and serving its own mailbox; the attention side hands every rank the same rows and
folds the partial outputs in rank order with fp32 accumulation, as the GPU Fabric does (no FFN rank waits for
another). The reference tests its topologies the same way, with one child process per PE
(src/xpool-dev/xtest/harness/native/fabric/topology.py).

Every entry point takes a preset name (random tensors) or a checkpoint directory (``config.json`` + safetensors): the
attention process then loads every tensor except the decoder FFNs, each FFN process its shard through the production
loader. Since the PyTorch oracle implements every supported attention form (rotary GQA, LayerNorm with learned
positions, sliding windows with sinks, latent attention), all architectures run disaggregated here, including the ones
the GPU attention engine does not run.
"""

from __future__ import annotations

import ctypes
import multiprocessing as mp
import os
from dataclasses import dataclass

import torch

from ..models import config as model_config
from ..models.reference import ReferenceModel, ffn_forward
from ..models.weights import random_attention_weights, random_ffn_layer
from ..native import runtime as rt


def _is_checkpoint(source: str) -> bool:
    return source not in model_config.PRESETS


def attention_side(source: str, seed: int):
    """Config and attention-side tensors of ``source``: a preset (random tensors from ``seed``) or a checkpoint
    directory (``config.json`` + safetensors; every tensor except the decoder FFNs)."""
    cfg = model_config.load(source)
    if _is_checkpoint(source):
        from ..models.weights import load_attention_from_safetensors

        return cfg, load_attention_from_safetensors(cfg, source, dtype=torch.float32)
    return cfg, random_attention_weights(cfg, seed, dtype=torch.float32)


def ffn_side(source: str, seed: int, rank: int = 0, size: int = 1, moe_parallel: str = "tp"):
    """Config and one FFN rank's share of every layer: rows ``rank`` of ``size`` of the intermediate dimension, or with
    ``moe_parallel="ep"`` its range of experts (shared experts ride with the rank that owns expert 0). A checkpoint
    directory goes through the production path: FFN description, coverage check, sharded loader."""
    cfg = model_config.load(source)
    ep = moe_parallel == "ep"
    if not _is_checkpoint(source):
        out = []
        for l in range(cfg.num_layers):
            if cfg.layer_is_moe(l) and ep:
                per = cfg.num_experts // size
                out.append(random_ffn_layer(cfg, l, seed, dtype=torch.float32, expert_range=(rank * per, (rank + 1) * per)))
            else:
                out.append(random_ffn_layer(cfg, l, seed, dtype=torch.float32, tp_rank=rank, tp_size=size))
        return cfg, out
    import json
    from pathlib import Path

    from ..models import adapters
    from . import checkpoint as ck
    from . import loader

    view = ck.read_checkpoint_key_view(source)
    spec = adapters.compile_ffn_spec(cfg.name, json.loads((Path(source) / "config.json").read_text()), view.keys())
    ck.validate_ffn_coverage(spec, view)
    out = []
    for l in range(cfg.num_layers):
        if cfg.layer_is_moe(l) and ep:
            per = cfg.num_experts // size
            w = loader.materialize_layer_weights(spec, view, l, dtype=torch.float32, experts=range(rank * per, (rank + 1) * per))
            if rank != 0:
                w.shared_gate_up = w.shared_down = None
        else:
            w = loader.materialize_layer_weights(spec, view, l, dtype=torch.float32, tp_rank=rank, tp_size=size)
        out.append(w)
    return cfg, out


def arena_view(address: int, rows: int, hidden: int) -> torch.Tensor:
    """``rows x hidden`` fp32 view of an arena's input or output region."""
    buf = (ctypes.c_float * (rows * hidden)).from_address(address)
    return torch.frombuffer(buf, dtype=torch.float32).view(rows, hidden)


def ffn_role_main(arena_name: str, preset: str, seed: int, max_rows: int, ready, idle_timeout_s: float = 30.0
                  ) -> None:
    """FFN role: serve FFN invocations from the mailbox until it is shut down or closed."""
    torch.set_num_threads(1)
    cfg, weights = ffn_side(preset, seed)
    mb = rt.CpuMailbox.attach(arena_name, max_rows, cfg.hidden_size * 4)
    mb.activate()
    ready.set()
    try:
        while True:
            rc, req = mb.take(idle_timeout_s)
            if rc != rt.WAIT_READY:
                break
            rows, layer, mode, _seq = req
            if layer >= cfg.num_layers or rows > max_rows:
                mb.complete(rt.RESULT_PROTOCOL_MISMATCH)
                break
            x = arena_view(mb.input_address, rows, cfg.hidden_size)
            y = arena_view(mb.output_address, rows, cfg.hidden_size)
            if mode == rt.MODE_IDLE:
                y.zero_()
            else:
                with torch.no_grad():
                    y.copy_(ffn_forward(x, weights[layer], cfg))
            mb.complete(rt.RESULT_OK)
    finally:
        mb.close()


@dataclass
class PlumbingResult:
    tokens: list[list[int]]
    logits: list[torch.Tensor]
    invocations: int


class RemoteFfn:
    """Attention-side shim: one blocking FFN call through the mailbox (the CPU counterpart of the
    ``ffn_shim`` op, src/xpool/ops.py)."""

    def __init__(self, mailbox: rt.CpuMailbox, hidden: int, timeout_s: float = 10.0):
        self.mb, self.hidden, self.timeout_s, self.calls = mailbox, hidden, timeout_s, 0

    def __call__(self, layer: int, x: torch.Tensor, mode: int | None = None) -> torch.Tensor:
        x = x.contiguous()
        y = torch.empty_like(x)
        mode = mode if mode is not None else (rt.MODE_DECODE if x.shape[0] == 1 else rt.MODE_PREFILL)
        rc = self.mb.submit(x.data_ptr(), y.data_ptr(), x.shape[0], layer, mode, timeout_s=self.timeout_s)
        self.calls += 1
        if rc != rt.RESULT_OK:
            raise RuntimeError(f"FFN invocation failed with result code {rc}")
        return y


def run(preset: str = "tiny-qwen3", seed: int = 0, requests: int = 8, prompt_len: int = 32, new_tokens: int = 16
        ) -> PlumbingResult:
    """Runs the acceptance workload: ``requests`` prompts of uniform random ids, greedy decoding."""
    torch.set_num_threads(1)
    cfg, attn = attention_side(preset, seed)
    max_rows = max(prompt_len, 1)
    name = f"/xpool-cpu-{os.getpid()}-{seed}"
    mb = rt.CpuMailbox.create(name, max_rows, cfg.hidden_size * 4)
    ctx = mp.get_context("spawn")
    ready = ctx.Event()
    proc = ctx.Process(target=ffn_role_main, args=(name, preset, seed, max_rows, ready), daemon=True)
    proc.start()
    try:
        if not ready.wait(120):
            raise RuntimeError("FFN role did not come up")
        if mb.wait_status(rt.MBOX_IDLE, 10.0) != rt.WAIT_READY:
            raise RuntimeError("mailbox never became idle")
        model = ReferenceModel(cfg, attn, ffn=[])
        shim = RemoteFfn(mb, cfg.hidden_size)
        gen = torch.Generator().manual_seed(seed + 12345)
        tokens, logits = [], []
        for _ in range(requests):
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen)
            t, l = model.generate(prompt, new_tokens, ffn=shim)
            tokens.append(t)
            logits.append(l)
        return PlumbingResult(tokens, logits, shim.calls)
    finally:
        mb.shutdown()
        proc.join(10)
        if proc.is_alive():
            proc.kill()
        mb.close()


def ffn_rank_main(arena_name: str, preset: str, seed: int, max_rows: int, ready, tp_rank: int, tp_size: int, moe_parallel: str,
                  idle_timeout_s: float = 30.0) -> None:
    """One rank of an FFN tier: holds its shard of every layer only (rows ``tp_rank`` of ``tp_size`` of the
    intermediate dimension, or with ``moe_parallel="ep"`` its range of experts) and answers with its partial sum."""
    torch.set_num_threads(1)
    cfg, weights = ffn_side(preset, seed, tp_rank, tp_size, moe_parallel)
    mb = rt.CpuMailbox.attach(arena_name, max_rows, cfg.hidden_size * 4)
    mb.activate()
    ready.set()
    try:
        while True:
            rc, req = mb.take(idle_timeout_s)
            if rc != rt.WAIT_READY:
                break
            rows, layer, mode, _seq = req
            if layer >= cfg.num_layers or rows > max_rows:
                mb.complete(rt.RESULT_PROTOCOL_MISMATCH)
                break
            x = arena_view(mb.input_address, rows, cfg.hidden_size)
            y = arena_view(mb.output_address, rows, cfg.hidden_size)
            if mode == rt.MODE_IDLE:
                y.zero_()
            else:
                with torch.no_grad():
                    y.copy_(ffn_forward(x, weights[layer], cfg))
            mb.complete(rt.RESULT_OK)
    finally:
        mb.close()


class RemoteFfnTier:
    """Attention-side shim of an FFN tier: every rank receives the same rows (one thread per rank drives its
    mailbox; the native calls release the interpreter lock), the partials are summed in rank order."""

    def __init__(self, mailboxes: list[rt.CpuMailbox], hidden: int, timeout_s: float = 20.0):
        self.ranks = [RemoteFfn(mb, hidden, timeout_s) for mb in mailboxes]
        self.calls = 0

    def __call__(self, layer: int, x: torch.Tensor, mode: int | None = None) -> torch.Tensor:
        import threading

        parts: list = [None] * len(self.ranks)
        errors: list = []

        def one(i):
            try:
                parts[i] = self.ranks[i](layer, x, mode)
            except Exception as e:   # surfaced on the calling thread
                errors.append(e)

        threads = [threading.Thread(target=one, args=(i,)) for i in range(len(self.ranks))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        self.calls += 1
        out = parts[0].clone()
        for p in parts[1:]:          # fixed order: the result does not depend on which rank answered first
            out += p
        return out


class FfnTierProcesses:
    """``ranks`` FFN processes, each with its own shard of ``source`` and its own mailbox; ``shim`` is the attention
    side's handle on all of them. A context manager: leaving it shuts the mailboxes down and reaps the processes."""

    def __init__(self, source: str, ranks: int = 2, moe_parallel: str = "tp", seed: int = 0, max_rows: int = 64, tag: str = "r"):
        cfg = model_config.load(source)
        if moe_parallel == "ep" and (not cfg.is_moe or cfg.num_experts % ranks):
            raise ValueError("expert parallelism needs a MoE model whose experts divide over the FFN ranks")
        self.cfg, self.source, self.ranks, self.moe_parallel, self.seed, self.max_rows = cfg, source, ranks, moe_parallel, seed, max_rows
        self.tag = tag
        self.boxes: list[rt.CpuMailbox] = []
        self.procs: list = []
        self.shim: RemoteFfnTier | None = None

    def __enter__(self) -> "FfnTierProcesses":
        ctx = mp.get_context("spawn")
        try:
            for r in range(self.ranks):
                name = f"/xpool-cpu-{os.getpid()}-{self.seed}-{self.tag}{r}"
                self.boxes.append(rt.CpuMailbox.create(name, self.max_rows, self.cfg.hidden_size * 4))
                ready = ctx.Event()
                p = ctx.Process(target=ffn_rank_main, daemon=True,
                                args=(name, self.source, self.seed, self.max_rows, ready, r, self.ranks, self.moe_parallel))
                p.start()
                self.procs.append((p, ready))
            for r, (p, ready) in enumerate(self.procs):
                if not ready.wait(120):
                    raise RuntimeError(f"FFN rank {r} did not come up")
                if self.boxes[r].wait_status(rt.MBOX_IDLE, 10.0) != rt.WAIT_READY:
                    raise RuntimeError(f"mailbox of FFN rank {r} never became idle")
        except BaseException:
            self.__exit__(None, None, None)
            raise
        self.shim = RemoteFfnTier(self.boxes, self.cfg.hidden_size)
        return self

    def __exit__(self, *exc) -> None:
        for mb in self.boxes:
            mb.shutdown()
        for p, _ in self.procs:
            p.join(10)
            if p.is_alive():
                p.kill()
        for mb in self.boxes:
            mb.close()
        self.boxes, self.procs = [], []


def run_topology(preset: str = "tiny-qwen3", ffn_ranks: int = 2, moe_parallel: str = "tp", seed: int = 0, requests: int = 4,
                 prompt_len: int = 24, new_tokens: int = 8) -> PlumbingResult:
    """One attention process (the caller) and ``ffn_ranks`` FFN processes, each with its own shard and mailbox."""
    torch.set_num_threads(1)
    cfg, attn = attention_side(preset, seed)
    with FfnTierProcesses(preset, ffn_ranks, moe_parallel, seed, max_rows=max(prompt_len, 1)) as tier:
        model = ReferenceModel(cfg, attn, ffn=[])
        gen = torch.Generator().manual_seed(seed + 12345)
        tokens, logits = [], []
        for _ in range(requests):
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen)
            t, l = model.generate(prompt, new_tokens, ffn=tier.shim)
            tokens.append(t)
            logits.append(l)
        return PlumbingResult(tokens, logits, tier.shim.calls)


def run_monolithic(preset: str = "tiny-qwen3", seed: int = 0, requests: int = 8, prompt_len: int = 32,
                   new_tokens: int = 16) -> PlumbingResult:
    torch.set_num_threads(1)
    cfg, attn = attention_side(preset, seed)
    model = ReferenceModel(cfg, attn, ffn_side(preset, seed)[1])
    gen = torch.Generator().manual_seed(seed + 12345)
    tokens, logits = [], []
    for _ in range(requests):
        prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen)
        t, l = model.generate(prompt, new_tokens)
        tokens.append(t)
        logits.append(l)
    return PlumbingResult(tokens, logits, 0)


# ------------------------------------------------------------------ data-parallel attention ranks

DP_LAYOUTS = {"packed": rt.DP_PACKED_BY_RANK, "uniform": rt.DP_UNIFORM_BY_RANK}


def dp_ffn_main(names: list[str], preset: str, seed: int, max_rows: int, ready, layout: int, stats,
                idle_timeout_s: float = 30.0) -> None:
    """FFN role of an Instance whose attention runs data-parallel: one mailbox per attention rank. Every layer call
    is a rendezvous: the role takes one invocation from every rank (in rank order), checks the row table with the
    native ``dp_inspect_rows``, evaluates the layer ONCE over the rows of all non-idle ranks and scatters the slices
    back, so a rank that has nothing to run still takes part with an Idle invocation. A table that does not add up,
    or ranks that disagree about the layer, end every rank's call with a protocol mismatch. Reference:
    src/cext/fabric/coordinator.cu:55-117 (row inspection), src/cext/fabric/executor.cu (merged evaluation)."""
    torch.set_num_threads(1)
    cfg, weights = ffn_side(preset, seed)
    hidden = cfg.hidden_size
    boxes = [rt.CpuMailbox.attach(n, max_rows, hidden * 4) for n in names]
    for mb in boxes:
        mb.activate()
    ready.set()
    try:
        while True:
            reqs = []
            for mb in boxes:
                rc, req = mb.take(idle_timeout_s)
                if rc != rt.WAIT_READY:
                    return
                reqs.append(req)
            modes = [q[2] for q in reqs]
            rows = [q[0] for q in reqs]
            layer = reqs[0][1]
            payload = sum(rows)
            table = rt.dp_inspect_rows(layout, payload, modes, rows) if len(boxes) > 1 else (modes[0], [0])
            if table is None or any(q[1] != layer for q in reqs) or layer >= cfg.num_layers:
                for mb in boxes:
                    mb.complete(rt.RESULT_PROTOCOL_MISMATCH)
                return
            merged_mode, offsets = table
            live = [r for r in range(len(boxes)) if modes[r] != rt.MODE_IDLE]
            x = torch.cat([arena_view(boxes[r].input_address, rows[r], hidden) for r in live])
            with torch.no_grad():
                y = ffn_forward(x, weights[layer], cfg)
            at = 0
            for r in live:
                arena_view(boxes[r].output_address, rows[r], hidden).copy_(y[at:at + rows[r]])
                at += rows[r]
            stats[0] += 1                                   # merged evaluations
            stats[1] += len(boxes) - len(live)              # idle participations
            stats[2] += int(merged_mode == rt.MODE_PREFILL and any(modes[r] == rt.MODE_DECODE for r in live))
            for mb in boxes:
                mb.complete(rt.RESULT_OK)
    finally:
        for mb in boxes:
            mb.close()


def _dp_attention_main(rank: int, dp: int, name: str, preset: str, seed: int, max_rows: int, requests: int, prompt_len: int,
                       new_tokens: int, layout: int, barrier, table, out_q) -> None:
    """One data-parallel attention rank: its own requests, its own KV, its own mailbox. Before every forward the
    ranks exchange (mode, rows) on the host (a serving engine gathers the same table for its batch metadata); a rank
    without work joins the layer calls with Idle invocations until every rank is done. ``table`` holds 2 words per
    rank: forward mode and row count of the coming forward (mode 0 = this rank is finished for good)."""
    torch.set_num_threads(1)
    cfg, attn = attention_side(preset, seed)
    mb = rt.CpuMailbox.attach(name, max_rows, cfg.hidden_size * 4)
    model = ReferenceModel(cfg, attn, ffn=[])
    shim = RemoteFfn(mb, cfg.hidden_size, timeout_s=30.0)
    gen = torch.Generator().manual_seed(seed + 12345 + 1000 * rank)
    hidden = cfg.hidden_size

    def rendezvous(mode: int, rows: int) -> tuple[bool, int]:
        table[2 * rank], table[2 * rank + 1] = mode, rows
        barrier.wait(60)
        snap = list(table)
        barrier.wait(60)                 # nobody overwrites the table before everyone has read it
        return all(snap[2 * r] == 0 for r in range(dp)), max(snap[2 * r + 1] for r in range(dp))

    def forward(ids, positions, cache):
        mode = rt.MODE_DECODE if ids.numel() == 1 else rt.MODE_PREFILL
        _, widest = rendezvous(mode, ids.numel())
        if layout == rt.DP_UNIFORM_BY_RANK and widest > ids.numel():
            pad = widest - ids.numel()   # uniform layout: every rank ships the widest rank's row count

            def padded(layer, x, _mode=None):
                y = shim(layer, torch.cat([x, x.new_zeros(pad, hidden)]), mode)
                return y[:x.shape[0]]
            return model.forward(ids, positions, cache, padded)
        return model.forward(ids, positions, cache, lambda layer, x: shim(layer, x, mode))

    tokens, logits = [], []
    try:
        for i in range(requests):
            n = prompt_len + 3 * ((rank + i) % 3)          # unequal lengths: prefill and decode steps interleave over ranks
            prompt = torch.randint(0, cfg.vocab_size, (n,), generator=gen)
            cache = model.new_cache()
            lg = forward(prompt, torch.arange(n), cache)[-1:]
            out, per = [], []
            for t in range(new_tokens):
                per.append(lg[-1])
                nxt = int(lg[-1].argmax())
                out.append(nxt)
                if t + 1 == new_tokens:
                    break
                lg = forward(torch.tensor([nxt]), torch.tensor([n + t]), cache)
            tokens.append(out)
            logits.append(torch.stack(per))
        while True:                                         # finished: keep the others' layer calls complete
            all_done, widest = rendezvous(0, 0)
            if all_done:
                break
            rows = widest if layout == rt.DP_UNIFORM_BY_RANK else 0
            x = torch.zeros(rows, hidden)
            for layer in range(cfg.num_layers):
                shim(layer, x, rt.MODE_IDLE)
        out_q.put((rank, tokens, [l.numpy() for l in logits], shim.calls, None))
    except Exception as e:                                  # reported to the parent, which fails the run
        barrier.abort()
        out_q.put((rank, [], [], shim.calls, repr(e)))
    finally:
        mb.close()


@dataclass
class DpPlumbingResult:
    ranks: list[PlumbingResult]       # per attention rank
    merged_evaluations: int           # layer evaluations the FFN role ran (one per rendezvous)
    idle_participations: int          # Idle invocations that took part in them
    mixed_mode_evaluations: int       # evaluations that merged a prefilling rank with a decoding one


def dp_rank_requests(rank: int, requests: int) -> int:
    """Requests of attention rank ``rank``: later ranks get one fewer each (at least one), so they finish early."""
    return max(1, requests - rank)


def dp_rank_new_tokens(rank: int, new_tokens: int) -> int:
    """Output length of rank ``rank``'s requests: one more per rank, so the ranks fall out of step and a prefill of
    one meets decode steps of another in the same rendezvous."""
    return new_tokens + rank


def run_dp_topology(preset: str = "tiny-qwen3", dp: int = 2, layout: str = "packed", seed: int = 0, requests: int = 3,
                    prompt_len: int = 12, new_tokens: int = 6) -> DpPlumbingResult:
    """``dp`` attention processes of one Instance (data parallel: different requests, same weights) and one FFN
    process that evaluates every layer once per rendezvous over all ranks' rows."""
    import queue

    cfg = model_config.load(preset)
    code = DP_LAYOUTS[layout]
    max_rows = prompt_len + 6
    ctx = mp.get_context("spawn")
    names = [f"/xpool-cpu-{os.getpid()}-{seed}-dp{r}" for r in range(dp)]
    boxes = [rt.CpuMailbox.create(n, max_rows, cfg.hidden_size * 4) for n in names]
    ready, barrier = ctx.Event(), ctx.Barrier(dp)
    table, stats = ctx.Array("i", 2 * dp, lock=False), ctx.Array("q", 3, lock=False)
    out_q = ctx.Queue()
    ffn = ctx.Process(target=dp_ffn_main, args=(names, preset, seed, max_rows, ready, code, stats), daemon=True)
    ffn.start()
    ranks = []
    try:
        if not ready.wait(120):
            raise RuntimeError("FFN role did not come up")
        for mb in boxes:
            if mb.wait_status(rt.MBOX_IDLE, 10.0) != rt.WAIT_READY:
                raise RuntimeError("a mailbox never became idle")
        for r in range(dp):
            p = ctx.Process(target=_dp_attention_main, daemon=True,
                            args=(r, dp, names[r], preset, seed, max_rows, dp_rank_requests(r, requests), prompt_len,
                                  dp_rank_new_tokens(r, new_tokens),
                                  code, barrier, table, out_q))
            p.start()
            ranks.append(p)
        got: dict[int, PlumbingResult] = {}
        for _ in range(dp):
            try:
                rank, tokens, logits, calls, err = out_q.get(timeout=300)
            except queue.Empty:
                raise RuntimeError("an attention rank did not finish") from None
            if err:
                raise RuntimeError(f"attention rank {rank} failed: {err}")
            got[rank] = PlumbingResult(tokens, [torch.from_numpy(l) for l in logits], calls)
        return DpPlumbingResult([got[r] for r in range(dp)], int(stats[0]), int(stats[1]), int(stats[2]))
    finally:
        for mb in boxes:
            mb.shutdown()
        for p in ranks + [ffn]:
            p.join(10)
            if p.is_alive():
                p.kill()
        for mb in boxes:
            mb.close()


def run_dp_monolithic(preset: str = "tiny-qwen3", dp: int = 2, seed: int = 0, requests: int = 3, prompt_len: int = 12,
                      new_tokens: int = 6) -> list[PlumbingResult]:
    """What every attention rank of ``run_dp_topology`` must produce, from one undivided model."""
    torch.set_num_threads(1)
    cfg, attn = attention_side(preset, seed)
    model = ReferenceModel(cfg, attn, ffn_side(preset, seed)[1])
    out = []
    for rank in range(dp):
        gen = torch.Generator().manual_seed(seed + 12345 + 1000 * rank)
        tokens, logits = [], []
        for i in range(dp_rank_requests(rank, requests)):
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len + 3 * ((rank + i) % 3),), generator=gen)
            t, l = model.generate(prompt, dp_rank_new_tokens(rank, new_tokens))
            tokens.append(t)
            logits.append(l)
        out.append(PlumbingResult(tokens, logits, 0))
    return out
