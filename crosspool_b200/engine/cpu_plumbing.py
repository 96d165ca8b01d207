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
"""

from __future__ import annotations

import ctypes
import multiprocessing as mp
import os
from dataclasses import dataclass

import torch

from ..models import config as model_config
from ..models.reference import ReferenceModel, ffn_forward
from ..models.weights import random_attention_weights, random_ffn_layer, random_ffn_weights
from ..native import runtime as rt


def _view(address: int, rows: int, hidden: int) -> torch.Tensor:
    buf = (ctypes.c_float * (rows * hidden)).from_address(address)
    return torch.frombuffer(buf, dtype=torch.float32).view(rows, hidden)


def ffn_role_main(arena_name: str, preset: str, seed: int, max_rows: int, ready, idle_timeout_s: float = 30.0
                  ) -> None:
    """FFN role: serve FFN invocations from the mailbox until it is shut down or closed."""
    torch.set_num_threads(1)
    cfg = model_config.preset(preset)
    weights = random_ffn_weights(cfg, seed, dtype=torch.float32)
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
            x = _view(mb.input_address, rows, cfg.hidden_size)
            y = _view(mb.output_address, rows, cfg.hidden_size)
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
    cfg = model_config.preset(preset)
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
        model = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), ffn=[])
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
    cfg = model_config.preset(preset)
    weights = []
    for l in range(cfg.num_layers):
        if cfg.layer_is_moe(l) and moe_parallel == "ep":
            per = cfg.num_experts // tp_size
            weights.append(random_ffn_layer(cfg, l, seed, dtype=torch.float32, expert_range=(tp_rank * per, (tp_rank + 1) * per)))
        else:
            weights.append(random_ffn_layer(cfg, l, seed, dtype=torch.float32, tp_rank=tp_rank, tp_size=tp_size))
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
            x = _view(mb.input_address, rows, cfg.hidden_size)
            y = _view(mb.output_address, rows, cfg.hidden_size)
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


def run_topology(preset: str = "tiny-qwen3", ffn_ranks: int = 2, moe_parallel: str = "tp", seed: int = 0, requests: int = 4,
                 prompt_len: int = 24, new_tokens: int = 8) -> PlumbingResult:
    """One attention process (the caller) and ``ffn_ranks`` FFN processes, each with its own shard and mailbox."""
    torch.set_num_threads(1)
    cfg = model_config.preset(preset)
    if moe_parallel == "ep" and (not cfg.is_moe or cfg.num_experts % ffn_ranks):
        raise ValueError("expert parallelism needs a MoE model whose experts divide over the FFN ranks")
    max_rows = max(prompt_len, 1)
    ctx = mp.get_context("spawn")
    boxes, procs = [], []
    try:
        for r in range(ffn_ranks):
            name = f"/xpool-cpu-{os.getpid()}-{seed}-r{r}"
            boxes.append(rt.CpuMailbox.create(name, max_rows, cfg.hidden_size * 4))
            ready = ctx.Event()
            p = ctx.Process(target=ffn_rank_main, args=(name, preset, seed, max_rows, ready, r, ffn_ranks, moe_parallel), daemon=True)
            p.start()
            procs.append((p, ready))
        for r, (p, ready) in enumerate(procs):
            if not ready.wait(120):
                raise RuntimeError(f"FFN rank {r} did not come up")
            if boxes[r].wait_status(rt.MBOX_IDLE, 10.0) != rt.WAIT_READY:
                raise RuntimeError(f"mailbox of FFN rank {r} never became idle")
        model = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32), ffn=[])
        shim = RemoteFfnTier(boxes, cfg.hidden_size)
        gen = torch.Generator().manual_seed(seed + 12345)
        tokens, logits = [], []
        for _ in range(requests):
            prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen)
            t, l = model.generate(prompt, new_tokens, ffn=shim)
            tokens.append(t)
            logits.append(l)
        return PlumbingResult(tokens, logits, shim.calls)
    finally:
        for mb in boxes:
            mb.shutdown()
        for p, _ in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
        for mb in boxes:
            mb.close()


def run_monolithic(preset: str = "tiny-qwen3", seed: int = 0, requests: int = 8, prompt_len: int = 32,
                   new_tokens: int = 16) -> PlumbingResult:
    torch.set_num_threads(1)
    cfg = model_config.preset(preset)
    model = ReferenceModel(cfg, random_attention_weights(cfg, seed, dtype=torch.float32),
                           random_ffn_weights(cfg, seed, dtype=torch.float32))
    gen = torch.Generator().manual_seed(seed + 12345)
    tokens, logits = [], []
    for _ in range(requests):
        prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen)
        t, l = model.generate(prompt, new_tokens)
        tokens.append(t)
        logits.append(l)
    return PlumbingResult(tokens, logits, 0)
