"""CPU plumbing deployment: attention role and FFN role as separate processes.

The attention process owns embedding, attention, norms, KV and the LM head; every decoder FFN runs
in another process that only ever loaded the FFN tensors. Hidden states cross through a Transport
arena in POSIX shared memory driven by the native mailbox state machine (claim → stage → publish →
evaluate → acknowledge), exactly the protocol the GPU data plane speaks, with CPU threads in place of
kernels. It exists to prove the plumbing: the logits must equal the monolithic forward.
"""

from __future__ import annotations

import ctypes
import multiprocessing as mp
import os
from dataclasses import dataclass

import torch

from ..models import config as model_config
from ..models.reference import ReferenceModel, ffn_forward
from ..models.weights import random_attention_weights, random_ffn_weights
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
