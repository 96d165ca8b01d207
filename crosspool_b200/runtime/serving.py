"""Request serving for the Instances hosted by one attention process.

``EngineLoop`` owns the :class:`Deployment` on a dedicated thread: it drains newly submitted requests
into the engines, steps every Instance, and hands each produced token to the request's queue.
``create_serving_app`` exposes it over HTTP: ``POST /generate`` with ``input_ids`` (or ``text`` when a
tokenizer is configured), ``max_new_tokens`` and ``stream``; streaming answers are server-sent events,
one per token, in the shape the reference's benchmark client consumes from SGLang
(``/generate`` with ``stream: true``, src/xpool-dev/xbench/harness/serving/api.py:61-80).
"""

from __future__ import annotations

import asyncio
import json
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Optional, Protocol

from pydantic import BaseModel


class SteppedDeployment(Protocol):
    def add_request(self, model_id: str, prompt: list[int], max_new_tokens: int, arrival: float | None = None): ...
    def step(self): ...
    @property
    def has_work(self) -> bool: ...


@dataclass
class Pending:
    model_id: str
    prompt: list[int]
    max_new_tokens: int
    arrival: float
    temperature: float = 0.0
    seed: int = 0
    out: "queue.Queue[tuple[int, bool] | Exception] | None" = field(default_factory=queue.Queue)
    # set by an asyncio consumer: tokens are then also handed to its event loop, so that it never has to poll
    aio_loop: object = None
    aio_queue: object = None
    tag: object = None   # opaque to the loop; an in-process consumer (``EngineLoop.sink``) finds its own record here

    def deliver(self, item) -> None:
        if self.out is not None:
            self.out.put(item)
        if self.aio_loop is not None:
            self.aio_loop.call_soon_threadsafe(self.aio_queue.put_nowait, item)


def deliver_batch(batch: list[tuple[Pending, object]]) -> None:
    """Hands one engine step's tokens to their consumers: one wake-up of the event loop per step, not per token."""
    by_loop: dict = {}
    for p, item in batch:
        if p.out is not None:
            p.out.put(item)
        if p.aio_loop is not None:
            by_loop.setdefault(p.aio_loop, []).append((p.aio_queue, item))
    for loop, items in by_loop.items():
        loop.call_soon_threadsafe(_fan_out, items)


def _fan_out(items) -> None:
    for q, item in items:
        q.put_nowait(item)


class EngineLoop:
    """``sink``: an in-process consumer called on the loop thread once per engine step with that step's
    ``[(Pending, (token, finished))]`` and a ``time.perf_counter()`` stamp taken after the step's tokens reached the
    host; requests submitted with ``queued=False`` are delivered to it alone (no per-request queue)."""

    def __init__(self, deployment: SteppedDeployment, idle_sleep: float = 0.0005, sink=None):
        self.dep = deployment
        self.sink = sink
        self._calls: "queue.Queue" = queue.Queue()
        self._inbox: "queue.Queue[Pending]" = queue.Queue()
        self._by_seq: dict[int, Pending] = {}
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self.idle_sleep = idle_sleep
        # a deployment of several co-located Instances is stepped event-driven (each Instance as soon as its own step
        # has finished) when it offers that; otherwise in lockstep
        self._step = getattr(deployment, "step_async", None) or deployment.step
        self.error: Exception | None = None
        self.steps = 0
        self.tokens = 0
        self.metrics = None      # runtime/metrics.py::InstanceMetrics once an HTTP endpoint serves GET /metrics

    def submit(self, model_id: str, prompt: list[int], max_new_tokens: int, temperature: float = 0.0, seed: int = 0,
               aio: bool = False, queued: bool = True, tag: object = None) -> Pending:
        """``aio``: called from a running event loop that will ``await p.aio_queue.get()``."""
        p = Pending(model_id, prompt, max_new_tokens, time.monotonic(), temperature, seed, tag=tag)
        if not queued:
            p.out = None
        if aio:
            p.aio_loop, p.aio_queue = asyncio.get_running_loop(), asyncio.Queue()
        self._inbox.put(p)
        return p

    def _admit(self) -> None:
        while True:
            try:
                p = self._inbox.get_nowait()
            except queue.Empty:
                return
            try:
                kw = {"temperature": p.temperature, "seed": p.seed} if p.temperature > 0 else {}
                seq = self.dep.add_request(p.model_id, p.prompt, p.max_new_tokens, arrival=p.arrival, **kw)
                self._by_seq[(p.model_id, seq.seq_id)] = p
            except Exception as e:  # bad request: answer it, keep serving
                p.deliver(e)

    def call_between_steps(self, fn) -> None:
        """Runs ``fn()`` on the loop thread between two of its iterations (a benchmark records its window boundaries
        this way). With event-driven stepping an Instance's step may be in flight at that moment; its tokens count
        when they are collected."""
        self._calls.put(fn)

    def _run_calls(self) -> None:
        while True:
            try:
                fn = self._calls.get_nowait()
            except queue.Empty:
                return
            fn()

    def _idle(self) -> None:
        tick = getattr(self.dep, "idle_tick", None)
        if tick is not None:
            tick()          # idle Instances still answer elastic-KV capacity commands
        time.sleep(self.idle_sleep)

    def _run(self) -> None:
        try:
            while not self._stop.is_set():
                self._run_calls()
                self._admit()
                if not self.dep.has_work:
                    self._idle()
                    continue
                res = self._step()
                self.steps += 1
                batch: list[tuple[Pending, tuple[int, bool]]] = []
                for model_id, pairs in res.tokens.items():
                    for seq, tok in pairs:
                        p = self._by_seq.get((model_id, seq.seq_id))
                        if p is None:
                            continue
                        done = seq.finished
                        batch.append((p, (tok, done)))
                        self.tokens += 1
                        if done:
                            del self._by_seq[(model_id, seq.seq_id)]
                            if self.metrics is not None:
                                try:
                                    self.metrics.finished(model_id, seq)
                                except Exception:      # a statistic must never stop the serving loop
                                    pass
                if self.sink is not None:
                    self.sink(batch, time.perf_counter())
                deliver_batch(batch)
        except Exception as e:  # device failure: fail every waiting request, stop (fail-stop)
            self.error = e
            for p in self._by_seq.values():
                p.deliver(e)

    def start(self) -> None:
        self._thread = threading.Thread(target=self._run, daemon=True, name="engine-loop")
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread:
            self._thread.join(30)


class GenerateRequest(BaseModel):
    model: Optional[str] = None
    input_ids: Optional[list[int]] = None
    text: Optional[str] = None
    max_new_tokens: int = 16
    stream: bool = False
    temperature: float = 0.0
    seed: int = 0


def load_tokenizers(checkpoints: dict[str, str | None]) -> dict:
    """Tokenizers of the models whose checkpoint directory ships one (``tokenizer.json`` or ``tokenizer_config.json``),
    through ``transformers.AutoTokenizer``; models without one (presets, weights-only directories) are served by token
    ids only. A tokenizer that fails to load is skipped with a warning: text is a convenience of this endpoint, not a
    reason to refuse serving."""
    import os

    out: dict = {}
    for model_id, path in checkpoints.items():
        if not path or not any(os.path.exists(os.path.join(path, f)) for f in ("tokenizer.json", "tokenizer_config.json")):
            continue
        try:
            from transformers import AutoTokenizer

            out[model_id] = AutoTokenizer.from_pretrained(path, local_files_only=True)
        except Exception as e:       # pragma: no cover - depends on the files found
            from ..logging import get_logger, kv

            get_logger().warning(kv(event="tokenizer_skipped", model=model_id, error=repr(e)[:200]))
    return out


def create_serving_app(loop: EngineLoop, models: list[str], tokenizer=None):
    """``tokenizer``: one tokenizer for every model, or ``{model id: tokenizer}`` (see :func:`load_tokenizers`)."""
    def tok_for(model: str):
        return tokenizer.get(model) if isinstance(tokenizer, dict) else tokenizer

    from fastapi import FastAPI, HTTPException
    from fastapi.responses import StreamingResponse

    from fastapi.responses import PlainTextResponse

    from .metrics import InstanceMetrics

    app = FastAPI(title="xpool instance")
    if loop is not None and loop.metrics is None:
        loop.metrics = InstanceMetrics()

    @app.get("/metrics", response_class=PlainTextResponse)
    def metrics():
        m = loop.metrics if loop is not None else None
        return (m or InstanceMetrics()).render(loop)

    @app.get("/health")
    def health():
        if loop.error is not None:
            raise HTTPException(status_code=503, detail=repr(loop.error))
        return {"status": "ok", "models": models, "steps": loop.steps, "tokens": loop.tokens}

    async def _next(p: Pending):
        return await p.aio_queue.get()

    @app.post("/generate")
    async def generate(req: GenerateRequest):
        model = req.model or models[0]
        if model not in models:
            raise HTTPException(status_code=404, detail=f"model {model} is not served here")
        ids = req.input_ids
        tok_model = tok_for(model)
        if ids is None:
            if req.text is None or tok_model is None:
                raise HTTPException(status_code=422, detail="input_ids required (no tokenizer configured)")
            ids = tok_model.encode(req.text)
        p = loop.submit(model, list(ids), req.max_new_tokens, req.temperature, req.seed, aio=True)
        if req.stream:
            async def sse():
                n = 0
                while True:
                    item = await _next(p)
                    if isinstance(item, Exception):
                        yield f"data: {json.dumps({'error': str(item)})}\n\n"
                        break
                    tok, done = item
                    n += 1
                    yield f"data: {json.dumps({'token_id': tok, 'index': n, 'finished': done})}\n\n"
                    if done:
                        break
                yield "data: [DONE]\n\n"

            return StreamingResponse(sse(), media_type="text/event-stream")
        out = []
        while True:
            item = await _next(p)
            if isinstance(item, Exception):
                raise HTTPException(status_code=422 if isinstance(item, ValueError) else 500, detail=str(item))
            out.append(item[0])
            if item[1]:
                break
        return {"output_ids": out, "text": tok_model.decode(out) if tok_model else None}

    return app
