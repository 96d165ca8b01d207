"""Data-parallel attention front end: one HTTP endpoint per model in front of its Instance ranks.

With ``atn_dp_size > 1`` a model runs as several independent Instance ranks (own GPU, own KV cache, same
weights; the FFN tier serves each rank through its own slot). Requests are spread over the ranks'
serving listeners by least outstanding tokens (prompt + remaining output), the policy an engine's DP
controller applies (reference: SGLang ``--enable-dp-attention`` as driven by
src/xpool/integrations/sglang/server_args.py:75-110). Streaming responses are passed through unchanged.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse


@dataclass
class Backend:
    url: str
    outstanding_tokens: int = 0
    inflight: int = 0
    served: int = 0
    healthy: bool = True


@dataclass
class DpRouter:
    backends: dict[str, list[Backend]] = field(default_factory=dict)   # model -> ranks

    def register(self, model: str, url: str) -> None:
        ranks = self.backends.setdefault(model, [])
        if all(b.url != url for b in ranks):
            ranks.append(Backend(url))

    def pick(self, model: str, cost: int) -> Backend:
        ranks = [b for b in self.backends.get(model, ()) if b.healthy]
        if not ranks:
            raise LookupError(f"no healthy Instance rank serves {model}")
        b = min(ranks, key=lambda r: (r.outstanding_tokens, r.inflight, r.served))
        b.outstanding_tokens += cost
        b.inflight += 1
        return b

    def done(self, b: Backend, cost: int, ok: bool = True) -> None:
        b.outstanding_tokens -= cost
        b.inflight -= 1
        b.served += 1
        if not ok:
            b.healthy = False

    def snapshot(self) -> dict:
        return {m: [vars(b) for b in r] for m, r in self.backends.items()}


def create_router_app(router: DpRouter, transport=None):
    """FastAPI app: ``POST /generate`` (same body as an Instance's endpoint) and ``GET /ranks``."""
    import httpx

    app = FastAPI(title="xpool dp router")
    client = httpx.AsyncClient(timeout=600.0, transport=transport)

    @app.get("/ranks")
    def ranks():
        return router.snapshot()

    @app.post("/generate")
    async def generate(request: Request):
        body = await request.json()
        model = body.get("model") or next(iter(router.backends), None)
        cost = len(body.get("input_ids") or []) + int(body.get("max_new_tokens", 16))
        try:
            b = router.pick(model, cost)
        except LookupError as e:
            raise HTTPException(status_code=503, detail=str(e))
        if not body.get("stream"):
            try:
                r = await client.post(b.url + "/generate", json=body)
                router.done(b, cost, ok=r.status_code < 500)
                return JSONResponse(r.json(), status_code=r.status_code)
            except httpx.HTTPError as e:
                router.done(b, cost, ok=False)
                raise HTTPException(status_code=502, detail=f"{b.url}: {e}")

        async def relay():
            ok = True
            try:
                async with client.stream("POST", b.url + "/generate", json=body) as r:
                    async for chunk in r.aiter_bytes():
                        yield chunk
            except httpx.HTTPError as e:
                ok = False
                yield f"data: {json.dumps({'error': str(e)})}\n\ndata: [DONE]\n\n".encode()
            finally:
                router.done(b, cost, ok=ok)

        return StreamingResponse(relay(), media_type="text/event-stream")

    return app


def discover_ranks(router: DpRouter, daemon_url: str, models: list[str] | None = None, http=None) -> int:
    """Registers the serving listeners the daemon knows (``GET /instances``: every initialised Instance rank that
    published one) with ``router``; ``models`` restricts it. Returns how many ranks are registered afterwards. Ranks
    that disappeared from the daemon's table are marked unhealthy, new ones are added: call it periodically."""
    import httpx

    get = (http or httpx).get
    table = get(daemon_url.rstrip("/") + "/instances", timeout=5).json()
    seen: dict[str, set[str]] = {}
    for key, info in table.items():
        model = key.rsplit(":", 1)[0]
        if (models and model not in models) or not info.get("initialized") or not info.get("listener"):
            continue
        url = "http://" + info["listener"]
        router.register(model, url)
        seen.setdefault(model, set()).add(url)
    for model, ranks in router.backends.items():
        for b in ranks:
            if b.url in seen.get(model, ()):
                b.healthy = True
            elif not models or model in models:
                b.healthy = False
    return sum(len(v) for v in seen.values())


def serve_router(daemon_url: str, host: str, port: int, models: list[str] | None = None, refresh_s: float = 2.0) -> int:
    """``xpool router``: one endpoint in front of every data-parallel rank the daemon lists, refreshed every
    ``refresh_s`` seconds."""
    import threading

    import uvicorn

    router = DpRouter()
    stop = threading.Event()

    def refresh():
        while not stop.is_set():
            try:
                discover_ranks(router, daemon_url, models)
            except Exception:
                pass            # the daemon may be restarting: keep the ranks already known
            stop.wait(refresh_s)

    threading.Thread(target=refresh, daemon=True, name="dp-router-discovery").start()
    try:
        uvicorn.run(create_router_app(router), host=host, port=port, log_level="warning")
    finally:
        stop.set()
    return 0
