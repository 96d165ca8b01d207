"""An engine process of its own around a ``transformers`` model: one Instance rank that serves ``POST /generate``.

    xpool --config deployment.toml daemon serve &
    xpool --config deployment.toml ffnagent --device 1 --backend cpu &
    xpool --config deployment.toml atnagent --device 0 --backend cpu &      # brokers the arena of the external rank
    XPOOL_CONFIG=deployment.toml python -m crosspool_b200.integrations.transformers.serve --model-id acme/model --port 30100

The deployment marks the model ``external = true``. The process loads the model from the model's configured path,
joins the deployment as the model's Instance rank (``instance.py::ExternalInstance``), keeps attention, KV cache and
sampling (the library's own ``generate``, greedy), and sends every decoder FFN to the FFN tier. It is the stand-in for
a serving engine with the plugin and serves any architecture the library implements, including the attention forms the
GPU attention engine of this repository does not compute. Requests are handled one at a time.
"""

from __future__ import annotations

import argparse
import json
import signal
import sys
import threading
from typing import Optional

from pydantic import BaseModel


class GenerateRequest(BaseModel):
    model: Optional[str] = None
    input_ids: Optional[list[int]] = None
    text: Optional[str] = None
    max_new_tokens: int = 16
    stream: bool = False


def build_app(model, tokenizer, model_id: str, instance):
    import torch
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import StreamingResponse

    app = FastAPI(title="xpool external instance")
    lock = threading.Lock()
    device = next(model.parameters()).device
    vocab = int(model.config.vocab_size)

    @app.get("/health")
    def health():
        return {"status": "ok", "models": [model_id], "ffn_calls": instance.ffn_calls, "state": instance.runtime.state}

    @app.post("/generate")
    def generate(req: GenerateRequest):
        if req.model not in (None, model_id):
            raise HTTPException(status_code=404, detail=f"model {req.model} is not served here")
        ids = req.input_ids
        if ids is None:
            if req.text is None or tokenizer is None:
                raise HTTPException(status_code=422, detail="input_ids required (no tokenizer configured)")
            ids = tokenizer.encode(req.text)
        if not ids or req.max_new_tokens < 1 or min(ids) < 0 or max(ids) >= vocab:
            raise HTTPException(status_code=422, detail="empty prompt, token id outside the vocabulary or max_new_tokens < 1")
        with lock, torch.no_grad():
            out = model.generate(torch.tensor([ids], device=device), max_new_tokens=req.max_new_tokens, do_sample=False)[0, len(ids):].tolist()
        if req.stream:
            def sse():
                for i, tok in enumerate(out):
                    yield f"data: {json.dumps({'token_id': tok, 'index': i + 1, 'finished': i + 1 == len(out)})}\n\n"
                yield "data: [DONE]\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")
        return {"output_ids": out, "text": tokenizer.decode(out) if tokenizer else None}

    return app


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.integrations.transformers.serve")
    ap.add_argument("--config", default=None, help="deployment TOML (default: XPOOL_CONFIG)")
    ap.add_argument("--model-id", required=True)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, required=True)
    ap.add_argument("--device", default="cpu", help="cpu, or cuda:N next to GPU agents")
    ns = ap.parse_args(argv)

    import torch
    import transformers
    import uvicorn

    from ... import config as C
    from ...runtime.serving import load_tokenizers
    from .instance import ExternalInstance

    cfg = C.load_config({"config": ns.config} if ns.config else None)
    path = cfg.model_path(ns.model_id)
    if path is None:
        print(f"serve: model {ns.model_id} has no checkpoint path (presets have no files)", file=sys.stderr)
        return 2
    on_gpu = ns.device != "cpu"
    model = transformers.AutoModelForCausalLM.from_pretrained(str(path), local_files_only=True,
                                                              torch_dtype=torch.bfloat16 if on_gpu else torch.float32).to(ns.device).eval()
    inst = ExternalInstance(cfg, ns.model_id, ns.rank)
    rep = inst.join(model, listener=(ns.host, ns.port))
    print(f"serve: {ns.model_id} rank {ns.rank} joined generation {inst.runtime.generation}; {len(rep.shims)} FFN layers on the tier",
          file=sys.stderr, flush=True)
    tok = load_tokenizers({ns.model_id: str(path)}).get(ns.model_id)
    server = uvicorn.Server(uvicorn.Config(build_app(model, tok, ns.model_id, inst), host=ns.host, port=ns.port, log_level="warning"))
    signal.signal(signal.SIGTERM, lambda *_: setattr(server, "should_exit", True))
    try:
        server.run()
    finally:
        ok = inst.leave()
        print(f"serve: left the deployment ({'clean' if ok else 'unconfirmed'})", file=sys.stderr, flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
