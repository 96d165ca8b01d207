"""Served-output qualification: does a deployment answer what the model's own implementation answers?

For a checkpoint directory (or the tiny configuration of an architecture, written by the ``transformers`` model class)
the tool starts a whole deployment on the CPU data plane (daemon, FFN agents that load their shards through the
production loader, an attention agent), sends prompts over ``POST /generate`` and compares the greedy tokens with the
``transformers`` model's own ``generate``. It is the per-model suite of the reference (tests/suites/models/: served
output against the stock engine's) with the library model as the stock side.

    python -m crosspool_b200.devtools.served_qualification --arch all
    python -m crosspool_b200.devtools.served_qualification --checkpoint /models/Qwen3-0.6B --ffn-ranks 2 --prompts 4
"""

from __future__ import annotations

import argparse
import json
import socket
import sys
import tempfile
from pathlib import Path


def _free_ports(n: int) -> list[int]:
    socks, out = [], []
    try:
        for _ in range(n):
            s = socket.socket()
            s.bind(("127.0.0.1", 0))
            socks.append(s)
            out.append(s.getsockname()[1])
    finally:
        for s in socks:
            s.close()
    return out


def qualify_served(checkpoint: str | Path, model=None, *, ffn_ranks: int = 2, prompts: int = 3, prompt_len: int = 12, new_tokens: int = 6,
                   seed: int = 0, model_id: str = "qualify/model") -> dict:
    """``model``: the loaded library model (default: loaded from ``checkpoint``). Returns a report with one entry per
    prompt and ``ok`` when every served answer equals the library's."""
    import httpx
    import torch
    import transformers

    from ..bench.serve_case import LocalDeployment

    if model is None:
        model = transformers.AutoModelForCausalLM.from_pretrained(str(checkpoint), local_files_only=True, torch_dtype=torch.float32).eval()
    g = torch.Generator().manual_seed(seed)
    vocab = int(model.config.vocab_size)
    cases = [torch.randint(0, vocab, (prompt_len + 2 * i,), generator=g).tolist() for i in range(prompts)]
    with torch.no_grad():
        want = [model.generate(torch.tensor([p]), max_new_tokens=new_tokens, do_sample=False)[0, len(p):].tolist() for p in cases]
    dport, sport = _free_ports(2)
    ffn = list(range(1, ffn_ranks + 1))
    rows = max(64, prompt_len + 2 * prompts + new_tokens + 8)
    toml = (f"[daemon]\nport = {dport}\n[atn]\ndevices = [0]\n[ffn]\ndevices = {ffn}\n[scheduler.slo]\nttft_ms = 2000\ntbt_ms = 50\n"
            f"[serving]\nbase_port = {sport}\n[[models]]\nid = \"{model_id}\"\npath = \"{checkpoint}\"\nffn_tp_size = {ffn_ranks}\n")
    env = {"XPOOL_MAX_ROWS": str(rows), "XPOOL_MAX_BATCH": "4", "XPOOL_MAX_SEQ_LEN": str(rows)}
    results = []
    with LocalDeployment(toml, [0], ffn, dport, env, backend="cpu", serving_port=sport) as dep:
        url = dep.targets([model_id])[model_id]
        for p, w in zip(cases, want):
            r = httpx.post(url + "/generate", json={"input_ids": p, "max_new_tokens": new_tokens}, timeout=600)
            got = r.json().get("output_ids") if r.status_code == 200 else None
            results.append({"prompt_tokens": len(p), "served": got, "library": w, "equal": got == w, "status": r.status_code})
    arch = (getattr(model.config, "architectures", None) or [type(model).__name__])[0]
    return {"architecture": arch, "checkpoint": str(checkpoint), "ffn_ranks": ffn_ranks, "ok": all(x["equal"] for x in results), "prompts": results}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.devtools.served_qualification")
    ap.add_argument("--arch", default=None, help="an architecture of the tiny configurations (or 'all'): the library writes the checkpoint")
    ap.add_argument("--checkpoint", default=None, help="a checkpoint directory to qualify as it is")
    ap.add_argument("--ffn-ranks", type=int, default=2)
    ap.add_argument("--prompts", type=int, default=3)
    ap.add_argument("--new-tokens", type=int, default=6)
    ap.add_argument("--json", action="store_true")
    ns = ap.parse_args(argv)
    if (ns.arch is None) == (ns.checkpoint is None):
        ap.error("give exactly one of --arch and --checkpoint")
    reports = []
    if ns.checkpoint:
        reports.append(qualify_served(ns.checkpoint, ffn_ranks=ns.ffn_ranks, prompts=ns.prompts, new_tokens=ns.new_tokens))
    else:
        from . import hf_parity
        from .qualification import TINY_CONFIGS

        names = [a for a in sorted(TINY_CONFIGS) if "+" not in a] + sorted(hf_parity.VARIANTS) if ns.arch == "all" else [ns.arch]
        for name in names:
            if not hf_parity.available(name):
                print(f"{name}: SKIPPED (the installed transformers has no such class)")
                continue
            with tempfile.TemporaryDirectory(prefix="xp-served-") as d:
                model = hf_parity.build_tiny_model(name)
                model.save_pretrained(d, safe_serialization=True)
                rep = qualify_served(d, model, ffn_ranks=ns.ffn_ranks, prompts=ns.prompts, new_tokens=ns.new_tokens)
                rep["configuration"] = name
                reports.append(rep)
    for rep in reports:
        if ns.json:
            print(json.dumps(rep))
        else:
            same = sum(x["equal"] for x in rep["prompts"])
            print(f"{rep.get('configuration', rep['checkpoint'])}: {'PASS' if rep['ok'] else 'FAIL'} ({same}/{len(rep['prompts'])} prompts answered as the library answers)")
    return 0 if all(r["ok"] for r in reports) else 1


if __name__ == "__main__":
    sys.exit(main())
