"""Try the disaggregated path with a ``transformers`` model and no GPU:

    python -m crosspool_b200.integrations.transformers --checkpoint /models/Qwen3-0.6B --ffn-ranks 2 --prompt "Hello"
    python -m crosspool_b200.integrations.transformers --checkpoint DIR --ffn-ranks 2 --moe-parallel ep --ids 1 2 3 --verify

The model is loaded from a local directory (nothing is downloaded), its decoder FFNs are detached, ``--ffn-ranks`` FFN
processes load their tensor-parallel shards (or expert ranges) of the same checkpoint through the production loader,
and the library's own ``generate`` runs attention here and every FFN over shared-memory mailboxes. ``--verify`` first
generates with the whole model and checks that the tokens are the same.
"""

from __future__ import annotations

import argparse
import sys
import time


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.integrations.transformers")
    ap.add_argument("--checkpoint", required=True, help="directory with config.json and *.safetensors")
    ap.add_argument("--ffn-ranks", type=int, default=2)
    ap.add_argument("--moe-parallel", choices=("tp", "ep"), default="tp")
    ap.add_argument("--prompt", default=None, help="text (needs the checkpoint's tokenizer)")
    ap.add_argument("--ids", type=int, nargs="*", default=None, help="token ids instead of text")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--verify", action="store_true", help="compare with the whole model's generation")
    ns = ap.parse_args(argv)

    import torch
    import transformers

    from ...engine.cpu_plumbing import FfnTierProcesses
    from . import bind_cpu_tier, detach_ffn, unbind

    torch.set_num_threads(max(1, torch.get_num_threads()))
    model = transformers.AutoModelForCausalLM.from_pretrained(ns.checkpoint, local_files_only=True, torch_dtype=torch.float32).eval()
    tok = None
    if ns.ids:
        ids = torch.tensor([ns.ids])
    else:
        if ns.prompt is None:
            ap.error("give --prompt or --ids")
        tok = transformers.AutoTokenizer.from_pretrained(ns.checkpoint, local_files_only=True)
        ids = torch.tensor([tok.encode(ns.prompt)])
    want = None
    if ns.verify:
        with torch.no_grad():
            want = model.generate(ids, max_new_tokens=ns.max_new_tokens, do_sample=False)[0, ids.shape[1]:].tolist()
    rep = detach_ffn(model)
    print(f"detached {len(rep.shims)} FFN layers: {rep.freed_parameters:,} parameters left the model, {rep.kept_parameters:,} stay",
          file=sys.stderr)
    rows = ids.shape[1] + ns.max_new_tokens
    with FfnTierProcesses(ns.checkpoint, ns.ffn_ranks, ns.moe_parallel, max_rows=max(64, rows), tag="hfdemo") as tier:
        bind_cpu_tier(tier.shim)
        try:
            t0 = time.perf_counter()
            with torch.no_grad():
                out = model.generate(ids, max_new_tokens=ns.max_new_tokens, do_sample=False)[0, ids.shape[1]:].tolist()
            dt = time.perf_counter() - t0
        finally:
            unbind()
        print(f"{len(out)} tokens in {dt:.2f} s through {tier.shim.calls} FFN invocations on {ns.ffn_ranks} ranks", file=sys.stderr)
    print(tok.decode(out) if tok is not None else " ".join(map(str, out)))
    if want is not None:
        same = out == want
        print("verify: " + ("same tokens as the whole model" if same else f"DIFFERENT from the whole model: {want}"), file=sys.stderr)
        return 0 if same else 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
