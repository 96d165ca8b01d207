"""Kernel microbenchmarks with roofline fractions.

``python -m crosspool_b200.bench.kernels gemm --rows 64 --n 3072 --k 1024 --dual 1``
``python -m crosspool_b200.bench.kernels decode-attn --batch 64``
``python -m crosspool_b200.bench.kernels norm --rows 256 --hidden 1024``
``python -m crosspool_b200.bench.kernels moe --rows 64``

Each case runs ``--warmup`` untimed iterations, then times ``--iters`` launches with CUDA events on
the launching stream, writing a buffer larger than L2 between launches, and prints one JSON line:
median microseconds, achieved GB/s and TFLOP/s, and the fractions of the measured copy bandwidth and
cuBLAS bf16 throughput (``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s
and 1.59 PFLOP/s, reported as "fallback"). ``--iters 1 --warmup 1 --no-flush`` gives a small
fixed-launch run suitable for a profiler.
"""

from __future__ import annotations

import argparse
import json
import random
import statistics
from pathlib import Path

import torch


def peaks() -> dict:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, iters: int, warmup: int, flush: bool):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return statistics.median(ts)


def report(name: str, us: float, bytes_moved: float, flops: float, extra: dict) -> dict:
    pk = peaks()
    gbs, tfl = bytes_moved / us / 1e3, flops / us / 1e6
    out = {"kernel": name, "us": round(us, 2), "gbs": round(gbs, 1), "tflops": round(tfl, 2),
           f"frac_hbm_of_{pk['source']}": round(gbs / pk["hbm_gbs"], 3),
           f"frac_bf16_of_{pk['source']}": round(tfl / pk["bf16_tflops"], 3), **extra}
    print(json.dumps(out), flush=True)
    return out


def bench_gemm(ns, timer: Timer) -> dict:
    from ..ops import gemm

    dev = torch.device("cuda")
    x = (torch.randn(ns.rows, ns.k, device=dev) * 0.5).bfloat16()
    w = (torch.randn(ns.n * (2 if ns.dual else 1), ns.k, device=dev) * 0.05).bfloat16()
    out = torch.empty(ns.rows, ns.n, dtype=torch.bfloat16, device=dev)
    if ns.fp8:
        # block-scaled e4m3 weights; the timed op is what a layer pays: activation quantisation + GEMM
        from ..quantization import Fp8Block

        q = Fp8Block().quantize(w[:ns.n])
        wq, wscale = q["weight"], q["scale"].contiguous()
        us = timer(lambda: gemm.linear_fp8(x, wq, wscale, out=out, splits=ns.splits, bn=ns.bn))
        gemm.check_status(dev)
        byts = wq.numel() + wscale.numel() * 4 + (x.numel() + out.numel()) * 2
        return report("gemm_ws_fp8_block", us, byts, 2.0 * ns.rows * ns.n * ns.k,
                      {"rows": ns.rows, "n": ns.n, "k": ns.k, "includes": "activation quantisation kernel"})
    wk = gemm.tile_weight(w) if ns.tiled else w      # 128 x 64 blocks stored contiguously (one 16 KB run per TMA box)
    fn = (lambda: gemm.gateup_swiglu(x, wk, out=out, splits=ns.splits, bn=ns.bn)) if ns.dual else \
        (lambda: gemm.linear(x, wk, out=out, splits=ns.splits, bn=ns.bn))
    us = timer(fn)
    gemm.check_status(dev)
    plan = gemm.plan_shape(ns.n, ns.k, ns.rows, int(ns.dual))
    byts = (w.numel() + x.numel() + out.numel()) * 2
    return report("gemm_ws" + ("_swiglu" if ns.dual else ""), us, byts, 2.0 * ns.rows * w.shape[0] * ns.k,
                  {"rows": ns.rows, "n": ns.n, "k": ns.k, "bn": ns.bn or plan["bn"], "splits": ns.splits or plan["splits"],
                   "tiled": int(ns.tiled)})


def bench_decode_attn(ns, timer: Timer) -> dict:
    from ..ops import attention as A

    B, hq, hkv, d, page = ns.batch, ns.q_heads, ns.kv_heads, ns.head_dim, 16
    rnd = random.Random(0)
    lens = [rnd.randint(ns.min_len, ns.max_len) for _ in range(B)]
    maxb = (max(lens) + page - 1) // page
    total = sum((l + page - 1) // page for l in lens) + 8
    perm = torch.randperm(total, device="cuda").int()
    table = torch.zeros(B, maxb, dtype=torch.int32, device="cuda")
    c = 0
    for b, l in enumerate(lens):
        n = (l + page - 1) // page
        table[b, :n] = perm[c:c + n]
        c += n
    kc = torch.randn(total, page, hkv, d, device="cuda").bfloat16()
    vc = torch.randn(total, page, hkv, d, device="cuda").bfloat16()
    q = torch.randn(B, hq, d, device="cuda").bfloat16()
    sl = torch.tensor(lens, device="cuda", dtype=torch.int32)
    out = torch.empty_like(q)
    splits, chunk = A.decode_plan(B, hkv, ns.max_len)
    if ns.chunk > 0:
        splits, chunk = (ns.max_len + ns.chunk - 1) // ns.chunk, ns.chunk
    ws = torch.empty(B * hq * max(splits, 1) * (d + 2), dtype=torch.float32, device="cuda")
    us = timer(lambda: A.paged_decode(q, kc, vc, table, sl, out=out, num_splits=splits, ws=ws, chunk_tokens=chunk))
    kv_bytes = sum(lens) * hkv * d * 2 * 2
    return report("paged_decode_attention", us, kv_bytes, 4.0 * sum(lens) * hq * d,
                  {"batch": B, "tokens": sum(lens), "splits": splits, "chunk_tokens": chunk})


def bench_prefill_attn(ns, timer: Timer) -> dict:
    """Causal prefill attention of ``--seqs`` prompts of ``--len`` tokens each (no cached context)."""
    from ..ops import attention as A

    S, L, hq, hkv, d, page = ns.seqs, ns.len, ns.q_heads, ns.kv_heads, ns.head_dim, ns.page
    blocks = (L + page - 1) // page
    table = torch.arange(S * blocks, dtype=torch.int32, device="cuda").view(S, blocks)
    kc = torch.randn(S * blocks, page, hkv, d, device="cuda").bfloat16()
    vc = torch.randn(S * blocks, page, hkv, d, device="cuda").bfloat16()
    q = torch.randn(S * L, hq, d, device="cuda").bfloat16()
    q_starts = (torch.arange(S, device="cuda", dtype=torch.int32) * L).contiguous()
    q_lens = torch.full((S,), L, dtype=torch.int32, device="cuda")
    ctx = torch.zeros(S, dtype=torch.int32, device="cuda")
    out = torch.empty_like(q)
    us = timer(lambda: A.paged_prefill(q, kc, vc, table, q_starts, q_lens, ctx, L, out=out, force_simple=ns.kernel))
    flops = 4.0 * S * (L * (L + 1) / 2) * hq * d          # QK^T and PV over the causal half
    byts = (q.numel() + out.numel() + kc.numel() + vc.numel()) * 2
    return report("paged_prefill_attention", us, byts, flops, {"seqs": S, "len": L, "q_heads": hq, "kv_heads": hkv,
                                                               "kernel": ns.kernel, "page": page})


def bench_norm(ns, timer: Timer) -> dict:
    from ..ops import norm

    h = torch.randn(ns.rows, ns.hidden, device="cuda").bfloat16()
    part = torch.randn(ns.rows, ns.hidden, device="cuda").bfloat16()
    w = torch.ones(ns.hidden, device="cuda").bfloat16()
    out = torch.empty_like(h)
    us = timer(lambda: norm.add_rmsnorm([part], w, 1e-6, resid=h, out=out))
    return report("add_rmsnorm", us, 4 * h.numel() * 2, 0.0, {"rows": ns.rows, "hidden": ns.hidden})


def bench_norm_publish(ns, timer: Timer) -> dict:
    """The transport producer on one GPU: fold ``parts`` partials and the residual, RMSNorm, store the rows into
    ``dests`` destination buffers (local memory standing in for the FFN ranks' slots) and release their sequence words."""
    from ..ops import norm

    rows, hidden = ns.rows, ns.hidden
    h = torch.randn(rows, hidden, device="cuda").bfloat16()
    parts = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(ns.parts)]
    w = torch.ones(hidden, device="cuda").bfloat16()
    out = torch.empty_like(h)
    dst = [torch.zeros(rows, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(ns.dests)]
    flags = torch.zeros(ns.dests, 8, device="cuda", dtype=torch.int32)
    meta = torch.zeros(ns.dests, 4, device="cuda", dtype=torch.int32)
    seq = [0]

    def run():
        seq[0] += 1
        norm.add_rmsnorm(parts, w, 1e-6, resid=h, out=out, peer_ptrs=[d.data_ptr() for d in dst],
                         peer_flag_ptrs=[flags[i].data_ptr() for i in range(ns.dests)],
                         peer_meta_ptrs=[meta[i].data_ptr() for i in range(ns.dests)], publish_seq=seq[0], meta=(0, 2, 0))

    us = timer(run)
    byts = (ns.parts + 2 + 1 + ns.dests) * h.numel() * 2     # partials + residual read/write + normed output + pushes
    return report("norm_publish", us, byts, 0.0, {"rows": rows, "hidden": hidden, "parts": ns.parts, "dests": ns.dests})


def bench_lane(ns, timer: Timer) -> dict:
    """One Executor-Lane iteration of a dense layer on one GPU: the invocation is published before the iteration is
    enqueued (nothing waits for another launch), then lane_wait, gate/up + SwiGLU, down, lane_complete run from the
    descriptor table. Weight bytes are the roofline at decode sizes, FLOPs at prefill sizes."""
    from ..models import config as mc
    from ..parallel import fabric as F

    cfg = mc.preset(ns.model).with_layers(ns.layers)
    ffn = F.FfnRankRuntime("cuda", n_lanes=1, tile_weights=bool(ns.tiled))
    cap = max(128, ns.rows)
    place = F.InstancePlacement("m0", cfg, seed=1, atn_rank=0, ffn_ranks=(1,), capacity_rows=cap)
    st = ffn.add_instance(place, 0)
    buf = F.PeerBuffer(F.atn_slot_layout(place).total_bytes)
    st.atn_base = buf.ptr
    ffn.install()
    try:
        flay = F.ffn_slot_layout(place)
        x = (torch.randn(ns.rows, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
        st.slot.tensor(flay.input_offset, (cap, cfg.hidden_size), torch.bfloat16, "cuda")[:ns.rows] = x
        rec = st.slot.tensor(flay.record_offset, (64,), torch.int32, "cuda")
        host = torch.zeros(64, dtype=torch.int32).pin_memory()
        seq = [0]

        def run():
            seq[0] += 1
            host[0], host[1], host[2], host[3], host[8] = ns.rows, (seq[0] - 1) % ns.layers, 2, 0, seq[0]
            rec.copy_(host, non_blocking=True)        # the invocation record, as the attention side would publish it
            ffn.launch_once(0, lease_ms=50)

        us = timer(run)
        stats = ffn.stats()
        if stats["status"] != 0:
            raise RuntimeError(f"lane iteration failed: {stats}")
        served, launched = int(stats["served"][0]), seq[0]
    finally:
        ffn.close()
    inter = cfg.intermediate_size
    byts = 3 * cfg.hidden_size * inter * 2 + 2 * ns.rows * cfg.hidden_size * 2
    note = "includes one 256-byte host-to-device copy of the invocation record"
    if served != launched:
        # an iteration whose lease ran out before its record arrived serves nothing and is still timed: say so
        note += f"; {served} of {launched} iterations found their invocation (the others timed an empty lease)"
    return report(f"lane_iteration({ns.model})", us, byts, 6.0 * ns.rows * cfg.hidden_size * inter,
                  {"rows": ns.rows, "served": served, "launched": launched, "note": note})


def bench_moe(ns, timer: Timer) -> dict:
    from ..models.config import PRESETS
    from ..models.weights import random_ffn_layer
    from ..ops import gemm, moe

    cfg = PRESETS["Qwen/Qwen3-30B-A3B"]
    w = random_ffn_layer(cfg, 0, 1, "cuda", torch.bfloat16)
    x = (torch.randn(ns.rows, cfg.hidden_size, device="cuda") * 0.5).bfloat16()
    out = torch.empty_like(x)
    ws = moe.workspace(x.device, ns.rows, cfg, cfg.moe_intermediate_size, cfg.num_experts)
    us = timer(lambda: moe.moe_forward(x, w, cfg, out=out, ws=ws))
    gemm.check_status(x.device)
    routes = ns.rows * cfg.num_experts_per_tok
    touched = min(cfg.num_experts, routes)  # upper bound on experts whose weights are read
    byts = touched * 3 * cfg.hidden_size * cfg.moe_intermediate_size * 2
    return report("moe_forward(Qwen3-30B-A3B layer)", us, byts, 6.0 * routes * cfg.hidden_size * cfg.moe_intermediate_size,
                  {"rows": ns.rows, "routes": routes})


def bench_prefill_step(ns, timer: Timer) -> dict:
    """Prefill chunks of one Instance on the loopback engine: a prompt of ``chunks`` x ``chunk`` tokens goes through
    the engine chunk by chunk (launched eagerly), each step timed on the device."""
    from ..engine.atn_engine import AttentionEngine, EngineConfig
    from ..engine.ffn_local import LocalFfnPort
    from ..models import config as mc
    from ..models.weights import random_attention_weights, random_ffn_weights
    from ..ops import gemm

    cfg = mc.preset(ns.model)
    aw = random_attention_weights(cfg, 0, "cuda", torch.bfloat16)
    fw = random_ffn_weights(cfg, 0, "cuda", torch.bfloat16)
    total = ns.chunk * ns.chunks
    eng = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), EngineConfig(
        max_batch=8, prefill_chunk=ns.chunk, max_seq_len=total + 64, decode_buckets=[8], use_cuda_graph=False))
    eng.warmup()
    rnd = random.Random(0)
    ts = []
    for rep in range(timer.warmup + timer.iters):
        eng.add_request([rnd.randrange(cfg.vocab_size) for _ in range(total)], 1)
        per = []
        while eng.has_work:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(eng.stream)
            eng.step()
            b.record(eng.stream)
            torch.cuda.synchronize()
            per.append(a.elapsed_time(b))
        if rep >= timer.warmup:
            ts.append(per[:ns.chunks])
    gemm.check_status(eng.device)
    med = [statistics.median(t[i] for t in ts) for i in range(ns.chunks)]
    out = {"kernel": "prefill_step", "model": ns.model, "chunk_tokens": ns.chunk, "ms_per_chunk_by_position": [round(m, 3) for m in med],
           "prompt_tokens_per_s": round(total / (sum(med) / 1e3))}
    print(json.dumps(out), flush=True)
    return out


def bench_kv_vmm(ns, timer: Timer) -> dict:
    """Elastic KV: time to map and to unmap one KV Page Bundle (one physical chunk per layer and K/V buffer behind
    stable addresses) of a model, and the ECS seqlock channel's command/completion round trip on the host."""
    import time

    from ..ecs import vmm
    from ..models import config as mc
    from ..native.runtime import EcsChannel

    cfg = mc.preset(ns.model)
    drv, quota = vmm.Driver.real(), vmm.MemoryQuota(1 << 62)
    ppb, chunk = vmm.bundle_geometry(cfg, 16)
    cache = vmm.elastic_kv_cache(cfg, ns.bundles * ppb, 16, "cuda", drv, quota, initial_bundles=1)
    base = cache.k[0].data_ptr()
    grow_us, shrink_us = [], []
    for _ in range(timer.iters):
        take = cache.allocator.unmapped_bundles()[: ns.bundles - 1]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert vmm.grow(cache, take) == 0
        t1 = time.perf_counter()
        for b in take:
            cache.allocator.begin_retirement(b)
        cache.backing.unmap(take)
        t2 = time.perf_counter()
        grow_us.append((t1 - t0) * 1e6 / len(take))
        shrink_us.append((t2 - t1) * 1e6 / len(take))
    assert cache.k[0].data_ptr() == base            # addresses never move
    ch = EcsChannel.create(f"/xp-bench-ecs-{time.time_ns() & 0xffffff}", 1, 2, 1)
    try:
        t0 = time.perf_counter()
        n = 20000
        for i in range(1, n + 1):
            ch.publish_command(0, i, i << 20)
            seq, _ = ch.read_command(0)
            ch.publish_completion(0, seq, i << 20)
            ch.read_completion(0)
        ecs_us = (time.perf_counter() - t0) * 1e6 / n
    finally:
        ch.close()
    out = {"kernel": "kv_vmm_bundle", "model": ns.model, "bundle_mib": round(chunk * 2 * cfg.num_layers / 2 ** 20, 1),
           "chunks_per_bundle": 2 * cfg.num_layers, "pages_per_bundle": ppb,
           "map_us_per_bundle": round(statistics.median(grow_us), 1), "unmap_us_per_bundle": round(statistics.median(shrink_us), 1),
           "ecs_command_completion_round_trip_us": round(ecs_us, 2)}
    print(json.dumps(out), flush=True)
    return out


def bench_decode_step(ns, timer: Timer) -> dict:
    """One Instance's decode step on the loopback engine, launched eagerly (no CUDA graph) over
    sequences whose KV is taken as already cached -- the workload for a per-launch time list."""
    from ..engine.atn_engine import AttentionEngine, EngineConfig, Sequence
    from ..engine.ffn_local import LocalFfnPort
    from ..models import config as mc
    from ..models.weights import random_attention_weights, random_ffn_weights
    from ..ops import gemm

    cfg = mc.preset(ns.model)
    aw = random_attention_weights(cfg, 0, "cuda", torch.bfloat16)
    fw = random_ffn_weights(cfg, 0, "cuda", torch.bfloat16)
    rnd = random.Random(0)
    lens = [rnd.randint(ns.min_len, ns.max_len) for _ in range(ns.batch)]
    steps = timer.iters + timer.warmup
    pages = sum((l + steps + 32) // 16 + 1 for l in lens) + 64
    eng = AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), EngineConfig(
        max_batch=ns.batch, prefill_chunk=256, max_seq_len=ns.max_len + steps + 64, num_pages=pages,
        decode_buckets=[ns.batch], use_cuda_graph=bool(ns.graph)))
    eng.warmup()
    for i, l in enumerate(lens):
        s = Sequence(i, [1] * l, steps + 8)
        s.computed, s.generated = l, [2]
        eng.kv.ensure(s.seq_id, l + 1)
        eng.running.append(s)
    torch.cuda.synchronize()
    for _ in range(timer.warmup):
        eng.step()
    torch.cuda.synchronize()
    ts = []
    for _ in range(timer.iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(eng.stream)
        eng.step()
        b.record(eng.stream)
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    gemm.check_status(torch.device("cuda"))
    us = statistics.median(ts)
    kv_bytes = sum(lens) * cfg.kv_bytes_per_token()
    w_bytes = cfg.attention_param_bytes() - 2 * cfg.vocab_size * cfg.hidden_size * (0 if cfg.tie_word_embeddings else 1) + \
        sum(cfg.ffn_param_bytes_per_layer(l) for l in range(cfg.num_layers))
    return report(f"decode_step({ns.model})", us, kv_bytes + w_bytes, 0.0,
                  {"batch": ns.batch, "tokens_cached": sum(lens), "graph": bool(ns.graph), "tok_per_s": round(ns.batch / us * 1e6)})


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m crosspool_b200.bench.kernels")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--rows", type=int, default=64)
    g.add_argument("--n", type=int, default=3072)
    g.add_argument("--k", type=int, default=1024)
    g.add_argument("--dual", type=int, default=0)
    g.add_argument("--splits", type=int, default=0)
    g.add_argument("--bn", type=int, default=0)
    g.add_argument("--tiled", type=int, default=0, help="1: weights pre-tiled into contiguous 128 x 64 blocks")
    g.add_argument("--fp8", type=int, default=0, help="1: block-scaled e4m3 weights and activations")
    a = sub.add_parser("decode-attn")
    a.add_argument("--batch", type=int, default=256)
    a.add_argument("--q-heads", type=int, default=16)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--min-len", type=int, default=128)
    a.add_argument("--max-len", type=int, default=2048)
    a.add_argument("--chunk", type=int, default=-1, help="KV slice length (-1: the planner's choice, 0: even split)")
    pa = sub.add_parser("prefill-attn")
    pa.add_argument("--seqs", type=int, default=4)
    pa.add_argument("--len", type=int, default=1024)
    pa.add_argument("--q-heads", type=int, default=16)
    pa.add_argument("--kv-heads", type=int, default=8)
    pa.add_argument("--head-dim", type=int, default=128)
    pa.add_argument("--page", type=int, default=16, help="tokens per KV page")
    pa.add_argument("--kernel", default="umma", choices=["umma", "umma-alt", "mma", "simple"],
                    help="umma: tcgen05 kernel; mma: TMA-fed mma.sync kernel; simple: plain mma.sync kernel")
    n = sub.add_parser("norm")
    n.add_argument("--rows", type=int, default=256)
    n.add_argument("--hidden", type=int, default=1024)
    npub = sub.add_parser("norm-publish")
    npub.add_argument("--rows", type=int, default=4096)
    npub.add_argument("--hidden", type=int, default=4096)
    npub.add_argument("--parts", type=int, default=2)
    npub.add_argument("--dests", type=int, default=2)
    ln = sub.add_parser("lane")
    ln.add_argument("--model", default="Qwen/Qwen3-8B")
    ln.add_argument("--rows", type=int, default=64)
    ln.add_argument("--layers", type=int, default=4)
    ln.add_argument("--tiled", type=int, default=0)
    m = sub.add_parser("moe")
    m.add_argument("--rows", type=int, default=64)
    ps = sub.add_parser("prefill-step")
    ps.add_argument("--model", default="Qwen/Qwen3-0.6B")
    ps.add_argument("--chunk", type=int, default=2048)
    ps.add_argument("--chunks", type=int, default=4)
    v = sub.add_parser("kv-vmm")
    v.add_argument("--model", default="Qwen/Qwen3-0.6B")
    v.add_argument("--bundles", type=int, default=9)
    d = sub.add_parser("decode-step")
    d.add_argument("--model", default="Qwen/Qwen3-0.6B")
    d.add_argument("--batch", type=int, default=256)
    d.add_argument("--min-len", type=int, default=128)
    d.add_argument("--max-len", type=int, default=2048)
    d.add_argument("--graph", type=int, default=0)
    ns = ap.parse_args(argv)
    timer = Timer(ns.iters, ns.warmup, not ns.no_flush)
    {"gemm": bench_gemm, "decode-attn": bench_decode_attn, "norm": bench_norm, "moe": bench_moe,
     "decode-step": bench_decode_step, "prefill-attn": bench_prefill_attn, "kv-vmm": bench_kv_vmm,
     "prefill-step": bench_prefill_step, "norm-publish": bench_norm_publish, "lane": bench_lane}[ns.case](ns, timer)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
