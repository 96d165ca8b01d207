"""Elastic KV on a real device: two engines share a physical budget through the capacity channel; the
daemon policy moves bundles from the idle engine to the busy one; tokens equal a fixed-cache run."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _engine(cfg, seed, kv, **kw):
    from crosspool_b200.engine.atn_engine import AttentionEngine, EngineConfig
    from crosspool_b200.engine.ffn_local import LocalFfnPort
    from crosspool_b200.models.weights import random_attention_weights, random_ffn_weights

    aw = random_attention_weights(cfg, seed, "cuda", torch.bfloat16)
    fw = random_ffn_weights(cfg, seed, "cuda", torch.bfloat16)
    return AttentionEngine(cfg, aw, LocalFfnPort(cfg, fw), EngineConfig(**kw), kv=kv)


def test_bundles_move_between_engines_and_results_match_a_fixed_cache():
    from crosspool_b200.ecs import reconciler as R
    from crosspool_b200.ecs import vmm
    from crosspool_b200.models import config as mc
    from crosspool_b200.native.runtime import EcsChannel
    from crosspool_b200.service.daemon.ecs import CapacityPolicy, Partition

    cfg = mc.preset("tiny-qwen3")
    kw = dict(max_batch=64, prefill_chunk=2048, max_seq_len=256, use_cuda_graph=True)
    ppb, chunk = vmm.bundle_geometry(cfg, 16)
    drv, quota = vmm.Driver.real(), vmm.MemoryQuota(1 << 40)
    ch = EcsChannel.create(f"/xp-test-elastic-{os.getpid()}", 1, 2, 1)
    engines, recs = [], []
    try:
        for i in (0, 1):
            kv = vmm.elastic_kv_cache(cfg, max_pages=2 * ppb, page_size=16, device="cuda", driver=drv, quota=quota,
                                      initial_bundles=1)
            eng = _engine(cfg, 3 + i, kv, **kw)
            rec = R.CapacityReconciler(kv, ch, i, gate_factory=lambda e=eng: R.cuda_event_gate(e.stream))
            eng.attach_capacity(rec)
            eng.warmup()
            engines.append(eng)
            recs.append(rec)
        bb = recs[0].bundle_bytes
        parts = [Partition(i, f"m{i}:0", 0, bb, 2 * bb, bb, mapped_bytes=bb) for i in (0, 1)]
        pol = CapacityPolicy(ch, parts, {0: 0}, utilization=1.0)
        ch.publish_report(0, 1 * bb, 100 * bb, 0)    # budget: the two mapped floors + one spare bundle
        pol.freeze_pools()
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(0, cfg.vocab_size, (190,), generator=g).tolist() for _ in range(64)]  # > one bundle of tokens

        def run(eng):
            seqs = [eng.add_request(p, 8) for p in prompts]
            steps = 0
            while eng.has_work and steps < 2000:
                pol.tick()
                for e in engines:
                    if e is not eng:
                        e.launch_step()      # idle engines still service capacity commands
                        e.collect_step()
                eng.step()
                steps += 1
            assert not eng.has_work
            return [s.generated for s in seqs]

        out_a = run(engines[0])
        assert recs[0].mapped_bundles == 2 and recs[1].mapped_bundles == 1      # A took the spare bundle
        out_b = run(engines[1])
        assert recs[1].mapped_bundles == 2 and recs[0].mapped_bundles == 1      # A gave its extra bundle back to B
        kinds = [e.kind for e in pol.events]
        assert "grow" in kinds and "shrink" in kinds
        assert quota.charged == 3 * bb
        # same models on fixed caches produce the same tokens
        for i, got in ((0, out_a), (1, out_b)):
            ref = _engine(cfg, 3 + i, None, **kw)
            ref.warmup()
            want = ref.generate(prompts, 8)
            same = sum(a == b for a, b in zip(got, want))
            assert same >= 60, same   # batch composition differs (admission order), so allow rare bf16 argmax flips
        from crosspool_b200.ops import gemm
        gemm.check_status(torch.device("cuda"))
    finally:
        for e in engines:
            torch.cuda.synchronize()
        ch.close()
