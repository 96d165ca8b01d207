"""Memory ledger / calibration fit and quantization formats (CPU)."""
import pytest
import torch

from crosspool_b200 import memory as M
from crosspool_b200 import quantization as Q


def _features(w=10 << 30, lanes=2, inst=3, **kw):
    return M.DeviceMemoryFeatures(weight_bytes=w, n_instances=inst, n_layers=28 * inst, slot_bytes=64 << 20, lanes=lanes,
                                  ws_bytes_per_lane=64 << 20, **kw)


def test_ledger_counts_every_allocation_class_and_rounds_to_granules():
    est = M.DeviceMemoryEstimator()
    e = est.analytic(_features())
    assert e.weights == 10 << 30 and e.slots == 64 << 20 and e.workspaces == 2 * ((64 << 20) + (64 << 10))
    assert e.moe_scratch == 0 and e.tables % (2 << 20) == 0 and e.lane_state % (2 << 20) == 0
    moe = est.analytic(_features(moe_routes=4096 * 8, moe_hidden=2048, moe_inter=768, moe_experts_padded=128, moe_rows=4096))
    assert moe.moe_scratch >= 2 * (2 * 32768 * 2048 * 2 + 32768 * 768 * 2)   # xp + yp + act per lane
    assert est.estimate(_features()).total > e.total
    assert M.allocator_reservation_bytes([100, 600, 3 << 20, 50 << 20]) == (2 << 20) + (20 << 20) + (50 << 20)


def test_calibration_fit_recovers_the_overhead_model_and_profiles_are_bound_to_their_environment(tmp_path):
    true = M.FfnMemoryCalibrationCoefficients(700e6, 12e6, 2e6, 0.01)
    gen = M.DeviceMemoryEstimator(true)
    feats = [_features(w << 30, l, i) for w, l, i in [(1, 1, 1), (8, 2, 2), (20, 4, 3), (40, 1, 6), (64, 8, 4), (3, 2, 8)]]
    samples = [(f, gen.estimate(f).total) for f in feats]
    coef, resid = M.fit_coefficients(samples)
    assert abs(coef.context_bytes - 700e6) < 1e6 and abs(coef.per_lane_bytes - 12e6) < 1e5 and abs(coef.weight_slack - 0.01) < 1e-4
    assert resid < 1 << 20
    env = M.MemoryCalibrationEnvironment("NVIDIA B200", "580.159", "12.9", "torch 2.11", "abc")
    prof = M.XpoolMemoryCalibrationProfile(env, coef, len(samples), resid)
    prof.save(tmp_path / "p.json")
    assert M.XpoolMemoryCalibrationProfile.load(tmp_path / "p.json", expect=env).coefficients == coef
    other = M.MemoryCalibrationEnvironment("NVIDIA B200", "590.0", "12.9", "torch 2.11", "abc")
    with pytest.raises(ValueError, match="different environment"):
        M.XpoolMemoryCalibrationProfile.load(tmp_path / "p.json", expect=other)
    with pytest.raises(ValueError):
        M.fit_coefficients(samples[:3])


def test_resolve_accepts_known_methods_only():
    assert isinstance(Q.resolve(None), Q.Unquantized) and isinstance(Q.resolve("mxfp4"), Q.Mxfp4)
    assert isinstance(Q.resolve("fp8_block"), Q.Fp8Block)
    with pytest.raises(ValueError, match="unsupported weight quantization method: awq"):
        Q.resolve("awq")


def test_mxfp4_round_trip_slicing_and_exact_code_points():
    q = Q.Mxfp4()
    g = torch.Generator().manual_seed(0)
    w = torch.randn(4, 64, 128, generator=g)          # [experts, n, k]
    st = q.quantize(w)
    assert st["blocks"].shape == (4, 64, 64) and st["scales"].shape == (4, 64, 4) and st["blocks"].dtype == torch.uint8
    back = q.dequantize(st, torch.float32)
    blk_max = w.reshape(4, 64, 4, 32).abs().amax(-1).repeat_interleave(32, -1)
    assert ((back - w).abs() <= 0.26 * blk_max + 1e-6).all()        # half of the widest e2m1 step (2 of 6) plus scale rounding
    exact = torch.tensor([[0.5, -6.0, 3.0, 0.0] * 8]) * 4.0       # code points times a power of two survive exactly
    assert torch.equal(q.dequantize(q.quantize(exact), torch.float32), exact)
    sl = q.slice(st, 16, 48, 32, 96)
    assert torch.equal(q.dequantize(sl, torch.float32), back[:, 16:48, 32:96])
    with pytest.raises(ValueError, match="cuts a scale block"):
        q.slice(st, 0, 64, 16, 128)
    assert q.stored_bytes(64, 128) == 64 * 64 + 64 * 4


def test_fp8_block_round_trip_and_quanta():
    q = Q.Fp8Block()
    w = torch.randn(256, 384) * 3
    st = q.quantize(w)
    assert st["weight"].dtype == torch.float8_e4m3fn and st["scale"].shape == (2, 3)
    back = q.dequantize(st, torch.float32)
    assert ((back - w).abs() <= 0.07 * w.abs() + 0.02 * w.abs().max()).all()
    assert torch.equal(q.dequantize(q.slice(st, 128, 256, 0, 256), torch.float32), back[128:, :256])
    with pytest.raises(ValueError):
        q.slice(st, 64, 256, 0, 128)


def test_calibration_runner_fits_from_an_injected_measurement():
    from crosspool_b200.runtime import memory_calibration as mcal

    true = M.DeviceMemoryEstimator(M.FfnMemoryCalibrationCoefficients(650e6, 9e6, 3e6, 0.0))
    env = M.MemoryCalibrationEnvironment("fake", "0", "12.9", "torch", "x")
    prof = mcal.calibrate(measure=lambda e: true.estimate(mcal.features_of(e)).total, environment=env)
    assert prof.samples == len(mcal.DEFAULT_CORPUS) and prof.max_abs_error_bytes < 4 << 20
    assert abs(prof.coefficients.per_lane_bytes - 9e6) < 1e6
    f = mcal.features_of(mcal.Experiment("Qwen/Qwen3-0.6B", 28, 1, 2))
    assert f.weight_bytes == 28 * 3 * 1024 * 3072 * 2 and f.slot_bytes > 512 * 1024 * 2


def test_calibration_evidence_persists_and_a_rerun_only_measures_what_is_missing(tmp_path):
    from crosspool_b200.runtime import memory_calibration as mcal

    env = M.MemoryCalibrationEnvironment("B200", "580", "12.9", "torch", "abc")
    measured = []

    def fake_measure(exp):
        measured.append(exp)
        f = mcal.features_of(exp)
        return M.DeviceMemoryEstimator().analytic(f).total + int(500e6 + 6e6 * f.lanes + 2e6 * f.n_instances)

    corpus = mcal.DEFAULT_CORPUS[:5]
    p1 = mcal.calibrate(corpus, fake_measure, env, evidence_root=tmp_path)
    assert len(measured) == 5 and p1.samples == 5
    store = mcal.EvidenceStore(tmp_path, env)
    assert len(store.all()) == 5 and store.load(corpus[0]) is not None
    # a second run with a larger corpus measures only the new experiments and fits on everything stored
    p2 = mcal.calibrate(mcal.DEFAULT_CORPUS[:7], fake_measure, env, evidence_root=tmp_path)
    assert len(measured) == 7 and p2.samples == 7
    assert abs(p2.coefficients.context_bytes - 500e6) < 5e6 and abs(p2.coefficients.per_lane_bytes - 6e6) < 1e6
    # another environment has its own evidence
    other = M.MemoryCalibrationEnvironment("B200", "999", "12.9", "torch", "abc")
    assert mcal.EvidenceStore(tmp_path, other).all() == []
