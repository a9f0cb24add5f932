"""The numpy quantization / QAT front-end against (a) golden outputs produced by the reference's own
code (tests/golden/make_golden.py) and (b) the known-answer tests the reference holds for this API."""
import json
from pathlib import Path

import numpy as np
import pytest

from zenith_b200 import qat as zq
from zenith_b200 import quantization as zp

G = np.load(Path(__file__).parent / "golden" / "quant_golden.npz")
CFG1 = json.loads((Path(__file__).parent / "golden" / "config1_golden.json").read_text())


def rng(seed):
    return np.random.default_rng(seed)


# ---- golden: PTQ ----------------------------------------------------------------------------
def test_params_quantize_truncates_like_reference():
    x = (rng(11).standard_normal(4096) * 3).astype(np.float32)
    assert np.array_equal(zp.QuantizationParams(0.1, 0).quantize(x), G["ptq_params_quantize"])
    q = zp.QuantizationParams(0.07, 5).quantize(x)
    assert np.array_equal(q, G["ptq_params_quantize_zp"])
    assert np.array_equal(zp.QuantizationParams(0.07, 5).dequantize(q), G["ptq_params_dequantize"])
    # truncation, not rounding (zenith/optimization/quantization.py:49-53)
    assert zp.QuantizationParams(0.1, 0).quantize(np.array([0.26, 0.19, -0.26], np.float32)).tolist() == [2, 1, -2]


@pytest.mark.parametrize("name,make", [
    ("minmax_sym", lambda: zp.MinMaxCalibrator(True)), ("minmax_asym", lambda: zp.MinMaxCalibrator(False)),
    ("pct_sym", lambda: zp.PercentileCalibrator(99.9, True)), ("pct_asym", lambda: zp.PercentileCalibrator(99.0, False)),
    ("ent_sym", lambda: zp.EntropyCalibrator(True)), ("ent_asym", lambda: zp.EntropyCalibrator(False))])
def test_calibrators_match_reference(name, make):
    st = zp.TensorStats()
    for s in (12, 13, 14):
        st.update((rng(s).standard_normal((64, 96)) * (1 + 0.3 * (s - 12))).astype(np.float32))
    p = make().compute_params(st)
    assert p.scale == G[f"ptq_cal_{name}"][0] and p.zero_point == int(G[f"ptq_cal_{name}"][1])
    if name == "minmax_sym":
        assert np.array_equal(st.histogram, G["ptq_stats_hist"])
        assert [st.min_val, st.max_val] == G["ptq_stats_minmax"].tolist()


def test_quantize_function_and_static_ptq_match_reference():
    q, s, z = zp.quantize(rng(15).standard_normal((8, 768)).astype(np.float32))
    assert np.array_equal(q, G["ptq_quantize_fn_q"]) and [s, z] == G["ptq_quantize_fn_sz"].tolist()
    weights = {"w0": (rng(16).standard_normal((48, 32)) * 0.02).astype(np.float32),
               "w1": (rng(17).standard_normal((32, 48)) * 0.05).astype(np.float32)}
    cal = [rng(18 + i).standard_normal((16, 32)).astype(np.float32) for i in range(3)]
    qm = zp.quantize_model_static(weights, cal, ["in0", "in0", "in1"])
    for k in weights:
        assert qm.get_weight(k).dtype == np.int8
        assert np.array_equal(qm.get_weight(k), G[f"ptq_static_{k}"])
        assert qm.weight_params[k].scale == G[f"ptq_static_{k}_scale"][0]
    assert [qm.activation_params["in0"].scale, qm.activation_params["in1"].scale] == G["ptq_static_act_scales"].tolist()
    err = zp.measure_quantization_error(weights["w0"], qm, "w0")
    assert np.allclose([err["mse"], err["max_abs_error"], err["snr_db"]], G["ptq_static_err"], rtol=1e-12)
    assert np.array_equal(zp.QATSimulator().simulate_forward(weights["w1"], cal[0]), G["ptq_sim_forward"])


# ---- golden: QAT ----------------------------------------------------------------------------
@pytest.mark.parametrize("name,kw", [
    ("pt_sym", dict()), ("pt_asym", dict(symmetric=False)), ("pc_sym", dict(per_channel=True, channel_axis=0)),
    ("pt_4bit", dict(num_bits=4)), ("pc_axis1", dict(per_channel=True, channel_axis=1))])
def test_fake_quantize_matches_reference(name, kw):
    xa = (rng(21).standard_normal((32, 64)) * 2).astype(np.float32)
    fq = zq.FakeQuantize(**kw)
    y = fq.forward(xa)
    assert np.array_equal(np.asarray(y, np.float64), G[f"qat_fq_{name}_y"])
    assert np.array_equal(np.asarray(fq.scale, np.float64), G[f"qat_fq_{name}_scale"])
    assert np.array_equal(np.asarray(fq.zero_point, np.int64), G[f"qat_fq_{name}_zp"])


def test_ema_observer_ste_trainer_and_converter_match_reference():
    fq = zq.FakeQuantize()
    for s in (22, 23, 24, 25):
        fq.observe((rng(s).standard_normal((16, 16)) * (s - 20)).astype(np.float32))
    assert np.array_equal(np.asarray(fq.scale, np.float64), G["qat_ema_scale"])
    assert [fq.min_val[0], fq.max_val[0]] == G["qat_ema_minmax"].tolist()
    xa = (rng(21).standard_normal((32, 64)) * 2).astype(np.float32)
    g = rng(26).standard_normal(xa.shape).astype(np.float32)
    assert np.array_equal(zq.FakeQuantize().forward_with_ste(xa * 100, g)[1], G["qat_ste_grad"])
    W = (rng(27).standard_normal((24, 40)) * 0.02).astype(np.float32)
    acts = [rng(28 + i).standard_normal((8, 40)).astype(np.float32) for i in range(4)]
    tr = zq.prepare_model_for_qat({"fc": W.shape})
    tr.calibrate("fc", W, acts)
    tr.qat_modules["fc"].freeze_observers()
    assert np.array_equal(np.asarray(tr.qat_modules["fc"].weight_fake_quant.scale, np.float64), G["qat_trainer_w_scale"])
    assert np.array_equal(np.asarray(tr.qat_modules["fc"].activation_fake_quant.scale, np.float64), G["qat_trainer_a_scale"])
    sim = zq.simulate_qat_forward(tr, "fc", W, acts[0])
    assert np.array_equal(np.asarray(sim, np.float64), G["qat_sim_forward"])
    cq, cp = zq.convert_qat_to_quantized(tr, {"fc": W})["fc"]
    assert cq.dtype == np.int8 and np.array_equal(cq, G["qat_convert_q"])
    assert [cp.scale, cp.zero_point] == G["qat_convert_scale"].tolist()
    e = zq.measure_qat_error(acts[0] @ W.T, sim)
    assert np.allclose([e["mse"], e["mae"], e["max_error"], e["snr_db"], e["relative_error"]], G["qat_error"], rtol=1e-12)
    # the per-channel converter uses every channel's scale and the observer's rounding
    q, s = zq.convert_per_channel(tr, {"fc": W})["fc"]
    fqs = np.asarray(tr.qat_modules["fc"].weight_fake_quant.scale)
    assert q.dtype == np.int8 and np.array_equal(q, np.clip(np.round(W / fqs[:, None]), -128, 127).astype(np.int8))
    assert s.dtype == np.float32 and s.shape == (24,)


def test_config1_calibration_matches_reference_digests():
    import hashlib

    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    M = 1234
    W = (rng(M + 100).standard_normal((3072, 768)) * 0.02).astype(np.float32)
    quant = zp.Quantizer(zp.QuantizationMode.STATIC, zp.CalibrationMethod.MINMAX)
    for i in range(1, 9):
        x = rng(M + i).standard_normal((128, 768)).astype(np.float32)
        quant.collect_stats(np.array([x.min(), x.max()]), "x")  # min/max only: same running extrema
    assert quant.compute_params("x").scale == CFG1["s_x"]
    tr = zq.prepare_model_for_qat({"fc": W.shape})
    tr.calibrate("fc", W, [])
    tr.qat_modules["fc"].freeze_observers()
    q, s = zq.convert_per_channel(tr, {"fc": W})["fc"]
    assert sha(s) == CFG1["s_w_sha256"] and sha(q) == CFG1["Wq_sha256"]
    assert int((q == -128).sum()) == CFG1["Wq_minus128"] > 0  # the full [-128, 127] range occurs
    assert sha(np.asarray(tr.qat_modules["fc"].fake_quantize_weight(W), np.float32)) == CFG1["fake_quant_W_sha256"]


# ---- the reference's own known-answer tests for this API -------------------------------------
def test_bounds_and_symmetry():  # tests/test_qat.py:22-41,72-102
    assert (zq.FakeQuantize(8, True).qmin, zq.FakeQuantize(8, True).qmax) == (-128, 127)
    assert (zq.FakeQuantize(8, False).qmin, zq.FakeQuantize(8, False).qmax) == (0, 255)
    assert (zq.FakeQuantize(4, True).qmin, zq.FakeQuantize(4, True).qmax) == (-8, 7)
    fq = zq.FakeQuantize()
    x = rng(1).standard_normal((10, 10)).astype(np.float32)
    y = fq.forward(x)
    assert np.all(fq.zero_point == 0)
    assert np.max(np.abs(x - y)) <= fq.scale[0] + 1e-6


def test_per_channel_scales_differ():  # tests/test_qat.py:165-179
    fq = zq.FakeQuantize(per_channel=True, channel_axis=0)
    w = rng(2).standard_normal((8, 16)).astype(np.float32) * np.arange(1, 9, dtype=np.float32)[:, None]
    fq.forward(w)
    assert fq.scale.shape == (8,) and len(set(fq.scale.tolist())) == 8


def test_frozen_observer_keeps_scale():  # tests/test_qat.py:334-354
    m = zq.QATModule((4, 4))
    m.fake_quantize_activation(rng(3).standard_normal((4, 4)).astype(np.float32))
    before = m.activation_fake_quant.scale.copy()
    m.freeze_observers()
    m.fake_quantize_activation(100 * rng(4).standard_normal((4, 4)).astype(np.float32))
    assert np.array_equal(before, m.activation_fake_quant.scale)


def test_minmax_known_answer():  # tests/test_quantization.py:79-91
    st = zp.TensorStats()
    st.update(np.array([-3.0, 1.0, 2.5], np.float32))
    assert zp.MinMaxCalibrator(True).compute_params(st).scale == 3.0 / 127.0


def test_fake_quant_quality_bars():  # tests/test_qat.py:512-553; tests/test_qat_cuda.py:34-60
    x = (rng(42).standard_normal(1000) * 3).astype(np.float32)
    fq = zq.FakeQuantize()
    y = fq.forward(x)
    s = fq.scale[0]
    np.testing.assert_array_almost_equal(y, np.clip(np.round(x / s), -128, 127) * s, decimal=5)
    snr = 10 * np.log10(np.mean(x**2) / np.mean((x - y) ** 2))
    assert snr > 20


def test_reexported_names_resolve():  # zenith/optimization/__init__.py:96-118
    for n in ("QuantizationMode", "CalibrationMethod", "QuantizationParams", "Quantizer", "QATSimulator",
              "quantize_model_static", "measure_quantization_error"):
        assert hasattr(zp, n)
    for n in ("QATScheme", "ObserverType", "QATConfig", "FakeQuantize", "QATModule", "QATTrainer",
              "prepare_model_for_qat", "convert_qat_to_quantized", "simulate_qat_forward", "measure_qat_error"):
        assert hasattr(zq, n)


def test_scale_table_round_trips_through_a_file(tmp_path):
    from zenith_b200.calibrate import activation_scales_from_ranges, quantize_weights
    from zenith_b200.encoder import ACT_POINTS, EncoderConfig, Int8Scales, init_params

    cfg = EncoderConfig(layers=2, hidden=64, heads=2, ffn=128, vocab=100, max_pos=16)
    params = init_params(cfg, 5)
    ranges = {p: [[(-1.0 - li, 2.0 + i)] for li in range(cfg.layers)] for i, p in enumerate(ACT_POINTS)}
    scales = Int8Scales(act=activation_scales_from_ranges(ranges, cfg.layers), weights=quantize_weights(params))
    path = tmp_path / "scales.npz"
    scales.save(path)
    back = Int8Scales.load(path)
    assert back.act == scales.act
    for a, b in zip(scales.weights, back.weights):
        assert a.keys() == b.keys()
        for k in a:
            assert b[k][0].dtype == np.int8 and np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1])
