"""Generates tests/golden/quant_golden.npz and config1_golden.json by IMPORTING THE REFERENCE
(vibeswithkk/ZENITH, read-only tree) and running its own quantization / QAT code on seeded inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference
    (or with the environment variable ZENITH_REFERENCE set to that path)

The outputs are committed; the tests never need the reference tree.  Inputs are regenerated in the
tests from the seeds below, only the reference's OUTPUTS are stored.
"""
import hashlib
import importlib.util
import json
import os
import sys
from pathlib import Path

import numpy as np

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ZENITH_REFERENCE")
if not REF or not (Path(REF) / "zenith").is_dir():
    raise SystemExit("usage: make_golden.py /path/to/reference   (the directory that holds the `zenith` package)")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

from zenith.optimization import qat as rq  # noqa: E402
from zenith.optimization import quantization as rp  # noqa: E402

HERE = Path(__file__).resolve().parent
out = {}


def rng(seed):
    return np.random.default_rng(seed)


# ---- PTQ (zenith/optimization/quantization.py) ----------------------------------------------
x = (rng(11).standard_normal(4096) * 3).astype(np.float32)
out["ptq_params_quantize"] = rp.QuantizationParams(0.1, 0).quantize(x)
out["ptq_params_quantize_zp"] = rp.QuantizationParams(0.07, 5).quantize(x)
out["ptq_params_dequantize"] = rp.QuantizationParams(0.07, 5).dequantize(out["ptq_params_quantize_zp"])
for name, cal in (("minmax_sym", rp.MinMaxCalibrator(True)), ("minmax_asym", rp.MinMaxCalibrator(False)),
                  ("pct_sym", rp.PercentileCalibrator(99.9, True)), ("pct_asym", rp.PercentileCalibrator(99.0, False)),
                  ("ent_sym", rp.EntropyCalibrator(True)), ("ent_asym", rp.EntropyCalibrator(False))):
    st = rp.TensorStats()
    for s in (12, 13, 14):
        st.update((rng(s).standard_normal((64, 96)) * (1 + 0.3 * (s - 12))).astype(np.float32))
    p = cal.compute_params(st)
    out[f"ptq_cal_{name}"] = np.array([p.scale, p.zero_point], dtype=np.float64)
    if name == "minmax_sym":
        out["ptq_stats_hist"] = st.histogram.copy()
        out["ptq_stats_minmax"] = np.array([st.min_val, st.max_val])
q, s, z = rp.quantize((rng(15).standard_normal((8, 768))).astype(np.float32))
out["ptq_quantize_fn_q"], out["ptq_quantize_fn_sz"] = q, np.array([s, z], dtype=np.float64)
weights = {"w0": (rng(16).standard_normal((48, 32)) * 0.02).astype(np.float32),
           "w1": (rng(17).standard_normal((32, 48)) * 0.05).astype(np.float32)}
cal_data = [(rng(18 + i).standard_normal((16, 32))).astype(np.float32) for i in range(3)]
qm = rp.quantize_model_static(weights, cal_data, ["in0", "in0", "in1"])
for k in weights:
    out[f"ptq_static_{k}"] = qm.get_weight(k)
    out[f"ptq_static_{k}_scale"] = np.array([qm.weight_params[k].scale])
out["ptq_static_act_scales"] = np.array([qm.activation_params["in0"].scale, qm.activation_params["in1"].scale])
err = rp.measure_quantization_error(weights["w0"], qm, "w0")
out["ptq_static_err"] = np.array([err["mse"], err["max_abs_error"], err["snr_db"]])
sim = rp.QATSimulator()
out["ptq_sim_forward"] = sim.simulate_forward(weights["w1"], cal_data[0])  # [16,32] @ [32,48]

# ---- QAT (zenith/optimization/qat.py) -------------------------------------------------------
xa = (rng(21).standard_normal((32, 64)) * 2).astype(np.float32)
for name, kw in (("pt_sym", dict()), ("pt_asym", dict(symmetric=False)), ("pc_sym", dict(per_channel=True, channel_axis=0)),
                 ("pt_4bit", dict(num_bits=4)), ("pc_axis1", dict(per_channel=True, channel_axis=1))):
    fq = rq.FakeQuantize(**kw)
    y = fq.forward(xa)
    out[f"qat_fq_{name}_y"] = np.asarray(y, dtype=np.float64)
    out[f"qat_fq_{name}_scale"] = np.asarray(fq.scale, dtype=np.float64)
    out[f"qat_fq_{name}_zp"] = np.asarray(fq.zero_point, dtype=np.int64)
fq = rq.FakeQuantize()
for s in (22, 23, 24, 25):
    fq.observe((rng(s).standard_normal((16, 16)) * (s - 20)).astype(np.float32))
out["qat_ema_scale"] = np.asarray(fq.scale, dtype=np.float64)
out["qat_ema_minmax"] = np.array([fq.min_val[0], fq.max_val[0]], dtype=np.float64)
fq = rq.FakeQuantize()
g = rng(26).standard_normal(xa.shape).astype(np.float32)
_, gi = fq.forward_with_ste(xa * 100, g)
out["qat_ste_grad"] = gi
W = (rng(27).standard_normal((24, 40)) * 0.02).astype(np.float32)
acts = [(rng(28 + i).standard_normal((8, 40))).astype(np.float32) for i in range(4)]
tr = rq.prepare_model_for_qat({"fc": W.shape})
tr.calibrate("fc", W, acts)
tr.qat_modules["fc"].freeze_observers()
out["qat_trainer_w_scale"] = np.asarray(tr.qat_modules["fc"].weight_fake_quant.scale, dtype=np.float64)
out["qat_trainer_a_scale"] = np.asarray(tr.qat_modules["fc"].activation_fake_quant.scale, dtype=np.float64)
out["qat_sim_forward"] = np.asarray(rq.simulate_qat_forward(tr, "fc", W, acts[0]), dtype=np.float64)
cq, cp = rq.convert_qat_to_quantized(tr, {"fc": W})["fc"]
out["qat_convert_q"], out["qat_convert_scale"] = cq, np.array([cp.scale, cp.zero_point], dtype=np.float64)
e = rq.measure_qat_error(acts[0] @ W.T, out["qat_sim_forward"])
out["qat_error"] = np.array([e["mse"], e["mae"], e["max_error"], e["snr_db"], e["relative_error"]])

np.savez_compressed(HERE / "quant_golden.npz", **out)

# ---- config 1 at full size: only scalars and digests are stored -----------------------------
MASTER = 1234
X = rng(MASTER).standard_normal((128, 768)).astype(np.float32)
Wc = (rng(MASTER + 100).standard_normal((3072, 768)) * 0.02).astype(np.float32)
bc = (rng(MASTER + 101).standard_normal(3072) * 0.02).astype(np.float32)
quant = rp.Quantizer(rp.QuantizationMode.STATIC, rp.CalibrationMethod.MINMAX)
for i in range(1, 9):
    quant.collect_stats(rng(MASTER + i).standard_normal((128, 768)).astype(np.float32), "x")
s_x = quant.compute_params("x").scale
fqw = rq.FakeQuantize(per_channel=True, channel_axis=0)
fqw.observe(Wc)
fqw.disable_observer()
s_w = np.asarray(fqw.scale, dtype=np.float32)
Wq = np.clip(np.round(Wc / s_w[:, None]), -128, 127).astype(np.int8)
Xq = np.clip(np.round(X / np.float32(s_x)), -128, 127).astype(np.int8)
# the integer product by the reference's own function (benchmarks/int8_bench.py:42-45; unit scales: the float32
# result is exact, |acc| < 2^24)
_spec = importlib.util.spec_from_file_location("ref_int8_bench", Path(REF) / "benchmarks" / "int8_bench.py")
ib = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(ib)
acc = ib.int8_matmul_reference(Xq, np.ascontiguousarray(Wq.T), np.float32(1.0), np.float32(1.0)).astype(np.int32)
assert np.array_equal(acc, Xq.astype(np.int32) @ Wq.astype(np.int32).T)
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
# ... and that benchmark's own per-tensor pipeline on the same tensors (int8_bench.py:19-25, 42-45)
bqx, bsx, _ = ib.quantize_to_int8(X)
bqw, bsw, _ = ib.quantize_to_int8(Wc)
by = ib.int8_matmul_reference(bqx, np.ascontiguousarray(bqw.T), bsx, bsw)
cfg1 = {"s_x": float(s_x), "s_w_sha256": sha(s_w), "s_w_first": [float(v) for v in s_w[:4]],
        "Wq_sha256": sha(Wq), "Wq_minus128": int((Wq == -128).sum()), "Xq_sha256": sha(Xq),
        "acc_sha256": sha(acc), "acc_sum": int(acc.astype(np.int64).sum()),
        "fake_quant_W_sha256": sha(np.asarray(fqw.forward(Wc), dtype=np.float32)),
        "bench_sx": float(bsx), "bench_sw": float(bsw), "bench_qx_sha256": sha(bqx), "bench_qw_sha256": sha(bqw),
        "bench_y_sha256": sha(np.asarray(by, dtype=np.float32)), "bench_y_dtype": str(np.asarray(by).dtype)}
(HERE / "config1_golden.json").write_text(json.dumps(cfg1, indent=1))
print("wrote", HERE / "quant_golden.npz", (HERE / "quant_golden.npz").stat().st_size, "bytes;", cfg1)
