"""The running histogram kept on the device (zen_histogram_*) against the reference's own TensorStats: the golden
histogram tests/golden/quant_golden.npz holds was produced by the reference's code (tests/golden/make_golden.py),
and the percentile / entropy calibrators fed with the device statistics give the reference's scales."""
from pathlib import Path

import numpy as np
import pytest
import torch

from zenith_b200 import _capi, ops
from zenith_b200 import quantization as Q

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "quant_golden.npz")


def rng(seed):
    return np.random.default_rng(seed)


def batches():
    # the three calibration tensors of make_golden.py
    return [(rng(s).standard_normal((64, 96)) * (1 + 0.3 * (s - 12))).astype(np.float32) for s in (12, 13, 14)]


def test_device_histogram_equals_the_reference_statistics(cuda):
    obs = ops.HistogramObserver(cuda)
    for b in batches():
        obs.observe(torch.from_numpy(b).to(cuda))
    st = obs.stats()
    assert np.array_equal(np.array([st.min_val, st.max_val]), GOLD["ptq_stats_minmax"])
    assert st.histogram.dtype == np.int64 and np.array_equal(st.histogram, GOLD["ptq_stats_hist"])
    for name, cal in (("minmax_sym", Q.MinMaxCalibrator(True)), ("pct_sym", Q.PercentileCalibrator(99.9, True)),
                      ("pct_asym", Q.PercentileCalibrator(99.0, False)), ("ent_sym", Q.EntropyCalibrator(True)),
                      ("ent_asym", Q.EntropyCalibrator(False))):
        p = cal.compute_params(st)
        assert np.array_equal(np.array([p.scale, p.zero_point], dtype=np.float64), GOLD[f"ptq_cal_{name}"]), name
    assert _capi.device_status() == 0


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n,bins", [(1, 2048), (1000, 2048), (1_000_003, 2048), (4097, 128), (70_000, 4096)])
def test_device_histogram_equals_numpy(cuda, dtype, n, bins):
    """Several updates with a growing range, NaNs and values on bin edges; numpy sees the same values as float32."""
    obs = ops.HistogramObserver(cuda, num_bins=bins)
    ref = Q.TensorStats(num_bins=bins)
    for k in range(3):
        x = (rng(n + k).standard_normal(n) * (1 + k)).astype(dtype)
        if n > 10:
            x[3] = np.nan
            x[5], x[6] = np.nanmin(x), np.nanmax(x)  # values on the outer edges, twice
        xs = x.astype(np.float32)
        # numpy's min / max would propagate the NaN; the observers skip it, so the reference sees the tensor without it
        clean = xs[~np.isnan(xs)]
        ref.update(clean)
        obs.observe(torch.from_numpy(x).to(cuda))
    st = obs.stats()
    assert st.min_val == ref.min_val and st.max_val == ref.max_val
    assert np.array_equal(st.histogram, ref.histogram)
    assert int(st.histogram.sum()) == int(ref.histogram.sum())


def test_constant_tensor_uses_the_unit_range(cuda):
    obs = ops.HistogramObserver(cuda)
    x = np.full(500, 0.25, np.float32)
    obs.observe(torch.from_numpy(x).to(cuda))
    ref = Q.TensorStats()
    ref.update(x)
    assert np.array_equal(obs.stats().histogram, ref.histogram)  # min == max: binned over (0, 1) like the reference


def test_encoder_calibration_with_percentile_and_entropy(cuda):
    """The encoder's calibration pass with the histogram observers: the scales come out of the reference's
    calibrators, differ from the min-max ones the way clipping must (never larger), and the int8 encoder built from
    them still tracks the fp16 encoder."""
    from zenith_b200.calibrate import calibrate
    from zenith_b200.encoder import EncoderConfig, Fp16Encoder, Int8Encoder, init_params

    cfg = EncoderConfig(layers=2, hidden=256, heads=4, ffn=512, vocab=2000, max_pos=128)
    params = init_params(cfg, 7, random_affine=True)
    mk = lambda s: (torch.from_numpy(rng(s).integers(0, cfg.vocab, (4, 96))).to(cuda), torch.tensor([96, 80, 64, 96], dtype=torch.int32, device=cuda))
    cal = [mk(s) for s in range(3)]
    mm = calibrate(cfg, params, cal, cuda)
    pct = calibrate(cfg, params, cal, cuda, method="percentile", percentile=99.9)
    ent = calibrate(cfg, params, cal, cuda, method="entropy")
    for li in range(cfg.layers):
        for k, v in mm.act[li].items():
            assert 0 < pct.act[li][k] <= v * 1.001  # clipping never widens the range
            # The reference's entropy search measures its threshold from min_val (quantization.py:206-207); on a range
            # that starts below zero it can end at or below zero and then falls back to scale 1.0.  Whatever it
            # returns, it is what its calibrator computes from the statistics gathered on the device.
            assert ent.act[li][k] > 0 and np.isfinite(ent.act[li][k])
    ids, lens = mk(9)
    want = Fp16Encoder(cfg, params, cuda).forward(ids, lens).float()
    got = Int8Encoder(cfg, params, pct, cuda).forward(ids, lens).float()
    assert (got - want).abs().mean().item() < 0.06
    assert _capi.device_status() == 0
