"""Calibration reductions on the device against numpy: running min / max, per-row absmax and the per-channel
int8 conversion are exact (they select among, or divide and round, the same fp32 values)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import _capi, ops
from zenith_b200.calibrate import quantize_weights, quantize_weights_on_device
from zenith_b200.encoder import EncoderConfig, Fp16Encoder, init_params

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("n,offset", [(1, 0), (7, 0), (4096, 0), (100003, 0), (100003, 3), (3_000_001, 1)])
def test_range_observer_is_exact(cuda, dtype, n, offset):
    x = (rng(n).standard_normal(n + offset) * 3).astype(dtype)
    t = torch.from_numpy(x).to(cuda)[offset:]  # offset: a start address that is not 16-byte aligned
    obs = ops.RangeObserver(cuda)
    obs.observe(t)
    assert obs.range() == (float(x[offset:].min()), float(x[offset:].max()))
    # a second tensor only widens the range; NaNs are skipped
    y = (rng(n + 1).standard_normal(1000) * 10).astype(dtype)
    y[::7] = np.nan
    obs.observe(torch.from_numpy(y).to(cuda))
    lo = min(float(x[offset:].min()), float(np.nanmin(y)))
    hi = max(float(x[offset:].max()), float(np.nanmax(y)))
    assert obs.range() == (lo, hi)
    assert _capi.device_status() == 0


def test_range_observer_rejects_what_it_cannot_read(cuda):
    obs = ops.RangeObserver(cuda)
    with pytest.raises(RuntimeError):
        obs.observe(torch.zeros(4))
    with pytest.raises(RuntimeError):
        obs.observe(torch.zeros(4, dtype=torch.int32, device=cuda))
    obs.observe(torch.zeros(0, dtype=torch.float32, device=cuda))  # nothing to see: the range stays empty
    assert obs.range() == (float("inf"), float("-inf"))


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 7), (768, 768), (3072, 770), (33, 4096)])
def test_per_channel_observer_and_conversion(cuda, rows, cols):
    w = (rng(rows * cols).standard_normal((rows, cols)) * 0.02).astype(np.float32)
    w[0, 0] = -1.0  # the peak of a row may be negative
    t = torch.from_numpy(w).to(cuda)
    peak = ops.absmax_rows(t).cpu().numpy()
    assert np.array_equal(peak, np.abs(w).max(axis=1))
    scale = np.maximum(peak / np.float32(127.5), np.float32(1e-8)).astype(np.float32)
    q = ops.quantize_rows(t, torch.from_numpy(scale).to(cuda)).cpu().numpy()
    want = np.stack([O.quantize(w[r], float(scale[r])) for r in range(rows)])
    assert np.array_equal(q, want)
    # a row view with a stride (columns of a wider matrix)
    wide = torch.from_numpy(np.concatenate([w, w], axis=1)).to(cuda)
    assert np.array_equal(ops.absmax_rows(wide[:, :cols]).cpu().numpy(), peak)
    assert _capi.device_status() == 0


def test_device_weight_quantization_equals_the_numpy_front_end(cuda):
    cfg = EncoderConfig(layers=2, hidden=128, heads=2, ffn=256, vocab=500, max_pos=64)
    params = init_params(cfg, 3)
    host = quantize_weights(params)
    dev = quantize_weights_on_device(params, cuda)
    for a, b in zip(host, dev):
        for k in a:
            assert np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1])


def test_ranges_accumulate_over_passes(cuda):
    cfg = EncoderConfig(layers=2, hidden=128, heads=2, ffn=256, vocab=500, max_pos=64)
    params = init_params(cfg, 3, random_affine=True)
    enc = Fp16Encoder(cfg, params, cuda)
    batches = [(torch.from_numpy(rng(s).integers(0, cfg.vocab, (3, 48))).to(cuda), None) for s in range(3)]
    single = [enc.forward_with_taps(i, l) for i, l in batches]
    observers = enc.make_observers()
    for i, l in batches:
        assert enc.forward_with_taps(i, l, observers) is None
    for p, per_layer in observers.items():
        for li, o in enumerate(per_layer):
            lo = min(s[p][li][0] for s in single)
            hi = max(s[p][li][1] for s in single)
            assert o.range() == (lo, hi)
