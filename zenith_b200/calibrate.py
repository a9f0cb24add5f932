"""Calibration of the W8A8 encoder: per-output-channel int8 weights and per-tensor activation scales.

Cold path.  Weights go through the QAT front-end exactly as a user of the reference would do it
(``QATTrainer.calibrate`` observing each weight once, zenith/optimization/qat.py:576-600, then the
observers are frozen); activation ranges are true running min / max over the calibration batches,
fed to ``Quantizer.collect_stats`` / ``MinMaxCalibrator`` (zenith/optimization/quantization.py:
95-116, 311-321).  The activations themselves come from one fp16 pass of the encoder per batch on
the device.
"""
from __future__ import annotations

import numpy as np

from .encoder import ACT_POINTS, LAYER_WEIGHTS, EncoderConfig, Fp16Encoder, Int8Scales
from .qat import QATConfig, convert_per_channel, prepare_model_for_qat
from .quantization import CalibrationMethod, QuantizationMode, Quantizer


def quantize_weights(params: dict) -> list:
    """``[{name: (int8 [N,K], float32 scale [N])}]`` per layer, symmetric per-output-channel."""
    out = []
    for lp in params["layers"]:
        weights = {k: lp[k] for k in LAYER_WEIGHTS}
        trainer = prepare_model_for_qat({k: w.shape for k, w in weights.items()}, QATConfig())
        for k, w in weights.items():
            trainer.calibrate(k, w, [])
            trainer.qat_modules[k].freeze_observers()
        out.append(convert_per_channel(trainer, weights))
    return out


def activation_scales_from_ranges(ranges: dict, n_layers: int) -> list:
    """``ranges[point][layer]`` = list of (min, max) per batch -> per-layer scale dicts (absmax / 127)."""
    quantizer = Quantizer(mode=QuantizationMode.STATIC, calibration_method=CalibrationMethod.MINMAX, symmetric=True)
    for point in ACT_POINTS:
        for li in range(n_layers):
            for lo, hi in ranges[point][li]:
                quantizer.collect_stats(np.array([lo, hi], dtype=np.float32), f"layer{li}.{point}")
    return [{point: float(quantizer.compute_params(f"layer{li}.{point}").scale) for point in ACT_POINTS}
            for li in range(n_layers)]


def activation_scales_from_stats(stats: dict, n_layers: int, method: CalibrationMethod, percentile: float = 99.99) -> list:
    """``stats[point][layer]`` = ``TensorStats`` (range + histogram) -> per-layer scale dicts through the
    reference's calibrators (zenith/optimization/quantization.py:95-214), symmetric."""
    from .quantization import EntropyCalibrator, MinMaxCalibrator, PercentileCalibrator

    cal = {CalibrationMethod.MINMAX: MinMaxCalibrator(True), CalibrationMethod.PERCENTILE: PercentileCalibrator(percentile, True),
           CalibrationMethod.ENTROPY: EntropyCalibrator(True)}[method]
    return [{point: float(cal.compute_params(stats[point][li]).scale) for point in ACT_POINTS} for li in range(n_layers)]


def calibrate(cfg: EncoderConfig, params: dict, batches, device="cuda:0", method: CalibrationMethod | str = CalibrationMethod.MINMAX,
              percentile: float = 99.99) -> Int8Scales:
    """``batches``: iterable of ``(ids [B,S] integer tensor, kv_lens [B] int32 tensor or None)``.

    The activation statistics accumulate on the device over all batches and are read back once: the running min /
    max (``ops.RangeObserver``, the statistic of ``TensorStats.update``) for min-max calibration - min / max select
    among the inputs, so the scales are those the per-batch host observers would give - and, for ``method``
    "percentile" / "entropy", also the running 2048-bin histogram (``ops.HistogramObserver``), which the reference's
    calibrators then turn into a clipping range."""
    method = CalibrationMethod(method) if not isinstance(method, CalibrationMethod) else method
    enc = Fp16Encoder(cfg, params, device)
    observers = enc.make_observers(histogram=method != CalibrationMethod.MINMAX)
    for ids, kv_lens in batches:
        enc.forward_with_taps(ids, kv_lens, observers)
    if method == CalibrationMethod.MINMAX:
        ranges = {p: [[observers[p][li].range()] for li in range(cfg.layers)] for p in ACT_POINTS}
        act = activation_scales_from_ranges(ranges, cfg.layers)
    else:
        stats = {p: [observers[p][li].stats() for li in range(cfg.layers)] for p in ACT_POINTS}
        act = activation_scales_from_stats(stats, cfg.layers, method, percentile)
    return Int8Scales(act=act, weights=quantize_weights(params))


def quantize_weights_on_device(params: dict, device="cuda:0") -> list:
    """``quantize_weights`` with the observer and the conversion on the device (``ops.absmax_rows``,
    ``ops.quantize_rows``): same int8 weights and scales, bit for bit (symmetric per-output-channel,
    ``scale = absmax / 127.5`` floored at 1e-8, zenith/optimization/qat.py:222-228)."""
    import torch

    from . import ops

    out = []
    for lp in params["layers"]:
        layer = {}
        for k in LAYER_WEIGHTS:
            w = torch.as_tensor(lp[k], dtype=torch.float32).to(device).contiguous()
            peak = ops.absmax_rows(w)
            # tensor / tensor: a true fp32 division (torch turns a Python-scalar divisor into a reciprocal multiply)
            scale = torch.clamp_min(peak / torch.full_like(peak, 127.5), 1e-8)
            layer[k] = (ops.quantize_rows(w, scale).cpu().numpy(), scale.cpu().numpy())
        out.append(layer)
    return out
