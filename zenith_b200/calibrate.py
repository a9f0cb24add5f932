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


def calibrate(cfg: EncoderConfig, params: dict, batches, device="cuda:0") -> Int8Scales:
    """``batches``: iterable of ``(ids [B,S] integer tensor, kv_lens [B] int32 tensor or None)``."""
    enc = Fp16Encoder(cfg, params, device)
    ranges = {p: [[] for _ in range(cfg.layers)] for p in ACT_POINTS}
    for ids, kv_lens in batches:
        taps = enc.forward_with_taps(ids, kv_lens)
        for p in ACT_POINTS:
            for li, mm in enumerate(taps[p]):
                ranges[p][li].append(mm)
    return Int8Scales(act=activation_scales_from_ranges(ranges, cfg.layers), weights=quantize_weights(params))
