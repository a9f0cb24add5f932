"""Post-training INT8 quantization front-end (host side, numpy).

API-compatible with the reference's ``zenith.optimization.quantization`` (same class and function
names, constructor arguments and numeric results; zenith/optimization/quantization.py:24-561), so
calibration code written against the reference runs unchanged and produces the scale tables the
sm_100a kernels of this package consume.  Nothing here touches the device: calibration is the
cold path, the kernels take scales as inputs.

Numeric conventions kept from the reference (they differ from the QAT module on purpose):
  * symmetric scale = absmax / 127 (quantization.py:101-107);
  * ``QuantizationParams.quantize`` truncates toward zero (``clip(...).astype(int8)``,
    quantization.py:49-53) — the device equivalent is ``round="trunc"``.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from enum import Enum

import numpy as np

__all__ = [
    "QuantizationMode", "CalibrationMethod", "QuantizationParams", "TensorStats", "Calibrator",
    "MinMaxCalibrator", "PercentileCalibrator", "EntropyCalibrator", "QuantizationModel", "Quantizer",
    "QATSimulator", "quantize_model_static", "measure_quantization_error", "quantize", "dequantize",
]

_INT8_MIN, _INT8_MAX = -128, 127


class QuantizationMode(Enum):
    STATIC = "static"
    DYNAMIC = "dynamic"
    QAT = "qat"


class CalibrationMethod(Enum):
    MINMAX = "minmax"
    PERCENTILE = "percentile"
    ENTROPY = "entropy"


@dataclass
class QuantizationParams:
    """Scale / zero point of one tensor (quantization.py:40-57)."""

    scale: float
    zero_point: int
    dtype: str = "int8"
    symmetric: bool = True

    def quantize(self, tensor: np.ndarray) -> np.ndarray:
        # astype(int8) after the clip drops the fraction: truncation toward zero
        return np.clip(tensor / self.scale + self.zero_point, _INT8_MIN, _INT8_MAX).astype(np.int8)

    def dequantize(self, tensor: np.ndarray) -> np.ndarray:
        return (tensor.astype(np.float32) - self.zero_point) * self.scale


@dataclass
class TensorStats:
    """Running min / max and a 2048-bin histogram over calibration batches (quantization.py:60-83)."""

    min_val: float = float("inf")
    max_val: float = float("-inf")
    histogram: np.ndarray | None = None
    num_bins: int = 2048

    def update(self, tensor: np.ndarray) -> None:
        self.min_val = min(self.min_val, float(np.min(tensor)))
        self.max_val = max(self.max_val, float(np.max(tensor)))
        if self.histogram is None:
            self.histogram = np.zeros(self.num_bins, dtype=np.int64)
        # the histogram range follows the running extrema, as in the reference
        span = (self.min_val, self.max_val) if self.min_val < self.max_val else (0, 1)
        counts, _ = np.histogram(np.ravel(tensor), bins=self.num_bins, range=span)
        self.histogram += counts


class Calibrator(ABC):
    @abstractmethod
    def compute_params(self, stats: TensorStats) -> QuantizationParams:
        ...


def _symmetric_params(abs_max: float) -> QuantizationParams:
    return QuantizationParams(scale=abs_max / 127.0 if abs_max > 0 else 1.0, zero_point=0, symmetric=True)


def _unsigned_params(upper: float) -> QuantizationParams:
    return QuantizationParams(scale=upper / 255.0 if upper > 0 else 1.0, zero_point=0, symmetric=False)


class MinMaxCalibrator(Calibrator):
    """Observed extrema (quantization.py:95-116)."""

    def __init__(self, symmetric: bool = True):
        self.symmetric = symmetric

    def compute_params(self, stats: TensorStats) -> QuantizationParams:
        if self.symmetric:
            return _symmetric_params(max(abs(stats.min_val), abs(stats.max_val)))
        scale = (stats.max_val - stats.min_val) / 255.0
        if not scale > 0:
            scale = 1.0
        zp = int(np.clip(int(-stats.min_val / scale), _INT8_MIN, _INT8_MAX))
        return QuantizationParams(scale=scale, zero_point=zp, symmetric=False)


class PercentileCalibrator(Calibrator):
    """Clip at a percentile of the calibration histogram (quantization.py:119-150)."""

    def __init__(self, percentile: float = 99.99, symmetric: bool = True):
        self.percentile = percentile
        self.symmetric = symmetric

    def compute_params(self, stats: TensorStats) -> QuantizationParams:
        if stats.histogram is None:
            return MinMaxCalibrator(self.symmetric).compute_params(stats)
        running = np.cumsum(stats.histogram)
        first_bin = np.searchsorted(running, running[-1] * (self.percentile / 100.0))
        width = (stats.max_val - stats.min_val) / len(stats.histogram)
        upper = stats.min_val + (first_bin + 1) * width
        return _symmetric_params(upper) if self.symmetric else _unsigned_params(upper)


class EntropyCalibrator(Calibrator):
    """KL-divergence threshold search over the histogram (quantization.py:153-214)."""

    def __init__(self, symmetric: bool = True):
        self.symmetric = symmetric

    def compute_params(self, stats: TensorStats) -> QuantizationParams:
        if stats.histogram is None:
            return MinMaxCalibrator(self.symmetric).compute_params(stats)
        hist = stats.histogram.astype(np.float64)
        hist = hist / (np.sum(hist) + 1e-10)
        nbins = len(hist)
        best_kl, best_t = float("inf"), nbins
        levels = np.arange(129)
        for t in range(128, nbins):
            ref = hist[:t]
            if np.sum(ref) == 0:
                continue
            # 128 coarse bins with the reference's integer edges int(i * t / 128), last edge capped at t
            edges = np.minimum((levels * (t / 128.0)).astype(np.int64), t)
            widths = np.diff(edges)
            mass = np.array([np.sum(ref[edges[i]:edges[i + 1]]) for i in range(128)], dtype=np.float64)
            spread = np.zeros(t, dtype=np.float64)
            for i in range(128):
                if widths[i] > 0:
                    spread[edges[i]:edges[i + 1]] = mass[i] / widths[i]
            keep = (ref > 0) & (spread > 0)
            if not np.any(keep):
                continue
            kl = np.sum(ref[keep] * np.log(ref[keep] / spread[keep]))
            if kl < best_kl:
                best_kl, best_t = kl, t
        width = (stats.max_val - stats.min_val) / nbins
        upper = stats.min_val + best_t * width
        return _symmetric_params(upper) if self.symmetric else _unsigned_params(upper)


class QuantizationModel:
    """Quantized weights plus the parameter tables of a model (quantization.py:217-269)."""

    def __init__(self, name: str = "quantized_model"):
        self.name = name
        self.weight_params: dict[str, QuantizationParams] = {}
        self.activation_params: dict[str, QuantizationParams] = {}
        self.quantized_weights: dict[str, np.ndarray] = {}

    def add_weight(self, name: str, weight: np.ndarray, params: QuantizationParams) -> None:
        self.weight_params[name] = params
        self.quantized_weights[name] = params.quantize(weight)

    def add_activation_params(self, name: str, params: QuantizationParams) -> None:
        self.activation_params[name] = params

    def quantize_activation(self, name: str, tensor: np.ndarray) -> np.ndarray:
        params = self.activation_params.get(name)
        if params is not None:
            return params.quantize(tensor)
        # unknown activation: dynamic per-tensor scale, truncating cast as in the reference
        peak = np.max(np.abs(tensor))
        return (tensor / (peak / 127.0 if peak > 0 else 1.0)).astype(np.int8)

    def get_weight(self, name: str) -> np.ndarray:
        return self.quantized_weights.get(name)

    def get_weight_dequantized(self, name: str) -> np.ndarray | None:
        if name not in self.quantized_weights:
            return None
        return self.weight_params[name].dequantize(self.quantized_weights[name])


_CALIBRATORS = {
    CalibrationMethod.MINMAX: lambda sym: MinMaxCalibrator(sym),
    CalibrationMethod.PERCENTILE: lambda sym: PercentileCalibrator(symmetric=sym),
    CalibrationMethod.ENTROPY: lambda sym: EntropyCalibrator(sym),
}


def _make_calibrator(method, symmetric: bool) -> Calibrator:
    return _CALIBRATORS.get(method, _CALIBRATORS[CalibrationMethod.MINMAX])(symmetric)


def _stats_of(tensor: np.ndarray) -> TensorStats:
    stats = TensorStats()
    stats.update(tensor)
    return stats


class Quantizer:
    """Collects activation statistics and produces a ``QuantizationModel`` (quantization.py:272-369)."""

    def __init__(self, mode: QuantizationMode = QuantizationMode.STATIC,
                 calibration_method: CalibrationMethod = CalibrationMethod.MINMAX, symmetric: bool = True):
        self.mode = mode
        self.calibration_method = calibration_method
        self.symmetric = symmetric
        self.tensor_stats: dict[str, TensorStats] = {}
        self._calibrator = _make_calibrator(calibration_method, symmetric)

    def collect_stats(self, tensor: np.ndarray, name: str) -> None:
        self.tensor_stats.setdefault(name, TensorStats()).update(tensor)

    def compute_params(self, name: str) -> QuantizationParams | None:
        stats = self.tensor_stats.get(name)
        return None if stats is None else self._calibrator.compute_params(stats)

    def quantize_weights(self, weights: dict[str, np.ndarray]) -> QuantizationModel:
        model = QuantizationModel()
        for name, weight in weights.items():
            model.add_weight(name, weight, self._calibrator.compute_params(_stats_of(weight)))
        for name, stats in self.tensor_stats.items():
            model.add_activation_params(name, self._calibrator.compute_params(stats))
        return model

    def quantize_tensor(self, tensor: np.ndarray, name: str | None = None) -> tuple[np.ndarray, QuantizationParams]:
        stats = self.tensor_stats[name] if name and name in self.tensor_stats else _stats_of(tensor)
        params = self._calibrator.compute_params(stats)
        return params.quantize(tensor), params


class QATSimulator:
    """Quantize-dequantize simulation on top of ``Quantizer`` (quantization.py:372-428)."""

    def __init__(self, calibration_method: CalibrationMethod = CalibrationMethod.MINMAX, symmetric: bool = True):
        self.quantizer = Quantizer(mode=QuantizationMode.QAT, calibration_method=calibration_method,
                                   symmetric=symmetric)

    def fake_quantize(self, tensor: np.ndarray, name: str | None = None) -> np.ndarray:
        q, params = self.quantizer.quantize_tensor(tensor, name)
        return params.dequantize(q)

    def simulate_forward(self, weight: np.ndarray, activation: np.ndarray, weight_name: str | None = None,
                         activation_name: str | None = None) -> np.ndarray:
        w = self.fake_quantize(weight, weight_name)
        a = self.fake_quantize(activation, activation_name)
        return np.matmul(a, w)

    def get_quantized_model(self, weights: dict[str, np.ndarray]) -> QuantizationModel:
        return self.quantizer.quantize_weights(weights)


def quantize_model_static(weights: dict[str, np.ndarray], calibration_data: list[np.ndarray],
                          activation_names: list[str] | None = None,
                          method: CalibrationMethod = CalibrationMethod.MINMAX) -> QuantizationModel:
    """Static PTQ in one call (quantization.py:431-460)."""
    quantizer = Quantizer(mode=QuantizationMode.STATIC, calibration_method=method)
    if activation_names:
        for i, batch in enumerate(calibration_data):
            quantizer.collect_stats(batch, activation_names[i] if i < len(activation_names) else f"act_{i}")
    return quantizer.quantize_weights(weights)


def measure_quantization_error(original: np.ndarray, quantized_model: QuantizationModel, weight_name: str) -> dict:
    """MSE, max abs error and SNR of one dequantized weight (quantization.py:463-493)."""
    restored = quantized_model.get_weight_dequantized(weight_name)
    if restored is None:
        return {"error": "Weight not found"}
    mse = float(np.mean((original - restored) ** 2))
    snr = 10 * np.log10(np.mean(original**2) / (mse + 1e-10))
    return {"mse": mse, "max_abs_error": float(np.max(np.abs(original - restored))), "snr_db": float(snr)}


def quantize(tensor: np.ndarray, num_bits: int = 8, method: CalibrationMethod = CalibrationMethod.MINMAX,
             symmetric: bool = True) -> tuple[np.ndarray, float, int]:
    """``(int8 tensor, scale, zero_point)`` of one tensor (quantization.py:496-538)."""
    calibrator = (MinMaxCalibrator(symmetric) if method == CalibrationMethod.MINMAX
                  else PercentileCalibrator(symmetric=symmetric) if method == CalibrationMethod.PERCENTILE
                  else EntropyCalibrator(symmetric))
    params = calibrator.compute_params(_stats_of(tensor))
    return params.quantize(tensor), params.scale, params.zero_point


def dequantize(tensor: np.ndarray, scale: float, zero_point: int = 0) -> np.ndarray:
    """Inverse of ``quantize`` (quantization.py:541-561)."""
    return QuantizationParams(scale=scale, zero_point=zero_point).dequantize(tensor)
