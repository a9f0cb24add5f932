"""Quantization-aware-training front-end (host side, numpy): observers, fake quantization,
calibration and conversion to real int8.

API-compatible with the reference's ``zenith.optimization.qat`` (zenith/optimization/qat.py:40-813):
``QATScheme``, ``ObserverType``, ``QATConfig``, ``FakeQuantize``, ``QATModule``, ``QATTrainer``,
``prepare_model_for_qat``, ``convert_qat_to_quantized``, ``simulate_qat_forward`` and
``measure_qat_error`` keep their names, arguments and numeric results.  Batch-norm folding (a
CNN training helper of the reference) is not part of the encoder inference path and is absent.

Conventions kept from the reference:
  * symmetric scale = absmax / ((qmax - qmin) / 2) = absmax / 127.5 for 8 bits, floored at 1e-8
    (qat.py:222-228) — note the PTQ module divides by 127;
  * rounding is ``np.round`` (half to even, qat.py:267) — the device equivalent is
    ``round="nearest_even"``;
  * ``observe`` keeps an exponential moving average of min / max after its first call
    (qat.py:205-212), and ``forward`` observes before it quantizes (qat.py:248-249): freeze the
    observers (``disable_observer`` / ``QATModule.freeze_observers``) before snapshotting scales.

One addition on top of the reference: ``FakeQuantize.quantize_int8`` / ``convert_per_channel``
return real int8 weights using the FULL per-channel scale vector.  The reference's
``get_quantization_params`` keeps only channel 0 (qat.py:329-331) and its converter truncates
with that single scale; that behaviour is reproduced unchanged by ``convert_qat_to_quantized``.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import numpy as np

from .quantization import QuantizationParams

__all__ = [
    "QATScheme", "ObserverType", "QATConfig", "FakeQuantize", "QATModule", "QATTrainer",
    "prepare_model_for_qat", "convert_qat_to_quantized", "convert_per_channel", "simulate_qat_forward",
    "measure_qat_error",
]


class QATScheme(Enum):
    PER_TENSOR = "per_tensor"
    PER_CHANNEL = "per_channel"


class ObserverType(Enum):
    MINMAX = "minmax"
    MOVING_AVERAGE = "moving_average"
    HISTOGRAM = "histogram"


@dataclass
class QATConfig:
    """Field names and defaults of the reference's configuration (qat.py:61-92)."""

    weight_bits: int = 8
    activation_bits: int = 8
    weight_scheme: QATScheme = QATScheme.PER_CHANNEL
    activation_scheme: QATScheme = QATScheme.PER_TENSOR
    observer_type: ObserverType = ObserverType.MOVING_AVERAGE
    averaging_constant: float = 0.01
    freeze_bn_after_epochs: int = 0
    start_qat_after_epochs: int = 0
    calibration_batches: int = 100
    per_channel_weights: bool = True
    symmetric_weights: bool = True
    symmetric_activations: bool = True


class FakeQuantize:
    """Observer + quantize-dequantize with a straight-through estimator (qat.py:100-341)."""

    def __init__(self, num_bits: int = 8, symmetric: bool = True, per_channel: bool = False, channel_axis: int = 0,
                 averaging_constant: float = 0.01):
        self.num_bits = num_bits
        self.symmetric = symmetric
        self.per_channel = per_channel
        self.channel_axis = channel_axis
        self.averaging_constant = averaging_constant
        if symmetric:
            self.qmin, self.qmax = -(2 ** (num_bits - 1)), 2 ** (num_bits - 1) - 1
        else:
            self.qmin, self.qmax = 0, 2**num_bits - 1
        self.scale: np.ndarray | None = None
        self.zero_point: np.ndarray | None = None
        self.min_val: np.ndarray | None = None
        self.max_val: np.ndarray | None = None
        self.enabled = True
        self.observer_enabled = True

    # -- switches ---------------------------------------------------------------------------
    def enable(self) -> None:
        self.enabled = True

    def disable(self) -> None:
        self.enabled = False

    def enable_observer(self) -> None:
        self.observer_enabled = True

    def disable_observer(self) -> None:
        self.observer_enabled = False

    def reset_stats(self) -> None:
        self.min_val = self.max_val = self.scale = self.zero_point = None

    # -- observation ------------------------------------------------------------------------
    def observe(self, x: np.ndarray) -> None:
        if not self.observer_enabled:
            return
        if self.per_channel:
            other_axes = tuple(a for a in range(x.ndim) if a != self.channel_axis)
            lo, hi = np.min(x, axis=other_axes), np.max(x, axis=other_axes)
        else:
            lo, hi = np.array([np.min(x)]), np.array([np.max(x)])
        if self.min_val is None:
            self.min_val, self.max_val = lo, hi
        else:
            a = self.averaging_constant
            self.min_val = (1 - a) * self.min_val + a * lo
            self.max_val = (1 - a) * self.max_val + a * hi
        self._compute_qparams()

    def _compute_qparams(self) -> None:
        if self.min_val is None or self.max_val is None:
            return
        if self.symmetric:
            peak = np.maximum(np.abs(self.min_val), np.abs(self.max_val))
            self.scale = np.maximum(peak / ((self.qmax - self.qmin) / 2), 1e-8)
            self.zero_point = np.zeros_like(self.scale, dtype=np.int32)
        else:
            self.scale = np.maximum((self.max_val - self.min_val) / (self.qmax - self.qmin), 1e-8)
            zp = np.round(self.qmin - self.min_val / self.scale).astype(np.int32)
            self.zero_point = np.clip(zp, self.qmin, self.qmax)

    # -- quantization -----------------------------------------------------------------------
    def _broadcast_qparams(self, ndim: int):
        if self.per_channel:
            shape = [1] * ndim
            shape[self.channel_axis] = -1
            return self.scale.reshape(shape), self.zero_point.reshape(shape)
        return self.scale[0], self.zero_point[0]

    def forward(self, x: np.ndarray) -> np.ndarray:
        self.observe(x)
        if not self.enabled or self.scale is None:
            return x
        scale, zp = self._broadcast_qparams(x.ndim)
        levels = np.clip(np.round(x / scale) + zp, self.qmin, self.qmax)
        return (levels - zp) * scale

    def forward_with_ste(self, x: np.ndarray, grad_output: np.ndarray | None = None):
        out = self.forward(x)
        if grad_output is None:
            return out, None
        if self.scale is None:
            return out, grad_output
        scale, zp = self._broadcast_qparams(x.ndim)
        raw = np.round(x / scale) + zp
        inside = (raw >= self.qmin) & (raw <= self.qmax)
        return out, grad_output * inside.astype(grad_output.dtype)

    def quantize_int8(self, x: np.ndarray) -> np.ndarray:
        """Integer levels ``clip(round(x / scale) + zp)`` with the full (per-channel) scale, as int8.

        Same arithmetic as the quantize half of ``forward`` (qat.py:267), without observing.
        """
        if self.scale is None:
            raise RuntimeError("FakeQuantize has not observed any tensor yet")
        if self.num_bits != 8 or not self.symmetric:
            raise RuntimeError("int8 conversion needs the symmetric 8-bit scheme")
        scale, zp = self._broadcast_qparams(x.ndim)
        return np.clip(np.round(x / scale) + zp, self.qmin, self.qmax).astype(np.int8)

    def get_quantization_params(self) -> QuantizationParams | None:
        if self.scale is None:
            return None
        # the reference reports a single (scale, zero_point): element 0, also for per-channel
        return QuantizationParams(scale=float(np.asarray(self.scale).flat[0]),
                                  zero_point=int(np.asarray(self.zero_point).flat[0]),
                                  dtype=f"int{self.num_bits}", symmetric=self.symmetric)


class QATModule:
    """Weight and activation fake-quantizers of one layer (qat.py:349-412)."""

    def __init__(self, weight_shape: tuple, config: QATConfig = QATConfig(), has_bias: bool = True):
        self.config = config
        self.weight_shape = weight_shape
        self.has_bias = has_bias
        self.weight_fake_quant = FakeQuantize(num_bits=config.weight_bits, symmetric=config.symmetric_weights,
                                              per_channel=config.per_channel_weights, channel_axis=0)
        self.activation_fake_quant = FakeQuantize(num_bits=config.activation_bits,
                                                  symmetric=config.symmetric_activations, per_channel=False)
        self.bias_fake_quant = None

    def fake_quantize_weight(self, weight: np.ndarray) -> np.ndarray:
        return self.weight_fake_quant.forward(weight)

    def fake_quantize_activation(self, activation: np.ndarray) -> np.ndarray:
        return self.activation_fake_quant.forward(activation)

    def freeze_observers(self) -> None:
        self.weight_fake_quant.disable_observer()
        self.activation_fake_quant.disable_observer()

    def enable_fake_quant(self) -> None:
        self.weight_fake_quant.enable()
        self.activation_fake_quant.enable()

    def disable_fake_quant(self) -> None:
        self.weight_fake_quant.disable()
        self.activation_fake_quant.disable()


class QATTrainer:
    """Registers layers, calibrates them and applies fake quantization (qat.py:531-678)."""

    def __init__(self, config: QATConfig = QATConfig()):
        self.config = config
        self.qat_modules: dict[str, QATModule] = {}
        self.epoch = 0
        self.calibration_complete = False

    def register_layer(self, name: str, weight_shape: tuple, has_bias: bool = True) -> QATModule:
        module = QATModule(weight_shape, self.config, has_bias)
        self.qat_modules[name] = module
        return module

    def calibrate(self, layer_name: str, weight: np.ndarray, activations: list[np.ndarray]) -> None:
        if layer_name not in self.qat_modules:
            raise ValueError(f"Layer '{layer_name}' not registered")
        module = self.qat_modules[layer_name]
        module.weight_fake_quant.observe(weight)
        for act in activations:
            module.activation_fake_quant.observe(act)

    def start_epoch(self, epoch: int) -> None:
        self.epoch = epoch
        active = epoch >= self.config.start_qat_after_epochs
        for module in self.qat_modules.values():
            module.enable_fake_quant() if active else module.disable_fake_quant()
        if epoch >= self.config.freeze_bn_after_epochs > 0:
            for module in self.qat_modules.values():
                module.freeze_observers()

    def fake_quantize_weights(self, weights: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
        return {name: self.qat_modules[name].fake_quantize_weight(w) if name in self.qat_modules else w
                for name, w in weights.items()}

    def fake_quantize_activation(self, layer_name: str, activation: np.ndarray) -> np.ndarray:
        module = self.qat_modules.get(layer_name)
        return activation if module is None else module.fake_quantize_activation(activation)

    def get_quantization_params(self) -> dict[str, dict[str, QuantizationParams]]:
        return {name: {"weight": m.weight_fake_quant.get_quantization_params(),
                       "activation": m.activation_fake_quant.get_quantization_params()}
                for name, m in self.qat_modules.items()}


def prepare_model_for_qat(layer_shapes: dict[str, tuple], config: QATConfig = QATConfig()) -> QATTrainer:
    trainer = QATTrainer(config)
    for name, shape in layer_shapes.items():
        trainer.register_layer(name, shape)
    return trainer


def _dynamic_params(weight: np.ndarray) -> QuantizationParams:
    peak = np.max(np.abs(weight))
    return QuantizationParams(scale=peak / 127.0 if peak > 0 else 1.0, zero_point=0)


def convert_qat_to_quantized(trainer: QATTrainer,
                             weights: dict[str, np.ndarray]) -> dict[str, tuple[np.ndarray, QuantizationParams]]:
    """The reference's converter, unchanged in behaviour (qat.py:708-748): one scale per layer
    (channel 0 of a per-channel observer) and the truncating ``QuantizationParams.quantize``."""
    result = {}
    for name, weight in weights.items():
        params = None
        if name in trainer.qat_modules:
            params = trainer.qat_modules[name].weight_fake_quant.get_quantization_params()
        if params is None:
            params = _dynamic_params(weight)
        result[name] = (params.quantize(weight), params)
    return result


def convert_per_channel(trainer: QATTrainer, weights: dict[str, np.ndarray]) -> dict[str, tuple[np.ndarray, np.ndarray]]:
    """``name -> (int8 weight, float32 scale vector)`` using every channel's scale and the
    observer's own rounding: ``Wq[n,k] = clip(rint(W[n,k] / s[n]), -128, 127)``.  These are the
    operands the W8A8 kernels take."""
    out = {}
    for name, weight in weights.items():
        fq = trainer.qat_modules[name].weight_fake_quant
        out[name] = (fq.quantize_int8(weight), np.asarray(fq.scale, dtype=np.float32).reshape(-1))
    return out


def simulate_qat_forward(trainer: QATTrainer, layer_name: str, weight: np.ndarray, activation: np.ndarray) -> np.ndarray:
    """Fake-quantized ``activation @ weight.T`` (qat.py:751-776)."""
    w = trainer.fake_quantize_weights({layer_name: weight})[layer_name]
    a = trainer.fake_quantize_activation(layer_name, activation)
    return np.matmul(a, w.T)


def measure_qat_error(original_output: np.ndarray, qat_output: np.ndarray) -> dict[str, float]:
    """MSE / MAE / max error / SNR / mean relative error (qat.py:779-813)."""
    diff = original_output - qat_output
    mse = float(np.mean(diff**2))
    snr = 10 * np.log10(np.mean(original_output**2) / (mse + 1e-10))
    return {
        "mse": mse,
        "mae": float(np.mean(np.abs(diff))),
        "max_error": float(np.max(np.abs(diff))),
        "snr_db": float(snr),
        "relative_error": float(np.mean(np.abs(diff) / (np.abs(original_output) + 1e-10))),
    }
