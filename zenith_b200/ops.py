"""Typed operators over ``torch`` CUDA tensors, each one C-ABI call on torch's current stream.

torch is used for device memory and streams only; every computation below runs in the
hand-written sm_100a kernels of ``libzenith_b200.so``.  There is no CPU path: a CPU tensor, a
missing extension or a non-zero status raises.
"""
from __future__ import annotations

import math

import torch

from . import _capi
from ._capi import (ACT_GELU, ACT_NONE, ACT_RELU, DT_F16, DT_F32, DT_S8, DT_S32, ROUND_NEAREST_EVEN,  # noqa: F401
                    ROUND_TRUNC)

_ACT = {"none": ACT_NONE, None: ACT_NONE, "gelu": ACT_GELU, "relu": ACT_RELU}
_ROUND = {"nearest_even": ROUND_NEAREST_EVEN, "trunc": ROUND_TRUNC}
_OUT = {torch.int32: DT_S32, torch.float32: DT_F32, torch.float16: DT_F16, torch.int8: DT_S8}

# number of kernels this module has launched (read by the benchmark's `gpu_launches`)
launch_count = 0


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(t: torch.Tensor, name: str, dtype=None, ndim=None, rows_may_be_strided: bool = False) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError(f"{name} must be {ndim}-D, got {t.dim()}-D")
    if rows_may_be_strided and t.dim() == 2 and (t.shape[1] <= 1 or t.stride(1) == 1) and t.stride(0) >= t.shape[1]:
        return
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def launch_count_add(n: int) -> None:
    global launch_count
    launch_count += n


def _call(fn: str, *args) -> None:
    global launch_count
    _capi.call(fn, *args)
    launch_count += 1


# --------------------------------------------------------------------------------------------
# GEMMs
# --------------------------------------------------------------------------------------------
def _pair_flag(pair) -> int:
    return 0 if pair is None else (_capi.GEMM_PAIR if pair else _capi.GEMM_NO_PAIR)


def linear_int8(xq, wq, x_scale: float, w_scale=None, bias=None, *, act="none", out_dtype=torch.float32,
                out_scale: float | None = None, round="nearest_even", out=None, prefetch=(), constant_weights=False,
                tile_n: int = 0, pair: bool | None = None):
    """W8A8 Linear: ``acc = xq @ wq.T`` in int32, then the fused epilogue.

    ``out_dtype=torch.int32`` returns the raw accumulators.  Otherwise
    ``y = (float(acc) * x_scale) * w_scale[n] + bias[n]``, optional activation, then fp32 / fp16
    output or requantisation ``clamp(round(y / out_scale))`` to int8.
    Follows core/src/cuda_kernels.cu:1010-1049 (fused_int8_linear_kernel) with per-output-channel
    weight scales (zenith/optimization/qat.py:195-199).

    ``prefetch``: up to two CUDA tensors (e.g. the weights of the GEMMs that follow) that the kernel
    hints into L2 while it runs; they are not read and the result does not depend on them.
    ``constant_weights``: promise that ``wq`` is not being written by work still queued on the device
    (``ZEN_GEMM_CONST_WEIGHTS``, for this call only); ``tile_n`` forces the tile width and ``pair`` the choice
    between the CTA-pair kernel (True) and the one-CTA kernel (False); both are benchmark / test hooks.
    """
    _require(xq, "xq", torch.int8, 2)
    _require(wq, "wq", torch.int8, 2)
    M, K = xq.shape
    N, K2 = wq.shape
    if len(prefetch) > 2 or any(not t.is_cuda for t in prefetch):
        raise RuntimeError("prefetch takes at most two CUDA tensors")
    if K != K2:
        raise RuntimeError(f"inner dimensions differ: xq {tuple(xq.shape)} vs wq {tuple(wq.shape)}")
    if w_scale is not None:
        _require(w_scale, "w_scale", torch.float32, 1)
        if w_scale.numel() != N:
            raise RuntimeError("w_scale must have one entry per output channel")
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
        if bias.numel() != N:
            raise RuntimeError("bias must have one entry per output channel")
    if out_dtype not in _OUT:
        raise RuntimeError(f"unsupported out_dtype {out_dtype}")
    if out_dtype == torch.int8 and out_scale is None:
        raise RuntimeError("out_scale is required for int8 output")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    else:
        _require(out, "out", out_dtype, 2)
    if M == 0 or N == 0:
        return out
    hint = [v for t in prefetch for v in (t.data_ptr(), t.numel() * t.element_size())] + [None, 0] * (2 - len(prefetch))
    flags = (_capi.GEMM_CONST_WEIGHTS if constant_weights else 0) | _capi.gemm_tile_n(tile_n) | _pair_flag(pair)
    _call("zen_linear_i8_ex", xq.data_ptr(), K, wq.data_ptr(), K, M, N, K, float(x_scale), _ptr(w_scale),
          _ptr(bias), _ACT[act], _OUT[out_dtype], float(out_scale if out_scale is not None else 1.0), _ROUND[round],
          out.data_ptr(), out.stride(0), *hint, flags, _stream())
    return out


def linear_int8_add_layernorm(xq, wq, x_scale: float, w_scale, bias, residual, gamma, beta, eps: float, *,
                              out_scale: float | None = None, round="nearest_even", constant_weights=False):
    """``LayerNorm(dequant(xq @ wq.T) + bias + residual) * gamma + beta`` in one kernel (hidden size 768).

    Returns fp16 ``y`` and, with ``out_scale``, also the int8 copy ``quantize(y, out_scale)``.
    """
    _require(xq, "xq", torch.int8, 2)
    _require(wq, "wq", torch.int8, 2)
    _require(residual, "residual", torch.float16, 2)
    _require(gamma, "gamma", torch.float16, 1)
    _require(beta, "beta", torch.float16, 1)
    M, K = xq.shape
    N = wq.shape[0]
    if wq.shape[1] != K or tuple(residual.shape) != (M, N):
        raise RuntimeError("shape mismatch")
    if w_scale is not None:
        _require(w_scale, "w_scale", torch.float32, 1)
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    y = torch.empty((M, N), dtype=torch.float16, device=xq.device)
    yq = torch.empty((M, N), dtype=torch.int8, device=xq.device) if out_scale is not None else None
    if M:
        _call("zen_linear_i8_add_layernorm_ex", xq.data_ptr(), K, wq.data_ptr(), K, M, N, K, float(x_scale), _ptr(w_scale),
              _ptr(bias), residual.data_ptr(), N, gamma.data_ptr(), beta.data_ptr(), float(eps), y.data_ptr(), _ptr(yq),
              float(out_scale or 1.0), _ROUND[round], _capi.GEMM_CONST_WEIGHTS if constant_weights else 0, _stream())
    return y if yq is None else (y, yq)


def linear_fp16_add_layernorm(x, w, bias, residual, gamma, beta, eps: float, *, out_scale: float | None = None,
                              round="nearest_even", constant_weights=False):
    """``LayerNorm(x @ w.T + bias + residual) * gamma + beta`` with fp16 operands in one kernel (hidden 768 or
    1024).  Returns fp16 ``y`` and, with ``out_scale``, also ``quantize(y, out_scale)``."""
    _require(x, "x", torch.float16, 2)
    _require(w, "w", torch.float16, 2)
    _require(residual, "residual", torch.float16, 2)
    _require(gamma, "gamma", torch.float16, 1)
    _require(beta, "beta", torch.float16, 1)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(residual.shape) != (M, N):
        raise RuntimeError("shape mismatch")
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    y = torch.empty((M, N), dtype=torch.float16, device=x.device)
    yq = torch.empty((M, N), dtype=torch.int8, device=x.device) if out_scale is not None else None
    if M:
        _call("zen_linear_f16_add_layernorm_ex", x.data_ptr(), K, w.data_ptr(), K, M, N, K, _ptr(bias), residual.data_ptr(), N,
              gamma.data_ptr(), beta.data_ptr(), float(eps), y.data_ptr(), _ptr(yq), float(out_scale or 1.0), _ROUND[round],
              _capi.GEMM_CONST_WEIGHTS if constant_weights else 0, _stream())
    return y if yq is None else (y, yq)


def linear_fp16(x, w, bias=None, *, act="none", out_dtype=torch.float16, out=None, tile_n: int = 0,
                pair: bool | None = None):
    """``act(x @ w.T + bias)`` with fp16 operands, fp32 accumulation (core/src/fp16_kernels.cu:92-122)."""
    _require(x, "x", torch.float16, 2, rows_may_be_strided=True)
    _require(w, "w", torch.float16, 2)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise RuntimeError(f"inner dimensions differ: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    if out_dtype not in (torch.float16, torch.float32):
        raise RuntimeError(f"unsupported out_dtype {out_dtype}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    if M == 0 or N == 0:
        return out
    _call("zen_linear_f16_ex", x.data_ptr(), x.stride(0) if M > 1 else K, w.data_ptr(), K, M, N, K, _ptr(bias), _ACT[act], _OUT[out_dtype],
          out.data_ptr(), out.stride(0), _capi.gemm_tile_n(tile_n) | _pair_flag(pair), _stream())
    return out


def linear_fp32(x, w, bias=None, *, act="none"):
    """``act(x @ w.T + bias)`` in fp32 storage, TF32 tensor-core math (python/src/bindings.cpp:1454-1496)."""
    _require(x, "x", torch.float32, 2)
    _require(w, "w", torch.float32, 2)
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise RuntimeError(f"inner dimensions differ: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    if M and N:
        _call("zen_linear_f32", x.data_ptr(), K, w.data_ptr(), K, M, N, K, _ptr(bias), _ACT[act], out.data_ptr(), N,
              _stream())
    return out


def wmma_matmul(a, b):
    """``C f32[M,N] = A f16[M,K] @ B f16[K,N]`` (core/bindings/cuda_bindings.cpp:110-132)."""
    if not a.is_cuda or not b.is_cuda:
        raise RuntimeError("Inputs must be CUDA tensors")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("Inputs must be 2D")
    if a.dtype != torch.float16 or b.dtype != torch.float16:
        raise RuntimeError("Inputs must be FP16")
    if a.shape[1] != b.shape[0]:
        raise RuntimeError("Inner dimensions must match")
    a = a.contiguous()
    b = b.contiguous()
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    if M and N:
        _call("zen_wmma_matmul_f16", a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, _stream())
    return c


def matmul_f32(a, b):
    """``C = A @ B`` for fp32 operands on the tensor cores in TF32 (core/bindings/cuda_bindings.cpp:73-88)."""
    if not a.is_cuda or not b.is_cuda:
        raise RuntimeError("Inputs must be CUDA tensors")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("Inputs must be 2D")
    if a.shape[1] != b.shape[0]:
        raise RuntimeError("Inner dimensions must match")
    _require(a.contiguous(), "A", torch.float32)
    a = a.contiguous()
    b = b.contiguous()
    _require(b, "B", torch.float32)
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    if M and N:
        nbytes = _capi.lib().zen_matmul_f32_workspace_bytes(N, K)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=a.device)  # B transposed to [N, K]
        _call("zen_matmul_f32", a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, workspace.data_ptr(), nbytes,
              _stream())
        launch_count_add(1)
    return c


# --------------------------------------------------------------------------------------------
# elementwise / row kernels
# --------------------------------------------------------------------------------------------
def gelu(x):
    """tanh-form GELU (core/src/cuda_kernels.cu:115-126), fp32 or fp16, any shape."""
    if x.dtype == torch.float32:
        _require(x, "input", torch.float32)
        y = torch.empty_like(x)
        if x.numel():
            _call("zen_gelu_f32", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
        return y
    _require(x, "input", torch.float16)
    y = torch.empty_like(x)
    if x.numel():
        _call("zen_gelu_f16", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
    return y


def tanh(x):
    """Elementwise tanh, fp32 or fp16 (the pooler's activation)."""
    if x.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("input must be fp32 or fp16")
    _require(x, "input", x.dtype)
    y = torch.empty_like(x)
    if x.numel():
        _call("zen_tanh_f32" if x.dtype == torch.float32 else "zen_tanh_f16", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
    return y


def relu(x):
    _require(x, "input", torch.float32)
    y = torch.empty_like(x)
    if x.numel():
        _call("zen_relu_f32", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
    return y


def bias_gelu(x, bias):
    """``gelu(x + bias[col])`` over [rows, features] (core/src/fused_kernels.cu:47-62)."""
    _require(x, "input", torch.float32, 2)
    _require(bias, "bias", torch.float32, 1)
    y = torch.empty_like(x)
    if x.numel():
        _call("zen_bias_gelu_f32", x.data_ptr(), bias.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], _stream())
    return y


def layernorm(x, gamma, beta, eps: float = 1e-5):
    """Row LayerNorm of a 2-D tensor, fp32 or fp16 (core/bindings/cuda_bindings.cpp:58-71)."""
    if x.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("input must be fp32 or fp16")
    _require(x, "input", x.dtype, 2)
    _require(gamma, "gamma", x.dtype, 1)
    _require(beta, "beta", x.dtype, 1)
    y = torch.empty_like(x)
    fn = "zen_layernorm_f32" if x.dtype == torch.float32 else "zen_layernorm_f16"
    if x.numel():
        _call(fn, x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], float(eps),
              _stream())
    return y


def add_layernorm(x, residual, gamma, beta, eps: float = 1e-5, *, out_scale: float | None = None,
                  round="nearest_even"):
    """``LayerNorm(x + residual)`` (core/src/fused_kernels.cu:145-221).

    With ``out_scale`` (fp16 only) also returns the int8 copy ``quantize(y, out_scale)``.
    """
    if x.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("input must be fp32 or fp16")
    _require(x, "input", x.dtype, 2)
    _require(residual, "residual", x.dtype, 2)
    _require(gamma, "gamma", x.dtype, 1)
    _require(beta, "beta", x.dtype, 1)
    if residual.shape != x.shape:
        raise RuntimeError("residual must have the shape of the input")
    y = torch.empty_like(x)
    rows, hidden = x.shape
    if x.dtype == torch.float32:
        if out_scale is not None:
            raise RuntimeError("the int8 copy is available for fp16 inputs only")
        if x.numel():
            _call("zen_add_layernorm_f32", x.data_ptr(), residual.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                  y.data_ptr(), rows, hidden, float(eps), _stream())
        return y
    yq = torch.empty(x.shape, dtype=torch.int8, device=x.device) if out_scale is not None else None
    if x.numel():
        _call("zen_add_layernorm_f16", x.data_ptr(), residual.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
              y.data_ptr(), _ptr(yq), float(out_scale or 1.0), _ROUND[round], rows, hidden, float(eps), _stream())
    return y if yq is None else (y, yq)


def quantize(x, scale: float, zero_point: int = 0, *, round="nearest_even"):
    """``clamp(round(x / scale + zero_point), -128, 127)`` (core/src/cuda_kernels.cu:918-929)."""
    if x.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("input must be fp32 or fp16")
    _require(x, "input", x.dtype)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    fn = "zen_quantize_f32" if x.dtype == torch.float32 else "zen_quantize_f16"
    if x.numel():
        _call(fn, x.data_ptr(), q.data_ptr(), x.numel(), float(scale), int(zero_point), _ROUND[round], _stream())
    return q


def dequantize(q, scale: float, zero_point: int = 0):
    """``(q - zero_point) * scale`` (core/src/cuda_kernels.cu:941-950)."""
    _require(q, "input", torch.int8)
    x = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    if q.numel():
        _call("zen_dequantize_f32", q.data_ptr(), x.data_ptr(), q.numel(), float(scale), int(zero_point), _stream())
    return x


class RangeObserver:
    """Running (min, max) of every tensor shown to it, kept on the device: two floats and no host
    read-back until ``range()`` is called.  Same statistic as ``TensorStats.update``
    (zenith/optimization/quantization.py:69-72); NaNs are skipped."""

    def __init__(self, device):
        self.minmax = torch.tensor([float("inf"), float("-inf")], dtype=torch.float32, device=device)
        nbytes = _capi.lib().zen_minmax_workspace_bytes()
        self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def observe(self, x: torch.Tensor) -> None:
        if not x.is_cuda or x.dtype not in (torch.float16, torch.float32) or not x.is_contiguous():
            raise RuntimeError("RangeObserver.observe wants a contiguous CUDA fp16 / fp32 tensor")
        fn = "zen_minmax_f16" if x.dtype == torch.float16 else "zen_minmax_f32"
        _call(fn, x.data_ptr(), x.numel(), self.minmax.data_ptr(), self._workspace.data_ptr(), self._workspace.numel(),
              _stream())
        launch_count_add(1)  # two launches in all: _call counted the first

    def range(self) -> tuple:
        lo, hi = self.minmax.tolist()
        return lo, hi


class HistogramObserver(RangeObserver):
    """``RangeObserver`` that also keeps the running histogram of ``TensorStats.update``
    (zenith/optimization/quantization.py:69-83) on the device: after each tensor's min / max have gone into the
    running range, the tensor is binned over that range (``num_bins`` equal bins, numpy's binning) and added to the
    histogram - the statistics the percentile and entropy calibrators need.  Nothing is read back until ``stats()``."""

    def __init__(self, device, num_bins: int = 2048):
        super().__init__(device)
        self.num_bins = int(num_bins)
        self.hist = torch.zeros(self.num_bins, dtype=torch.int64, device=device)

    def observe(self, x: torch.Tensor) -> None:
        super().observe(x)
        fn = "zen_histogram_f16" if x.dtype == torch.float16 else "zen_histogram_f32"
        _call(fn, x.data_ptr(), x.numel(), self.minmax.data_ptr(), self.num_bins, self.hist.data_ptr(), _stream())

    def stats(self):
        """The observations as a ``quantization.TensorStats`` (host): min, max and the int64 histogram."""
        from .quantization import TensorStats

        lo, hi = self.range()
        return TensorStats(min_val=lo, max_val=hi, histogram=self.hist.cpu().numpy().copy(), num_bins=self.num_bins)


def absmax_rows(w):
    """``max_c |w[r, c]|`` per row of a CUDA fp32 matrix: the per-output-channel weight observer
    (zenith/optimization/qat.py:195-199)."""
    _require(w, "w", torch.float32, 2, rows_may_be_strided=True)
    out = torch.empty(w.shape[0], dtype=torch.float32, device=w.device)
    if w.shape[0]:
        _call("zen_absmax_rows_f32", w.data_ptr(), w.shape[0], w.shape[1], w.stride(0), out.data_ptr(), _stream())
    return out


def quantize_rows(w, scale, *, round="nearest_even"):
    """``clamp(round(w[r, c] / scale[r]), -128, 127)`` as int8: per-output-channel weight conversion."""
    _require(w, "w", torch.float32, 2, rows_may_be_strided=True)
    _require(scale, "scale", torch.float32, 1)
    if scale.numel() != w.shape[0]:
        raise RuntimeError("scale must have one entry per row")
    q = torch.empty(w.shape, dtype=torch.int8, device=w.device)
    if w.numel():
        _call("zen_quantize_rows_f32", w.data_ptr(), scale.data_ptr(), w.shape[0], w.shape[1], w.stride(0), q.data_ptr(),
              q.stride(0), _ROUND[round], _stream())
    return q


def to_fp16(x):
    _require(x, "input", torch.float32)
    y = torch.empty(x.shape, dtype=torch.float16, device=x.device)
    if x.numel():
        _call("zen_convert_f32_to_f16", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
    return y


def to_fp32(x):
    _require(x, "input", torch.float16)
    y = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    if x.numel():
        _call("zen_convert_f16_to_f32", x.data_ptr(), y.data_ptr(), x.numel(), _stream())
    return y


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def flash_attention_strided(q, k, v, out, B, H, S, D, q_strides, k_strides, v_strides, o_strides, *, kv_lens=None,
                            causal=False, scale=None, out_q=None, out_scale=None):
    """Attention over strided fp16 views: strides are (batch, head, seq) in elements, d contiguous."""
    if kv_lens is not None:
        _require(kv_lens, "kv_lens", torch.int32, 1)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    _call("zen_flash_attention_f16", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), _ptr(out_q),
          float(out_scale or 1.0), B, H, S, D, *q_strides, *k_strides, *v_strides, *o_strides, _ptr(kv_lens),
          1 if causal else 0, scale, _stream())
    return out


def flash_attention(q, k, v, *, causal: bool = False, kv_lens=None, scale: float | None = None):
    """``softmax(scale * Q K^T) V`` for ``[batch, heads, seq, dim]`` tensors.

    fp16 inputs run directly; fp32 inputs (the reference binding's dtype,
    core/bindings/cuda_bindings.cpp:90-106) are converted to fp16 on the device, run on the
    tensor cores with fp32 softmax and accumulation, and returned as fp32.
    ``kv_lens[b]`` masks keys at positions >= kv_lens[b]; a row with no valid key yields zeros.
    """
    if not q.is_cuda:
        raise RuntimeError("Q must be CUDA tensor")
    if q.dim() != 4:
        raise RuntimeError("Q must be 4D [batch, heads, seq, dim]")
    if k.shape != q.shape or v.shape != q.shape:
        raise RuntimeError("K and V must have the shape of Q")
    B, H, S, D = q.shape
    if q.dtype == torch.float32:
        qh, kh, vh = (to_fp16(t.contiguous()) for t in (q, k, v))
        oh = flash_attention(qh, kh, vh, causal=causal, kv_lens=kv_lens, scale=scale)
        return to_fp32(oh)
    for name, t in (("Q", q), ("K", k), ("V", v)):
        _require(t, name, torch.float16, 4)
    out = torch.empty_like(q)
    st = (H * S * D, S * D, D)
    flash_attention_strided(q, k, v, out, B, H, S, D, st, st, st, st, kv_lens=kv_lens, causal=causal, scale=scale)
    return out


def qkv_attention_int8(xq, wqkv, x_scale: float, w_scale, bias, B: int, S: int, heads: int, *, kv_lens=None,
                       scale: float | None = None, out_scale: float | None = None, emit_qkv: bool = False,
                       constant_weights=False, prefetch=()):
    """W8A8 QKV projection + attention in one kernel (``zen_qkv_attention_i8``): sequences of at most 128 tokens,
    head size 64.  ``xq`` int8 ``[B*S, K]``, ``wqkv`` int8 ``[3*heads*64, K]``.  Returns fp16 ``ctx [B*S, heads*64]``,
    then (with ``out_scale``) its int8 copy, then (with ``emit_qkv``) the fp16 projection ``[B*S, 3*heads*64]``.
    Bit-identical to ``linear_int8(..., out_dtype=float16)`` followed by ``flash_attention_strided``."""
    _require(xq, "xq", torch.int8, 2)
    _require(wqkv, "wqkv", torch.int8, 2)
    hidden = heads * 64
    T, K = xq.shape
    if T != B * S or tuple(wqkv.shape) != (3 * hidden, K):
        raise RuntimeError("shape mismatch")
    if w_scale is not None:
        _require(w_scale, "w_scale", torch.float32, 1)
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    if kv_lens is not None:
        _require(kv_lens, "kv_lens", torch.int32, 1)
    if len(prefetch) > 2:
        raise RuntimeError("prefetch takes at most two CUDA tensors")
    ctx = torch.empty((T, hidden), dtype=torch.float16, device=xq.device)
    ctxq = torch.empty((T, hidden), dtype=torch.int8, device=xq.device) if out_scale is not None else None
    qkv = torch.empty((T, 3 * hidden), dtype=torch.float16, device=xq.device) if emit_qkv else None
    hint = [v for t in prefetch for v in (t.data_ptr(), t.numel() * t.element_size())] + [None, 0] * (2 - len(prefetch))
    _call("zen_qkv_attention_i8", xq.data_ptr(), K, wqkv.data_ptr(), K, B, S, heads, K, float(x_scale), _ptr(w_scale),
          _ptr(bias), _ptr(kv_lens), float(1.0 / math.sqrt(64) if scale is None else scale), ctx.data_ptr(), _ptr(ctxq),
          float(out_scale or 1.0), _ptr(qkv), *hint, _capi.GEMM_CONST_WEIGHTS if constant_weights else 0, _stream())
    out = [ctx]
    if ctxq is not None:
        out.append(ctxq)
    if qkv is not None:
        out.append(qkv)
    return out[0] if len(out) == 1 else tuple(out)


# --------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------
def embed_layernorm(ids, type_ids, word, pos, typ, gamma, beta, eps: float, seq: int, *, out_scale=None,
                    round="nearest_even"):
    """``LayerNorm(word[ids] + pos[t % seq] + type[type_ids])`` in fp16, optional int8 copy.

    The reference's embedding kernel gathers the word table only
    (core/src/transformer_kernels.cu:236-262); position / type tables and the LayerNorm are the
    BERT embedding block that precedes the encoder.
    """
    _require(ids, "ids", torch.int32, 1)
    if type_ids is not None:
        _require(type_ids, "type_ids", torch.int32, 1)
    for name, t in (("word", word), ("pos", pos), ("type", typ)):
        _require(t, name, torch.float16, 2)
    _require(gamma, "gamma", torch.float16, 1)
    _require(beta, "beta", torch.float16, 1)
    tokens = ids.numel()
    hidden = word.shape[1]
    if pos.shape[0] < seq:
        raise RuntimeError("position table shorter than the sequence")
    y = torch.empty((tokens, hidden), dtype=torch.float16, device=word.device)
    yq = torch.empty((tokens, hidden), dtype=torch.int8, device=word.device) if out_scale is not None else None
    if tokens:
        _call("zen_embed_layernorm_f16", ids.data_ptr(), _ptr(type_ids), word.data_ptr(), pos.data_ptr(),
              typ.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), _ptr(yq), float(out_scale or 1.0),
              _ROUND[round], tokens, int(seq), hidden, word.shape[0], float(eps), _stream())
    return y if yq is None else (y, yq)


# --------------------------------------------------------------------------------------------
# unpadded batches: the valid tokens packed back to back
# --------------------------------------------------------------------------------------------
def pack_tokens(ids, kv_lens, capacity: int, type_ids=None):
    """From padded ``ids [B, S]`` (int32) and key lengths ``kv_lens [B]`` to ``(cu_seqlens [B+1], ids_packed,
    pos_packed, type_packed or None)`` of ``capacity`` rows (``zen_pack_tokens_i32``); rows beyond the total
    carry id 0 / position 0."""
    _require(ids, "ids", torch.int32, 2)
    _require(kv_lens, "kv_lens", torch.int32, 1)
    if type_ids is not None:
        _require(type_ids, "type_ids", torch.int32, 2)
    B, S = ids.shape
    d = ids.device
    cu = torch.empty(B + 1, dtype=torch.int32, device=d)
    ids_p = torch.empty(capacity, dtype=torch.int32, device=d)
    pos_p = torch.empty(capacity, dtype=torch.int32, device=d)
    type_p = torch.empty(capacity, dtype=torch.int32, device=d) if type_ids is not None else None
    _call("zen_pack_tokens_i32", ids.data_ptr(), _ptr(type_ids), kv_lens.data_ptr(), B, S, int(capacity), cu.data_ptr(),
          ids_p.data_ptr(), pos_p.data_ptr(), _ptr(type_p), _stream())
    return cu, ids_p, pos_p, type_p


def unpad_rows(packed, cu_seqlens, B: int, S: int):
    """Padded ``[B*S, hidden]`` fp16 copy of packed rows: zeros at padding positions (``zen_unpad_rows_f16``)."""
    _require(packed, "packed", torch.float16, 2)
    _require(cu_seqlens, "cu_seqlens", torch.int32, 1)
    if cu_seqlens.numel() != B + 1:
        raise RuntimeError("cu_seqlens must hold B + 1 offsets")
    out = torch.empty((B * S, packed.shape[1]), dtype=torch.float16, device=packed.device)
    _call("zen_unpad_rows_f16", packed.data_ptr(), cu_seqlens.data_ptr(), B, S, packed.shape[1], packed.shape[0],
          out.data_ptr(), _stream())
    return out


def embed_layernorm_unpadded(ids_packed, pos_packed, type_packed, word, pos, typ, gamma, beta, eps: float, *,
                             out_scale=None, round="nearest_even"):
    """``embed_layernorm`` on packed rows: the position of each row comes from ``pos_packed``."""
    _require(ids_packed, "ids_packed", torch.int32, 1)
    _require(pos_packed, "pos_packed", torch.int32, 1)
    if type_packed is not None:
        _require(type_packed, "type_packed", torch.int32, 1)
    for name, t in (("word", word), ("pos", pos), ("type", typ)):
        _require(t, name, torch.float16, 2)
    _require(gamma, "gamma", torch.float16, 1)
    _require(beta, "beta", torch.float16, 1)
    rows = ids_packed.numel()
    hidden = word.shape[1]
    y = torch.empty((rows, hidden), dtype=torch.float16, device=word.device)
    yq = torch.empty((rows, hidden), dtype=torch.int8, device=word.device) if out_scale is not None else None
    if rows:
        _call("zen_embed_layernorm_unpadded_f16", ids_packed.data_ptr(), pos_packed.data_ptr(), _ptr(type_packed),
              word.data_ptr(), pos.data_ptr(), typ.data_ptr(), gamma.data_ptr(), beta.data_ptr(), y.data_ptr(), _ptr(yq),
              float(out_scale or 1.0), _ROUND[round], rows, pos.shape[0], hidden, word.shape[0], float(eps), _stream())
    return y if yq is None else (y, yq)


def qkv_attention_unpadded_int8(xq, wqkv, x_scale: float, w_scale, bias, cu_seqlens, heads: int, *,
                                scale: float | None = None, out_scale: float | None = None, emit_qkv: bool = False,
                                constant_weights=False):
    """``qkv_attention_int8`` on packed rows (``zen_qkv_attention_unpadded_i8``): ``xq`` int8 ``[rows, K]``, sequence b
    in rows ``cu_seqlens[b] .. cu_seqlens[b+1]-1`` (at most 128 each).  Rows that belong to no sequence are left
    unwritten in the outputs (which start as zeros here)."""
    _require(xq, "xq", torch.int8, 2)
    _require(wqkv, "wqkv", torch.int8, 2)
    _require(cu_seqlens, "cu_seqlens", torch.int32, 1)
    hidden = heads * 64
    T, K = xq.shape
    if tuple(wqkv.shape) != (3 * hidden, K):
        raise RuntimeError("shape mismatch")
    if w_scale is not None:
        _require(w_scale, "w_scale", torch.float32, 1)
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    B = cu_seqlens.numel() - 1
    ctx = torch.zeros((T, hidden), dtype=torch.float16, device=xq.device)
    ctxq = torch.zeros((T, hidden), dtype=torch.int8, device=xq.device) if out_scale is not None else None
    qkv = torch.zeros((T, 3 * hidden), dtype=torch.float16, device=xq.device) if emit_qkv else None
    _call("zen_qkv_attention_unpadded_i8", xq.data_ptr(), K, wqkv.data_ptr(), K, B, T, cu_seqlens.data_ptr(), heads, K,
          float(x_scale), _ptr(w_scale), _ptr(bias), float(1.0 / math.sqrt(64) if scale is None else scale),
          ctx.data_ptr(), _ptr(ctxq), float(out_scale or 1.0), _ptr(qkv), None, 0, None, 0,
          _capi.GEMM_CONST_WEIGHTS if constant_weights else 0, _stream())
    out = [ctx]
    if ctxq is not None:
        out.append(ctxq)
    if qkv is not None:
        out.append(qkv)
    return out[0] if len(out) == 1 else tuple(out)


# --------------------------------------------------------------------------------------------
# FP8 (e4m3) operands
# --------------------------------------------------------------------------------------------
def quantize_e4m3(x, scale: float):
    """e4m3 bit patterns (uint8) of ``x / scale``: round to nearest even, saturating at +-448."""
    if x.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("input must be fp32 or fp16")
    _require(x, "input", x.dtype)
    q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    fn = "zen_quantize_e4m3_f32" if x.dtype == torch.float32 else "zen_quantize_e4m3_f16"
    if x.numel():
        _call(fn, x.data_ptr(), q.data_ptr(), x.numel(), float(scale), _stream())
    return q


def linear_fp8(xq, wq, x_scale: float, w_scale=None, bias=None, *, act="none", out_dtype=torch.float16, out=None,
               constant_weights=False, tile_n: int = 0):
    """``act((xq @ wq.T) * x_scale * w_scale + bias)`` with e4m3 operands (uint8 bit patterns) and fp32 accumulation on
    the tensor cores (``zen_linear_f8``); a tolerance path like ``linear_fp16``."""
    _require(xq, "xq", torch.uint8, 2, rows_may_be_strided=True)
    _require(wq, "wq", torch.uint8, 2)
    M, K = xq.shape
    N, K2 = wq.shape
    if K != K2:
        raise RuntimeError(f"inner dimensions differ: xq {tuple(xq.shape)} vs wq {tuple(wq.shape)}")
    if w_scale is not None:
        _require(w_scale, "w_scale", torch.float32, 1)
    if bias is not None:
        _require(bias, "bias", torch.float32, 1)
    if out_dtype not in (torch.float16, torch.float32):
        raise RuntimeError(f"unsupported out_dtype {out_dtype}")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    if M == 0 or N == 0:
        return out
    _call("zen_linear_f8", xq.data_ptr(), xq.stride(0) if M > 1 else K, wq.data_ptr(), K, M, N, K, float(x_scale), _ptr(w_scale),
          _ptr(bias), _ACT[act], _OUT[out_dtype], out.data_ptr(), out.stride(0),
          (_capi.GEMM_CONST_WEIGHTS if constant_weights else 0) | _capi.gemm_tile_n(tile_n), _stream())
    return out


def flash_attention_unpadded(qkv, cu_seqlens, heads: int, head_dim: int, max_seqlen: int, *, causal: bool = False,
                             scale: float | None = None, out_scale: float | None = None):
    """Attention on packed rows (``zen_flash_attention_unpadded_f16``): ``qkv`` fp16 ``[rows, 3 * heads * head_dim]``
    (columns Q | K | V, each head's columns together), sequence b in rows ``cu_seqlens[b] .. cu_seqlens[b+1]-1`` (any
    length up to ``max_seqlen``).  Returns the context ``[rows, heads * head_dim]`` (rows of no sequence stay zero),
    and with ``out_scale`` its int8 copy."""
    _require(qkv, "qkv", torch.float16, 2)
    _require(cu_seqlens, "cu_seqlens", torch.int32, 1)
    hidden = heads * head_dim
    rows = qkv.shape[0]
    if qkv.shape[1] != 3 * hidden:
        raise RuntimeError("qkv must be [rows, 3 * heads * head_dim]")
    ctx = torch.zeros((rows, hidden), dtype=torch.float16, device=qkv.device)
    ctxq = torch.zeros((rows, hidden), dtype=torch.int8, device=qkv.device) if out_scale is not None else None
    B = cu_seqlens.numel() - 1
    e = qkv.element_size()
    _call("zen_flash_attention_unpadded_f16", qkv.data_ptr(), qkv.data_ptr() + hidden * e, qkv.data_ptr() + 2 * hidden * e,
          ctx.data_ptr(), _ptr(ctxq), float(out_scale or 1.0), B, heads, int(max_seqlen), head_dim, rows, 3 * hidden, head_dim,
          3 * hidden, head_dim, 3 * hidden, head_dim, hidden, head_dim, cu_seqlens.data_ptr(), 1 if causal else 0,
          float(1.0 / math.sqrt(head_dim) if scale is None else scale), _stream())
    return ctx if ctxq is None else (ctx, ctxq)
