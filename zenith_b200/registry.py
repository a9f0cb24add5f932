"""Plug-in registration for the reference's kernel registry.

``register(registry)`` installs one ``KernelSpec`` per operator family under the op-type strings the
reference uses (zenith/runtime/kernel_registry.py:227-286, :450-488; zenith/runtime/
triton_kernels.py:435-444) at a priority above every kernel the reference registers itself (its
highest is 30), so ``KernelRegistry.get_kernel`` (kernel_registry.py:118-153) picks these.  The
callables follow the argument order ``KernelDispatcher._call_kernel`` uses
(zenith/runtime/dispatcher.py:235-315): ``fn(x, w, b)`` for Linear, ``fn(x, gamma, beta, eps)`` for
LayerNorm, ``fn(q, k, v)`` for Attention, ``fn(x)`` for GELU / ReLU,
``fn(x, residual, gamma, beta, eps)`` for FusedAddLayerNorm.

If the reference package is importable its own ``KernelSpec`` / ``Precision`` classes are used, so the
specs are instances of the types its registry expects; otherwise structurally identical stand-ins.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Optional

import torch

from . import ops

PRIORITY = 40

try:  # pragma: no cover - depends on the host application
    from zenith.runtime.kernel_registry import KernelSpec, Precision  # type: ignore
except Exception:  # the reference is not installed: same fields, same names

    class Precision(Enum):
        FP32 = "fp32"
        FP16 = "fp16"
        BF16 = "bf16"
        INT8 = "int8"

    @dataclass
    class KernelSpec:
        name: str
        op_types: list
        precision: Precision
        kernel_fn: Optional[Callable] = None
        input_constraints: dict = field(default_factory=dict)
        priority: int = 0
        estimated_flops: Optional[Callable] = None
        requires_gpu: bool = True

        def supports_op(self, op_type: str) -> bool:
            return op_type in self.op_types


def _as_2d(x):
    return x.reshape(-1, x.shape[-1]).contiguous(), x.shape[:-1]


def linear(x, w, b=None, *, act="none"):
    """``fn(input, weight, bias)`` with a ``[out, in]`` weight, or ``fn(a, b)`` as a plain matmul when the
    shapes only fit ``a @ b``.  fp32 tensors run in TF32, fp16 tensors in fp16, both with fp32 accumulation."""
    x2, lead = _as_2d(x)
    as_linear = x2.shape[1] == w.shape[1] and (b is not None or x2.shape[1] != w.shape[0])
    if not as_linear:
        if x2.dtype == torch.float16:
            return ops.wmma_matmul(x2, w).to(torch.float16).reshape(*lead, w.shape[1])
        return ops.matmul_f32(x2, w).reshape(*lead, w.shape[1])
    bias = None if b is None else b.float().contiguous()
    if x2.dtype == torch.float16:
        y = ops.linear_fp16(x2, w.contiguous(), bias, act=act)
    else:
        y = ops.linear_fp32(x2, w.contiguous(), bias, act=act)
    return y.reshape(*lead, w.shape[0])


def linear_gelu(x, w, b=None):
    return linear(x, w, b, act="gelu")


def layernorm(x, gamma, beta=None, eps=1e-5):
    x2, lead = _as_2d(x)
    if beta is None:
        beta = torch.zeros_like(gamma)
    return ops.layernorm(x2, gamma.contiguous(), beta.contiguous(), eps).reshape(*lead, x.shape[-1])


def add_layernorm(x, residual, gamma, beta, eps=1e-5):
    x2, lead = _as_2d(x)
    r2, _ = _as_2d(residual)
    return ops.add_layernorm(x2, r2, gamma.contiguous(), beta.contiguous(), eps).reshape(*lead, x.shape[-1])


def bias_gelu(x, bias):
    x2, lead = _as_2d(x)
    return ops.bias_gelu(x2, bias.contiguous()).reshape(*lead, x.shape[-1])


def attention(q, k=None, v=None):
    if k is None or v is None:
        raise RuntimeError("attention needs separate Q, K, V tensors [batch, heads, seq, dim]")
    return ops.flash_attention(q.contiguous(), k.contiguous(), v.contiguous())


def _specs():
    for prec in (Precision.FP32, Precision.FP16):
        tag = prec.value
        yield KernelSpec(f"b200_linear_{tag}", ["MatMul", "Gemm", "matmul", "Linear"], prec, linear, priority=PRIORITY)
        yield KernelSpec(f"b200_linear_gelu_{tag}", ["FusedLinearGELU", "Linear+GELU", "Gemm+GELU"], prec, linear_gelu,
                         priority=PRIORITY)
        yield KernelSpec(f"b200_gelu_{tag}", ["Gelu", "GELU", "gelu"], prec, ops.gelu, priority=PRIORITY)
        yield KernelSpec(f"b200_layernorm_{tag}", ["LayerNorm", "LayerNormalization", "layer_norm"], prec, layernorm,
                         priority=PRIORITY)
        yield KernelSpec(f"b200_add_layernorm_{tag}", ["FusedAddLayerNorm", "Add+LayerNorm", "AddLayerNorm"], prec,
                         add_layernorm, priority=PRIORITY)
        yield KernelSpec(f"b200_attention_{tag}", ["Attention", "MultiHeadAttention", "flash_attention"], prec,
                         attention, priority=PRIORITY)
    yield KernelSpec("b200_relu_fp32", ["Relu", "ReLU", "relu"], Precision.FP32, ops.relu, priority=PRIORITY)
    yield KernelSpec("b200_bias_gelu_fp32", ["FusedBiasGeLU", "Bias+GELU", "BiasGeLU"], Precision.FP32, bias_gelu,
                     priority=PRIORITY)
    yield KernelSpec("b200_linear_int8", ["QuantizedLinear", "Linear"], Precision.INT8, ops.linear_int8,
                     priority=PRIORITY)


def register(registry) -> int:
    """Install every spec into ``registry`` (anything with ``register(spec)``); returns how many."""
    n = 0
    for spec in _specs():
        spec.requires_gpu = True
        registry.register(spec)
        n += 1
    return n
