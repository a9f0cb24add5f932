"""Drop-in for the reference's ``zenith_cuda`` torch extension.

Same six functions, argument order, dtype contract, error type (``RuntimeError``) and output
ownership (a new tensor per call) as core/bindings/cuda_bindings.cpp:134-145, served by the
sm_100a kernels of this package and launched on torch's current stream (the reference used the
legacy default stream).  Typed extensions that the reference does not have (fp16 / int8 paths,
masks) keep the positional contract and add keyword-only arguments.

``zenith_b200.install_as_zenith_cuda()`` registers this module under the name ``zenith_cuda``
so that ``import zenith_cuda`` in zenith/runtime/kernel_registry.py:225 and
zenith/optimization/fx_patterns.py:43 resolves to it.
"""
from __future__ import annotations

import torch

from . import ops

__all__ = ["relu", "gelu", "layernorm", "matmul", "flash_attention", "wmma_matmul",
           "linear_int8", "linear_fp16", "add_layernorm", "quantize", "dequantize", "embed_layernorm"]


def _check_cuda_contig(t, what="Input"):
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{what} must be contiguous")


def relu(input):
    """ReLU, fp32 (core/bindings/cuda_bindings.cpp:39-46)."""
    _check_cuda_contig(input)
    return ops.relu(input)


def gelu(input):
    """GELU, fp32 as in the reference (core/bindings/cuda_bindings.cpp:48-56); fp16 also accepted."""
    _check_cuda_contig(input)
    return ops.gelu(input)


def layernorm(input, gamma, beta, eps: float = 1e-5):
    """LayerNorm of a 2-D [batch, hidden] tensor (core/bindings/cuda_bindings.cpp:58-71)."""
    if not input.is_cuda:
        raise RuntimeError("Input must be CUDA tensor")
    if input.dim() != 2:
        raise RuntimeError("Input must be 2D [batch, hidden]")
    return ops.layernorm(input.contiguous(), gamma.contiguous(), beta.contiguous(), eps)


def matmul(A, B):
    """``A[M,K] @ B[K,N]`` in fp32 storage, TF32 tensor-core math (core/bindings/cuda_bindings.cpp:73-88)."""
    return ops.matmul_f32(A, B)


def flash_attention(Q, K, V, *, causal: bool = False, kv_lens=None, scale=None):
    """Attention over ``[batch, heads, seq, dim]`` (core/bindings/cuda_bindings.cpp:90-106)."""
    return ops.flash_attention(Q, K, V, causal=causal, kv_lens=kv_lens, scale=scale)


def wmma_matmul(A, B):
    """``A f16[M,K] @ B f16[K,N] -> f32[M,N]`` (core/bindings/cuda_bindings.cpp:110-132)."""
    return ops.wmma_matmul(A, B)


# typed extensions
linear_int8 = ops.linear_int8
linear_fp16 = ops.linear_fp16
add_layernorm = ops.add_layernorm
quantize = ops.quantize
dequantize = ops.dequantize
embed_layernorm = ops.embed_layernorm
