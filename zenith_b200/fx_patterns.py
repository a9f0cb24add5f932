"""FX graph patterns that route a traced PyTorch model onto this package's kernels.

Same surface as the reference's pattern module (zenith/optimization/fx_patterns.py:60-230: ``FXPattern``,
``sdpa_pattern`` / ``zenith_sdpa_replacement``, ``causal_sdpa_pattern``, ``gelu_tanh_pattern``,
``layernorm_pattern``, ``get_*_patterns``), with three differences: the replacements call the B200 kernels
and nothing else (no PyTorch fallback: they raise on CPU tensors); the causal pattern, which the reference
defines but never returns from ``get_attention_patterns`` (fx_patterns.py:117-135, 187-196), is registered;
and two fused patterns the kernels support are added (Linear -> tanh-GELU, residual add -> LayerNorm).

``apply_patterns(gm)`` rewrites a ``torch.fx.GraphModule`` in place; ``zenith_backend`` is a
``torch.compile(model, backend=zenith_backend)`` entry that applies them to the captured graph.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.fx
import torch.nn.functional as F

from . import ops


@dataclass
class FXPattern:
    """A subgraph to find and the function to put in its place (zenith/optimization/fx_patterns.py:60-68)."""

    name: str
    pattern_fn: Callable
    replacement_fn: Callable
    priority: int = 10
    enabled: bool = True


# ---------------------------------------------------------------------------------------------
# leaves: calls into the kernels (opaque to the tracer, so they survive as single graph nodes)
# ---------------------------------------------------------------------------------------------
def _attention(q, k, v, causal):
    dt = q.dtype
    out = ops.flash_attention(q.to(torch.float16).contiguous(), k.to(torch.float16).contiguous(),
                              v.to(torch.float16).contiguous(), causal=causal)
    return out.to(dt)


@torch.fx.wrap
def zenith_flash_attention(q, k, v):
    """softmax(q k^T / sqrt(d)) v on ``[batch, heads, seq, d]`` tensors (d = 64 or 128)."""
    return _attention(q, k, v, False)


@torch.fx.wrap
def zenith_causal_flash_attention(q, k, v):
    return _attention(q, k, v, True)


@torch.fx.wrap
def zenith_gelu(x):
    if x.dtype == torch.float16:
        return ops.gelu(x.contiguous())
    return ops.gelu(x.float().contiguous()).to(x.dtype)


@torch.fx.wrap
def zenith_layernorm(x, weight, bias, eps):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    return ops.layernorm(x2, weight.to(x.dtype), bias.to(x.dtype), float(eps)).reshape(x.shape)


@torch.fx.wrap
def zenith_add_layernorm(x, residual, weight, bias, eps):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    r2 = residual.reshape(-1, x.shape[-1]).contiguous()
    return ops.add_layernorm(x2, r2, weight.to(x.dtype), bias.to(x.dtype), float(eps)).reshape(x.shape)


@torch.fx.wrap
def zenith_linear_gelu(x, weight, bias):
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    if x.dtype == torch.float16:
        y = ops.linear_fp16(x2, weight.contiguous(), None if bias is None else bias.float(), act="gelu")
    else:
        y = ops.linear_fp32(x2.float(), weight.float().contiguous(), None if bias is None else bias.float(), act="gelu").to(x.dtype)
    return y.reshape(*x.shape[:-1], weight.shape[0])


# ---------------------------------------------------------------------------------------------
# patterns (what a hand-written model looks like after symbolic tracing) and their replacements
# ---------------------------------------------------------------------------------------------
def sdpa_pattern(q, k, v):
    scale = q.shape[-1] ** -0.5
    weights = F.softmax(torch.matmul(q, k.transpose(-2, -1)) * scale, dim=-1)
    return torch.matmul(weights, v)


def zenith_sdpa_replacement(q, k, v):
    return zenith_flash_attention(q, k, v)


def causal_sdpa_pattern(q, k, v, mask):
    scale = q.shape[-1] ** -0.5
    weights = torch.matmul(q, k.transpose(-2, -1)) * scale
    weights = F.softmax(weights + mask, dim=-1)
    return torch.matmul(weights, v)


def zenith_causal_sdpa_replacement(q, k, v, mask):
    """``mask`` is taken to be the additive lower-triangular mask the pattern's name promises (the reference
    makes the same assumption: it passes ``is_causal=True``, fx_patterns.py:127-130); it is not read."""
    return zenith_causal_flash_attention(q, k, v)


def gelu_tanh_pattern(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def zenith_gelu_replacement(x):
    return zenith_gelu(x)


def layernorm_pattern(x, weight, bias, eps=1e-5):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def zenith_layernorm_replacement(x, weight, bias, eps=1e-5):
    return zenith_layernorm(x, weight, bias, eps)


def linear_gelu_pattern(x, weight, bias):
    return F.gelu(F.linear(x, weight, bias), approximate="tanh")


def zenith_linear_gelu_replacement(x, weight, bias):
    return zenith_linear_gelu(x, weight, bias)


def make_add_layernorm_pattern(hidden: int, eps: float) -> FXPattern:
    """``layer_norm(x + residual)`` for one (hidden size, eps) pair: both are literals in a traced graph."""

    def pattern(x, residual, weight, bias):
        return F.layer_norm(x + residual, (hidden,), weight, bias, eps)

    def replacement(x, residual, weight, bias):
        return zenith_add_layernorm(x, residual, weight, bias, eps)

    return FXPattern(f"add_layernorm_{hidden}", pattern, replacement, priority=15)


def get_attention_patterns() -> list:
    return [FXPattern("causal_sdpa_to_flash", causal_sdpa_pattern, zenith_causal_sdpa_replacement, priority=21),
            FXPattern("sdpa_to_flash", sdpa_pattern, zenith_sdpa_replacement, priority=20)]


def get_activation_patterns() -> list:
    return [FXPattern("linear_gelu_to_fused", linear_gelu_pattern, zenith_linear_gelu_replacement, priority=12),
            FXPattern("gelu_tanh_to_native", gelu_tanh_pattern, zenith_gelu_replacement, priority=10)]


def get_normalization_patterns() -> list:
    return [make_add_layernorm_pattern(768, 1e-12), make_add_layernorm_pattern(1024, 1e-12),
            FXPattern("manual_layernorm_to_native", layernorm_pattern, zenith_layernorm_replacement, priority=10)]


def get_all_patterns() -> list:
    return get_attention_patterns() + get_activation_patterns() + get_normalization_patterns()


def apply_patterns(gm: torch.fx.GraphModule, patterns: list | None = None) -> dict:
    """Rewrite ``gm`` in place, highest priority first; returns ``{pattern name: matches replaced}``."""
    from torch.fx import subgraph_rewriter

    counts = {}
    for pat in sorted(patterns if patterns is not None else get_all_patterns(), key=lambda p: -p.priority):
        if not pat.enabled:
            continue
        counts[pat.name] = len(subgraph_rewriter.replace_pattern(gm, pat.pattern_fn, pat.replacement_fn))
    gm.recompile()
    return counts


def zenith_backend(gm: torch.fx.GraphModule, example_inputs):
    """``torch.compile(model, backend=zenith_backend)``: apply the patterns to the captured graph, run it eagerly."""
    apply_patterns(gm)
    return gm.forward
