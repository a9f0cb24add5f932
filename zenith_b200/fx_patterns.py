"""FX graph patterns that route a traced PyTorch model onto this package's kernels.

Same surface as the reference's pattern module (zenith/optimization/fx_patterns.py:60-230: ``FXPattern``,
``sdpa_pattern`` / ``zenith_sdpa_replacement``, ``causal_sdpa_pattern``, ``gelu_tanh_pattern``,
``layernorm_pattern``, ``get_*_patterns``), with these differences: the replacements call the B200 kernels
(a CPU tensor of a supported shape raises; there is no CPU path); the masked pattern, which the reference
defines but never returns from ``get_attention_patterns`` (fx_patterns.py:117-135, 187-196), is registered,
and its replacement READS the mask: a lower-triangular additive mask runs the causal kernel, a key-padding
mask (the same suffix of keys masked for every query of a sequence) becomes per-sequence key lengths, and
any other mask - like any head size or width the kernels do not cover - is computed with the original
PyTorch expression, so a rewrite never changes what a model computes and never makes a working model fail;
patterns for ``F.scaled_dot_product_attention`` (the form a HuggingFace encoder traces to) are added, and so
are two fused patterns the kernels support (Linear -> tanh-GELU, residual add -> LayerNorm).

``apply_patterns(gm)`` rewrites a ``torch.fx.GraphModule`` in place; ``zenith_backend`` is a
``torch.compile(model, backend=zenith_backend)`` entry that applies them to the captured graph.
"""
from __future__ import annotations

import math
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
_SUPPORTED_HEAD_DIMS = (64, 128)
_MASKED = -1.0e4  # additive-mask entries at or below this count as "masked" (HuggingFace uses the dtype's minimum)


def _reference_attention(q, k, v, mask=None, causal=False, scale=None):
    """The expression the patterns match, evaluated by PyTorch: what runs when the kernels do not cover a case."""
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    w = torch.matmul(q, k.transpose(-2, -1)) * scale
    if causal:
        S = q.shape[-2]
        w = w.masked_fill(torch.ones(S, k.shape[-2], dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    if mask is not None:
        w = w.masked_fill(~mask, float("-inf")) if mask.dtype == torch.bool else w + mask
    return torch.matmul(F.softmax(w, dim=-1), v)


def classify_mask(mask, batch: int, q_len: int, k_len: int):
    """What an additive attention mask means for the kernels: ``("none", None)`` (all zeros), ``("causal", None)``
    (0 on and below the diagonal, masked above, the same for every batch / head), ``("kv_lens", lengths)`` (for
    every query of sequence b the keys from ``lengths[b]`` on are masked and the others are 0), or
    ``("other", None)``.  ``mask`` broadcasts against ``[batch, heads, q_len, k_len]`` and is additive (0 / very
    negative) or boolean (True = attend), the two forms ``F.scaled_dot_product_attention`` takes."""
    if mask is None:
        return "none", None
    m = mask
    while m.dim() < 4:
        m = m.unsqueeze(0)
    if m.shape[-1] != k_len or m.shape[1] != 1 or m.shape[0] not in (1, batch) or m.shape[2] not in (1, q_len):
        return "other", None
    if m.dtype == torch.bool:  # the boolean form: True = attend
        masked = ~m
    else:
        masked = m <= _MASKED
        if not bool(((m == 0) | masked).all()):
            return "other", None
    if not bool(masked.any()):
        return "none", None
    if m.shape[2] == q_len and q_len == k_len and m.shape[0] == 1:
        tri = torch.ones(q_len, k_len, dtype=torch.bool, device=m.device).triu(1)
        if bool((masked[0, 0] == tri).all()):
            return "causal", None
    rows = masked if m.shape[2] == 1 else masked[:, :, :1]
    if m.shape[2] != 1 and not bool((masked == rows).all()):
        return "other", None  # the mask differs between queries and is not the causal one
    key = rows[:, 0, 0]  # [1 or batch, k_len]
    lengths = (~key).sum(dim=-1)
    prefix = torch.arange(k_len, device=m.device)[None, :] < lengths[:, None]
    if not bool((prefix == ~key).all()):
        return "other", None  # masked keys are not a suffix
    return "kv_lens", lengths.expand(batch).to(torch.int32).contiguous()


def _kernel_covers(q, k, v) -> bool:
    return (q.dim() == 4 and q.shape == k.shape == v.shape and q.shape[-1] in _SUPPORTED_HEAD_DIMS and q.is_floating_point())


def _attention(q, k, v, causal=False, kv_lens=None, scale=None):
    dt = q.dtype
    out = ops.flash_attention(q.to(torch.float16).contiguous(), k.to(torch.float16).contiguous(),
                              v.to(torch.float16).contiguous(), causal=causal, kv_lens=kv_lens, scale=scale)
    return out.to(dt)


@torch.fx.wrap
def zenith_flash_attention(q, k, v):
    """softmax(q k^T / sqrt(d)) v on ``[batch, heads, seq, d]`` tensors; d = 64 or 128 run on the kernels, any
    other shape is computed by PyTorch."""
    if not _kernel_covers(q, k, v):
        return _reference_attention(q, k, v)
    return _attention(q, k, v)


@torch.fx.wrap
def zenith_masked_flash_attention(q, k, v, mask, scale=None, is_causal=False):
    """softmax(scale q k^T + mask) v.  The mask is read (``classify_mask``): causal and key-padding masks run on
    the kernels, anything else is computed by PyTorch with the mask as given."""
    if not _kernel_covers(q, k, v):
        return _reference_attention(q, k, v, mask, is_causal, scale)
    kind, lens = classify_mask(mask, q.shape[0], q.shape[-2], k.shape[-2])
    if kind == "other":
        return _reference_attention(q, k, v, mask, is_causal, scale)
    return _attention(q, k, v, bool(is_causal) or kind == "causal", lens, scale)


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
    if residual.shape != x.shape or residual.dtype != x.dtype:  # a broadcast add (embedding sums): add first
        return zenith_layernorm(x + residual, weight, bias, eps)
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    r2 = residual.reshape(-1, x.shape[-1]).contiguous()
    return ops.add_layernorm(x2, r2, weight.to(x.dtype), bias.to(x.dtype), float(eps)).reshape(x.shape)


@torch.fx.wrap
def zenith_linear_gelu(x, weight, bias):
    if x.shape[-1] % 8 or x.dtype not in (torch.float16, torch.float32):  # widths the GEMM kernels do not take
        return F.gelu(F.linear(x, weight, bias), approximate="tanh")
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
    """The pattern matches ANY additive mask (a key-padding mask as well as the causal one the reference's name
    promises, fx_patterns.py:117-135), so the replacement hands the mask on and the leaf decides what it is."""
    return zenith_masked_flash_attention(q, k, v, mask)


def functional_sdpa_pattern(q, k, v):
    return F.scaled_dot_product_attention(q, k, v)


def functional_sdpa_masked_pattern(q, k, v, mask):
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=0.0, is_causal=False)


def functional_sdpa_masked_replacement(q, k, v, mask):
    return zenith_masked_flash_attention(q, k, v, mask)


def gelu_tanh_pattern(x):
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def zenith_gelu_replacement(x):
    return zenith_gelu(x)


def gelu_new_pattern(x):
    """The tanh GELU as HuggingFace writes it (``NewGELUActivation``: the cube through ``torch.pow``)."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * torch.pow(x, 3.0))))


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
            FXPattern("sdpa_to_flash", sdpa_pattern, zenith_sdpa_replacement, priority=20),
            FXPattern("functional_sdpa_masked_to_flash", functional_sdpa_masked_pattern, functional_sdpa_masked_replacement,
                      priority=19),
            FXPattern("functional_sdpa_to_flash", functional_sdpa_pattern, zenith_sdpa_replacement, priority=18)]


def get_activation_patterns() -> list:
    return [FXPattern("linear_gelu_to_fused", linear_gelu_pattern, zenith_linear_gelu_replacement, priority=12),
            FXPattern("gelu_tanh_to_native", gelu_tanh_pattern, zenith_gelu_replacement, priority=10),
            FXPattern("gelu_new_to_native", gelu_new_pattern, zenith_gelu_replacement, priority=10)]


def get_normalization_patterns() -> list:
    return [make_add_layernorm_pattern(768, 1e-12), make_add_layernorm_pattern(1024, 1e-12),
            FXPattern("manual_layernorm_to_native", layernorm_pattern, zenith_layernorm_replacement, priority=10)]


def get_all_patterns() -> list:
    return get_attention_patterns() + get_activation_patterns() + get_normalization_patterns()


def rewrite_calls(gm: torch.fx.GraphModule) -> dict:
    """Node-by-node rewrites of calls whose arguments vary too much for a fixed pattern - the forms a HuggingFace
    encoder traces to under ``torch.compile``:

    * ``dropout(x, p, training=False)`` and ``dropout(x, 0.0, ...)`` are removed (identity at inference);
    * ``F.scaled_dot_product_attention(q, k, v, attn_mask=, dropout_p=0.0, scale=, is_causal=)`` with any mask /
      scale / causal arguments becomes ``zenith_masked_flash_attention`` (which reads the mask at run time);
    * ``F.layer_norm(x + r, (H,), w, b, eps)`` becomes ``zenith_add_layernorm``, a plain ``F.layer_norm`` over the
      last dimension ``zenith_layernorm``;
    * ``zenith_gelu(F.linear(x, w, b))`` becomes ``zenith_linear_gelu``.
    Returns ``{rewrite name: count}``."""
    import operator

    counts = {"dropout_removed": 0, "functional_sdpa_call_to_flash": 0, "add_layer_norm_call": 0, "layer_norm_call": 0,
              "linear_then_gelu": 0}
    g = gm.graph

    def is_fn(n, *fns):
        return n.op == "call_function" and any(n.target is f for f in fns)

    for n in list(g.nodes):
        if is_fn(n, F.dropout, torch.dropout):
            a = list(n.args) + [None] * 4
            p_ = n.kwargs.get("p", a[1] if a[1] is not None else 0.5)
            training = n.kwargs.get("training", n.kwargs.get("train", a[2] if a[2] is not None else True))
            if training is False or p_ == 0.0:
                n.replace_all_uses_with(n.args[0])
                g.erase_node(n)
                counts["dropout_removed"] += 1
    for n in list(g.nodes):
        if is_fn(n, F.scaled_dot_product_attention):
            kw = dict(n.kwargs)
            a = list(n.args)
            mask = kw.get("attn_mask", a[3] if len(a) > 3 else None)
            drop = kw.get("dropout_p", a[4] if len(a) > 4 else 0.0)
            causal = kw.get("is_causal", a[5] if len(a) > 5 else False)
            scale = kw.get("scale", None)
            if drop != 0.0 or kw.get("enable_gqa", False) or isinstance(causal, torch.fx.Node):
                continue
            with g.inserting_before(n):
                new = g.call_function(zenith_masked_flash_attention, (a[0], a[1], a[2], mask, scale, causal))
            n.replace_all_uses_with(new)
            g.erase_node(n)
            counts["functional_sdpa_call_to_flash"] += 1
    for n in list(g.nodes):
        if is_fn(n, F.layer_norm):
            a = list(n.args)
            shape = n.kwargs.get("normalized_shape", a[1] if len(a) > 1 else None)
            w = n.kwargs.get("weight", a[2] if len(a) > 2 else None)
            b = n.kwargs.get("bias", a[3] if len(a) > 3 else None)
            eps = n.kwargs.get("eps", a[4] if len(a) > 4 else 1e-5)
            if not isinstance(shape, (tuple, list)) or len(shape) != 1 or w is None or b is None:
                continue
            src = a[0]
            with g.inserting_before(n):
                if isinstance(src, torch.fx.Node) and is_fn(src, operator.add, torch.add) and len(src.users) == 1 and \
                        len(src.args) == 2 and all(isinstance(t, torch.fx.Node) for t in src.args) and not src.kwargs:
                    new = g.call_function(zenith_add_layernorm, (src.args[0], src.args[1], w, b, eps))
                    counts["add_layer_norm_call"] += 1
                else:
                    src = None
                    new = g.call_function(zenith_layernorm, (a[0], w, b, eps))
                    counts["layer_norm_call"] += 1
            n.replace_all_uses_with(new)
            g.erase_node(n)
            if src is not None:
                g.erase_node(src)
    for n in list(g.nodes):
        if is_fn(n, zenith_gelu):
            src = n.args[0]
            if isinstance(src, torch.fx.Node) and is_fn(src, F.linear) and len(src.users) == 1:
                a = list(src.args)
                w = src.kwargs.get("weight", a[1] if len(a) > 1 else None)
                b = src.kwargs.get("bias", a[2] if len(a) > 2 else None)
                with g.inserting_before(n):
                    new = g.call_function(zenith_linear_gelu, (a[0], w, b))
                n.replace_all_uses_with(new)
                g.erase_node(n)
                g.erase_node(src)
                counts["linear_then_gelu"] += 1
    g.lint()
    gm.recompile()
    return counts


def apply_patterns(gm: torch.fx.GraphModule, patterns: list | None = None, calls: bool = True) -> dict:
    """Rewrite ``gm`` in place, highest priority first, then (``calls``) the node-by-node rewrites of
    ``rewrite_calls``; returns ``{name: matches replaced}``."""
    from torch.fx import subgraph_rewriter

    counts = {}
    for pat in sorted(patterns if patterns is not None else get_all_patterns(), key=lambda p: -p.priority):
        if not pat.enabled:
            continue
        counts[pat.name] = len(subgraph_rewriter.replace_pattern(gm, pat.pattern_fn, pat.replacement_fn))
    gm.recompile()
    if calls and patterns is None:
        counts.update(rewrite_calls(gm))
    return counts


last_backend_counts: dict = {}


def zenith_backend(gm: torch.fx.GraphModule, example_inputs):
    """``torch.compile(model, backend=zenith_backend)``: apply the patterns to the captured graph, run it eagerly.
    The rewrite counts of the most recent graph are left in ``last_backend_counts``."""
    counts = apply_patterns(gm)
    last_backend_counts.clear()
    last_backend_counts.update(counts)
    return gm.forward
