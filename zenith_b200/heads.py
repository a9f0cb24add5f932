"""What sits on top of the encoder's hidden states: the BERT pooler and task heads.

The reference's encoder benchmarks measure themselves against HuggingFace's ``BertModel``, which ends in a pooler
(benchmarks/bert_hybrid.py:188-196); the reference itself stops at the last LayerNorm.  These heads keep the
[CLS] rows on the device and read them IN PLACE: the GEMM takes the hidden states ``[batch * seq, hidden]`` with a
row stride of ``seq * hidden`` elements, so no gather kernel runs.

    pooled = tanh(h[:, 0] @ Wp^T + bp)            Pooler
    logits = pooled @ Wc^T + bc                    ClassificationHead
    logits[t] = h[t] @ Wt^T + bt                   TokenClassificationHead (every token)
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops


def _f16(a, device):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=torch.float32).to(device=device, dtype=torch.float16)


def _f32(a, device):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=torch.float32).to(device)


class Pooler:
    """``tanh(dense(hidden_states[:, 0]))``: fp16 tensor-core GEMM over the [CLS] rows, fp32 accumulation."""

    def __init__(self, weight, bias, device="cuda:0"):
        self.w, self.b = _f16(weight, device), _f32(bias, device)
        if self.w.shape[0] != self.w.shape[1] or self.b.numel() != self.w.shape[0]:
            raise RuntimeError("the pooler is a square Linear with one bias per output")

    def __call__(self, hidden: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """``hidden``: fp16 ``[batch * seq, H]`` (the encoder's output buffer); returns fp16 ``[batch, H]``."""
        if hidden.dtype != torch.float16 or tuple(hidden.shape) != (batch * seq, self.w.shape[1]) or not hidden.is_contiguous():
            raise RuntimeError("hidden must be contiguous fp16 [batch * seq, hidden]")
        cls_rows = hidden.view(batch, seq, -1)[:, 0, :]  # a view: row stride seq * H
        return ops.tanh(ops.linear_fp16(cls_rows, self.w, self.b))


class ClassificationHead:
    """``pooled @ W^T + b`` -> fp32 logits ``[batch, classes]``."""

    def __init__(self, weight, bias, device="cuda:0"):
        self.w, self.b = _f16(weight, device), _f32(bias, device)
        if self.w.shape[1] % 8:
            raise RuntimeError("the input width must be a multiple of 8")

    def __call__(self, pooled: torch.Tensor) -> torch.Tensor:
        return ops.linear_fp16(pooled, self.w, self.b, out_dtype=torch.float32)


class TokenClassificationHead(ClassificationHead):
    """The same Linear applied to every token: fp32 logits ``[batch * seq, classes]``."""

    def __call__(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear_fp16(hidden, self.w, self.b, out_dtype=torch.float32)
