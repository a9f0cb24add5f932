"""FX patterns: a hand-written attention / GELU / LayerNorm module is rewritten onto the kernel leaves
(graph structure only; the kernels themselves are checked on the GPU)."""
import torch
import torch.fx
import torch.nn.functional as F

from zenith_b200 import fx_patterns as P


class Block(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.w = torch.nn.Parameter(torch.ones(64))
        self.b = torch.nn.Parameter(torch.zeros(64))
        self.fc = torch.nn.Linear(64, 128)

    def forward(self, q, k, v, mask):
        a = P.sdpa_pattern(q, k, v)
        c = P.causal_sdpa_pattern(q, k, v, mask)
        g = P.gelu_tanh_pattern(a + c)
        n = P.layernorm_pattern(g, self.w, self.b, 1e-5)
        return F.gelu(F.linear(n, self.fc.weight, self.fc.bias), approximate="tanh")


def targets(gm):
    return [n.target.__name__ for n in gm.graph.nodes if n.op == "call_function" and hasattr(n.target, "__name__")]


def test_patterns_are_found_and_replaced_by_kernel_leaves():
    gm = torch.fx.symbolic_trace(Block())
    before = targets(gm)
    assert "softmax" in before and "tanh" in before
    counts = P.apply_patterns(gm)
    assert counts["sdpa_to_flash"] == 1 and counts["causal_sdpa_to_flash"] == 1
    assert counts["gelu_tanh_to_native"] == 1 and counts["manual_layernorm_to_native"] == 1
    assert counts["linear_gelu_to_fused"] == 1
    after = targets(gm)
    for leaf in ("zenith_flash_attention", "zenith_causal_flash_attention", "zenith_gelu", "zenith_layernorm",
                 "zenith_linear_gelu"):
        assert leaf in after
    assert "softmax" not in after and "tanh" not in after and "sqrt" not in after


def test_pattern_lists_mirror_the_reference_names():
    names = {p.name for p in P.get_all_patterns()}
    assert {"sdpa_to_flash", "gelu_tanh_to_native", "manual_layernorm_to_native"} <= names
    assert "causal_sdpa_to_flash" in names  # defined but never registered in the reference
    assert all(callable(p.pattern_fn) and callable(p.replacement_fn) for p in P.get_all_patterns())


def test_add_layernorm_pattern_matches_the_encoder_form():
    class Res(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ln = torch.nn.LayerNorm(768, eps=1e-12)

        def forward(self, x, r):
            return F.layer_norm(x + r, (768,), self.ln.weight, self.ln.bias, 1e-12)

    gm = torch.fx.symbolic_trace(Res())
    counts = P.apply_patterns(gm)
    assert counts["add_layernorm_768"] == 1 and "zenith_add_layernorm" in targets(gm)


def test_replacements_refuse_cpu_tensors():
    import pytest

    x = torch.zeros(1, 1, 4, 64)
    with pytest.raises(RuntimeError):
        P.zenith_flash_attention(x, x, x)
    with pytest.raises(RuntimeError):
        P.zenith_gelu(x)
