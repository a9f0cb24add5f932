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
    for leaf in ("zenith_flash_attention", "zenith_masked_flash_attention", "zenith_gelu", "zenith_layernorm",
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


def test_the_masked_pattern_keeps_the_mask_and_the_leaf_reads_it():
    """A key-padding mask must not be turned into causal attention: the rewritten node still receives the mask,
    and the classifier tells the three kinds of mask apart."""
    class Att(torch.nn.Module):
        def forward(self, q, k, v, mask):
            return P.causal_sdpa_pattern(q, k, v, mask)

    gm = torch.fx.symbolic_trace(Att())
    assert P.apply_patterns(gm)["causal_sdpa_to_flash"] == 1
    node = next(n for n in gm.graph.nodes if n.op == "call_function" and n.target is P.zenith_masked_flash_attention)
    assert len(node.args) == 4 and node.args[3].name == "mask"
    B, S = 3, 16
    neg = torch.finfo(torch.float32).min
    causal = torch.zeros(S, S).masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), neg)
    assert P.classify_mask(causal, B, S, S)[0] == "causal"
    assert P.classify_mask(causal[None, None], B, S, S)[0] == "causal"
    lens = torch.tensor([16, 9, 1])
    pad = torch.zeros(B, 1, 1, S).masked_fill(torch.arange(S)[None, None, None, :] >= lens[:, None, None, None], neg)
    kind, got = P.classify_mask(pad, B, S, S)
    assert kind == "kv_lens" and got.tolist() == [16, 9, 1] and got.dtype == torch.int32
    kind, got = P.classify_mask(pad.expand(B, 1, S, S), B, S, S)  # the same mask, materialised per query
    assert kind == "kv_lens" and got.tolist() == [16, 9, 1]
    assert P.classify_mask(torch.zeros(B, 1, 1, S), B, S, S)[0] == "none"
    holes = pad.clone()
    holes[1, 0, 0, 2] = neg  # a masked key in the middle: not a suffix
    assert P.classify_mask(holes, B, S, S)[0] == "other"
    assert P.classify_mask(torch.randn(B, 1, S, S), B, S, S)[0] == "other"  # a relative-position bias
    keep = torch.arange(S)[None, None, None, :] < lens[:, None, None, None]  # boolean form: True = attend
    kind, got = P.classify_mask(keep, B, S, S)
    assert kind == "kv_lens" and got.tolist() == [16, 9, 1]
    assert P.classify_mask(torch.ones(B, 1, 1, S, dtype=torch.bool), B, S, S)[0] == "none"
    assert P.classify_mask(torch.ones(S, S, dtype=torch.bool).tril(), B, S, S)[0] == "causal"


def test_shapes_the_kernels_do_not_cover_are_computed_by_pytorch():
    """head size 32 (no kernel) and a bias-like mask: the leaves return what the original expression returns, on
    any device, instead of raising."""
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(2, 3, 10, 32, generator=g) for _ in range(3))
    mask = torch.randn(2, 1, 10, 10, generator=g)
    assert torch.allclose(P.zenith_flash_attention(q, k, v), P.sdpa_pattern(q, k, v), atol=1e-6)
    assert torch.allclose(P.zenith_masked_flash_attention(q, k, v, mask), P.causal_sdpa_pattern(q, k, v, mask), atol=1e-6)
    x, w, b = torch.randn(5, 12, generator=g), torch.randn(7, 12, generator=g), torch.randn(7, generator=g)
    assert torch.allclose(P.zenith_linear_gelu(x, w, b), P.linear_gelu_pattern(x, w, b), atol=1e-6)


def test_functional_sdpa_calls_are_rewritten():
    class Att(torch.nn.Module):
        def forward(self, q, k, v, mask):
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=0.0, is_causal=False)
            return a + F.scaled_dot_product_attention(q, k, v)

    gm = torch.fx.symbolic_trace(Att())
    counts = P.apply_patterns(gm)
    assert counts["functional_sdpa_masked_to_flash"] == 1 and counts["functional_sdpa_to_flash"] == 1
    assert "scaled_dot_product_attention" not in targets(gm)


def test_a_huggingface_bert_traces_onto_the_kernel_leaves():
    """``torch.compile(BertModel, backend=...)``: in the graph Dynamo hands the backend, every layer's attention, both
    residual LayerNorms and the Linear + GELU are rewritten (zenith/adapters/pytorch_adapter.py:606-744 is the
    reference's hook for the same thing; its pattern set only knows the hand-written softmax form).  The rewritten
    graph is inspected, the original one is run (this host has no GPU)."""
    import copy

    import pytest

    transformers = pytest.importorskip("transformers")
    cfg = transformers.BertConfig(hidden_size=128, num_attention_heads=2, num_hidden_layers=2, intermediate_size=256,
                                  hidden_act="gelu_new", vocab_size=1000, max_position_embeddings=64)
    model = transformers.BertModel(cfg, add_pooling_layer=False).eval()
    seen = []

    def backend(gm, example_inputs):
        g2 = copy.deepcopy(gm)
        seen.append((P.apply_patterns(g2), targets(g2)))
        return gm.forward

    ids = torch.randint(0, 1000, (2, 32))
    mask = torch.ones(2, 32, dtype=torch.long)
    mask[1, 20:] = 0
    with torch.no_grad():
        torch.compile(model, backend=backend)(input_ids=ids, attention_mask=mask)
    counts, after = seen[0]
    layers = cfg.num_hidden_layers
    assert counts["functional_sdpa_call_to_flash"] == layers
    assert counts["add_layer_norm_call"] >= 2 * layers
    assert counts["linear_then_gelu"] == layers and counts["gelu_new_to_native"] == layers
    assert "scaled_dot_product_attention" not in after and "layer_norm" not in after and "tanh" not in after
    assert after.count("zenith_masked_flash_attention") == layers and after.count("zenith_linear_gelu") == layers
