"""The `zenith_cuda` drop-in surface: the six functions of core/bindings/cuda_bindings.cpp:134-145 with the
reference's argument order, dtypes, shapes and error type, plus registration as a kernel plug-in."""
import sys

import numpy as np
import pytest
import torch

import zenith_b200
from zenith_b200 import _capi, registry

pytestmark = pytest.mark.gpu


def test_import_name_and_smoke_shapes(cuda):
    zenith_b200.install_as_zenith_cuda()
    import zenith_cuda  # the name zenith/runtime/kernel_registry.py:225 imports

    assert sys.modules["zenith_cuda"] is zenith_cuda
    x = torch.randn(64, 768, device=cuda)
    # zenith/build_cuda.py:114-131 smoke sequence
    assert zenith_cuda.relu(x).shape == x.shape
    assert zenith_cuda.gelu(x).shape == x.shape
    g, b = torch.ones(768, device=cuda), torch.zeros(768, device=cuda)
    y = zenith_cuda.layernorm(x, g, b)  # eps defaults to 1e-5
    assert torch.allclose(y, torch.nn.functional.layer_norm(x, (768,), g, b, 1e-5), atol=1e-4, rtol=1e-4)
    assert torch.allclose(zenith_cuda.gelu(x), torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-5)
    a, w = torch.randn(128, 64, device=cuda), torch.randn(64, 256, device=cuda)
    c = zenith_cuda.matmul(a, w)
    assert c.shape == (128, 256) and c.dtype == torch.float32
    assert (c - a.double() @ w.double()).abs().max().item() < 0.1  # TF32
    # BENCHMARK_REPORT.md:178-185: A[128,64] f16 . B[64,256] f16 -> C[128,256] f32
    c = zenith_cuda.wmma_matmul(a.half(), w.half())
    assert c.shape == (128, 256) and c.dtype == torch.float32
    assert (c - a.half().double() @ w.half().double()).abs().max().item() < 1e-3
    q = torch.randn(1, 12, 32, 64, device=cuda)
    o = zenith_cuda.flash_attention(q, q, q)
    assert o.shape == q.shape and o.dtype == torch.float32
    ref = torch.nn.functional.scaled_dot_product_attention(q, q, q)
    assert (o - ref).abs().max().item() < 1e-2


def test_argument_checks_raise_runtime_error(cuda):
    from zenith_b200 import zenith_cuda

    with pytest.raises(RuntimeError):
        zenith_cuda.layernorm(torch.zeros(2, 3, 4, device=cuda), torch.ones(4, device=cuda), torch.zeros(4, device=cuda))
    with pytest.raises(RuntimeError):
        zenith_cuda.wmma_matmul(torch.zeros(16, 16, device=cuda), torch.zeros(16, 16, device=cuda))  # not fp16
    with pytest.raises(RuntimeError):
        zenith_cuda.matmul(torch.zeros(16, 8, device=cuda), torch.zeros(16, 8, device=cuda))  # inner dims
    with pytest.raises(RuntimeError):
        zenith_cuda.flash_attention(torch.zeros(2, 3, 4, device=cuda), None, None)


def test_runs_on_the_current_torch_stream(cuda):
    s = torch.cuda.Stream()
    x = torch.randn(1 << 20, device=cuda)
    from zenith_b200 import zenith_cuda

    with torch.cuda.stream(s):
        y = zenith_cuda.gelu(x)
    s.synchronize()
    assert torch.allclose(y, torch.nn.functional.gelu(x, approximate="tanh"), atol=1e-5)


def test_registry_plugin(cuda):
    """Registers KernelSpecs the way zenith/runtime/kernel_registry.py:215-286 does for `zenith_cuda`,
    into a registry object with the reference's `register(spec)` method, and dispatches like
    zenith/runtime/dispatcher.py:235-315."""

    class FakeRegistry:
        def __init__(self):
            self.specs = []

        def register(self, spec):
            self.specs.append(spec)

    reg = FakeRegistry()
    n = registry.register(reg)
    assert n == len(reg.specs) >= 6
    by_op = {}
    for s in reg.specs:
        assert s.priority > 30 and s.requires_gpu
        for op in s.op_types:
            by_op.setdefault(op, s)
    for op in ("Linear", "MatMul", "Gelu", "LayerNorm", "Attention", "FusedAddLayerNorm", "FusedLinearGELU",
               "FusedBiasGeLU"):
        assert op in by_op
    x = torch.randn(32, 64, device=cuda)
    w = torch.randn(128, 64, device=cuda)
    b = torch.randn(128, device=cuda)
    y = by_op["Linear"].kernel_fn(x, w, b)  # dispatcher calls fn(x, w, b)
    assert (y - torch.nn.functional.linear(x, w, b)).abs().max().item() < 0.1
    y = by_op["FusedLinearGELU"].kernel_fn(x, w, b)
    assert (y - torch.nn.functional.gelu(torch.nn.functional.linear(x, w, b), approximate="tanh")).abs().max().item() < 0.1
    g, be = torch.ones(64, device=cuda), torch.zeros(64, device=cuda)
    r = torch.randn(32, 64, device=cuda)
    y = by_op["FusedAddLayerNorm"].kernel_fn(x, r, g, be, 1e-5)
    assert torch.allclose(y, torch.nn.functional.layer_norm(x + r, (64,), g, be, 1e-5), atol=1e-4, rtol=1e-4)


def test_fx_rewritten_module_matches_the_original(cuda):
    """A traced attention + GELU + LayerNorm + Linear-GELU block, rewritten onto the kernels by the FX patterns,
    computes what the PyTorch original computes (fp16 attention / TF32 GEMM tolerances)."""
    import torch.fx
    import torch.nn.functional as F

    from zenith_b200 import fx_patterns as P

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.w = torch.nn.Parameter(1 + 0.1 * torch.randn(64))
            self.b = torch.nn.Parameter(0.1 * torch.randn(64))
            self.fc = torch.nn.Linear(64, 128)

        def forward(self, q, k, v, mask):
            a = P.sdpa_pattern(q, k, v)
            c = P.causal_sdpa_pattern(q, k, v, mask)
            g = P.gelu_tanh_pattern(a + c)
            n = P.layernorm_pattern(g, self.w, self.b, 1e-5)
            return F.gelu(F.linear(n, self.fc.weight, self.fc.bias), approximate="tanh")

    torch.manual_seed(0)
    blk = Block().to(cuda)
    q, k, v = (torch.randn(2, 4, 96, 64, device=cuda) for _ in range(3))
    mask = torch.full((96, 96), float("-inf"), device=cuda).triu(1)
    want = blk(q, k, v, mask)
    gm = torch.fx.symbolic_trace(blk)
    counts = P.apply_patterns(gm)
    assert sum(counts.values()) == 5
    got = gm(q, k, v, mask)
    assert got.shape == want.shape and (got - want).abs().max().item() < 2e-2
    assert _capi.device_status() == 0


def test_torch_compile_of_a_huggingface_bert_runs_on_the_kernels(cuda):
    """A stock HuggingFace ``BertModel`` (BERT-base widths, tanh GELU, random init) through
    ``torch.compile(model, backend=zenith_backend)``: per layer the attention (with the key-padding mask turned into
    key lengths), both residual LayerNorms and the Linear + GELU run on this library's kernels, and the hidden
    states match eager PyTorch within the fp16-attention / TF32-GEMM tolerance.  This is the use the reference's
    torch.compile backend exists for (zenith/adapters/pytorch_adapter.py:606-744, fx_patterns.py:95-114)."""
    transformers = pytest.importorskip("transformers")
    from zenith_b200 import fx_patterns as P
    from zenith_b200 import ops

    torch.manual_seed(0)
    layers = 2
    cfg = transformers.BertConfig(hidden_act="gelu_new", num_hidden_layers=layers, vocab_size=2000, max_position_embeddings=128)
    model = transformers.BertModel(cfg, add_pooling_layer=False).eval().to(cuda)
    ids = torch.randint(0, 2000, (3, 96), device=cuda)
    mask = torch.ones(3, 96, dtype=torch.long, device=cuda)
    mask[1, 70:] = 0
    mask[2, 33:] = 0
    with torch.no_grad():
        want = model(input_ids=ids, attention_mask=mask).last_hidden_state
        before = ops.launch_count
        got = torch.compile(model, backend=P.zenith_backend)(input_ids=ids, attention_mask=mask).last_hidden_state
    counts = dict(P.last_backend_counts)
    assert counts["functional_sdpa_call_to_flash"] == layers and counts["linear_then_gelu"] == layers
    assert counts["add_layer_norm_call"] >= 2 * layers
    assert ops.launch_count - before >= 4 * layers  # the leaves really launched this library's kernels
    assert got.shape == want.shape and not torch.isnan(got).any()
    err = (got - want).abs()
    assert err.max().item() < 3e-2 and err.mean().item() < 2e-3
    assert _capi.device_status() == 0
