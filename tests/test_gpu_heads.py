"""Pooler and task heads on the encoder's output, against the CPU oracle (fp16 operands: within 1e-2 of fp32)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import _capi, ops
from zenith_b200.heads import ClassificationHead, Pooler, TokenClassificationHead

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("n", [1, 7, 4099])
def test_tanh_bit_exact_with_the_oracle_and_close_to_libm(cuda, n):
    x = (3 * rng(n).standard_normal(n)).astype(np.float32)
    got = ops.tanh(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert np.array_equal(got.view(np.int32), O.tanh(x).view(np.int32))
    assert np.max(np.abs(got - O.tanh(x, libm=True))) < 5e-7
    h = x.astype(np.float16)
    assert np.array_equal(ops.tanh(torch.from_numpy(h).to(cuda)).cpu().numpy(), O.tanh(h.astype(np.float32)).astype(np.float16))


@pytest.mark.parametrize("B,S,H,C", [(32, 128, 768, 2), (3, 40, 256, 9), (1, 1, 64, 3)])
def test_pooler_and_heads(cuda, B, S, H, C):
    hidden = rng(1).standard_normal((B * S, H)).astype(np.float16)
    wp = (rng(2).standard_normal((H, H)) * 0.03).astype(np.float32)
    bp = (rng(3).standard_normal(H) * 0.1).astype(np.float32)
    wc = (rng(4).standard_normal((C, H)) * 0.05).astype(np.float32)
    bc = (rng(5).standard_normal(C) * 0.1).astype(np.float32)
    hd = torch.from_numpy(hidden).to(cuda)
    pooled = Pooler(wp, bp, cuda)(hd, B, S)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    cls = hidden.reshape(B, S, H)[:, 0].astype(np.float32)
    want = O.tanh(O.gemm_f32_nt(cls, f16(wp)) + bp, libm=True)
    got = pooled.float().cpu().numpy()
    assert pooled.dtype == torch.float16 and got.shape == (B, H)
    assert np.max(np.abs(got - want)) < 1e-2
    logits = ClassificationHead(wc, bc, cuda)(pooled).cpu().numpy()
    want_logits = O.gemm_f32_nt(got, f16(wc)) + bc
    assert logits.dtype == np.float32 and np.max(np.abs(logits - want_logits)) < 1e-2
    tok = TokenClassificationHead(wc, bc, cuda)(hd).cpu().numpy()
    assert tok.shape == (B * S, C)
    assert np.max(np.abs(tok - (O.gemm_f32_nt(hidden.astype(np.float32), f16(wc)) + bc))) < 1e-2 * max(1.0, np.abs(tok).max())
    assert _capi.device_status() == 0


def test_pooler_matches_huggingface(cuda):
    transformers = pytest.importorskip("transformers")
    torch.manual_seed(0)
    cfg = transformers.BertConfig(num_hidden_layers=1, vocab_size=100)
    pooler = transformers.models.bert.modeling_bert.BertPooler(cfg).eval().to(cuda)
    hidden = torch.randn(4, 32, 768, device=cuda).half()
    with torch.no_grad():
        want = pooler(hidden.float())
    got = Pooler(pooler.dense.weight.detach().cpu().numpy(), pooler.dense.bias.detach().cpu().numpy(), cuda)(
        hidden.reshape(4 * 32, 768).contiguous(), 4, 32)
    assert (got.float() - want).abs().max().item() < 1e-2
