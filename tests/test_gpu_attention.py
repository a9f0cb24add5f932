"""tcgen05 flash-attention forward against the fp32 CPU oracle (masks, causal, ragged lengths)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import ops

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


def run(cuda, B, H, S, D, causal=False, lens=None, seed=0, dtype=np.float16):
    q, k, v = (rng(seed + i).standard_normal((B, H, S, D)).astype(dtype) for i in range(3))
    kl = None if lens is None else np.array(lens, np.int32)
    o = ops.flash_attention(*(torch.from_numpy(a).to(cuda) for a in (q, k, v)), causal=causal,
                            kv_lens=None if kl is None else torch.from_numpy(kl).to(cuda))
    want = O.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), kl, causal)
    return o, want


@pytest.mark.parametrize("B,H,S,D,causal,lens", [
    (1, 12, 32, 64, False, None),            # the shape of benchmarks/flash_attention_benchmark.py:129-153
    (2, 3, 128, 64, False, [128, 96]),       # key-padding mask as in the encoder
    (1, 2, 256, 64, True, None), (1, 2, 200, 64, False, None), (1, 1, 129, 64, True, None),
    (1, 1, 128, 128, False, None), (2, 2, 384, 128, True, [384, 200]), (1, 2, 1024, 64, True, None),
    (1, 1, 1, 64, False, None), (2, 1, 300, 128, False, [1, 299])])
def test_attention_fp16(cuda, B, H, S, D, causal, lens):
    o, want = run(cuda, B, H, S, D, causal, lens)
    got = o.float().cpu().numpy()
    assert o.dtype == torch.float16 and not np.isnan(got).any()
    # fp16 path within 1e-2 (relative to the output scale) of the fp32 path
    assert np.max(np.abs(got - want)) < 1e-2 * max(1.0, np.abs(want).max())
    assert np.mean(np.abs(got - want)) < 2e-4


def test_fully_masked_batch_yields_zeros(cuda):
    o, want = run(cuda, 2, 2, 200, 64, lens=[0, 77])
    assert torch.all(o[0] == 0) and np.all(want[0] == 0)
    assert np.max(np.abs(o[1].float().cpu().numpy() - want[1])) < 1e-2


def test_fp32_binding_shape_and_dtype(cuda):
    """The reference binding takes and returns fp32 [batch, heads, seq, dim] (cuda_bindings.cpp:90-106)."""
    o, want = run(cuda, 1, 12, 32, 64, dtype=np.float32, seed=42)
    assert o.dtype == torch.float32 and tuple(o.shape) == (1, 12, 32, 64)
    assert np.max(np.abs(o.cpu().numpy() - want)) < 1e-2


def test_strided_qkv_and_int8_copy(cuda):
    """Q, K, V read in place from a fused [tokens, 3*hidden] projection; output written as [tokens, hidden]
    with an int8 copy, as the encoder does."""
    B, S, nh, hd = 2, 128, 4, 64
    H = nh * hd
    qkv = rng(1).standard_normal((B * S, 3 * H)).astype(np.float16)
    lens = np.array([128, 50], np.int32)
    t = torch.from_numpy(qkv).to(cuda)
    out = torch.empty((B * S, H), dtype=torch.float16, device=cuda)
    outq = torch.empty((B * S, H), dtype=torch.int8, device=cuda)
    qs, os_ = (S * 3 * H, hd, 3 * H), (S * H, hd, H)
    ops.flash_attention_strided(t, t[:, H:], t[:, 2 * H:], out, B, nh, S, hd, qs, qs, qs, os_,
                                kv_lens=torch.from_numpy(lens).to(cuda), out_q=outq, out_scale=0.02)
    f = qkv.astype(np.float32)
    split = lambda a: np.ascontiguousarray(a.reshape(B, S, nh, hd).transpose(0, 2, 1, 3))
    want = O.attention(split(f[:, :H]), split(f[:, H:2 * H]), split(f[:, 2 * H:]), lens)
    want = want.transpose(0, 2, 1, 3).reshape(B * S, H)
    got = out.float().cpu().numpy()
    assert np.max(np.abs(got - want)) < 1e-2
    assert np.array_equal(outq.cpu().numpy(), O.quantize(got, 0.02))


@pytest.mark.parametrize("S,lens,causal", [
    (128, [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 127], False),  # every kind of boundary inside a 32-key chunk
    (100, [100, 99, 37, 5], False), (100, [100, 64, 33, 1], True), (17, [17, 3], True), (128, [128, 96, 32, 0], True)])
def test_single_block_kernel_key_length_boundaries(cuda, S, lens, causal):
    """Sequences of at most 128 keys (the encoder's kernel): chunk-level masking and the shortened P V product."""
    o, want = run(cuda, len(lens), 2, S, 64, causal, lens, seed=7)
    got = o.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert np.max(np.abs(got - want)) < 1e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("S,hd", [(128, 128), (96, 128), (384, 64), (300, 128)])
def test_int8_copy_equals_quantized_output(cuda, S, hd):
    """Both kernels (one key block / pipelined), both head sizes, strided in and out with key lengths: the int8
    copy is exactly the quantization of the fp16 output beside it."""
    B, nh = 3, 2
    H = nh * hd
    qkv = rng(S + hd).standard_normal((B * S, 3 * H)).astype(np.float16)
    lens = np.array([S, max(1, S // 3), S - 1], np.int32)
    t = torch.from_numpy(qkv).to(cuda)
    out = torch.empty((B * S, H), dtype=torch.float16, device=cuda)
    outq = torch.empty((B * S, H), dtype=torch.int8, device=cuda)
    qs, os_ = (S * 3 * H, hd, 3 * H), (S * H, hd, H)
    ops.flash_attention_strided(t, t[:, H:], t[:, 2 * H:], out, B, nh, S, hd, qs, qs, qs, os_,
                                kv_lens=torch.from_numpy(lens).to(cuda), out_q=outq, out_scale=0.013)
    f = qkv.astype(np.float32)
    split = lambda a: np.ascontiguousarray(a.reshape(B, S, nh, hd).transpose(0, 2, 1, 3))
    want = O.attention(split(f[:, :H]), split(f[:, H:2 * H]), split(f[:, 2 * H:]), lens).transpose(0, 2, 1, 3).reshape(B * S, H)
    got = out.float().cpu().numpy()
    assert np.max(np.abs(got - want)) < 1e-2
    assert np.array_equal(outq.cpu().numpy(), O.quantize(got, 0.013))


def test_properties_at_encoder_size(cuda):
    """B = 32, H = 12, S = 128, d = 64 (too large for the CPU oracle in a test): rows of P sum to one, so
    V = 1 gives O = 1; permuting the keys (with their values) changes nothing beyond fp16 rounding; a key
    length is the same as truncating K and V."""
    B, H, S, D = 32, 12, 128, 64
    g = torch.Generator(device="cpu").manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D, generator=g).half().to(cuda) for _ in range(3))
    ones = ops.flash_attention(q, k, torch.ones_like(v))
    assert (ones.float() - 1).abs().max().item() < 2e-3
    base = ops.flash_attention(q, k, v)
    perm = torch.randperm(S, generator=g).to(cuda)
    assert (ops.flash_attention(q, k[:, :, perm], v[:, :, perm]).float() - base.float()).abs().max().item() < 4e-3
    lens = torch.full((B,), 77, dtype=torch.int32, device=cuda)
    cut = ops.flash_attention(q, k, v, kv_lens=lens)
    # the truncated call has 77 query rows as well (the binding wants equal shapes); compare those rows
    ref = ops.flash_attention(q[:, :, :77].contiguous(), k[:, :, :77].contiguous(), v[:, :, :77].contiguous())
    assert (cut[:, :, :77].float() - ref.float()).abs().max().item() < 2e-3
