"""The fused W8A8 QKV-projection + attention kernel (zen_qkv_attention_i8): bit-identical to the projection
(zen_linear_i8, fp16 output) followed by attention (zen_flash_attention_f16) on its column slices, and within the
attention tolerance of the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import _capi, ops

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def two_kernels(xq, wq, ws, b, B, S, heads, lens, out_scale, x_scale=0.02):
    H = heads * 64
    qkv = ops.linear_int8(xq, wq, x_scale, ws, b, out_dtype=torch.float16)
    ctx = torch.empty((B * S, H), dtype=torch.float16, device=xq.device)
    ctxq = torch.empty((B * S, H), dtype=torch.int8, device=xq.device)
    qs, os_ = (S * 3 * H, 64, 3 * H), (S * H, 64, H)
    ops.flash_attention_strided(qkv, qkv[:, H:], qkv[:, 2 * H:], ctx, B, heads, S, 64, qs, qs, qs, os_, kv_lens=lens,
                                out_q=ctxq, out_scale=out_scale)
    return qkv, ctx, ctxq


@pytest.mark.parametrize("B,S,heads,K,lens", [
    (1, 128, 1, 128, None), (2, 128, 2, 256, [128, 77]), (3, 96, 4, 256, [96, 64, 1]), (2, 17, 2, 64, [17, 5]),
    (2, 8, 1, 64, [8, 3]), (4, 128, 12, 768, [128, 100, 33, 0]), (5, 40, 3, 192, [40, 39, 16, 15, 0]),
    (32, 128, 12, 768, "ragged")])
def test_fused_equals_projection_then_attention(cuda, B, S, heads, K, lens):
    H = heads * 64
    x = rng(B * S + K).integers(-128, 128, (B * S, K), dtype=np.int8)
    w = rng(K).integers(-128, 128, (3 * H, K), dtype=np.int8)
    ws = ((rng(3).random(3 * H) + 0.5) * (0.009 / np.sqrt(K))).astype(np.float32)  # Q, K, V of unit scale
    b = (rng(4).standard_normal(3 * H) * 0.1).astype(np.float32)
    if isinstance(lens, str):
        lens = (S - rng(5).integers(0, 33, B)).tolist()
    kl = None if lens is None else dev(np.array(lens, np.int32), cuda)
    xd, wd, wsd, bd = dev(x, cuda), dev(w, cuda), dev(ws, cuda), dev(b, cuda)
    qkv2, ctx2, ctxq2 = two_kernels(xd, wd, wsd, bd, B, S, heads, kl, 0.02)
    ctx, ctxq, qkv = ops.qkv_attention_int8(xd, wd, 0.02, wsd, bd, B, S, heads, kv_lens=kl, out_scale=0.02, emit_qkv=True)
    assert _capi.device_status() == 0
    assert torch.equal(qkv, qkv2)
    assert torch.equal(ctx, ctx2)
    assert torch.equal(ctxq, ctxq2)
    # with the early weight request, without the int8 copy, without the copy of Q, K, V: same bits
    ctx3 = ops.qkv_attention_int8(xd, wd, 0.02, wsd, bd, B, S, heads, kv_lens=kl, constant_weights=True,
                                  prefetch=(wd,))
    assert torch.equal(ctx3, ctx)
    if B * S * heads <= 4096:
        # against the oracle: exact projection (fp16 bits), attention within 1e-2
        want_qkv = O.linear_int8(x, w, 0.02, ws, b, "none", "f16")
        assert np.array_equal(qkv.cpu().numpy().view(np.uint16), want_qkv.view(np.uint16))
        f = want_qkv.astype(np.float32)
        split = lambda a: np.ascontiguousarray(a.reshape(B, S, heads, 64).transpose(0, 2, 1, 3))
        o = O.attention(split(f[:, :H]), split(f[:, H:2 * H]), split(f[:, 2 * H:]), None if lens is None else np.array(lens, np.int32))
        o = o.transpose(0, 2, 1, 3).reshape(B * S, H)
        got = ctx.float().cpu().numpy()
        assert np.max(np.abs(got - o)) < 1e-2 * max(1.0, np.abs(o).max())
        assert np.array_equal(ctxq.cpu().numpy(), O.quantize(got, 0.02))


def test_fused_back_to_back_and_no_scale_no_bias(cuda):
    B, S, heads, K = 8, 128, 12, 768
    H = heads * 64
    x = dev(rng(1).integers(-128, 128, (B * S, K), dtype=np.int8), cuda)
    ws_ = [dev(rng(10 + i).integers(-16, 16, (3 * H, K), dtype=np.int8), cuda) for i in range(3)]
    ref = [ops.qkv_attention_int8(x, w, 1e-3, None, None, B, S, heads).clone() for w in ws_]
    for _ in range(10):
        outs = [ops.qkv_attention_int8(x, w, 1e-3, None, None, B, S, heads, constant_weights=True) for w in ws_]
    for a, b in zip(ref, outs):
        assert torch.equal(a, b)
    qkv2, ctx2, _ = two_kernels(x, ws_[0], None, None, B, S, heads, None, 0.02, x_scale=1e-3)
    assert torch.equal(ref[0], ctx2)
    assert _capi.device_status() == 0


def test_longer_sequences_are_refused(cuda):
    x = torch.zeros((256, 64), dtype=torch.int8, device=cuda)
    w = torch.zeros((192, 64), dtype=torch.int8, device=cuda)
    with pytest.raises(_capi.ZenithError) as e:
        ops.qkv_attention_int8(x, w, 1.0, None, None, 1, 256, 1)
    assert e.value.status == _capi.ERR_UNSUPPORTED
