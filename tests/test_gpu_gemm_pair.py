"""The CTA-pair GEMM kernel (tcgen05 cta_group::2, two CTAs per 256-row tile) against the CPU oracle, through the
C ABI with the pair kernel forced: integer results bit-exact, fp16 within 1e-2, and always identical to the
one-CTA kernel's output."""
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


@pytest.mark.parametrize("M,N,K,tile", [
    (256, 256, 128, 256), (256, 128, 256, 128), (256, 192, 128, 192),  # one tile, each width
    (1, 16, 16, 0), (100, 72, 80, 0), (129, 257, 400, 0), (300, 328, 512, 0), (333, 1000, 1024, 128),
    (512, 3072, 768, 0), (2048, 768, 3072, 192)])
def test_pair_int8_accumulators_bit_exact(cuda, M, N, K, tile):
    x = rng(M + N).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(K).integers(-128, 128, (N, K), dtype=np.int8)
    acc = ops.linear_int8(dev(x, cuda), dev(w, cuda), 1.0, out_dtype=torch.int32, tile_n=tile, pair=True).cpu().numpy()
    assert _capi.device_status() == 0
    assert np.array_equal(acc, O.gemm_s8(x, w))


@pytest.mark.parametrize("act", ["none", "gelu"])
@pytest.mark.parametrize("out", ["f32", "f16", "s8"])
def test_pair_int8_fused_epilogue_bit_exact(cuda, act, out):
    M, N, K = 600, 328, 512  # ragged in M and N (the second row block of the last tile is partly empty)
    x = rng(1).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(2).integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng(3).random(N) + 0.5) * 1e-3).astype(np.float32)
    b = (rng(4).standard_normal(N) * 0.1).astype(np.float32)
    tdt = {"f32": torch.float32, "f16": torch.float16, "s8": torch.int8}[out]
    kw = dict(act=act, out_dtype=tdt, out_scale=0.05 if out == "s8" else None)
    got = ops.linear_int8(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), pair=True, **kw)
    want = O.linear_int8(x, w, 0.02, ws, b, act, out, 0.05)
    assert np.array_equal(got.cpu().numpy().view(np.uint8), want.view(np.uint8))
    single = ops.linear_int8(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), pair=False, **kw)
    assert torch.equal(got, single)
    assert _capi.device_status() == 0


@pytest.mark.parametrize("N,kw", [(2304, dict(out_dtype=torch.float16)),
                                  (3072, dict(act="gelu", out_dtype=torch.int8, out_scale=0.05))])
@pytest.mark.parametrize("cw", [False, True])
def test_pair_encoder_shapes_whole_output_bit_exact(cuda, N, kw, cw):
    """The QKV and FFN1 GEMMs of BERT-base at 4096 tokens: two to three tiles per pair, with and without the
    early weight request."""
    M, K = 4096, 768
    x = rng(N).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(K + 1).integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng(3).random(N) + 0.5) * 4e-4).astype(np.float32)
    b = (rng(4).standard_normal(N) * 0.1).astype(np.float32)
    got = ops.linear_int8(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), constant_weights=cw, pair=True,
                          **kw).cpu().numpy()
    out = "s8" if kw["out_dtype"] == torch.int8 else "f16"
    want = O.linear_int8(x, w, 0.02, ws, b, kw.get("act", "none"), out, 0.05)
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
    assert _capi.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(256, 320, 520), (100, 72, 80), (4096, 768, 768)])
def test_pair_fp16_linear(cuda, M, N, K):
    x = rng(1).standard_normal((M, K)).astype(np.float16)
    w = (rng(2).standard_normal((N, K)) * 0.1).astype(np.float16)
    b = rng(3).standard_normal(N).astype(np.float32)
    want = (dev(x, cuda).double() @ dev(w, cuda).double().T + dev(b, cuda).double()).cpu().numpy()
    y32 = ops.linear_fp16(dev(x, cuda), dev(w, cuda), dev(b, cuda), out_dtype=torch.float32, pair=True)
    assert np.max(np.abs(y32.cpu().numpy() - want)) / np.abs(want).max() < 1e-4
    assert torch.equal(y32, ops.linear_fp16(dev(x, cuda), dev(w, cuda), dev(b, cuda), out_dtype=torch.float32, pair=False))
    assert _capi.device_status() == 0


def test_pair_back_to_back_launches(cuda):
    """Many launches in a row on one stream (programmatic dependent launch between them): the clusters of
    consecutive kernels overlap at their edges; every result is the same."""
    M, N, K = 1024, 768, 768
    x = dev(rng(1).integers(-128, 128, (M, K), dtype=np.int8), cuda)
    ws_ = [dev(rng(10 + i).integers(-128, 128, (N, K), dtype=np.int8), cuda) for i in range(4)]
    first = [ops.linear_int8(x, w, 1.0, out_dtype=torch.int32, pair=True).clone() for w in ws_]
    for _ in range(10):
        outs = [ops.linear_int8(x, w, 1.0, out_dtype=torch.int32, pair=True, constant_weights=True) for w in ws_]
    for a, b in zip(first, outs):
        assert torch.equal(a, b)
    assert torch.equal(first[0], ops.linear_int8(x, ws_[0], 1.0, out_dtype=torch.int32, pair=False))
    assert _capi.device_status() == 0
