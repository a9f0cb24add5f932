"""FP8 (e4m3) operands: quantization is bit-exact against the restated format; the GEMM (fp32 accumulation on the tensor
cores, order unspecified) is a tolerance path: 2e-3 of the output's magnitude plus the fp16 rounding of the output."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import ops

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("n,scale,spread", [(1, 1.0, 1.0), (1000, 0.02, 1.0), (4099, 0.5, 300.0), (1 << 20, 0.013, 3.0)])
def test_quantize_e4m3_bit_exact(cuda, n, scale, spread):
    x = (rng(n).standard_normal(n) * spread).astype(np.float32)
    x[: min(n, 8)] = np.array([0, -0.0, 448, 449, -1e9, 2**-9, 3 * 2**-10, 1e-12], np.float32)[: min(n, 8)] * np.float32(scale)
    got = ops.quantize_e4m3(dev(x, cuda), scale).cpu().numpy()
    assert np.array_equal(got, O.quantize_e4m3(x, scale))
    xh = x.astype(np.float16)
    got = ops.quantize_e4m3(dev(xh, cuda), scale).cpu().numpy()
    assert np.array_equal(got, O.quantize_e4m3(xh.astype(np.float32), scale))
    # an unaligned view takes the element-by-element form of the kernel
    if n > 16:
        got = ops.quantize_e4m3(dev(x, cuda)[3:], scale).cpu().numpy()
        assert np.array_equal(got, O.quantize_e4m3(x[3:], scale))


@pytest.mark.parametrize("M,N,K,act,out", [
    (128, 64, 128, "none", torch.float32), (200, 328, 272, "none", torch.float16), (4096, 768, 768, "none", torch.float16),
    (512, 3072, 768, "gelu", torch.float16), (384, 256, 3072, "relu", torch.float32), (1, 64, 16, "none", torch.float32)])
def test_linear_fp8_tracks_oracle(cuda, M, N, K, act, out):
    x = rng(M + K).standard_normal((M, K)).astype(np.float32)
    w = (rng(N + K).standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = (rng(3).standard_normal(N) * 0.1).astype(np.float32)
    x_scale = float(np.abs(x).max() / 448.0)
    w_scale = (np.abs(w).max(axis=1) / 448.0).astype(np.float32)
    xq = O.quantize_e4m3(x, x_scale)
    wq = O.e4m3_encode(w / w_scale[:, None])
    want = O.linear_fp8(xq, wq, x_scale, w_scale, b, act)
    got = ops.linear_fp8(dev(xq, cuda), dev(wq, cuda), x_scale, dev(w_scale, cuda), dev(b, cuda), act=act, out_dtype=out,
                         constant_weights=True).float().cpu().numpy()
    tol = 2e-3 * np.abs(want).max() + (1e-3 * np.abs(want) if out == torch.float16 else 0)
    assert np.all(np.abs(got - want) <= tol)
    # and the quantized product is a fair stand-in for the fp32 one (e4m3 keeps 3 mantissa bits: a few percent)
    if act == "none":
        exact = x @ w.T + b
        assert np.mean(np.abs(want - exact)) < 0.05 * np.mean(np.abs(exact)) + 0.02
    # the tile width does not change a value beyond the same tolerance
    got2 = ops.linear_fp8(dev(xq, cuda), dev(wq, cuda), x_scale, dev(w_scale, cuda), dev(b, cuda), act=act, out_dtype=out,
                          tile_n=64).float().cpu().numpy()
    assert np.all(np.abs(got2 - want) <= tol)
