"""W8A8 Linear + residual + LayerNorm in one cluster kernel, against the CPU oracle."""
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


@pytest.mark.parametrize("M,K,N", [(128, 768, 768), (300, 768, 768), (4096, 768, 768), (1000, 3072, 768),
                                   (4096, 3072, 768), (1, 128, 768), (700, 1024, 1024), (512, 4096, 1024)])
def test_linear_add_layernorm(cuda, M, K, N):
    x = rng(M).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(K).integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng(1).random(N) + 0.5) * 2e-4).astype(np.float32)
    b = (rng(2).standard_normal(N) * 0.1).astype(np.float32)
    res = rng(3).standard_normal((M, N)).astype(np.float16)
    g = (1 + 0.1 * rng(4).standard_normal(N)).astype(np.float16)
    be = (0.1 * rng(5).standard_normal(N)).astype(np.float16)
    y, yq = ops.linear_int8_add_layernorm(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), dev(res, cuda),
                                          dev(g, cuda), dev(be, cuda), 1e-12, out_scale=0.03)
    t = O.linear_int8(x, w, 0.02, ws, b, "none", "f32") + res.astype(np.float32)
    want = O.layernorm(t, g.astype(np.float32), be.astype(np.float32), 1e-12)
    got = y.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert np.max(np.abs(got - want)) < 1e-2 and np.mean(np.abs(got - want)) < 5e-4
    # the int8 copy is exactly the quantization of the fp16 tensor written beside it
    assert np.array_equal(yq.cpu().numpy(), O.quantize(got, 0.03))
    # without the int8 copy
    y2 = ops.linear_int8_add_layernorm(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), dev(res, cuda),
                                       dev(g, cuda), dev(be, cuda), 1e-12)
    assert torch.equal(y2, y)
    assert _capi.device_status() == 0


def test_statistics_are_robust_to_a_large_mean(cuda):
    """Rows whose mean is far larger than their spread: the pairwise-combined variance must not cancel."""
    M, K, N = 256, 128, 768
    x = rng(1).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(2).integers(-128, 128, (N, K), dtype=np.int8)
    res = (100 + rng(3).standard_normal((M, N))).astype(np.float16)
    g = np.ones(N, np.float16)
    be = np.zeros(N, np.float16)
    y = ops.linear_int8_add_layernorm(dev(x, cuda), dev(w, cuda), 1e-4, None, None, dev(res, cuda), dev(g, cuda),
                                      dev(be, cuda), 1e-5)
    t = O.linear_int8(x, w, 1e-4, None, None, "none", "f32") + res.astype(np.float32)
    want = O.layernorm(t, g.astype(np.float32), be.astype(np.float32), 1e-5)
    assert np.max(np.abs(y.float().cpu().numpy() - want)) < 2e-2


def test_unsupported_width_is_refused(cuda):
    x = torch.zeros((16, 64), dtype=torch.int8, device=cuda)
    w = torch.zeros((512, 64), dtype=torch.int8, device=cuda)
    r = torch.zeros((16, 512), dtype=torch.float16, device=cuda)
    g = torch.ones(512, dtype=torch.float16, device=cuda)
    with pytest.raises(_capi.ZenithError) as e:
        ops.linear_int8_add_layernorm(x, w, 1.0, None, None, r, g, g, 1e-5)
    assert e.value.status == _capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("M,K,N", [(128, 768, 768), (300, 256, 768), (4096, 3072, 768), (1, 8, 768), (700, 1024, 1024)])
def test_fp16_linear_add_layernorm(cuda, M, K, N):
    """The fp16-operand form of the cluster kernel against an fp32 computation of the same thing."""
    x = (rng(M).standard_normal((M, K)) * 0.5).astype(np.float16)
    w = (rng(K).standard_normal((N, K)) * 0.05).astype(np.float16)
    b = (rng(2).standard_normal(N) * 0.1).astype(np.float32)
    res = rng(3).standard_normal((M, N)).astype(np.float16)
    g = (1 + 0.1 * rng(4).standard_normal(N)).astype(np.float16)
    be = (0.1 * rng(5).standard_normal(N)).astype(np.float16)
    y, yq = ops.linear_fp16_add_layernorm(dev(x, cuda), dev(w, cuda), dev(b, cuda), dev(res, cuda), dev(g, cuda),
                                          dev(be, cuda), 1e-12, out_scale=0.03)
    t = x.astype(np.float32) @ w.astype(np.float32).T + b + res.astype(np.float32)
    want = O.layernorm(t, g.astype(np.float32), be.astype(np.float32), 1e-12)
    got = y.float().cpu().numpy()
    assert not np.isnan(got).any()
    assert np.max(np.abs(got - want)) < 1e-2 and np.mean(np.abs(got - want)) < 5e-4
    assert np.array_equal(yq.cpu().numpy(), O.quantize(got, 0.03))
    assert torch.equal(ops.linear_fp16_add_layernorm(dev(x, cuda), dev(w, cuda), dev(b, cuda), dev(res, cuda), dev(g, cuda),
                                                     dev(be, cuda), 1e-12), y)
    assert _capi.device_status() == 0
