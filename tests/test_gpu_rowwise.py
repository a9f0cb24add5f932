"""LayerNorm / add+LayerNorm / GELU / quantize kernels against the CPU oracle, through the C ABI."""
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


# shapes of tests/test_layernorm_parallel.py:45-100 plus odd ones (fallback kernel) and the encoder's
SHAPES = [(1, 32), (1, 768), (4, 128), (16, 256), (32, 512), (64, 768), (128, 1024), (7, 100), (5, 4096), (3, 2304),
          (4096, 768)]


@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_layernorm_fp32(cuda, rows, hidden):
    x = rng(rows).standard_normal((rows, hidden)).astype(np.float32)
    r = rng(1).standard_normal((rows, hidden)).astype(np.float32)
    g = (1 + 0.1 * rng(2).standard_normal(hidden)).astype(np.float32)
    b = (0.1 * rng(3).standard_normal(hidden)).astype(np.float32)
    y = ops.layernorm(dev(x, cuda), dev(g, cuda), dev(b, cuda), 1e-5).cpu().numpy()
    np.testing.assert_allclose(y, O.layernorm(x, g, b, 1e-5), rtol=1e-4, atol=1e-5)
    y = ops.add_layernorm(dev(x, cuda), dev(r, cuda), dev(g, cuda), dev(b, cuda), 1e-12).cpu().numpy()
    np.testing.assert_allclose(y, O.add_layernorm(x, r, g, b, 1e-12), rtol=1e-4, atol=1e-5)
    y = ops.layernorm(dev(100 * x, cuda), dev(g, cuda), dev(b, cuda), 1e-5).cpu().numpy()  # scaled inputs
    np.testing.assert_allclose(y, O.layernorm(100 * x, g, b, 1e-5), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("rows,hidden", SHAPES)
def test_layernorm_fp16_with_int8_copy(cuda, rows, hidden):
    x = rng(rows).standard_normal((rows, hidden)).astype(np.float16)
    r = rng(1).standard_normal((rows, hidden)).astype(np.float16)
    g = (1 + 0.1 * rng(2).standard_normal(hidden)).astype(np.float16)
    b = (0.1 * rng(3).standard_normal(hidden)).astype(np.float16)
    f = lambda a: a.astype(np.float32)
    y = ops.layernorm(dev(x, cuda), dev(g, cuda), dev(b, cuda), 1e-5).float().cpu().numpy()
    assert np.max(np.abs(y - O.layernorm(f(x), f(g), f(b), 1e-5))) < 1e-2
    y, yq = ops.add_layernorm(dev(x, cuda), dev(r, cuda), dev(g, cuda), dev(b, cuda), 1e-12, out_scale=0.031)
    assert np.max(np.abs(y.float().cpu().numpy() - O.add_layernorm(f(x), f(r), f(g), f(b), 1e-12))) < 1e-2
    # the int8 copy is exactly the quantization of the fp16 row that was written
    assert np.array_equal(yq.cpu().numpy(), O.quantize(y.float().cpu().numpy(), 0.031))


@pytest.mark.parametrize("n", [1, 7, 4096, 1_000_003])
def test_elementwise_bit_exact(cuda, n):
    x = (3 * rng(n).standard_normal(n)).astype(np.float32)
    xd = dev(x, cuda)
    assert np.array_equal(ops.gelu(xd).cpu().numpy().view(np.int32), O.gelu(x).view(np.int32))
    assert np.array_equal(ops.relu(xd).cpu().numpy(), np.maximum(x, 0))
    assert np.array_equal(ops.quantize(xd, 0.05).cpu().numpy(), O.quantize(x, 0.05))
    assert np.array_equal(ops.quantize(xd, 0.05, 3).cpu().numpy(), O.quantize(x, 0.05, 3))
    assert np.array_equal(ops.quantize(xd, 0.05, round="trunc").cpu().numpy(), O.quantize(x, 0.05, round="trunc"))
    h = x.astype(np.float16)
    assert np.array_equal(ops.gelu(dev(h, cuda)).cpu().numpy(), O.gelu(h.astype(np.float32)).astype(np.float16))
    assert np.array_equal(ops.quantize(dev(h, cuda), 0.05).cpu().numpy(), O.quantize(h.astype(np.float32), 0.05))
    q = rng(1).integers(-128, 128, n, dtype=np.int8)
    assert np.array_equal(ops.dequantize(dev(q, cuda), 0.05, 3).cpu().numpy(), O.dequantize(q, 0.05, 3))
    assert np.array_equal(ops.to_fp16(xd).cpu().numpy(), h)
    assert np.array_equal(ops.to_fp32(dev(h, cuda)).cpu().numpy(), h.astype(np.float32))


@pytest.mark.parametrize("off", [1, 3])
@pytest.mark.parametrize("n", [1, 37, 4099])
def test_elementwise_on_unaligned_views(cuda, n, off):
    """Contiguous views that start off a 16-byte boundary (``t[off:]``) take the element-by-element form of the
    kernel: results are those of the aligned call and nothing outside the output view is written."""
    x = (3 * rng(n + off).standard_normal(n + off)).astype(np.float32)
    h = x.astype(np.float16)
    q = rng(1).integers(-128, 128, n + off, dtype=np.int8)
    xs, hs, qs = x[off:], h[off:], q[off:]
    xd, hd, qd = dev(x, cuda)[off:], dev(h, cuda)[off:], dev(q, cuda)[off:]
    assert np.array_equal(ops.gelu(xd).cpu().numpy().view(np.int32), O.gelu(xs).view(np.int32))
    assert np.array_equal(ops.relu(xd).cpu().numpy(), np.maximum(xs, 0))
    assert np.array_equal(ops.gelu(hd).cpu().numpy(), O.gelu(hs.astype(np.float32)).astype(np.float16))
    assert np.array_equal(ops.quantize(xd, 0.05).cpu().numpy(), O.quantize(xs, 0.05))
    assert np.array_equal(ops.quantize(hd, 0.05, 3).cpu().numpy(), O.quantize(hs.astype(np.float32), 0.05, 3))
    assert np.array_equal(ops.dequantize(qd, 0.05, 3).cpu().numpy(), O.dequantize(qs, 0.05, 3))
    assert np.array_equal(ops.to_fp16(xd).cpu().numpy(), hs)
    assert np.array_equal(ops.to_fp32(hd).cpu().numpy(), hs.astype(np.float32))
    # unaligned OUTPUT through the C ABI: canaries on both sides of the view stay intact
    from zenith_b200 import _capi
    stream = torch.cuda.current_stream().cuda_stream
    for dt, fn, src, want in ((torch.int8, "zen_quantize_f16", hd, O.quantize(hs.astype(np.float32), 0.05)),
                              (torch.float16, "zen_gelu_f16", hd, O.gelu(hs.astype(np.float32)).astype(np.float16))):
        buf = torch.full((n + off + 16,), 77, dtype=dt, device=cuda)
        out = buf[off:off + n]
        args = (src.data_ptr(), out.data_ptr(), n) + ((0.05, 0, 0) if dt == torch.int8 else ()) + (stream,)
        _capi.call(fn, *args)
        got = buf.cpu().numpy()
        assert np.array_equal(got[off:off + n], want)
        assert np.all(got[:off] == 77) and np.all(got[off + n:] == 77)
    assert _capi.device_status() == 0


def test_gelu_meets_reference_tolerance(cuda):
    # benchmarks/bert_encoder.py:264-309: max_diff < 1e-4 against PyTorch
    x = torch.linspace(-8, 8, 100001, device=cuda)
    assert (ops.gelu(x) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max().item() < 1e-5


def test_bias_gelu(cuda):
    x = rng(1).standard_normal((33, 130)).astype(np.float32)
    b = rng(2).standard_normal(130).astype(np.float32)
    assert np.array_equal(ops.bias_gelu(dev(x, cuda), dev(b, cuda)).cpu().numpy(), O.gelu(x + b[None, :]))


def test_embed_layernorm(cuda):
    V, P, H, B, S = 1000, 64, 768, 3, 40
    word, pos, typ = (rng(i).standard_normal(s).astype(np.float16) * 0.5 for i, s in ((1, (V, H)), (2, (P, H)), (3, (2, H))))
    g = (1 + 0.1 * rng(4).standard_normal(H)).astype(np.float16)
    b = (0.1 * rng(5).standard_normal(H)).astype(np.float16)
    ids = rng(6).integers(0, V, B * S).astype(np.int32)
    tids = rng(7).integers(0, 2, B * S).astype(np.int32)
    y, yq = ops.embed_layernorm(dev(ids, cuda), dev(tids, cuda), dev(word, cuda), dev(pos, cuda), dev(typ, cuda),
                                dev(g, cuda), dev(b, cuda), 1e-12, S, out_scale=0.04)
    f = lambda a: a.astype(np.float32)
    e = f(word)[ids] + np.tile(f(pos)[:S], (B, 1)) + f(typ)[tids]
    assert np.max(np.abs(y.float().cpu().numpy() - O.layernorm(e, f(g), f(b), 1e-12))) < 1e-2
    assert np.array_equal(yq.cpu().numpy(), O.quantize(y.float().cpu().numpy(), 0.04))
