"""Parity of the tcgen05 GEMMs with the CPU oracle, through the C ABI.  Integer results are bit-exact;
fp16 / TF32 results are within 1e-2 relative of an fp32 / fp64 computation."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import _capi, ops

pytestmark = pytest.mark.gpu
CFG1 = json.loads((Path(__file__).parent / "golden" / "config1_golden.json").read_text())
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def rng(seed):
    return np.random.default_rng(seed)


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("M,N,K,tile", [
    (128, 64, 128, 64), (128, 128, 256, 128), (128, 192, 128, 192), (128, 256, 512, 256),
    (1, 16, 16, 0), (100, 72, 80, 0), (129, 257, 400, 0), (333, 1000, 1024, 128), (128, 3072, 768, 0),
    (4096, 768, 768, 0)])
def test_int8_accumulators_bit_exact(cuda, M, N, K, tile):
    x = rng(M + N).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(K).integers(-128, 128, (N, K), dtype=np.int8)
    acc = ops.linear_int8(dev(x, cuda), dev(w, cuda), 1.0, out_dtype=torch.int32, tile_n=tile).cpu().numpy()
    want = O.gemm_s8(x, w) if M * N * K <= 4e8 else (dev(x, cuda).double() @ dev(w, cuda).double().T).to(torch.int32).cpu().numpy()
    assert np.array_equal(acc, want)


def test_int8_extreme_operands(cuda):
    """-128 on both sides (it occurs in calibrated weights) and the largest possible accumulator."""
    K = 4096
    x = np.full((130, K), -128, np.int8)
    w = np.full((70, K), -128, np.int8)
    w[1::2] = 127
    acc = ops.linear_int8(dev(x, cuda), dev(w, cuda), 1.0, out_dtype=torch.int32).cpu().numpy()
    assert np.all(acc[:, 0::2] == 128 * 128 * K) and np.all(acc[:, 1::2] == -128 * 127 * K)


@pytest.mark.parametrize("act", ["none", "gelu", "relu"])
@pytest.mark.parametrize("out", ["f32", "f16", "s8"])
def test_int8_fused_epilogue_bit_exact(cuda, act, out):
    M, N, K = 300, 328, 512  # ragged in M and N, N not a multiple of 16
    x = rng(1).integers(-128, 128, (M, K), dtype=np.int8)
    w = rng(2).integers(-128, 128, (N, K), dtype=np.int8)
    ws = ((rng(3).random(N) + 0.5) * 1e-3).astype(np.float32)
    b = (rng(4).standard_normal(N) * 0.1).astype(np.float32)
    tdt = {"f32": torch.float32, "f16": torch.float16, "s8": torch.int8}[out]
    got = ops.linear_int8(dev(x, cuda), dev(w, cuda), 0.02, dev(ws, cuda), dev(b, cuda), act=act, out_dtype=tdt,
                          out_scale=0.05 if out == "s8" else None).cpu().numpy()
    want = O.linear_int8(x, w, 0.02, ws, b, act, out, 0.05)
    assert got.dtype == want.dtype
    assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


def test_prefetch_hint_changes_nothing(cuda):
    """zen_linear_i8_prefetch: odd sizes and unaligned ranges are accepted, the ranges are not modified and the
    result is that of the plain call."""
    M, N, K = 300, 520, 256
    x = dev(rng(1).integers(-128, 128, (M, K), dtype=np.int8), cuda)
    w = dev(rng(2).integers(-128, 128, (N, K), dtype=np.int8), cuda)
    ws = dev((rng(3).random(N) * 1e-3).astype(np.float32), cuda)
    nxt = torch.arange(3_000_001, dtype=torch.int32, device=cuda).to(torch.int8)
    keep = nxt.clone()
    kw = dict(act="gelu", out_dtype=torch.int8, out_scale=0.05)
    plain = ops.linear_int8(x, w, 0.02, ws, None, **kw)
    for hint in ((nxt,), (nxt[1:], nxt[5:77]), (nxt[3:4],)):
        assert torch.equal(ops.linear_int8(x, w, 0.02, ws, None, prefetch=hint, **kw), plain)
    assert torch.equal(nxt, keep)
    with pytest.raises(RuntimeError):
        ops.linear_int8(x, w, 0.02, ws, None, prefetch=(nxt, nxt, nxt), **kw)
    assert _capi.device_status() == 0


def test_constant_weights_promise_changes_nothing(cuda):
    """ZEN_GEMM_CONST_WEIGHTS: with the promise the kernels request weight tiles before their dependency
    wait; results are the same, for one tile per CTA and for several, plain and fused with LayerNorm."""
    for (M, N, K) in [(200, 520, 256), (4096, 3072, 768), (128, 768, 64)]:
        x = dev(rng(1).integers(-128, 128, (M, K), dtype=np.int8), cuda)
        w = dev(rng(2).integers(-128, 128, (N, K), dtype=np.int8), cuda)
        ws = dev((rng(3).random(N) * 1e-3).astype(np.float32), cuda)
        kw = dict(act="gelu", out_dtype=torch.int8, out_scale=0.05)
        res = dev(rng(4).standard_normal((M, 768)).astype(np.float16), cuda)
        g = torch.ones(768, dtype=torch.float16, device=cuda)
        outs = []
        for on in (False, True):
            o = [ops.linear_int8(x, w, 0.02, ws, None, constant_weights=on, **kw),
                 ops.linear_int8(x, w, 0.02, ws, None, out_dtype=torch.float16, constant_weights=on)]
            if N == 768:
                o += list(ops.linear_int8_add_layernorm(x, w, 0.02, ws, None, res, g, g, 1e-5, out_scale=0.03,
                                                        constant_weights=on))
            outs.append(o)
        for a, b in zip(*outs):
            assert torch.equal(a, b)
    assert _capi.device_status() == 0


def test_weights_written_by_the_previous_kernel_in_the_stream(cuda):
    """Without the constant-weights promise every operand is read after the dependency wait: a GEMM whose
    weight matrix is the int8 output of the GEMM launched just before it (same stream, programmatic dependent
    launch in between, no synchronisation) is still bit-exact.  Also after an encoder object exists: building
    one switches nothing process-wide."""
    from zenith_b200.encoder import EncoderConfig, Int8Encoder, Int8Scales, init_params  # noqa: F401
    M, N, K = 512, 768, 256
    a = rng(1).integers(-128, 128, (N, 512), dtype=np.int8)
    b = rng(2).integers(-20, 20, (K, 512), dtype=np.int8)
    x = rng(3).integers(-128, 128, (M, K), dtype=np.int8)
    ad, bd, xd = dev(a, cuda), dev(b, cuda), dev(x, cuda)
    want_w = O.linear_int8(a, b, 1e-3, None, None, "none", "s8", 0.7)  # [N, K] int8
    want = O.gemm_s8(x, want_w)
    for _ in range(20):  # back to back, so the second launch really overlaps the first one's tail
        wq = ops.linear_int8(ad, bd, 1e-3, out_dtype=torch.int8, out_scale=0.7)
        acc = ops.linear_int8(xd, wq, 1.0, out_dtype=torch.int32)
    assert np.array_equal(wq.cpu().numpy(), want_w)
    assert np.array_equal(acc.cpu().numpy(), want)


def test_int8_epilogue_trunc_rounding_and_no_scale_no_bias(cuda):
    x = rng(5).integers(-128, 128, (64, 64), dtype=np.int8)
    w = rng(6).integers(-128, 128, (48, 64), dtype=np.int8)
    got = ops.linear_int8(dev(x, cuda), dev(w, cuda), 0.001, act="none", out_dtype=torch.int8, out_scale=0.37,
                          round="trunc").cpu().numpy()
    assert np.array_equal(got, O.linear_int8(x, w, 0.001, None, None, "none", "s8", 0.37, "trunc"))


def test_config1_on_device_matches_reference_digests(cuda):
    """BASELINE config 1 end to end: quantize X on the device, int8 GEMM, dequant + bias + GELU."""
    M = 1234
    X = rng(M).standard_normal((128, 768)).astype(np.float32)
    W = (rng(M + 100).standard_normal((3072, 768)) * 0.02).astype(np.float32)
    b = (rng(M + 101).standard_normal(3072) * 0.02).astype(np.float32)
    s_w = np.maximum(np.abs(W).max(axis=1) / np.float32(127.5), np.float32(1e-8)).astype(np.float32)
    Wq = np.clip(np.round(W / s_w[:, None]), -128, 127).astype(np.int8)
    assert sha(Wq) == CFG1["Wq_sha256"]
    xq = ops.quantize(dev(X, cuda), CFG1["s_x"])
    assert sha(xq.cpu().numpy()) == CFG1["Xq_sha256"]
    acc = ops.linear_int8(xq, dev(Wq, cuda), 1.0, out_dtype=torch.int32).cpu().numpy()
    assert sha(acc) == CFG1["acc_sha256"]
    y = ops.linear_int8(xq, dev(Wq, cuda), CFG1["s_x"], dev(s_w, cuda), dev(b, cuda), act="gelu").cpu().numpy()
    want = O.linear_int8(xq.cpu().numpy(), Wq, CFG1["s_x"], s_w, b, "gelu", "f32")
    assert np.array_equal(y.view(np.int32), want.view(np.int32))
    fp = O.gelu_libm(X @ W.T + b)  # full-precision Linear+GELU: the quantized result tracks it
    assert np.sqrt(np.mean((y - fp) ** 2)) / np.sqrt(np.mean(fp**2)) < 0.05


def test_int8_linearity_and_checksum_at_encoder_size(cuda):
    """Size-independent properties at the FFN1 shape of the benchmark (4096 x 3072 x 768)."""
    g = torch.Generator(device="cpu").manual_seed(3)
    a = torch.randint(-64, 64, (4096, 768), dtype=torch.int8, generator=g).to(cuda)
    b2 = torch.randint(-64, 64, (4096, 768), dtype=torch.int8, generator=g).to(cuda)
    w = torch.randint(-128, 128, (3072, 768), dtype=torch.int8, generator=g).to(cuda)
    f = lambda t: ops.linear_int8(t, w, 1.0, out_dtype=torch.int32)
    assert torch.equal(f(a) + f(b2), f(a + b2))  # integer GEMM is linear (a + b stays in int8 range)
    colsum = w.double().sum(dim=0)  # [K]; every value below is an integer < 2^53, exact in fp64
    assert torch.equal(f(a).double().sum(dim=1), a.double() @ colsum)


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 320, 520), (100, 72, 80), (4096, 768, 768), (1, 8, 8)])
def test_fp16_linear(cuda, M, N, K):
    x = rng(1).standard_normal((M, K)).astype(np.float16)
    w = (rng(2).standard_normal((N, K)) * 0.1).astype(np.float16)
    b = rng(3).standard_normal(N).astype(np.float32)
    want = (dev(x, cuda).double() @ dev(w, cuda).double().T + dev(b, cuda).double()).cpu().numpy()
    ref_scale = np.abs(want).max()
    y32 = ops.linear_fp16(dev(x, cuda), dev(w, cuda), dev(b, cuda), out_dtype=torch.float32).cpu().numpy()
    assert np.max(np.abs(y32 - want)) / ref_scale < 1e-4
    y16 = ops.linear_fp16(dev(x, cuda), dev(w, cuda), dev(b, cuda), act="gelu").float().cpu().numpy()
    assert np.max(np.abs(y16 - O.gelu(want.astype(np.float32)))) / ref_scale < 1e-2


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 320, 520), (100, 72, 80), (16, 16, 16)])
def test_wmma_matmul_and_fp32_matmul(cuda, M, N, K):
    a = rng(1).standard_normal((M, K)).astype(np.float32)
    b = (rng(2).standard_normal((K, N)) * 0.1).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    c = ops.wmma_matmul(dev(a.astype(np.float16), cuda), dev(b.astype(np.float16), cuda))
    assert c.dtype == torch.float32 and tuple(c.shape) == (M, N)  # cuda_bindings.cpp:110-132: fp32 result
    assert np.max(np.abs(c.cpu().numpy() - want)) / np.abs(want).max() < 1e-2
    c = ops.matmul_f32(dev(a, cuda), dev(b, cuda))
    assert np.max(np.abs(c.cpu().numpy() - want)) / np.abs(want).max() < 1e-2
    y = ops.linear_fp32(dev(a, cuda), dev(np.ascontiguousarray(b.T), cuda))
    assert np.max(np.abs(y.cpu().numpy() - want)) / np.abs(want).max() < 1e-2


def test_no_device_timeout_recorded(cuda):
    assert _capi.device_status() == 0
