"""Pins the CPU oracle: against the reference-generated digests for config 1, against the reference's
known-answer values, against the reference's own compiled CPU GEMM (oracle/_ref) and against
independent numpy / torch formulations."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import encoder_ref as ER
from oracle import oracle as O

CFG1 = json.loads((Path(__file__).parent / "golden" / "config1_golden.json").read_text())
sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def rng(seed):
    return np.random.default_rng(seed)


def test_config1_integer_path_matches_reference_digests():
    """X -> Xq -> int32 accumulators of config 1, scales taken from the reference run."""
    M = 1234
    X = rng(M).standard_normal((128, 768)).astype(np.float32)
    W = (rng(M + 100).standard_normal((3072, 768)) * 0.02).astype(np.float32)
    absmax = np.abs(W).max(axis=1)
    s_w = np.maximum(absmax / np.float32(127.5), np.float32(1e-8)).astype(np.float32)
    assert sha(s_w) == CFG1["s_w_sha256"]
    Xq = O.quantize(X, CFG1["s_x"])
    assert sha(Xq) == CFG1["Xq_sha256"]
    Wq = np.stack([O.quantize(W[n], s_w[n]) for n in range(0, 3072)])
    assert sha(Wq) == CFG1["Wq_sha256"] and int((Wq == -128).sum()) == CFG1["Wq_minus128"]
    acc = O.gemm_s8(Xq, Wq)
    assert sha(acc) == CFG1["acc_sha256"] and int(acc.astype(np.int64).sum()) == CFG1["acc_sum"]


def test_int_gemm_and_epilogue_against_numpy():
    x = rng(0).integers(-128, 128, (37, 80), dtype=np.int8)
    w = rng(1).integers(-128, 128, (50, 80), dtype=np.int8)
    acc = O.gemm_s8(x, w)
    assert np.array_equal(acc, x.astype(np.int32) @ w.astype(np.int32).T)  # benchmarks/int8_bench.py:42-45
    ws = (rng(2).random(50).astype(np.float32) + 0.5) * 1e-3
    b = rng(3).standard_normal(50).astype(np.float32)
    y = O.epilogue(acc, 0.02, ws, b)
    want = (acc.astype(np.float32) * np.float32(0.02)) * ws[None, :] + b[None, :]  # cuda_kernels.cu:1035-1036
    assert np.array_equal(y.view(np.int32), want.astype(np.float32).view(np.int32))
    # extremes: -128 * -128 * K must not overflow or saturate
    big = O.gemm_s8(np.full((1, 4096), -128, np.int8), np.full((1, 4096), -128, np.int8))
    assert big[0, 0] == 128 * 128 * 4096


def test_quantize_rounding_modes_and_saturation():
    x = np.array([0.25, 0.35, -0.25, 0.15, 1e9, -1e9, 12.7, -12.85, np.nan], np.float32)
    q = O.quantize(x, 0.1)
    assert q.tolist() == [2, 4, -2, 2, 127, -128, 127, -128, -128]  # nearest-even; NaN -> -128
    assert O.quantize(np.array([0.26, 0.19, -0.26], np.float32), 0.1, round="trunc").tolist() == [2, 1, -2]
    xs = (rng(5).standard_normal(20000) * 3).astype(np.float32)
    assert np.array_equal(O.quantize(xs, 0.05), np.clip(np.round(xs / np.float32(0.05)), -128, 127).astype(np.int8))
    assert np.array_equal(O.dequantize(O.quantize(xs, 0.05), 0.05, 0), O.quantize(xs, 0.05).astype(np.float32) * np.float32(0.05))


def test_gelu_known_answers_and_distance_from_libm():
    # tests/test_cuda_cublas_bindings.py:36-56
    g = O.gelu(np.array([1.0, 0.0, -1.0], np.float32))
    assert abs(g[0] - 0.841) < 0.01 and g[1] == 0.0 and abs(g[2] + 0.159) < 0.01
    x = np.linspace(-12, 12, 2_000_001).astype(np.float32)
    det, libm = O.gelu(x), O.gelu_libm(x)
    x64 = x.astype(np.float64)
    exact = 0.5 * x64 * (1 + np.tanh(0.7978845608028654 * (x64 + 0.044715 * x64**3)))
    assert np.max(np.abs(det - exact)) < 1e-6  # the deterministic form is as close to the formula as libm's
    assert np.max(np.abs(det - libm)) < 2e-6
    # tests/python/test_fx_patterns.py:189-203
    t = torch.nn.functional.gelu(torch.from_numpy(x), approximate="tanh").numpy()
    assert np.max(np.abs(det - t)) < 1e-5
    assert np.isnan(O.gelu(np.array([np.nan], np.float32))[0])
    tails = O.gelu(np.array([-1e4, 1e4, -0.0], np.float32))
    assert abs(tails[0]) < 1e-30 and tails[1] == 1e4 and tails[2] == 0.0  # exp is clamped at 2^126


@pytest.mark.parametrize("rows,hidden", [(1, 32), (4, 128), (16, 768), (64, 1024), (7, 100)])
def test_layernorm_against_numpy(rows, hidden):  # tests/test_layernorm_parallel.py:45-100
    x = rng(rows).standard_normal((rows, hidden)).astype(np.float32)
    g = rng(1).standard_normal(hidden).astype(np.float32)
    b = rng(2).standard_normal(hidden).astype(np.float32)
    want = (x - x.mean(1, keepdims=True)) / np.sqrt(x.var(1, keepdims=True) + 1e-5) * g + b
    np.testing.assert_allclose(O.layernorm(x, g, b, 1e-5), want, rtol=1e-4, atol=1e-5)
    r = rng(3).standard_normal((rows, hidden)).astype(np.float32)
    v = x + r
    want = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-12) * g + b
    np.testing.assert_allclose(O.add_layernorm(x, r, g, b, 1e-12), want, rtol=1e-4, atol=1e-5)


def test_attention_against_torch_sdpa():
    q, k, v = (rng(i).standard_normal((2, 3, 40, 64)).astype(np.float32) for i in (1, 2, 3))
    tq, tk, tv = map(torch.from_numpy, (q, k, v))
    sdpa = torch.nn.functional.scaled_dot_product_attention
    assert np.max(np.abs(O.attention(q, k, v) - sdpa(tq, tk, tv).numpy())) < 1e-4  # flash_attention_benchmark.py:129-153
    assert np.max(np.abs(O.attention(q, k, v, causal=True) - sdpa(tq, tk, tv, is_causal=True).numpy())) < 1e-4
    lens = np.array([40, 9], np.int32)
    m = torch.arange(40)[None, None, None, :] < torch.tensor(lens.tolist())[:, None, None, None]
    assert np.max(np.abs(O.attention(q, k, v, lens) - sdpa(tq, tk, tv, attn_mask=m).numpy())) < 1e-4
    # a row with no valid key yields zeros (zenith/jax/primitives.py:302-310)
    assert np.all(O.attention(q, k, v, np.array([0, 5], np.int32))[0] == 0)
    assert np.max(np.abs(ER.attention_numpy(q, k, v, lens) - O.attention(q, k, v, lens))) < 1e-5


def test_reference_cpu_gemm_agrees_with_oracle():
    """oracle/_ref is the reference's own core/src/cpu_kernels.cpp compiled as it stands."""
    if O.ref_lib() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    a = rng(1).standard_normal((33, 70)).astype(np.float32)
    w = rng(2).standard_normal((41, 70)).astype(np.float32)
    got = O.ref_matmul_avx2(a, np.ascontiguousarray(w.T))
    np.testing.assert_allclose(got, O.gemm_f32_nt(a, w), rtol=1e-4, atol=1e-4)


def test_int8_encoder_oracle_tracks_fp32_encoder():
    from zenith_b200.calibrate import activation_scales_from_ranges, quantize_weights
    from zenith_b200.encoder import EncoderConfig, Int8Scales, init_params

    cfg = EncoderConfig(layers=2, hidden=128, heads=2, ffn=256, vocab=500, max_pos=32)
    params = init_params(cfg, 7, random_affine=True)
    mk = lambda s: (rng(s).integers(0, cfg.vocab, (2, 32)), np.array([32, 20], np.int32))
    scales = ER.calibrate_on_oracle(cfg, params, [mk(s) for s in range(4)], quantize_weights,
                                    activation_scales_from_ranges, Int8Scales)
    ids, lens = mk(99)
    ref = ER.encoder_fp32(cfg, params, ids, lens)
    q8 = ER.encoder_int8(cfg, params, scales, ids, lens).astype(np.float32)
    fq = ER.encoder_fake_quant(cfg, params, scales, ids, lens)
    assert np.max(np.abs(q8 - ref)) < 0.15 and np.mean(np.abs(q8 - ref)) < 0.02
    assert np.max(np.abs(fq - ref)) < 0.15


def test_attention_rows_is_a_row_subset_of_attention():
    r = np.random.default_rng(0)
    q, k, v = (r.standard_normal((2, 2, 70, 16)).astype(np.float32) for _ in range(3))
    rows = np.array([0, 3, 69, 17])
    for causal in (False, True):
        full = O.attention(q, k, v, [70, 33], causal)
        assert np.array_equal(full[:, :, rows], O.attention_rows(q, k, v, rows, [70, 33], causal))


def test_oracle_reproduces_the_reference_benchmark_pipeline_on_config1():
    """benchmarks/int8_bench.py:19-25, 42-45 run on the config-1 tensors (digests stored by make_golden.py): per-tensor
    symmetric quantization of X and W, int32 product, dequantised with the two scales."""
    cfg1 = json.loads((Path(__file__).parent / "golden" / "config1_golden.json").read_text())
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    M = 1234
    X = np.random.default_rng(M).standard_normal((128, 768)).astype(np.float32)
    W = (np.random.default_rng(M + 100).standard_normal((3072, 768)) * 0.02).astype(np.float32)
    sx, sw = np.float32(cfg1["bench_sx"]), np.float32(cfg1["bench_sw"])
    assert sx == np.abs(X).max() / np.float32(127.0) and sw == np.abs(W).max() / np.float32(127.0)
    qx, qw = O.quantize(X, sx), O.quantize(W, sw)
    assert sha(qx) == cfg1["bench_qx_sha256"] and sha(qw) == cfg1["bench_qw_sha256"]
    y = O.epilogue(O.gemm_s8(qx, qw), sx, np.full(3072, sw, np.float32), None, "none")
    assert sha(y) == cfg1["bench_y_sha256"]


def test_e4m3_restatement_matches_an_independent_conversion():
    """The oracle's e4m3 encode / decode against torch's float8_e4m3fn conversion on the CPU: all 256 codes, and
    a million values across the format's range (ties, subnormals, saturation)."""
    import torch
    bits = np.arange(256, dtype=np.uint8)
    t = torch.from_numpy(bits).view(torch.float8_e4m3fn).float().numpy()
    d = O.e4m3_decode(bits)
    assert np.array_equal(np.isnan(t), np.isnan(d)) and np.array_equal(t[~np.isnan(t)], d[~np.isnan(d)])
    r = np.random.default_rng(0)
    x = np.concatenate([r.standard_normal(200000).astype(np.float32) * np.float32(s) for s in (1e-3, 0.05, 1, 30, 300)] +
                       [np.array([0, -0.0, 448, 449, 464, 465, 480, 1e9, -1e9, 2**-9, 2**-10, 1.5 * 2**-9, 3 * 2**-10], np.float32)])
    want = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x), want)
    # decode(encode(v)) == v for every finite code
    finite = ~np.isnan(d)
    assert np.array_equal(O.e4m3_encode(d[finite]), bits[finite])
