"""Encoder drivers on the device against the CPU oracles.

fp16 encoder  : within 1e-2 (relative to the activation scale) of the fp32 oracle encoder.
int8 encoder  : every int8 GEMM of every layer is checked BIT-EXACTLY against the oracle on the int8
                inputs the device really produced (teacher forcing), the int8 copies are the exact
                quantization of the fp16 tensors beside them, and the final hidden states track the
                oracle's int8 encoder and the fp32 encoder.
"""
import numpy as np
import pytest
import torch

from oracle import encoder_ref as ER
from oracle import oracle as O
from zenith_b200 import _capi
from zenith_b200.calibrate import activation_scales_from_ranges, calibrate, quantize_weights
from zenith_b200.encoder import EncoderConfig, Fp16Encoder, Int8Encoder, Int8Scales, init_params

pytestmark = pytest.mark.gpu

CFG = EncoderConfig(layers=3, hidden=256, heads=4, ffn=512, vocab=2000, max_pos=128)


def rng(seed):
    return np.random.default_rng(seed)


def batch(seed, B=3, S=96):
    r = rng(seed)
    ids = r.integers(0, CFG.vocab, (B, S))
    lens = (S - r.integers(0, 33, B)).astype(np.int32)
    return ids, lens


def tdev(ids, lens, cuda):
    return torch.from_numpy(ids).to(cuda), torch.from_numpy(lens).to(cuda)


@pytest.fixture(scope="module")
def params():
    return init_params(CFG, 7, random_affine=True)


def test_fp16_encoder_tracks_fp32_oracle(cuda, params):
    enc = Fp16Encoder(CFG, params, cuda)
    ids, lens = batch(1)
    got = enc.forward(*tdev(ids, lens, cuda)).float().cpu().numpy()
    want = ER.encoder_fp32(CFG, params, ids, lens)
    assert np.max(np.abs(got - want)) < 1e-2 * np.abs(want).max() * 3  # 3 layers of fp16 storage
    assert np.mean(np.abs(got - want)) < 2e-3
    # CUDA-graph replay reproduces the eager pass bit for bit
    eager = enc.out.clone()
    enc.capture(*ids.shape)
    enc.set_inputs(*tdev(ids, lens, cuda))
    assert torch.equal(enc.replay(), eager)


def test_device_calibration_matches_oracle_calibration(cuda, params):
    batches = [batch(100 + i) for i in range(4)]
    dev_scales = calibrate(CFG, params, [tdev(i, l, cuda) for i, l in batches], cuda)
    cpu_scales = ER.calibrate_on_oracle(CFG, params, batches, quantize_weights, activation_scales_from_ranges, Int8Scales)
    for a, b in zip(dev_scales.act, cpu_scales.act):
        for k in a:
            assert abs(a[k] - b[k]) / b[k] < 0.03  # fp16 vs fp32 activations
    for a, b in zip(dev_scales.weights, cpu_scales.weights):
        for k in a:
            assert np.array_equal(a[k][0], b[k][0]) and np.array_equal(a[k][1], b[k][1])


def test_int8_encoder_gemms_bit_exact_and_output_tracks_oracle(cuda, params):
    batches = [batch(100 + i) for i in range(4)]
    scales = ER.calibrate_on_oracle(CFG, params, batches, quantize_weights, activation_scales_from_ranges, Int8Scales)
    enc = Int8Encoder(CFG, params, scales, cuda, fuse_layernorm=False, keep_qkv=True)
    ids, lens = batch(2)
    np_ = lambda t: t.cpu().numpy()
    for li, buf in enc.forward_layerwise(*tdev(ids, lens, cuda)):
        a, wq, lp = scales.act[li], scales.weights[li], params["layers"][li]
        # int8 copies == quantization of the fp16 tensor written beside them
        assert np.array_equal(np_(buf["xq"]), O.quantize(np_(buf["x"].float()), a["x"]))
        assert np.array_equal(np_(buf["ctxq"]), O.quantize(np_(buf["ctx"].float()), a["ctx"]))
        assert np.array_equal(np_(buf["h1q"]), O.quantize(np_(buf["h1"].float()), a["h1"]))
        # each GEMM, on the device's own int8 inputs, bit-exact through its fused epilogue
        want = O.linear_int8(np_(buf["xq"]), wq["wqkv"][0], a["x"], wq["wqkv"][1], lp["bqkv"], "none", "f16")
        assert np.array_equal(np_(buf["qkv"]).view(np.uint16), want.view(np.uint16))
        want = O.linear_int8(np_(buf["ctxq"]), wq["wo"][0], a["ctx"], wq["wo"][1], lp["bo"], "none", "f16")
        assert np.array_equal(np_(buf["ao"]).view(np.uint16), want.view(np.uint16))
        want = O.linear_int8(np_(buf["h1q"]), wq["w1"][0], a["h1"], wq["w1"][1], lp["b1"], "gelu", "s8", a["gelu"])
        assert np.array_equal(np_(buf["gq"]), want)
        want = O.linear_int8(np_(buf["gq"]), wq["w2"][0], a["gelu"], wq["w2"][1], lp["b2"], "none", "f16")
        assert np.array_equal(np_(buf["o"]).view(np.uint16), want.view(np.uint16))
        # float kernels on the device's own inputs, within tolerance
        f16 = lambda k: lp[k].astype(np.float16).astype(np.float32)
        want = O.add_layernorm(np_(buf["ao"].float()), np_(buf["x"].float()), f16("ln1_g"), f16("ln1_b"), CFG.eps)
        assert np.max(np.abs(np_(buf["h1"].float()) - want)) < 1e-2
    got = np_(enc.out.float())
    want8 = ER.encoder_int8(CFG, params, scales, ids, lens).astype(np.float32)
    want32 = ER.encoder_fp32(CFG, params, ids, lens)
    assert np.mean(np.abs(got - want8)) < 5e-3 and np.max(np.abs(got - want8)) < 0.1
    assert np.mean(np.abs(got - want32)) < 3e-2
    # graph replay == eager
    eager = enc.out.clone()
    enc.capture(*ids.shape)
    enc.set_inputs(*tdev(ids, lens, cuda))
    assert torch.equal(enc.replay(), eager)
    # QKV projection and attention as two kernels instead of one: bit-identical
    two = Int8Encoder(CFG, params, scales, cuda, fuse_layernorm=False, fuse_attention=False)
    assert torch.equal(two.forward(*tdev(ids, lens, cuda)), eager)
    assert two.launches_per_layer == 7 and enc.launches_per_layer == 6
    # concurrent micro-batches (sequences are independent): bit-identical, eager and replayed
    for n in (2, 3):
        enc_m = Int8Encoder(CFG, params, scales, cuda, micro_batches=n, fuse_layernorm=False)
        assert torch.equal(enc_m.forward(*tdev(ids, lens, cuda)), eager)
        enc_m.capture(*ids.shape)
        enc_m.set_inputs(*tdev(ids, lens, cuda))
        assert torch.equal(enc_m.replay(), eager)


def test_int8_encoder_with_fused_layernorm_kernels(cuda):
    """hidden 768: attention-output and FFN2 run as GEMM + residual + LayerNorm kernels (5 launches / layer)."""
    cfg = EncoderConfig(layers=2, hidden=768, heads=12, ffn=1024, vocab=2000, max_pos=128)
    params = init_params(cfg, 11, random_affine=True)
    mk = lambda s: (rng(s).integers(0, cfg.vocab, (2, 96)), np.array([96, 70], np.int32))
    scales = ER.calibrate_on_oracle(cfg, params, [mk(s) for s in range(3)], quantize_weights,
                                    activation_scales_from_ranges, Int8Scales)
    ids, lens = mk(50)
    enc = Int8Encoder(cfg, params, scales, cuda)
    assert enc.fuse_layernorm
    np_ = lambda t: t.cpu().numpy()
    for li, buf in enc.forward_layerwise(*tdev(ids, lens, cuda)):
        a, wq, lp = scales.act[li], scales.weights[li], params["layers"][li]
        f16 = lambda k: lp[k].astype(np.float16).astype(np.float32)
        # the fused kernel on the device's own inputs: LayerNorm(dequant(ctx_q . Wo) + bo + x)
        t = O.linear_int8(np_(buf["ctxq"]), wq["wo"][0], a["ctx"], wq["wo"][1], lp["bo"], "none", "f32") + np_(buf["x"].float())
        want = O.layernorm(t, f16("ln1_g"), f16("ln1_b"), cfg.eps)
        assert np.max(np.abs(np_(buf["h1"].float()) - want)) < 1e-2
        assert np.array_equal(np_(buf["h1q"]), O.quantize(np_(buf["h1"].float()), a["h1"]))
        want = O.linear_int8(np_(buf["h1q"]), wq["w1"][0], a["h1"], wq["w1"][1], lp["b1"], "gelu", "s8", a["gelu"])
        assert np.array_equal(np_(buf["gq"]), want)
        t = O.linear_int8(np_(buf["gq"]), wq["w2"][0], a["gelu"], wq["w2"][1], lp["b2"], "none", "f32") + np_(buf["h1"].float())
        want = O.layernorm(t, f16("ln2_g"), f16("ln2_b"), cfg.eps)
        assert np.max(np.abs(np_(buf["x_next"].float()) - want)) < 1e-2
    got = np_(enc.out.float())
    want8 = ER.encoder_int8(cfg, params, scales, ids, lens, fused_layernorm=True).astype(np.float32)
    assert np.mean(np.abs(got - want8)) < 5e-3 and np.max(np.abs(got - want8)) < 0.1
    assert enc.launches_per_layer == 4  # QKV + attention, attention-out + LN, FFN1, FFN2 + LN
    unfused = Int8Encoder(cfg, params, scales, cuda, fuse_layernorm=False).forward(*tdev(ids, lens, cuda)).float()
    assert (unfused - enc.out.float()).abs().mean().item() < 5e-3
    two = Int8Encoder(cfg, params, scales, cuda, fuse_attention=False)
    assert torch.equal(two.forward(*tdev(ids, lens, cuda)), enc.out) and two.launches_per_layer == 5
    eager = enc.out.clone()
    enc.capture(*ids.shape)
    enc.set_inputs(*tdev(ids, lens, cuda))
    assert torch.equal(enc.replay(), eager)


def test_host_pipeline_returns_every_batch(cuda):
    """HostPipeline: different batches streamed back to back from pinned host memory come back, in host
    memory, equal to what a plain forward pass gives for each of them."""
    from zenith_b200.serve import HostPipeline

    cfg = EncoderConfig(layers=2, hidden=768, heads=12, ffn=1024, vocab=2000, max_pos=128)
    params = init_params(cfg, 11, random_affine=True)
    mk = lambda s: (rng(s).integers(0, cfg.vocab, (4, 64)), rng(s + 100).integers(1, 65, 4).astype(np.int32))
    scales = ER.calibrate_on_oracle(cfg, params, [mk(s) for s in range(2)], quantize_weights,
                                    activation_scales_from_ranges, Int8Scales)
    enc = Int8Encoder(cfg, params, scales, cuda)
    batches = [mk(20 + i) for i in range(5)]
    want = [enc.forward(*tdev(i, l, cuda)).cpu().clone() for i, l in batches]
    pipe = HostPipeline(enc, 4, 64)
    host = [(torch.from_numpy(i).pin_memory(), torch.from_numpy(l).pin_memory()) for i, l in batches]
    got, prev = [], None
    for ids_h, lens_h in host:
        t = pipe.submit(ids_h, lens_h)
        if prev is not None:
            got.append(pipe.result(prev).clone())
        prev = t
    got.append(pipe.result(prev).clone())
    pipe.drain()
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    with pytest.raises(ValueError):
        pipe.result(0)  # its slot has been reused
    assert _capi.device_status() == 0


@pytest.mark.parametrize("micro_batches", [1, 2])
def test_capture_slots_have_their_own_inputs_and_results(cuda, micro_batches):
    """capture(..., slots=2): two graphs of the same pass, each with its own input block and result buffer; a slot's
    replay leaves the other slot's result alone and gives the bits of a plain forward pass."""
    cfg = EncoderConfig(layers=2, hidden=768, heads=12, ffn=1024, vocab=2000, max_pos=128)
    params = init_params(cfg, 11, random_affine=True)
    mk = lambda s: (rng(s).integers(0, cfg.vocab, (4, 64)), rng(s + 100).integers(1, 65, 4).astype(np.int32))
    scales = ER.calibrate_on_oracle(cfg, params, [mk(s) for s in range(2)], quantize_weights,
                                    activation_scales_from_ranges, Int8Scales)
    enc = Int8Encoder(cfg, params, scales, cuda, micro_batches=micro_batches)
    (ia, la), (ib, lb) = mk(31), mk(32)
    want_a = enc.forward(*tdev(ia, la, cuda)).clone()
    want_b = enc.forward(*tdev(ib, lb, cuda)).clone()
    enc.capture(4, 64, slots=2)
    pack = lambda i, l: torch.from_numpy(np.concatenate([i.reshape(-1), l]).astype(np.int32)).to(cuda)
    enc.inputs_of(0).copy_(pack(ia, la))
    enc.inputs_of(1).copy_(pack(ib, lb))
    ra = enc.replay(0)
    rb = enc.replay(1)
    assert ra.data_ptr() != rb.data_ptr() and ra.data_ptr() == enc.result_of(0).data_ptr()
    assert torch.equal(ra, want_a) and torch.equal(rb, want_b)
    enc.inputs_of(0).copy_(pack(ib, lb))
    assert torch.equal(enc.replay(0), want_b) and torch.equal(enc.result_of(1), want_b)
    if micro_batches != 1:
        return  # the unpadded form runs as one micro-batch
    # the unpadded form takes slots the same way
    cap = Int8Encoder.unpadded_capacity(la.tolist(), 64)
    enc.capture_unpadded(4, 64, max(cap, Int8Encoder.unpadded_capacity(lb.tolist(), 64)), slots=2)
    enc.inputs_of(1).copy_(pack(ia, la))
    got = enc.replay(1)
    rows = torch.from_numpy(np.concatenate([b * 64 + np.arange(int(n)) for b, n in enumerate(la)])).to(cuda)
    assert torch.equal(got[rows], want_a[rows])
    assert _capi.device_status() == 0


def test_fp16_encoder_with_fused_layernorm_kernels(cuda):
    """hidden 768: the fp16 encoder runs attention-output and FFN2 as GEMM + residual + LayerNorm kernels."""
    cfg = EncoderConfig(layers=2, hidden=768, heads=12, ffn=1024, vocab=2000, max_pos=128)
    params = init_params(cfg, 11, random_affine=True)
    ids = rng(50).integers(0, cfg.vocab, (2, 96))
    lens = np.array([96, 70], np.int32)
    enc = Fp16Encoder(cfg, params, cuda)
    assert enc.fuse_layernorm and enc.launches_per_layer == 5
    got = enc.forward(*tdev(ids, lens, cuda)).float().cpu().numpy()
    want = ER.encoder_fp32(cfg, params, ids, lens)
    assert np.max(np.abs(got - want)) < 3e-2 and np.mean(np.abs(got - want)) < 2e-3
    unfused = Fp16Encoder(cfg, params, cuda, fuse_layernorm=False).forward(*tdev(ids, lens, cuda)).float().cpu().numpy()
    assert np.mean(np.abs(unfused - got)) < 2e-3
    eager = enc.out.clone()
    enc.capture(*ids.shape)
    enc.set_inputs(*tdev(ids, lens, cuda))
    assert torch.equal(enc.replay(), eager)
    taps = enc.forward_with_taps(*tdev(ids, lens, cuda))
    assert len(taps["h1"]) == cfg.layers and all(lo < hi for lo, hi in taps["h1"])
