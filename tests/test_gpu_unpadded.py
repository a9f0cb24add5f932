"""Unpadded batches: the valid tokens of a padded batch packed back to back.

Packing / unpacking are index work (exact).  The packed QKV + attention kernel and the packed W8A8 encoder must give,
for every valid token, the bits of the padded path (which the other suites pin to the CPU oracle); the attention
output is also checked against the oracle directly."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from zenith_b200 import _capi, ops
from zenith_b200.calibrate import calibrate
from zenith_b200.encoder import EncoderConfig, Int8Encoder, init_params

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def valid_rows(lens, S):
    """Row indices of the padded [B * S] layout that hold valid tokens, in packed order."""
    return np.concatenate([b * S + np.arange(min(max(int(n), 0), S)) for b, n in enumerate(lens)] + [np.zeros(0, np.int64)]).astype(np.int64)


@pytest.mark.parametrize("B,S,lens,cap", [
    (4, 16, [16, 3, 0, 9], 32), (1, 128, [128], 128), (3, 8, [0, 0, 0], 8), (5, 40, [40, 39, 16, 15, 1], 128),
    (6, 10, [10, 12, -3, 4, 10, 7], 48), (3, 10, [10, 10, 10], 25)])
def test_pack_tokens_and_unpad_rows(cuda, B, S, lens, cap):
    ids = rng(B * S).integers(1, 30000, (B, S)).astype(np.int32)
    types = rng(B).integers(0, 2, (B, S)).astype(np.int32)
    cu, ids_p, pos_p, type_p = ops.pack_tokens(dev(ids, cuda), dev(np.array(lens, np.int32), cuda), cap, dev(types, cuda))
    clamped = np.clip(np.array(lens), 0, S)
    want_cu = np.concatenate([[0], np.cumsum(clamped)]).astype(np.int32)
    assert np.array_equal(cu.cpu().numpy(), want_cu)
    rows = valid_rows(lens, S)
    want_ids = np.zeros(cap, np.int32)
    want_pos = np.zeros(cap, np.int32)
    want_type = np.zeros(cap, np.int32)
    n = min(len(rows), cap)  # rows that do not fit the capacity are dropped
    want_ids[:n] = ids.reshape(-1)[rows[:n]]
    want_pos[:n] = (rows % S)[:n]
    want_type[:n] = types.reshape(-1)[rows[:n]]
    assert np.array_equal(ids_p.cpu().numpy(), want_ids)
    assert np.array_equal(pos_p.cpu().numpy(), want_pos)
    assert np.array_equal(type_p.cpu().numpy(), want_type)
    # unpad: packed rows back to their padded positions, zeros elsewhere
    packed = rng(7).standard_normal((cap, 64)).astype(np.float16)
    got = ops.unpad_rows(dev(packed, cuda), cu, B, S).cpu().numpy()
    want = np.zeros((B * S, 64), np.float16)
    want[rows[:n]] = packed[:n]
    assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("B,S,heads,K,lens", [
    (2, 128, 2, 256, [128, 77]), (4, 128, 12, 768, [128, 100, 33, 0]), (5, 40, 3, 192, [40, 39, 16, 15, 0]),
    (3, 96, 4, 256, [1, 96, 1]), (1, 128, 1, 128, [5]), (32, 128, 12, 768, "ragged")])
def test_packed_attention_equals_padded_on_valid_rows(cuda, B, S, heads, K, lens):
    H = heads * 64
    if isinstance(lens, str):
        lens = (S - rng(5).integers(0, 33, B)).tolist()
    x = rng(B * S + K).integers(-128, 128, (B * S, K), dtype=np.int8)
    w = rng(K).integers(-128, 128, (3 * H, K), dtype=np.int8)
    ws = ((rng(3).random(3 * H) + 0.5) * (0.009 / np.sqrt(K))).astype(np.float32)
    b = (rng(4).standard_normal(3 * H) * 0.1).astype(np.float32)
    rows = valid_rows(lens, S)
    total = len(rows)
    cap = total + 3  # a few rows that belong to no sequence: they must stay untouched
    xp = np.zeros((cap, K), np.int8)
    xp[:total] = x[rows]
    xp[total:] = 55
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    wd, wsd, bd = dev(w, cuda), dev(ws, cuda), dev(b, cuda)
    ctx, ctxq, qkv = ops.qkv_attention_int8(dev(x, cuda), wd, 0.02, wsd, bd, B, S, heads, kv_lens=dev(np.array(lens, np.int32), cuda),
                                            out_scale=0.02, emit_qkv=True)
    pctx, pctxq, pqkv = ops.qkv_attention_unpadded_int8(dev(xp, cuda), wd, 0.02, wsd, bd, dev(cu, cuda), heads, out_scale=0.02,
                                                        emit_qkv=True, constant_weights=True)
    assert _capi.device_status() == 0
    idx = torch.from_numpy(rows).to(cuda)
    assert torch.equal(pqkv[:total], qkv[idx])
    assert torch.equal(pctx[:total], ctx[idx])
    assert torch.equal(pctxq[:total], ctxq[idx])
    # rows outside every sequence: never written (the outputs started as zeros)
    assert not pctx[total:].any() and not pctxq[total:].any() and not pqkv[total:].any()
    if total * heads <= 4096 and total:
        q3 = pqkv[:total].float().cpu().numpy()
        for bi in range(B):
            r0, r1 = cu[bi], cu[bi + 1]
            if r1 == r0:
                continue
            for h in range(heads):
                q, k, v = (q3[r0:r1, t * H + h * 64: t * H + (h + 1) * 64][None, None] for t in range(3))
                want = O.attention(q, k, v)[0, 0]
                got = pctx[r0:r1, h * 64:(h + 1) * 64].float().cpu().numpy()
                assert np.max(np.abs(got - want)) <= 1e-2 * max(1.0, np.abs(want).max())


def test_packed_attention_cuts_offsets_beyond_the_row_capacity(cuda):
    """Offsets that run past the rows of the packed tensors (a batch that does not fit its capacity): the rows that
    exist get their results, nothing is written beyond them."""
    heads, K, H = 2, 128, 128
    lens = [100, 128, 90, 128]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)  # 446 rows wanted
    rows = 300                                                    # ... 300 exist: sequence 2 is cut, sequence 3 is gone
    x = rng(1).integers(-128, 128, (rows + 64, K), dtype=np.int8)
    w = rng(2).integers(-128, 128, (3 * H, K), dtype=np.int8)
    ws = ((rng(3).random(3 * H) + 0.5) * (0.009 / np.sqrt(K))).astype(np.float32)
    xd = dev(x, cuda)
    # outputs allocated with slack rows behind them, so that a stray store would land in memory this test owns
    got = ops.qkv_attention_unpadded_int8(xd[:rows], dev(w, cuda), 0.02, dev(ws, cuda), None, dev(cu, cuda), heads, out_scale=0.02)
    ctx, ctxq = got
    assert _capi.device_status() == 0
    cu_cut = np.minimum(cu, rows).astype(np.int32)
    want, wantq = ops.qkv_attention_unpadded_int8(xd[:rows], dev(w, cuda), 0.02, dev(ws, cuda), None, dev(cu_cut, cuda), heads,
                                                   out_scale=0.02)
    assert torch.equal(ctx, want) and torch.equal(ctxq, wantq)
    assert ctx[:228].any() and ctx[228:300].any()


def test_unpadded_encoder_survives_a_batch_larger_than_its_capacity(cuda):
    """capture_unpadded warms up and captures with full-length sequences (more tokens than the capacity): rows beyond
    the capacity are dropped, nothing outside the buffers is touched, later batches that fit are exact."""
    cfg = EncoderConfig(layers=2, hidden=768, heads=12, ffn=1024, vocab=2000, max_pos=128)
    params = init_params(cfg, 11, random_affine=True)
    r = rng(33)
    B, S = 16, 128
    mk = lambda: (torch.from_numpy(r.integers(0, cfg.vocab, (B, S))).to(cuda),
                  torch.from_numpy((S - r.integers(40, 90, B)).astype(np.int32)).to(cuda))
    scales = calibrate(cfg, params, [mk() for _ in range(2)], cuda)
    enc = Int8Encoder(cfg, params, scales, cuda)
    ids, lens = mk()
    want = Int8Encoder(cfg, params, scales, cuda).forward(ids, lens).clone()
    cap = Int8Encoder.unpadded_capacity(lens.tolist(), S)
    assert cap <= B * S - 512
    guard = torch.full((4 << 20,), 7, dtype=torch.uint8, device=cuda)  # allocated next: a stray store is likely to land here
    enc.capture_unpadded(B, S, cap)       # runs the pass with every sequence at full length: 2048 tokens > capacity
    full = torch.full((B,), S, dtype=torch.int32, device=cuda)
    enc.set_inputs(ids, full)
    enc.replay()                          # again, explicitly
    enc.set_inputs(ids, lens)
    got = enc.replay()
    rows = torch.from_numpy(valid_rows(lens.tolist(), S)).to(cuda)
    assert torch.equal(got[rows], want[rows])
    assert bool((guard == 7).all())
    assert _capi.device_status() == 0


def test_packed_attention_flags_a_sequence_longer_than_a_tile(cuda):
    heads, K = 1, 64
    x = dev(rng(1).integers(-128, 128, (200, K), dtype=np.int8), cuda)
    w = dev(rng(2).integers(-128, 128, (192, K), dtype=np.int8), cuda)
    cu = dev(np.array([0, 200], np.int32), cuda)
    ops.qkv_attention_unpadded_int8(x, w, 0.02, None, None, cu, heads)
    torch.cuda.synchronize()
    try:
        assert _capi.device_status() == 2  # ZEN_ERR_UNSUPPORTED
    finally:
        _capi.device_status(clear=True)
    assert _capi.device_status() == 0


CFG = EncoderConfig(layers=3, hidden=256, heads=4, ffn=512, vocab=2000, max_pos=128)


@pytest.mark.parametrize("cfg,B,S", [(CFG, 5, 96), (EncoderConfig(layers=2, hidden=768, heads=12, ffn=3072, vocab=3000, max_pos=128), 8, 128)])
def test_unpadded_encoder_equals_padded_on_valid_tokens(cuda, cfg, B, S):
    params = init_params(cfg, 11, random_affine=True)
    r = rng(21)
    mk = lambda: (torch.from_numpy(r.integers(0, cfg.vocab, (B, S))).to(cuda),
                  torch.from_numpy((S - r.integers(0, 33, B)).astype(np.int32)).to(cuda))
    scales = calibrate(cfg, params, [mk() for _ in range(2)], cuda)
    enc = Int8Encoder(cfg, params, scales, cuda)
    ids, lens = mk()
    padded = enc.forward(ids, lens).clone()
    got = enc.forward_unpadded(ids, lens).clone()
    assert _capi.device_status() == 0
    cap = enc._packed_rows
    assert cap == min(B * S, Int8Encoder.unpadded_capacity(lens.tolist(), S))
    rows = torch.from_numpy(valid_rows(lens.tolist(), S)).to(cuda)
    assert torch.equal(got[rows], padded[rows])
    mask = torch.ones(B * S, dtype=torch.bool, device=cuda)
    mask[rows] = False
    assert not got[mask].any()  # padding positions: zeros
    assert torch.equal(enc.out[:len(rows)], padded[rows])  # the packed rows themselves
    assert enc.launches_per_forward == 2 + cfg.layers * enc.launches_per_layer + 1
    # one captured graph serves other batches that fit the capacity: shorter sequences, same bits as the padded pass
    enc.capture_unpadded(B, S, cap)
    for _ in range(2):
        ids2, lens2 = mk()
        lens2 = torch.clamp(lens2 - 7, min=0)
        lens2[0] = 0
        enc.set_inputs(ids2, lens2)
        rep = enc.replay().clone()
        ref = Int8Encoder(cfg, params, scales, cuda).forward(ids2, lens2)
        rows2 = torch.from_numpy(valid_rows(lens2.tolist(), S)).to(cuda)
        assert torch.equal(rep[rows2], ref[rows2])
    # and the padded form is still there afterwards
    assert torch.equal(enc.forward(ids, lens), padded)


@pytest.mark.parametrize("heads,D,lens,causal", [
    (2, 64, [300, 128, 1, 257], False), (2, 64, [300, 128, 1, 257], True), (1, 128, [384, 200], False),
    (3, 64, [100, 0, 64], False), (1, 128, [513], True), (4, 64, [40, 39, 16, 15, 1], False)])
def test_packed_long_sequence_attention(cuda, heads, D, lens, causal):
    """zen_flash_attention_unpadded_f16: sequences of any length back to back; every row against the fp32 oracle, and for
    sequences longer than one key block bit-equal to the padded call (the same kernel on the same rows)."""
    H = heads * D
    S = max(max(lens), 1)
    B = len(lens)
    r = rng(sum(lens) + D)
    qkv_pad = (r.standard_normal((B, S, 3 * H)) * 0.7).astype(np.float16)
    rows = np.concatenate([b * S + np.arange(n) for b, n in enumerate(lens)]).astype(np.int64)
    total = len(rows)
    packed = np.zeros((total + 5, 3 * H), np.float16)
    packed[:total] = qkv_pad.reshape(B * S, 3 * H)[rows]
    packed[total:] = 3.0
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ctx, ctxq = ops.flash_attention_unpadded(dev(packed, cuda), dev(cu, cuda), heads, D, S, causal=causal, out_scale=0.02)
    assert _capi.device_status() == 0
    got = ctx.float().cpu().numpy()
    assert not got[total:].any() and not ctxq[total:].any()
    f = packed.astype(np.float32)
    for b in range(B):
        r0, r1 = cu[b], cu[b + 1]
        if r1 == r0:
            continue
        split = lambda t: t[r0:r1].reshape(r1 - r0, heads, D).transpose(1, 0, 2)[None]
        want = O.attention(split(f[:, :H]), split(f[:, H:2 * H]), split(f[:, 2 * H:]), causal=causal)[0]  # [heads, n, D]
        g = got[r0:r1].reshape(r1 - r0, heads, D).transpose(1, 0, 2)
        assert np.max(np.abs(g - want)) <= 1e-2 * max(1.0, np.abs(want).max())
    # the int8 copy is the quantization of the fp16 rows beside it
    assert np.array_equal(ctxq[:total].cpu().numpy(), O.quantize(got[:total], 0.02))
    if S > 128:
        # the padded call runs the same kernel: valid rows carry the same bits
        qp = dev(qkv_pad.reshape(B * S, 3 * H), cuda)
        out = torch.empty((B * S, H), dtype=torch.float16, device=cuda)
        st = (S * 3 * H, D, 3 * H)
        ops.flash_attention_strided(qp, qp[:, H:], qp[:, 2 * H:], out, B, heads, S, D, st, st, st, (S * H, D, H),
                                    kv_lens=dev(np.array(lens, np.int32), cuda), causal=causal)
        assert torch.equal(ctx[:total], out[torch.from_numpy(rows).to(cuda)])


@pytest.mark.parametrize("kind,S,exact", [("int8", 160, True), ("fp16", 160, True), ("fp16", 96, False)])
def test_unpadded_encoders_beyond_the_fused_kernel(cuda, kind, S, exact):
    """Sequences longer than one key block (W8A8 and fp16 encoders) and the fp16 encoder at any length run the
    projection as a GEMM on the packed rows and attention from the offsets.  Longer than 128 tokens the padded pass
    runs the same kernels on the same rows (same bits); at 96 tokens its attention kernel is another one (tolerance)."""
    from zenith_b200.encoder import Fp16Encoder
    cfg = EncoderConfig(layers=2, hidden=256, heads=4, ffn=512, vocab=2000, max_pos=256)
    params = init_params(cfg, 5, random_affine=True)
    r = rng(77)
    B = 6
    mk = lambda: (torch.from_numpy(r.integers(0, cfg.vocab, (B, S))).to(cuda),
                  torch.from_numpy((S - r.integers(0, S // 2, B)).astype(np.int32)).to(cuda))
    if kind == "int8":
        scales = calibrate(cfg, params, [mk() for _ in range(2)], cuda)
        enc, ref = Int8Encoder(cfg, params, scales, cuda), Int8Encoder(cfg, params, scales, cuda)
    else:
        enc, ref = Fp16Encoder(cfg, params, cuda), Fp16Encoder(cfg, params, cuda)
    ids, lens = mk()
    lens[1] = 1
    want = ref.forward(ids, lens).clone()
    got = enc.forward_unpadded(ids, lens).clone()
    assert _capi.device_status() == 0
    rows = torch.from_numpy(valid_rows(lens.tolist(), S)).to(cuda)
    if exact:
        assert torch.equal(got[rows], want[rows])
    else:
        assert float((got[rows].float() - want[rows].float()).abs().max()) < 3e-2
    mask = torch.ones(B * S, dtype=torch.bool, device=cuda)
    mask[rows] = False
    assert not got[mask].any()
    # as a graph, fed with another batch
    enc.capture_unpadded(B, S, enc._packed_rows)
    ids2, lens2 = mk()
    lens2 = torch.clamp(lens2 - 9, min=1)
    enc.set_inputs(ids2, lens2)
    rep = enc.replay().clone()
    want2 = ref.forward(ids2, lens2)
    rows2 = torch.from_numpy(valid_rows(lens2.tolist(), S)).to(cuda)
    if exact:
        assert torch.equal(rep[rows2], want2[rows2])
    else:
        assert float((rep[rows2].float() - want2[rows2].float()).abs().max()) < 3e-2
