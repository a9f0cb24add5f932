"""Encoder-level CPU oracles — TEST INFRASTRUCTURE, NOT PRODUCT.

``encoder_fp32``  : the FP32 path of a BERT-style post-LN encoder built from the oracle's ops, the
                    way the reference's drivers chain them (benchmarks/bert_hybrid.py:96-145:
                    linear x3 -> attention -> linear -> add+LayerNorm -> linear -> GELU -> linear ->
                    add+LayerNorm).  Also the CPU baseline of the benchmark ("numpy quantized
                    executor" uses ``encoder_fake_quant``).
``encoder_int8``  : the pinned W8A8 dataflow with the same fp16 rounding points as the device path.
                    The reference has no int8 encoder; this restatement is its definition here
                    (parity unpinned in the reference).
``encoder_fake_quant``: the reference's own CPU way of running a quantized Linear — fake-quantize
                    weight and activation, fp32 matmul (zenith/optimization/qat.py:751-776) — looped
                    over the encoder.  This is what ``bench.py --impl reference`` times.
"""
from __future__ import annotations

import numpy as np

from . import oracle as O

ACT_POINTS = ("x", "ctx", "h1", "gelu")


def _split_heads(t, B, S, nh, hd):
    return np.ascontiguousarray(t.reshape(B, S, nh, hd).transpose(0, 2, 1, 3))


def _merge_heads(t, B, S, nh, hd):
    return np.ascontiguousarray(t.transpose(0, 2, 1, 3)).reshape(B * S, nh * hd)


def embed(cfg, params, ids, dtype=np.float32):
    B, S = ids.shape
    word, pos, typ = (params[k].astype(dtype).astype(np.float32) for k in ("word", "pos", "type"))
    e = word[ids.reshape(-1)] + np.tile(pos[:S], (B, 1)) + typ[0][None, :]
    g = params["emb_ln_g"].astype(dtype).astype(np.float32)
    b = params["emb_ln_b"].astype(dtype).astype(np.float32)
    return O.layernorm(e, g, b, cfg.eps)


def encoder_fp32(cfg, params, ids, kv_lens=None, taps=None):
    """fp32 hidden states [B*S, H].  ``taps`` (dict) receives per-layer (min, max) at the four GEMM inputs."""
    B, S = ids.shape
    nh, hd = cfg.heads, cfg.head_dim
    x = embed(cfg, params, ids)
    for lp in params["layers"]:
        qkv = x @ lp["wqkv"].T + lp["bqkv"]
        q, k, v = (_split_heads(qkv[:, i * cfg.hidden:(i + 1) * cfg.hidden], B, S, nh, hd) for i in range(3))
        ctx = _merge_heads(O.attention(q, k, v, kv_lens), B, S, nh, hd)
        ao = ctx @ lp["wo"].T + lp["bo"]
        h1 = O.add_layernorm(ao, x, lp["ln1_g"], lp["ln1_b"], cfg.eps)
        g = O.gelu(h1 @ lp["w1"].T + lp["b1"])
        o = g @ lp["w2"].T + lp["b2"]
        if taps is not None:
            for name, t in (("x", x), ("ctx", ctx), ("h1", h1), ("gelu", g)):
                taps.setdefault(name, []).append((float(t.min()), float(t.max())))
        x = O.add_layernorm(o, h1, lp["ln2_g"], lp["ln2_b"], cfg.eps)
    return x


def _f16(a):
    return a.astype(np.float16).astype(np.float32)


def encoder_int8(cfg, params, scales, ids, kv_lens=None, trace=None, fused_layernorm=False):
    """Pinned W8A8 dataflow; returns fp16 hidden states [B*S, H].  ``trace`` (list) receives a dict of
    every intermediate per layer.  ``fused_layernorm``: the attention-output and FFN2 projections feed the
    residual add in fp32 (no fp16 rounding in between), as the fused GEMM + LayerNorm kernel does."""
    proj = "f32" if fused_layernorm else "f16"
    B, S = ids.shape
    nh, hd, H = cfg.heads, cfg.head_dim, cfg.hidden
    x = _f16(embed(cfg, params, ids, np.float16))
    xq = O.quantize(x, scales.act[0]["x"])
    n_layers = len(params["layers"])
    for li, (lp, wq) in enumerate(zip(params["layers"], scales.weights)):
        a = scales.act[li]
        ln = {k: _f16(lp[k]) for k in ("ln1_g", "ln1_b", "ln2_g", "ln2_b")}
        qkv = O.linear_int8(xq, wq["wqkv"][0], a["x"], wq["wqkv"][1], lp["bqkv"], "none", "f16").astype(np.float32)
        q, k, v = (_split_heads(qkv[:, i * H:(i + 1) * H], B, S, nh, hd) for i in range(3))
        ctx = _f16(_merge_heads(O.attention(q, k, v, kv_lens), B, S, nh, hd))
        ctxq = O.quantize(ctx, a["ctx"])
        ao = O.linear_int8(ctxq, wq["wo"][0], a["ctx"], wq["wo"][1], lp["bo"], "none", proj).astype(np.float32)
        h1 = _f16(O.add_layernorm(ao, x, ln["ln1_g"], ln["ln1_b"], cfg.eps))
        h1q = O.quantize(h1, a["h1"])
        gq = O.linear_int8(h1q, wq["w1"][0], a["h1"], wq["w1"][1], lp["b1"], "gelu", "s8", a["gelu"])
        o = O.linear_int8(gq, wq["w2"][0], a["gelu"], wq["w2"][1], lp["b2"], "none", proj).astype(np.float32)
        x_next = _f16(O.add_layernorm(o, h1, ln["ln2_g"], ln["ln2_b"], cfg.eps))
        xq_next = O.quantize(x_next, scales.act[li + 1]["x"]) if li + 1 < n_layers else None
        if trace is not None:
            trace.append(dict(x=x, xq=xq, qkv=qkv, ctx=ctx, ctxq=ctxq, ao=ao, h1=h1, h1q=h1q, gq=gq, o=o,
                              x_next=x_next, xq_next=xq_next))
        x, xq = x_next, xq_next
    return x.astype(np.float16)


def _fake_quant(x, scale, qmin=-128, qmax=127):
    # zenith/optimization/qat.py:267-268
    return (np.clip(np.round(x / scale), qmin, qmax) * scale).astype(np.float32)


def encoder_fake_quant(cfg, params, scales, ids, kv_lens=None):
    """The reference's CPU quantized executor, looped over the encoder: every Linear is
    ``fake_quant(x) @ fake_quant(W).T + b`` in fp32 (numpy BLAS), per-channel weight scales,
    per-tensor activation scales."""
    B, S = ids.shape
    nh, hd, H = cfg.heads, cfg.head_dim, cfg.hidden
    fqw = [{k: (v[0].astype(np.float32) * v[1][:, None]) for k, v in wq.items()} for wq in scales.weights]
    x = embed(cfg, params, ids)
    for li, lp in enumerate(params["layers"]):
        a, w = scales.act[li], fqw[li]
        qkv = _fake_quant(x, a["x"]) @ w["wqkv"].T + lp["bqkv"]
        q, k, v = (_split_heads(qkv[:, i * H:(i + 1) * H], B, S, nh, hd) for i in range(3))
        ctx = _merge_heads(attention_numpy(q, k, v, kv_lens), B, S, nh, hd)
        ao = _fake_quant(ctx, a["ctx"]) @ w["wo"].T + lp["bo"]
        h1 = layernorm_numpy(ao + x, lp["ln1_g"], lp["ln1_b"], cfg.eps)
        g = gelu_numpy(_fake_quant(h1, a["h1"]) @ w["w1"].T + lp["b1"])
        o = _fake_quant(g, a["gelu"]) @ w["w2"].T + lp["b2"]
        x = layernorm_numpy(o + h1, lp["ln2_g"], lp["ln2_b"], cfg.eps)
    return x


def gelu_numpy(x):
    # zenith/execution/operators/activation_ops.py:184-186 (tanh form)
    return (0.5 * x * (1.0 + np.tanh(np.float32(0.7978845608028654) * (x + np.float32(0.044715) * x**3)))).astype(np.float32)


def layernorm_numpy(x, gamma, beta, eps):
    # zenith/execution/operators/norm_ops.py:72-90
    mean = x.mean(axis=-1, keepdims=True)
    var = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    return ((x - mean) / np.sqrt(var + np.float32(eps)) * gamma + beta).astype(np.float32)


def attention_numpy(q, k, v, kv_lens=None):
    """Vectorised numpy attention (BLAS batched matmul) with a key-padding mask."""
    B, nh, S, hd = q.shape
    s = np.matmul(q, k.transpose(0, 1, 3, 2)) * np.float32(1.0 / np.sqrt(hd))
    if kv_lens is not None:
        mask = np.arange(S)[None, :] >= np.asarray(kv_lens)[:, None]
        s = np.where(mask[:, None, None, :], -np.inf, s)
    with np.errstate(invalid="ignore"):
        s = s - np.max(s, axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / np.sum(p, axis=-1, keepdims=True)
    p = np.nan_to_num(p, nan=0.0).astype(np.float32)
    return np.matmul(p, v)


def calibrate_on_oracle(cfg, params, batches, quantize_weights, scales_from_ranges, scales_cls):
    """Activation scales from min-max over ``batches`` run through ``encoder_fp32``.  The product's
    weight-quantization and range-to-scale helpers are passed in by the test so that the oracle
    does not import the product."""
    ranges = {p: [[] for _ in range(cfg.layers)] for p in ACT_POINTS}
    for ids, kv_lens in batches:
        taps = {}
        encoder_fp32(cfg, params, ids, kv_lens, taps)
        for p in ACT_POINTS:
            for li, mm in enumerate(taps[p]):
                ranges[p][li].append(mm)
    return scales_cls(act=scales_from_ranges(ranges, cfg.layers), weights=quantize_weights(params))
