"""Kernel micro-benchmarks (one kernel per invocation, CUDA-event timing, L2 flushed between launches).

    python -m zenith_b200.microbench gemm_i8 --m 4096 --n 2304 --k 768 --epilogue f16 [--tile-n 256] [--iters 20]
    python -m zenith_b200.microbench add_ln  --rows 4096 --hidden 768
    python -m zenith_b200.microbench attention --b 32 --h 12 --s 128 --d 64 [--causal]
    python -m zenith_b200.microbench qkv_attn --b 32 --h 12 --s 128

Prints one JSON line.  The counterpart of the reference's benchmarks/int8_bench.py, wmma_bench.py,
layernorm_bench.py and flash_attention_benchmark.py; also the small, single-kernel command used for
profiler captures.
"""
from __future__ import annotations

import argparse
import json
import statistics

import torch

from . import ops


def _time(fn, iters, flush):
    for _ in range(3):
        fn()
    us = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        us.append(s.elapsed_time(e) * 1e3)
    return statistics.median(us), min(us)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm_i8", "gemm_i8_ln", "gemm_f16", "add_ln", "attention", "qkv_attn", "encoder"])
    ap.add_argument("--config", choices=["base", "large"], default="base")
    ap.add_argument("--dtype", choices=["int8", "fp16"], default="int8")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--epilogue", choices=["s32", "f32", "f16", "gelu_s8", "gelu_f16"], default="f16")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--pair", choices=["auto", "on", "off"], default="auto", help="CTA-pair kernel: forced on / off")
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=768)
    ap.add_argument("--b", type=int, default=32)
    ap.add_argument("--h", type=int, default=12)
    ap.add_argument("--s", type=int, default=128)
    ap.add_argument("--d", type=int, default=64)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {"case": a.case}
    pair = {"auto": None, "on": True, "off": False}[a.pair]
    if a.case == "gemm_i8":
        x = torch.randint(-128, 128, (a.m, a.k), dtype=torch.int8, device=dev)
        w = torch.randint(-128, 128, (a.n, a.k), dtype=torch.int8, device=dev)
        ws = torch.rand(a.n, device=dev) * 1e-3
        b = torch.randn(a.n, device=dev)
        kw = {"s32": dict(out_dtype=torch.int32), "f32": dict(out_dtype=torch.float32), "f16": dict(out_dtype=torch.float16),
              "gelu_s8": dict(act="gelu", out_dtype=torch.int8, out_scale=0.05),
              "gelu_f16": dict(act="gelu", out_dtype=torch.float16)}[a.epilogue]
        y = torch.empty((a.m, a.n), dtype=kw["out_dtype"], device=dev)
        med, best = _time(lambda: ops.linear_int8(x, w, 0.02, ws, b, out=y, tile_n=a.tile_n, pair=pair, **kw), a.iters, flush)
        out.update(m=a.m, n=a.n, k=a.k, epilogue=a.epilogue, tile_n=a.tile_n, pair=a.pair, us=med, us_min=best,
                   tops=2.0 * a.m * a.n * a.k / med / 1e6)
    elif a.case == "gemm_i8_ln":
        n = a.n if a.n in (768, 1024) else 768
        x = torch.randint(-128, 128, (a.m, a.k), dtype=torch.int8, device=dev)
        w = torch.randint(-128, 128, (n, a.k), dtype=torch.int8, device=dev)
        ws = torch.rand(n, device=dev) * 1e-3
        b = torch.randn(n, device=dev)
        res = torch.randn(a.m, n, device=dev, dtype=torch.float16)
        g = torch.ones(n, device=dev, dtype=torch.float16)
        be = torch.zeros_like(g)
        med, best = _time(lambda: ops.linear_int8_add_layernorm(x, w, 0.02, ws, b, res, g, be, 1e-12, out_scale=0.03),
                          a.iters, flush)
        out.update(m=a.m, n=n, k=a.k, us=med, us_min=best, tops=2.0 * a.m * n * a.k / med / 1e6)
    elif a.case == "gemm_f16":
        x = torch.randn(a.m, a.k, device=dev, dtype=torch.float16)
        w = torch.randn(a.n, a.k, device=dev, dtype=torch.float16)
        b = torch.randn(a.n, device=dev)
        y = torch.empty((a.m, a.n), dtype=torch.float16, device=dev)
        med, best = _time(lambda: ops.linear_fp16(x, w, b, out=y, tile_n=a.tile_n, pair=pair), a.iters, flush)
        out.update(m=a.m, n=a.n, k=a.k, tile_n=a.tile_n, us=med, us_min=best, tflops=2.0 * a.m * a.n * a.k / med / 1e6)
    elif a.case == "add_ln":
        x = torch.randn(a.rows, a.hidden, device=dev, dtype=torch.float16)
        r = torch.randn_like(x)
        g = torch.ones(a.hidden, device=dev, dtype=torch.float16)
        be = torch.zeros_like(g)
        med, best = _time(lambda: ops.add_layernorm(x, r, g, be, 1e-12, out_scale=0.03), a.iters, flush)
        nbytes = a.rows * a.hidden * 7  # 2 fp16 reads, 1 fp16 write, 1 int8 write
        out.update(rows=a.rows, hidden=a.hidden, us=med, us_min=best, gbs=nbytes / med / 1e3)
    elif a.case == "qkv_attn":
        hidden = a.h * 64
        x = torch.randint(-128, 128, (a.b * a.s, hidden), dtype=torch.int8, device=dev)
        w = torch.randint(-128, 128, (3 * hidden, hidden), dtype=torch.int8, device=dev)
        ws = torch.rand(3 * hidden, device=dev) * 1e-4
        b = torch.randn(3 * hidden, device=dev) * 0.1
        lens = torch.full((a.b,), max(1, a.s - 16), dtype=torch.int32, device=dev)
        med, best = _time(lambda: ops.qkv_attention_int8(x, w, 0.02, ws, b, a.b, a.s, a.h, kv_lens=lens, out_scale=0.02),
                          a.iters, flush)
        out.update(b=a.b, h=a.h, s=a.s, us=med, us_min=best, projection_tops=2.0 * a.b * a.s * 3 * hidden * hidden / med / 1e6,
                   attention_tflops=4.0 * a.b * a.h * a.s * a.s * 64 / med / 1e6)
    elif a.case == "encoder":
        import numpy as np

        from .calibrate import calibrate
        from .encoder import BERT_BASE, BERT_LARGE, Fp16Encoder, Int8Encoder, init_params

        cfg = BERT_BASE if a.config == "base" else BERT_LARGE
        params = init_params(cfg, 1234)
        rng = np.random.default_rng(0)

        def batch():
            ids = torch.from_numpy(rng.integers(0, cfg.vocab, (a.batch, a.seq)).astype(np.int32)).to(dev)
            lens = torch.from_numpy((a.seq - rng.integers(0, 33, a.batch)).astype(np.int32)).to(dev)
            return ids, lens

        if a.dtype == "int8":
            enc = Int8Encoder(cfg, params, calibrate(cfg, params, [batch() for _ in range(4)], dev), dev, gemm_pair=pair)
        else:
            enc = Fp16Encoder(cfg, params, dev, gemm_pair=pair)
        enc.capture(a.batch, a.seq)
        enc.set_inputs(*batch())
        med, best = _time(enc.replay, a.iters, flush)
        T = a.batch * a.seq
        gemm_ops = 2.0 * T * (4 * cfg.hidden**2 + 2 * cfg.hidden * cfg.ffn) * cfg.layers
        attn_flops = 4.0 * a.batch * cfg.heads * a.seq * a.seq * cfg.head_dim * cfg.layers
        out.update(config=a.config, dtype=a.dtype, batch=a.batch, seq=a.seq, pair=a.pair, us=med, us_min=best,
                   seq_per_s=a.batch / med * 1e6, gemm_tops=gemm_ops / med / 1e6, attn_tflops=attn_flops / med / 1e6,
                   launches=enc.launches_per_forward)
    else:
        q = torch.randn(a.b, a.h, a.s, a.d, device=dev, dtype=torch.float16)
        k = torch.randn_like(q)
        v = torch.randn_like(q)
        med, best = _time(lambda: ops.flash_attention(q, k, v, causal=a.causal), max(3, a.iters // 4), flush)
        fl = 4.0 * a.b * a.h * a.s * a.s * a.d * (0.5 if a.causal else 1.0)
        out.update(b=a.b, h=a.h, s=a.s, d=a.d, causal=a.causal, us=med, us_min=best, tflops=fl / med / 1e6)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
