#!/usr/bin/env python
"""Benchmark of the W8A8 BERT encoder on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config bert_base|bert_large]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

``--config bert_base`` (default, the headline): a step is one forward pass over one batch of 32 synthetic
sequences of 128 tokens per GPU (BASELINE.json configs[2]: 12 layers, hidden 768, 12 heads, FFN 3072, post-LN,
tanh-GELU, W8A8 with per-channel weight scales and min-max activation scales from 16 seeded batches; token ids
uniform over 30522 words, the last 0..32 positions of each row masked).  Ranks are independent replicas (weak
scaling, global batch 32 * N).  ``--config bert_large``: BASELINE.json configs[4], global batch 256 x 384 tokens
split over the ranks (strong scaling).  For N > 1 every step ends with the gather of the hidden states onto rank
0.  Rank 0 prints ONE JSON line.

`value`      sequences/s with token ids already in HBM (CUDA-graph replay of the launch list).
`e2e`        the same through the public host API (zenith_b200.serve.HostPipeline) with HOST buffers: every
             step copies pinned ids / lengths to the device and the fp16 hidden states back to pinned host
             memory inside the timed region; the copy back of step i overlaps the compute of step i + 1.
`sustained`  seconds of back-to-back replays under the clock sampler: the power-capped rate, beside the burst
             rate of the short timed region.
`roofline`   the launches of a layer that carry its int8 GEMM work: average launch durations measured with
             CUDA events inside a graph of 12 launches per shape, as the step runs them.
`secondary`  the other configurations of BASELINE.json measured in the same run (fp16 encoder, attention
             sweep, a BERT-large shard), kernel yardsticks (int8 8192^3 against the library GEMM, add+LayerNorm
             against the copy bandwidth).
`parity_check` one layer's FFN1 int8 output of the timed encoder against the CPU oracle, and replay == eager.
`cpu_baseline` the CPU restatement of the reference's quantized executor (fake-quant + fp32 BLAS matmul) on a
             bounded sample, plus the reference's two single-Linear CPU forms on BASELINE.json configs[0].
`--impl reference` times that CPU executor alone, on the same workload definition (32 sequences per step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

BATCH, SEQ = 32, 128
MASTER_SEED = 1234
CALIB_BATCHES = 16
METRIC = "bert_base_int8_seq128_sequences_per_sec"
WORKLOAD = "bert-base W8A8 encoder, batch 32 per GPU, seq 128 (BASELINE.json configs[2])"
LARGE_GLOBAL_BATCH, LARGE_SEQ = 256, 384
LARGE_METRIC = "bert_large_int8_seq384_sequences_per_sec"
LARGE_WORKLOAD = "bert-large W8A8 encoder, global batch 256 split over the GPUs, seq 384 (BASELINE.json configs[4])"


def make_batch(seed: int, vocab: int, batch: int = BATCH, seq: int = SEQ):
    """Token ids uniform over the vocabulary; attention mask all ones except the last 0..32 positions."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, (batch, seq)).astype(np.int32)
    lens = (seq - rng.integers(0, 33, batch)).astype(np.int32)
    return ids, lens


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": smax, "reasons": ["no samples"]}
        busy = [c for c, p in zip(sm, power) if p > 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's quantized executor restated (oracle/encoder_ref.py), host cores only
# ------------------------------------------------------------------------------------------------
def blas_threads_all() -> int:
    """Let numpy's BLAS use every host core (torchrun exports OMP_NUM_THREADS=1 to its workers) and return the
    number of threads it will really use."""
    n = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info, threadpool_limits

        threadpool_limits(limits=n)
        used = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
        return max(used) if used else 1
    except Exception:
        return int(os.environ.get("OMP_NUM_THREADS", n))


def cpu_executor(sample_seqs: int, steps: int, warmup: int, large: bool = False) -> dict:
    threads = blas_threads_all()
    from oracle import encoder_ref as ER
    from zenith_b200.calibrate import activation_scales_from_ranges, quantize_weights
    from zenith_b200.encoder import BERT_BASE, BERT_LARGE, Int8Scales, init_params

    cfg = BERT_LARGE if large else BERT_BASE
    seq = LARGE_SEQ if large else SEQ
    params = init_params(cfg, MASTER_SEED)
    cal = [make_batch(MASTER_SEED + 1 + i, cfg.vocab, batch=2, seq=seq) for i in range(2)]  # scales do not affect timing
    scales = ER.calibrate_on_oracle(cfg, params, cal, quantize_weights, activation_scales_from_ranges, Int8Scales)
    ids, lens = make_batch(MASTER_SEED, cfg.vocab, batch=sample_seqs, seq=seq)
    for _ in range(warmup):
        ER.encoder_fake_quant(cfg, params, scales, ids, lens)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        ER.encoder_fake_quant(cfg, params, scales, ids, lens)
        times.append(time.perf_counter() - t0)
    total = sum(times)
    return {"seq_per_s": sample_seqs * steps / total, "ms_per_step": 1e3 * total / steps,
            "cores": threads, "sample": f"{steps} passes of {sample_seqs} sequences x {seq} tokens "
            f"(numpy fake-quant + fp32 BLAS matmul on {threads} BLAS threads of {os.cpu_count()} host cores)"}


def cpu_single_linear_baselines() -> list:
    """The reference's two other CPU forms of a quantized Linear, on BASELINE.json configs[0] (X [128, 768],
    W [3072, 768]): the true-integer numpy product (benchmarks/int8_bench.py:42-45: int32 matmul, then dequant) and
    the reference's own AVX2 fp32 GEMM (core/src/cpu_kernels.cpp:129-165, compiled as it stands into oracle/_ref) on
    the dequantised operands.  Both are single-threaded by construction."""
    from oracle import oracle as O

    M, K, N = 128, 768, 3072
    rng = np.random.default_rng(MASTER_SEED)
    xq = rng.integers(-128, 128, (M, K), dtype=np.int8)
    wq = rng.integers(-128, 128, (N, K), dtype=np.int8)
    s_x, s_w = np.float32(0.03), np.float32(1e-3)

    def median_ms(fn, reps=10, warm=3):
        for _ in range(warm):
            fn()
        t = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            t.append(time.perf_counter() - t0)
        return 1e3 * statistics.median(t), 1e3 * min(t)

    out = []
    b32 = np.ascontiguousarray(wq.astype(np.int32).T)
    med, best = median_ms(lambda: (xq.astype(np.int32) @ b32).astype(np.float32) * s_x * s_w, reps=3, warm=1)
    out.append({"name": "true-integer numpy GEMM + dequant (int8_bench.py:42-45)", "workload": "configs[0]: 128 x 3072 x 768",
                "ms": round(med, 3), "ms_min": round(best, 3), "gops": round(2.0 * M * N * K / med / 1e6, 2), "cores": 1,
                "kind": "reference formula in numpy"})
    if O.ref_lib() is not None:
        xf = xq.astype(np.float32) * s_x
        wt = np.ascontiguousarray((wq.astype(np.float32) * s_w).T)  # [K, N]
        med, best = median_ms(lambda: O.ref_matmul_avx2(xf, wt))
        out.append({"name": "reference AVX2 fp32 GEMM on dequantised operands (cpu_kernels.cpp:129-165)",
                    "workload": "configs[0]: 128 x 3072 x 768", "ms": round(med, 3), "ms_min": round(best, 3),
                    "gflops": round(2.0 * M * N * K / med / 1e6, 2), "cores": 1, "kind": "reference"})
    else:
        out.append({"name": "reference AVX2 fp32 GEMM", "ms": None, "kind": "reference",
                    "why": "oracle/_ref was not built (the reference tree was not mounted when build() ran)"})
    return out


_RESULT_FD = None


def quiet_stdout() -> None:
    """Route everything libraries write to stdout (NCCL prints its version line there) to stderr and keep the
    real stdout for the one JSON line."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def workload_of(args, world: int) -> dict:
    """Metric, per-rank batch and names for the selected configuration."""
    if args.config == "bert_large":
        from zenith_b200.dist import shard_bounds

        rank = int(os.environ.get("RANK", "0"))
        _, local = shard_bounds(LARGE_GLOBAL_BATCH, world, rank)
        return {"metric": LARGE_METRIC, "workload": LARGE_WORKLOAD, "seq": LARGE_SEQ, "local_batch": local,
                "global_batch": LARGE_GLOBAL_BATCH, "scaling": "strong", "large": True}
    return {"metric": METRIC, "workload": WORKLOAD, "seq": SEQ, "local_batch": BATCH, "global_batch": BATCH * world,
            "scaling": "weak", "large": False}


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = workload_of(args, 1)
    # One step = the batch a GPU gets in a step of the other arm (32 sequences; BERT-large: a 4-sequence sample of
    # its 256), as long as K such steps fit a few minutes of host time (about 2 sequences/s for BERT-base, 0.2 for
    # BERT-large on these cores); beyond that the per-step sample shrinks so that the whole run stays bounded.
    full, budget = (BATCH, 320) if not wl["large"] else (4, 36)
    sample = max(1, min(full, budget // max(1, args.steps)))
    r = cpu_executor(sample, max(1, args.steps), 1 if args.warmup > 0 else 0, large=wl["large"])
    line = {
        "impl": "reference", "metric": wl["metric"], "value": r["seq_per_s"], "unit": "sequences/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32 (fake-quantized int8 values)", "data": "synthetic",
        "config": {"workload": wl["workload"], "global_batch": sample, "seq_len": wl["seq"],
                   "step_sample": f"{sample} sequences per step", "warmup_run": 1 if args.warmup > 0 else 0},
        "cpu_baseline": {"value": r["seq_per_s"], "unit": "sequences/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["seq_per_s"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def _graph_of(torch, fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def _event_us(torch, fn, reps, flush=None):
    us = []
    for _ in range(reps):
        if flush is not None:
            flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        us.append(s.elapsed_time(e) * 1e3)
    return statistics.median(us)


def time_gemm_shapes(torch, ops, dev, flush) -> dict:
    """The four launches of one encoder layer that carry its int8 GEMM work, with the epilogue each has in the
    encoder: QKV projection fused with attention, attention-out (+ residual + LayerNorm, cluster kernel), FFN1
    (+ GELU + requant), FFN2 (+ residual + LayerNorm), timed with CUDA events in two ways:

    * ``in_step``: as the step runs them - a CUDA graph of 12 back-to-back launches of the shape, one per layer,
      each with its own weight matrix, L2 flushed before every replay (so the weights come from HBM, as in the
      step); average launch duration = replay time / 12.  `roofline.achieved` uses these.
    * ``cold``: one launch alone, L2 flushed, launch latency included (the upper bound a profiler also sees).
    The plain QKV GEMM (the projection alone, as a two-kernel encoder runs it) is timed as well, for reference.
    """
    T, H, F, LAYERS, HEADS = BATCH * SEQ, 768, 3072, 12, 12

    def plain(N, K, **kw):
        x = torch.randint(-128, 128, (T, K), dtype=torch.int8, device=dev)
        ws_ = [torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(LAYERS)]
        ws, b = torch.rand(N, device=dev) * 1e-3, torch.randn(N, device=dev)
        out = torch.empty((T, N), dtype=kw["out_dtype"], device=dev)
        return lambda i: ops.linear_int8(x, ws_[i], 0.02, ws, b, out=out, constant_weights=True, **kw)

    def with_ln(K):
        x = torch.randint(-128, 128, (T, K), dtype=torch.int8, device=dev)
        ws_ = [torch.randint(-128, 128, (H, K), dtype=torch.int8, device=dev) for _ in range(LAYERS)]
        ws, b = torch.rand(H, device=dev) * 1e-3, torch.randn(H, device=dev)
        res = torch.randn(T, H, device=dev, dtype=torch.float16)
        g, be = torch.ones(H, device=dev, dtype=torch.float16), torch.zeros(H, device=dev, dtype=torch.float16)
        return lambda i: ops.linear_int8_add_layernorm(x, ws_[i], 0.02, ws, b, res, g, be, 1e-12, out_scale=0.03,
                                                       constant_weights=True)

    def qkv_attention():
        x = torch.randint(-128, 128, (T, H), dtype=torch.int8, device=dev)
        ws_ = [torch.randint(-128, 128, (3 * H, H), dtype=torch.int8, device=dev) for _ in range(LAYERS)]
        ws, b = torch.rand(3 * H, device=dev) * 1e-4, torch.randn(3 * H, device=dev) * 0.1
        lens = torch.full((BATCH,), SEQ - 16, dtype=torch.int32, device=dev)  # the mean key length of the workload
        return lambda i: ops.qkv_attention_int8(x, ws_[i], 0.02, ws, b, BATCH, SEQ, HEADS, kv_lens=lens, out_scale=0.02,
                                                constant_weights=True)

    # (name, GEMM N, GEMM K, launcher, counted in the family)
    shapes = [("qkv_projection_attention", 3 * H, H, qkv_attention(), True),
              ("attn_out_add_layernorm", H, H, with_ln(H), True),
              ("ffn1_gelu_requant", F, H, plain(F, H, act="gelu", out_dtype=torch.int8, out_scale=0.05), True),
              ("ffn2_add_layernorm", H, F, with_ln(F), True),
              ("qkv_projection_alone", 3 * H, H, plain(3 * H, H, out_dtype=torch.float16), False)]
    per_shape, tot_ops, tot_us, alg_bytes = {}, 0.0, 0.0, 0.0
    for name, N, K, fn, counted in shapes:
        def all_layers():
            for i in range(LAYERS):
                fn(i)
        graph = _graph_of(torch, all_layers)
        for _ in range(3):
            graph.replay()
        in_step = _event_us(torch, graph.replay, 9, flush) / LAYERS
        cold = _event_us(torch, lambda: fn(0), 9, flush)
        ops_ = 2.0 * T * N * K
        per_shape[name] = {"us": round(in_step, 2), "tops": round(ops_ / in_step / 1e6, 1), "cold_us": round(cold, 2)}
        if counted:
            tot_ops += ops_
            tot_us += in_step
    # operand, residual and output bytes of the four launches, from the shapes: int8 operands M K + N K, per-column
    # scale and bias 8 N, then what each launch writes (and, for the LayerNorm launches, the fp16 residual it reads)
    alg_bytes += T * H + 3 * H * H + 8 * 3 * H + T * H * (2 + 1)                # projection + attention: ctx fp16 + int8
    alg_bytes += T * H + H * H + 8 * H + T * H * (2 + 2 + 1)                    # attention-out: residual, y fp16, y int8
    alg_bytes += T * H + F * H + 8 * F + T * F                                  # FFN1: int8 out
    alg_bytes += T * F + H * F + 8 * H + T * H * (2 + 2 + 1)                    # FFN2
    return {"per_shape": per_shape, "ops_per_layer": tot_ops, "us_per_layer": tot_us, "algorithmic_bytes": alg_bytes}


def secondary_metrics(torch, ops, dev, flush, peaks, cfg_base, params_base) -> dict:
    """The other BASELINE.json configurations and two kernel yardsticks, measured in this run (CUDA events, L2
    flushed between launches, medians)."""
    from zenith_b200.encoder import BERT_LARGE, Fp16Encoder, Int8Encoder, Int8Scales, init_params

    out = {}

    def done(what):  # progress on stderr: a fault in a secondary measurement is then easy to place
        torch.cuda.synchronize()
        print(f"[bench] secondary: {what} done", file=sys.stderr, flush=True)

    # configs[1]: the fp16 encoder, batch 32 x 128
    enc = Fp16Encoder(cfg_base, params_base, dev)
    ids, lens = make_batch(MASTER_SEED + 1000, cfg_base.vocab)
    enc.capture(BATCH, SEQ)
    enc.set_inputs(torch.from_numpy(ids).to(dev), torch.from_numpy(lens).to(dev))
    for _ in range(3):
        enc.replay()
    us = _event_us(torch, enc.replay, 15, flush)
    out["bert_base_fp16_seq128"] = {"sequences_per_s": round(BATCH / us * 1e6, 1), "ms_per_step": round(us / 1e3, 4),
                                    "launches": enc.launches_per_forward, "workload": "BASELINE.json configs[1]"}
    del enc
    done("fp16 encoder")
    # configs[3]: attention forward sweep, B = 8, H = 16
    fp16_peak = peaks["bf16_tflops"]
    sweep = {}
    for D in (64, 128):
        for S in (512, 2048, 8192):
            q, k, v = (torch.randn(8, 16, S, D, device=dev, dtype=torch.float16) for _ in range(3))
            for causal in (False, True):
                fn = lambda: ops.flash_attention(q, k, v, causal=causal)
                for _ in range(2):
                    fn()
                us = _event_us(torch, fn, 5, flush)
                tf = 4.0 * 8 * 16 * S * S * D * (0.5 if causal else 1.0) / us / 1e6
                sweep[f"d{D}_s{S}_{'causal' if causal else 'full'}"] = {"tflops": round(tf, 1), "frac_of_fp16_peak": round(tf / fp16_peak, 3)}
            del q, k, v
    out["attention_fwd_b8_h16"] = {"cases": sweep, "peak_tflops": fp16_peak,
                                   "peak_source": f"{peaks['source']} bf16 GEMM burst", "workload": "BASELINE.json configs[3]"}
    done("attention sweep")
    # int8 GEMM yardstick: own kernel against the library GEMM on the same device in the same run
    n = 8192
    a = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev)
    b = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev)
    o16 = torch.empty((n, n), dtype=torch.float16, device=dev)
    ws = torch.rand(n, device=dev) * 1e-4
    own = lambda: ops.linear_int8(a, b, 0.02, ws, None, out=o16, out_dtype=torch.float16)
    lib = lambda: torch._int_mm(a, b.t())
    for f in (own, lib):
        for _ in range(2):
            f()
    us_own, us_lib = _event_us(torch, own, 7, flush), _event_us(torch, lib, 7, flush)
    out["int8_gemm_8192"] = {"own_tops": round(2.0 * n**3 / us_own / 1e6, 1), "library_int_mm_tops": round(2.0 * n**3 / us_lib / 1e6, 1),
                             "note": "own: fp16 output with per-column scales (CTA-pair kernel); library: torch._int_mm, int32 output"}
    del a, b, o16
    done("int8 GEMM 8192")
    # add + LayerNorm (fp16 in / out + int8 copy) against the measured copy bandwidth
    rows, hidden = 98304, 1024
    x = torch.randn(rows, hidden, device=dev, dtype=torch.float16)
    r = torch.randn_like(x)
    g, be = torch.ones(hidden, device=dev, dtype=torch.float16), torch.zeros(hidden, device=dev, dtype=torch.float16)
    fn = lambda: ops.add_layernorm(x, r, g, be, 1e-12, out_scale=0.03)
    for _ in range(2):
        fn()
    us = _event_us(torch, fn, 7, flush)
    gbs = rows * hidden * 7 / us / 1e3
    out["add_layernorm_98304x1024"] = {"gb_per_s": round(gbs, 1), "frac_of_hbm": round(gbs / peaks["hbm_gbs"], 3),
                                       "hbm_gbs": peaks["hbm_gbs"], "bytes_per_row": hidden * 7}
    del x, r
    done("add + LayerNorm")
    # unpadded batches where they pay: 128 sequences x 128 tokens (the headline's 32 x 128 needs the same number of
    # tile rounds packed or padded, so packing gains nothing there)
    try:
        from zenith_b200.calibrate import calibrate as _cal
        calb = [make_batch(MASTER_SEED + 1 + i, cfg_base.vocab) for i in range(2)]
        sc_b = _cal(cfg_base, params_base, [(torch.from_numpy(i).to(dev), torch.from_numpy(l).to(dev)) for i, l in calb], dev)
        ids, lens = make_batch(MASTER_SEED + 3000, cfg_base.vocab, batch=128, seq=SEQ)
        ids_d, lens_d = torch.from_numpy(ids).to(dev), torch.from_numpy(lens).to(dev)
        res = {}
        for form in ("padded", "unpadded"):
            enc = Int8Encoder(cfg_base, params_base, sc_b, dev)
            if form == "padded":
                enc.capture(128, SEQ)
            else:
                enc.capture_unpadded(128, SEQ, Int8Encoder.unpadded_capacity(lens.tolist(), SEQ))
            enc.set_inputs(ids_d, lens_d)
            for _ in range(3):
                enc.replay()
            us = _event_us(torch, enc.replay, 9, flush)
            res[form] = {"ms_per_step": round(us / 1e3, 4), "sequences_per_s": round(128 / us * 1e6, 1)}
            del enc
        res["valid_tokens"] = int(lens.sum())
        res["padded_tokens"] = int(ids.size)
        out["bert_base_int8_batch128_unpadded"] = res
    except Exception as exc:
        out["bert_base_int8_batch128_unpadded"] = {"error": str(exc)}
    done("batch 128 padded / unpadded")
    # configs[4]: one GPU's shard of the BERT-large run at 8 GPUs (32 sequences x 384 tokens)
    cfg = BERT_LARGE
    params = init_params(cfg, MASTER_SEED)
    from zenith_b200.calibrate import calibrate
    cal = [make_batch(MASTER_SEED + 1 + i, cfg.vocab, batch=8, seq=LARGE_SEQ) for i in range(2)]
    scales = calibrate(cfg, params, [(torch.from_numpy(i).to(dev), torch.from_numpy(l).to(dev)) for i, l in cal], dev)
    enc = Int8Encoder(cfg, params, scales, dev)
    ids, lens = make_batch(MASTER_SEED + 2000, cfg.vocab, batch=32, seq=LARGE_SEQ)
    enc.capture(32, LARGE_SEQ)
    enc.set_inputs(torch.from_numpy(ids).to(dev), torch.from_numpy(lens).to(dev))
    for _ in range(3):
        enc.replay()
    us = _event_us(torch, enc.replay, 9, flush)
    out["bert_large_int8_seq384_shard32"] = {"ms_per_step": round(us / 1e3, 3), "sequences_per_s": round(32 / us * 1e6, 1),
                                             "launches": enc.launches_per_forward,
                                             "workload": "BASELINE.json configs[4], the 32-sequence shard one of 8 GPUs holds"}
    try:  # the same shard unpadded (projection GEMM on the packed rows, attention from the offsets)
        enc.capture_unpadded(32, LARGE_SEQ, Int8Encoder.unpadded_capacity(lens.tolist(), LARGE_SEQ))
        enc.set_inputs(torch.from_numpy(ids).to(dev), torch.from_numpy(lens).to(dev))
        for _ in range(3):
            enc.replay()
        us_u = _event_us(torch, enc.replay, 9, flush)
        out["bert_large_int8_seq384_shard32"].update({"unpadded_ms_per_step": round(us_u / 1e3, 3),
                                                      "valid_tokens": int(lens.sum()), "padded_tokens": int(ids.size)})
    except Exception as exc:
        out["bert_large_int8_seq384_shard32"]["unpadded_error"] = str(exc)
    return out


def unpadded_metric(torch, cfg, params, scales, ids_np, lens_np, dev, flush, padded_out) -> dict:
    """The same batch through the unpadded form of the encoder (valid tokens packed back to back, GEMMs on the
    packed rows, attention from the offsets): time per step, and a check that every valid token's hidden state has
    the bits of the padded pass that was timed as the headline."""
    from zenith_b200.encoder import Int8Encoder

    B, S = ids_np.shape
    enc = Int8Encoder(cfg, params, scales, dev)
    cap = Int8Encoder.unpadded_capacity(lens_np.tolist(), S)
    enc.capture_unpadded(B, S, cap)
    enc.set_inputs(torch.from_numpy(ids_np).to(dev), torch.from_numpy(lens_np).to(dev))
    for _ in range(3):
        out = enc.replay()
    rows = torch.from_numpy(np.concatenate([b * S + np.arange(int(n)) for b, n in enumerate(lens_np)])).to(dev)
    same = bool(torch.equal(out[rows], padded_out[rows]))
    us = _event_us(torch, enc.replay, 15, flush)
    return {"sequences_per_s": round(B / us * 1e6, 1), "ms_per_step": round(us / 1e3, 4), "packed_rows": cap,
            "padded_rows": B * S, "valid_tokens": int(lens_np.sum()), "launches": enc.launches_per_forward,
            "valid_tokens_equal_padded_pass": same,
            "note": "not the headline: the reference computes the padding positions too; their hidden states are zeros here"}


def parity_check(torch, enc, scales, params, ids_np, lens_np, dev) -> dict:
    """The encoder that was timed, checked: the CUDA-graph replay equals the eager launch list bit for bit, and the
    FFN1 int8 output of one layer (GELU + requantisation epilogue) equals the CPU oracle on sampled rows, computed
    from the int8 input the device itself gave that GEMM."""
    from oracle import oracle as O

    enc.set_inputs(torch.from_numpy(ids_np).to(dev), torch.from_numpy(lens_np).to(dev))
    replayed = enc.replay().clone()
    layer = len(params["layers"]) // 2
    rows = np.arange(5, ids_np.size, max(1, ids_np.size // 96))
    ok, checked = True, 0
    for li, buf in enc.forward_layerwise(torch.from_numpy(ids_np).to(dev), torch.from_numpy(lens_np).to(dev)):
        if li == layer:
            a, wq, lp = scales.act[li], scales.weights[li], params["layers"][li]
            want = O.linear_int8(buf["h1q"].cpu().numpy()[rows], wq["w1"][0], a["h1"], wq["w1"][1], lp["b1"], "gelu", "s8", a["gelu"])
            got = buf["gq"].cpu().numpy()[rows]
            ok = bool(np.array_equal(got, want))
            checked = int(got.size)
    same = bool(torch.equal(enc.out, replayed))
    return {"status": "ok" if (ok and same) else "MISMATCH", "ffn1_int8_elements_checked": checked, "layer": layer,
            "replay_equals_eager": same}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from zenith_b200 import _capi, ops
    from zenith_b200.calibrate import calibrate
    from zenith_b200.dist import OutputGatherer, PeerGatherer, init_from_env
    from zenith_b200.encoder import BERT_BASE, BERT_LARGE, Int8Encoder, init_params
    from zenith_b200.serve import HostPipeline

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    rank, local_rank, world = init_from_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _capi.lib()
    wl = workload_of(args, world)
    cfg = BERT_LARGE if wl["large"] else BERT_BASE
    B, S = wl["local_batch"], wl["seq"]
    K, W = args.steps, max(3, args.warmup)

    params = init_params(cfg, MASTER_SEED)
    n_cal, cal_batch = (CALIB_BATCHES, BATCH) if not wl["large"] else (CALIB_BATCHES, 8)
    calib = [make_batch(MASTER_SEED + 1 + i, cfg.vocab, batch=cal_batch, seq=S) for i in range(n_cal)]
    scales = calibrate(cfg, params, [(torch.from_numpy(i).to(dev), torch.from_numpy(l).to(dev)) for i, l in calib], dev)
    enc = Int8Encoder(cfg, params, scales, dev, micro_batches=args.micro_batches)
    ids_np, lens_np = make_batch(MASTER_SEED + 1000 + rank, cfg.vocab, batch=B, seq=S)
    ids_h = torch.from_numpy(ids_np).pin_memory()
    lens_h = torch.from_numpy(lens_np).pin_memory()
    enc.capture(B, S)
    enc.set_inputs(ids_h.to(dev), lens_h.to(dev))
    # The gather of the hidden states onto rank 0, one per step.  "peer" (default): every rank pushes its shard into
    # rank 0's buffer with its copy engine over NVLink (zenith_b200.dist.PeerGatherer), the push of step i running
    # under the kernels of step i + 1; "nccl": an NCCL gather in the compute stream after every pass.
    gatherer = peer = None
    if world > 1 and args.gather == "nccl":
        gatherer = OutputGatherer(wl["global_batch"], S, cfg.hidden, torch.float16, dev, root=0)
    elif world > 1:
        peer = PeerGatherer(wl["global_batch"], S, cfg.hidden, torch.float16, dev, root=0, depth=3)
        parked = [torch.empty_like(enc.out) for _ in range(peer.depth)]
    ticket = [0]
    collected = [0]  # rank 0: tickets below this one have been waited for and released (each exactly once)

    l2_flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # 2 x the 126 MB L2

    def flush():
        l2_flush_buf.fill_(1)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_device():
        enc.replay()
        if gatherer is not None:
            gatherer.gather(enc.out)
        elif peer is not None:
            t = ticket[0]
            ticket[0] += 1
            buf = parked[t % peer.depth]
            buf.copy_(enc.out, non_blocking=True)  # the next pass overwrites the encoder's output buffer at once
            peer.push(buf, t)
            if t >= 1 and peer.pushed(t - 1) is not None:
                # the previous step's push is part of this step's timed region: it must have finished by now
                torch.cuda.current_stream().wait_event(peer.pushed(t - 1))
            lag = peer.depth - 1
            while rank == 0 and collected[0] <= t - lag:
                peer.wait(collected[0])  # host-side: every shard of that ticket has landed in rank 0's buffer
                peer.release(collected[0])
                collected[0] += 1

    def finish_gathers():
        """Rank 0 collects the tickets still in flight; every rank's queued copies complete."""
        if peer is None:
            return
        while rank == 0 and collected[0] < ticket[0]:
            peer.wait(collected[0])
            peer.release(collected[0])
            collected[0] += 1
        peer.drain()

    # End to end through the public host API (zenith_b200.serve.HostPipeline): every step copies its ids /
    # lengths from pinned host memory and its hidden states back to pinned host memory; the device->host
    # copy of step i runs on a copy stream while step i + 1 computes, and the host waits for step i - 1's
    # result before it queues step i + 1 (the loop a server would run).  With several GPUs every rank delivers
    # its own shard to host memory over its own PCIe link (host memory is where the shards meet).
    pipe = HostPipeline(enc, B, S)

    def timed_e2e(steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s.record()
        prev = None
        for _ in range(steps):
            t = pipe.submit(ids_h, lens_h)
            if prev is not None:
                pipe.result(prev)
            prev = t
        pipe.result(prev)
        pipe.drain()
        e.record()
        barrier()
        t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(step_fn, steps):
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        barrier()
        for i in range(steps):
            flush()
            starts[i].record()
            step_fn()
            if i == steps - 1 and peer is not None and peer.pushed(ticket[0] - 1) is not None:
                torch.cuda.current_stream().wait_event(peer.pushed(ticket[0] - 1))  # the last push ends inside the region
            ends[i].record()
        finish_gathers()
        barrier()
        ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sustained(seconds):
        """Back-to-back steps for `seconds`: no L2 flush (a step's working set exceeds the L2), one event pair."""
        sampler_ = ClockSampler(local_rank) if rank == 0 else None
        n_guess = max(10, int(seconds / max(1e-4, total_ms / K / 1e3)))
        barrier()
        if sampler_:
            sampler_.start()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n_guess):
            step_device()
        if peer is not None and peer.pushed(ticket[0] - 1) is not None:
            torch.cuda.current_stream().wait_event(peer.pushed(ticket[0] - 1))
        e.record()
        finish_gathers()
        barrier()
        clk = sampler_.stop() if sampler_ else None
        t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        return {"value": wl["global_batch"] * n_guess / (ms / 1e3) if wl["large"] else world * B * n_guess / (ms / 1e3),
                "unit": "sequences/s", "seconds": round(ms / 1e3, 2), "steps": n_guess, "ms_per_step": ms / n_guess,
                "clocks": clk, "how": "back-to-back steps, one event pair, no L2 flush between steps"}

    for _ in range(W):
        step_device()
    finish_gathers()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    launches0 = ops.launch_count
    total_ms = timed(step_device, K)
    launches = ops.launch_count - launches0
    timed_e2e(W)
    e2e_ms = timed_e2e(K)
    e2e_launches = enc.launches_per_forward  # the copies to and from the host run on the copy engines
    clocks = sampler.stop() if sampler else None
    sus = sustained(args.sustain_seconds) if args.sustain_seconds > 0 else None
    gather_check = None
    if peer is not None:
        # what the pushes delivered against an NCCL all_gather of the same tensors
        t = ticket[0]
        step_device()
        finish_gathers()
        barrier()
        ref = torch.empty((wl["global_batch"] * S, cfg.hidden), dtype=torch.float16, device=dev)
        if len({c for _, c in peer.bounds}) == 1:
            dist.all_gather_into_tensor(ref, enc.out.contiguous())
            if rank == 0:
                gather_check = "ok" if torch.equal(peer.data[t % peer.depth], ref) else "MISMATCH"
        else:
            gather_check = "not run (uneven shards)"
        barrier()
    status = _capi.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    seqs_per_step = wl["global_batch"] if wl["large"] else world * B
    value = seqs_per_step * K / (total_ms / 1e3)
    e2e_value = seqs_per_step * K / (e2e_ms / 1e3)
    peaks = measured_peaks()
    line = {
        "metric": wl["metric"], "value": value, "unit": "sequences/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None,
        "dtype": "s8 operands, s32 accumulators (fp16 LayerNorm / softmax / residual)", "data": "synthetic",
        "config": {"workload": wl["workload"], "global_batch": seqs_per_step, "seq_len": S,
                   "parallelism": f"replicas x{world}" + ("" if world == 1 else
                                                             ", NCCL gather of the hidden states onto rank 0 inside every step" if peer is None else
                                                             ", hidden states pushed onto rank 0 by the copy engines over NVLink every step "
                                                             "(peer-to-peer copies, the push of step i under the kernels of step i + 1)"),
                   "l2": "256 MB buffer written between timed steps",
                   "launch": f"CUDA-graph replay of {enc.launches_per_forward} kernels in {args.micro_batches} concurrent micro-batch(es)"},
        "e2e": {"value": e2e_value, "unit": "sequences/s", "ms_per_step": e2e_ms / K,
                "h2d_bytes_per_step": int(ids_h.numel() * ids_h.element_size() + lens_h.numel() * lens_h.element_size()),
                "d2h_bytes_per_step": int(pipe.host_out[0].numel() * 2),
                "how": "zenith_b200.serve.HostPipeline: one event pair around all steps; per step pinned-host ids -> device on an "
                       "input stream, replay of the slot's graph (own inputs, own result buffer), hidden states -> pinned host "
                       "on a copy stream; both copies overlap the neighbouring steps' compute; "
                       "no L2 flush in this loop (a step's working set of weights + activations exceeds the 126 MB L2); "
                       "with several GPUs every rank delivers its own shard to host memory (bytes are per rank)",
                "launches_per_step": e2e_launches},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "device_status": status,
    }
    if sus is not None:
        line["sustained"] = sus
    if gather_check is not None:
        line["gather_check"] = gather_check
    if world == 1 and not wl["large"]:
        g = time_gemm_shapes(torch, ops, dev, flush)
        int8_peak = 2.0 * peaks["bf16_tflops"]
        achieved = g["ops_per_layer"] / g["us_per_layer"] / 1e6
        line["roofline"] = {
            "kernel": "the launches of one layer that carry its int8 GEMM work: qkv_attn_kernel (QKV projection fused with "
                      "attention; only the projection's operations are counted), gemm_i8_ln_kernel (attention-out / FFN2 + "
                      "residual + LayerNorm) and gemm_tc_kernel (FFN1 + GELU + requant)",
            "bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
            "peak_source": f"2 x {peaks['source']} bf16 GEMM burst ({peaks['bf16_tflops']} TFLOP/s): int8 issues at "
                           "twice the bf16 rate; nominal dense int8 is 4500 TOP/s",
            "frac_of_nominal": achieved / 4500.0,
            "traffic": None,
            "traffic_note": "DRAM bytes per launch come from profiler captures, which cannot run inside this program: see the "
                            "committed summaries of the GEMM launches (reads only, equal to the operand + residual bytes; "
                            "outputs are still in L2 when a kernel ends)",
            "algorithmic_bytes": g["algorithmic_bytes"], "algorithmic_bytes_unit": "bytes per layer (4 launches), from the shapes",
            "per_shape": g["per_shape"],
            "gemm_share_of_step": len(params["layers"]) * g["us_per_layer"] / (total_ms / K * 1e3),
            "duration": "average launch duration inside a CUDA graph of 12 back-to-back launches of the shape (one per "
                        "layer, 12 different weight matrices, L2 flushed before every replay), CUDA events; cold_us: one "
                        "launch alone after an L2 flush, launch latency included"}
        try:
            line["parity_check"] = parity_check(torch, enc, scales, params, ids_np, lens_np, dev)
        except Exception as exc:
            line["parity_check"] = {"status": f"failed to run: {exc}"}
        try:
            enc.set_inputs(torch.from_numpy(ids_np).to(dev), torch.from_numpy(lens_np).to(dev))
            line["unpadded"] = unpadded_metric(torch, cfg, params, scales, ids_np, lens_np, dev, flush, enc.replay().clone())
        except Exception as exc:
            line["unpadded"] = {"error": str(exc)}
        if not args.no_secondary:
            try:
                line["secondary"] = secondary_metrics(torch, ops, dev, flush, peaks, cfg, params)
            except Exception as exc:  # a secondary measurement must never take the headline down with it
                line["secondary"] = {"error": str(exc)}
        try:
            r = cpu_executor(8, 3, 1)
            line["cpu_baseline"] = {"value": r["seq_per_s"], "unit": "sequences/s", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"], "others": cpu_single_linear_baselines()}
        except Exception as exc:  # the CPU leg must never take the GPU numbers down with it
            line["cpu_baseline"] = {"value": None, "unit": "sequences/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": f"failed: {exc}"}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", choices=["bert_base", "bert_large"], default="bert_base",
                    help="bert_base: BASELINE.json configs[2] (the headline); bert_large: configs[4], global batch 256 x 384")
    ap.add_argument("--micro-batches", type=int, default=1,
                    help="cut each GPU's batch into this many concurrently running micro-batches")
    ap.add_argument("--gather", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how the hidden states reach rank 0 (copy-engine pushes, or an NCCL gather in the compute stream)")
    ap.add_argument("--sustain-seconds", type=float, default=3.0, help="length of the sustained leg (0 = skip it)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements (other configurations)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
