#!/usr/bin/env python
"""Benchmark of the W8A8 BERT-base encoder (batch 32 per GPU, seq 128) on N B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one forward pass of the encoder over one batch of 32 synthetic sequences per GPU
(BASELINE.json configs[2]: 12 layers, hidden 768, 12 heads, FFN 3072, post-LN, tanh-GELU, W8A8 with
per-channel weight scales and min-max activation scales from 16 seeded batches; token ids uniform
over 30522 words, the last 0..32 positions of each row masked).  Ranks are independent replicas
(weak scaling, global batch 32 * N); for N > 1 each step ends with the NCCL gather of the hidden
states onto rank 0.  Rank 0 prints ONE JSON line.

`value`      sequences/s with token ids already in HBM (CUDA-graph replay of the 61 launches).
`e2e`        the same through the public host API (zenith_b200.serve.HostPipeline) with HOST buffers: every
             step copies pinned ids / lengths to the device and the fp16 hidden states back to pinned host
             memory inside the timed region; the copy back of step i overlaps the compute of step i + 1.
`roofline`   the int8 tcgen05 GEMM family (4 shapes x 12 layers per step): average launch durations measured with
             CUDA events inside a graph of 12 launches per shape, as the step runs them.
`cpu_baseline` the CPU restatement of the reference's quantized executor (fake-quant + fp32 BLAS
             matmul), timed on this host's cores on a bounded sample.
`--impl reference` times that CPU executor alone, on the same workload definition.
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


def cpu_executor(sample_seqs: int, steps: int, warmup: int) -> dict:
    threads = blas_threads_all()
    from oracle import encoder_ref as ER
    from zenith_b200.calibrate import activation_scales_from_ranges, quantize_weights
    from zenith_b200.encoder import BERT_BASE, Int8Scales, init_params

    cfg = BERT_BASE
    params = init_params(cfg, MASTER_SEED)
    cal = [make_batch(MASTER_SEED + 1 + i, cfg.vocab, batch=2) for i in range(2)]  # scales do not affect timing
    scales = ER.calibrate_on_oracle(cfg, params, cal, quantize_weights, activation_scales_from_ranges, Int8Scales)
    ids, lens = make_batch(MASTER_SEED, cfg.vocab, batch=sample_seqs)
    for _ in range(warmup):
        ER.encoder_fake_quant(cfg, params, scales, ids, lens)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        ER.encoder_fake_quant(cfg, params, scales, ids, lens)
        times.append(time.perf_counter() - t0)
    total = sum(times)
    return {"seq_per_s": sample_seqs * steps / total, "ms_per_step": 1e3 * total / steps,
            "cores": threads, "sample": f"{steps} passes of {sample_seqs} sequences x {SEQ} tokens "
            f"(numpy fake-quant + fp32 BLAS matmul on {threads} BLAS threads of {os.cpu_count()} host cores)"}


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


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 4
    r = cpu_executor(sample, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["seq_per_s"], "unit": "sequences/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (fake-quantized int8 values)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step_sample": f"{sample} sequences per step"},
        "cpu_baseline": {"value": r["seq_per_s"], "unit": "sequences/s", "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["seq_per_s"], "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def time_gemm_shapes(torch, ops, dev, flush) -> dict:
    """The four int8 GEMM launches of one encoder layer with the epilogue each has in the encoder: QKV (-> fp16),
    attention-out (+ residual + LayerNorm, cluster kernel), FFN1 (+ GELU + requant), FFN2 (+ residual +
    LayerNorm), timed with CUDA events in two ways:

    * ``in_step``: as the step runs them - a CUDA graph of 12 back-to-back launches of the shape, one per layer,
      each with its own weight matrix, L2 flushed before every replay (so the weights come from HBM, as in the
      step); average launch duration = replay time / 12.  `roofline.achieved` uses these.
    * ``cold``: one launch alone, L2 flushed, launch latency included (the upper bound a profiler also sees).
    """
    T, H, F, LAYERS = BATCH * SEQ, 768, 3072, 12

    def plain(N, K, **kw):
        x = torch.randint(-128, 128, (T, K), dtype=torch.int8, device=dev)
        ws_ = [torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(LAYERS)]
        ws, b = torch.rand(N, device=dev) * 1e-3, torch.randn(N, device=dev)
        out = torch.empty((T, N), dtype=kw["out_dtype"], device=dev)
        return lambda i: ops.linear_int8(x, ws_[i], 0.02, ws, b, out=out, **kw)

    def with_ln(K):
        x = torch.randint(-128, 128, (T, K), dtype=torch.int8, device=dev)
        ws_ = [torch.randint(-128, 128, (H, K), dtype=torch.int8, device=dev) for _ in range(LAYERS)]
        ws, b = torch.rand(H, device=dev) * 1e-3, torch.randn(H, device=dev)
        res = torch.randn(T, H, device=dev, dtype=torch.float16)
        g, be = torch.ones(H, device=dev, dtype=torch.float16), torch.zeros(H, device=dev, dtype=torch.float16)
        return lambda i: ops.linear_int8_add_layernorm(x, ws_[i], 0.02, ws, b, res, g, be, 1e-12, out_scale=0.03)

    shapes = [("qkv", 3 * H, H, plain(3 * H, H, out_dtype=torch.float16)),
              ("attn_out_add_layernorm", H, H, with_ln(H)),
              ("ffn1_gelu_requant", F, H, plain(F, H, act="gelu", out_dtype=torch.int8, out_scale=0.05)),
              ("ffn2_add_layernorm", H, F, with_ln(F))]

    def event_us(fn, reps):
        us = []
        for _ in range(reps):
            flush()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            e.synchronize()
            us.append(s.elapsed_time(e) * 1e3)
        return statistics.median(us)

    per_shape, tot_ops, tot_us = {}, 0.0, 0.0
    for name, N, K, fn in shapes:
        def all_layers():
            for i in range(LAYERS):
                fn(i)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            all_layers()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            all_layers()
        for _ in range(3):
            graph.replay()
        in_step = event_us(graph.replay, 9) / LAYERS
        cold = event_us(lambda: fn(0), 9)
        ops_ = 2.0 * T * N * K
        per_shape[name] = {"us": round(in_step, 2), "tops": round(ops_ / in_step / 1e6, 1), "cold_us": round(cold, 2)}
        tot_ops += ops_
        tot_us += in_step
    return {"per_shape": per_shape, "ops_per_layer": tot_ops, "us_per_layer": tot_us}


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from zenith_b200 import _capi, ops
    from zenith_b200.calibrate import calibrate
    from zenith_b200.dist import OutputGatherer, init_from_env
    from zenith_b200.encoder import BERT_BASE, Int8Encoder, init_params
    from zenith_b200.serve import HostPipeline

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    rank, local_rank, world = init_from_env()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _capi.lib()
    cfg = BERT_BASE
    K, W = args.steps, max(3, args.warmup)

    params = init_params(cfg, MASTER_SEED)
    calib = [make_batch(MASTER_SEED + 1 + i, cfg.vocab) for i in range(CALIB_BATCHES)]
    scales = calibrate(cfg, params, [(torch.from_numpy(i).to(dev), torch.from_numpy(l).to(dev)) for i, l in calib], dev)
    enc = Int8Encoder(cfg, params, scales, dev, micro_batches=args.micro_batches)
    ids_np, lens_np = make_batch(MASTER_SEED + 1000 + rank, cfg.vocab)
    ids_h = torch.from_numpy(ids_np).pin_memory()
    lens_h = torch.from_numpy(lens_np).pin_memory()
    enc.capture(BATCH, SEQ)
    enc.set_inputs(ids_h.to(dev), lens_h.to(dev))
    gatherer = OutputGatherer(BATCH * world, SEQ, cfg.hidden, torch.float16, dev, root=0) if world > 1 else None

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

    # End to end through the public host API (zenith_b200.serve.HostPipeline): every step copies its ids /
    # lengths from pinned host memory and its hidden states back to pinned host memory; the device->host
    # copy of step i runs on a copy stream while step i + 1 computes, and the host waits for step i - 1's
    # result before it queues step i + 1 (the loop a server would run).
    pipe = HostPipeline(enc, BATCH, SEQ, gatherer=gatherer)

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
        pipe.drain()  # the last gathers are ordered before the end event
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
            ends[i].record()
        barrier()
        ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(W):
        step_device()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    launches0 = ops.launch_count
    total_ms = timed(step_device, K)
    launches = ops.launch_count - launches0
    timed_e2e(W)
    e2e_ms = timed_e2e(K)
    e2e_launches = enc.launches_per_forward + 1  # + the device copy that parks the result for the copy stream
    clocks = sampler.stop() if sampler else None
    status = _capi.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    value = world * BATCH * K / (total_ms / 1e3)
    e2e_value = world * BATCH * K / (e2e_ms / 1e3)
    peaks = measured_peaks()
    line = {
        "metric": METRIC, "value": value, "unit": "sequences/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8 operands, s32 accumulators (fp16 LayerNorm / softmax / residual)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": f"replicas x{world}" + (", NCCL gather of the hidden states onto rank 0 inside every step" if world > 1 else ""),
                   "l2": "256 MB buffer written between timed steps", "launch": f"CUDA-graph replay of {enc.launches_per_forward} kernels in {args.micro_batches} concurrent micro-batch(es)"},
        "e2e": {"value": e2e_value, "unit": "sequences/s", "ms_per_step": e2e_ms / K,
                "h2d_bytes_per_step": int(ids_h.numel() * ids_h.element_size() + lens_h.numel() * lens_h.element_size()),
                "d2h_bytes_per_step": int(pipe.host_out[0].numel() * 2),
                "how": "zenith_b200.serve.HostPipeline: one event pair around all steps; per step pinned-host ids -> device, "
                       "graph replay, hidden states -> pinned host on a copy stream that overlaps the next step's compute; "
                       "no L2 flush in this loop (a step's working set, 85 MB of weights + 60 MB of activations, exceeds "
                       "the 126 MB L2; flushing changed the device-resident step time by 0.3 %)",
                "launches_per_step": e2e_launches},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "device_status": status,
    }
    if world == 1:
        g = time_gemm_shapes(torch, ops, dev, flush)
        int8_peak = 2.0 * peaks["bf16_tflops"]
        achieved = g["ops_per_layer"] / g["us_per_layer"] / 1e6
        line["roofline"] = {
            "kernel": "int8 tcgen05 GEMM family of one layer: gemm_tc_kernel (QKV, FFN1+GELU+requant) and "
                      "gemm_i8_ln_kernel (attention-out / FFN2 + residual + LayerNorm)",
            "bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
            "peak_source": f"2 x {peaks['source']} bf16 GEMM burst ({peaks['bf16_tflops']} TFLOP/s): int8 issues at "
                           "twice the bf16 rate; nominal dense int8 is 4500 TOP/s",
            "frac_of_nominal": achieved / 4500.0,
            # DRAM bytes of the same four launches from profiles/gemm_i8_bert_base_layer_shapes.md (ncu): reads
            # only and equal to the operand (+ residual) bytes; the outputs are still in L2 when each kernel ends
            "traffic": 42.0e6, "traffic_unit": "bytes per layer (4 launches)",
            "algorithmic_bytes": 92.1e6, "per_shape": g["per_shape"],
            "gemm_share_of_step": 12.0 * g["us_per_layer"] / (total_ms / K * 1e3),
            "duration": "average launch duration inside a CUDA graph of 12 back-to-back launches of the shape (one per "
                        "layer, 12 different weight matrices, L2 flushed before every replay), CUDA events; cold_us: one "
                        "launch alone after an L2 flush, launch latency included"}
        try:
            r = cpu_executor(8, 3, 1)
            line["cpu_baseline"] = {"value": r["seq_per_s"], "unit": "sequences/s", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"]}
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
    ap.add_argument("--micro-batches", type=int, default=1,
                    help="cut each GPU's batch into this many concurrently running micro-batches")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
