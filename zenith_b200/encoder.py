"""BERT-style post-LN encoder drivers over the sm_100a kernels: fp16 and W8A8 int8.

These play the role of the reference's hand-written encoder drivers
(benchmarks/bert_hybrid.py:96-145, benchmarks/bert_fp16_full.py:96-145): a fixed sequence of
kernel launches per layer, here 7 (int8) or 7 (fp16) launches instead of ~27, with every layout
change and elementwise op folded into a GEMM epilogue, the attention kernel or the LayerNorm
kernel.  All buffers of a (batch, seq) shape are allocated once; ``forward`` only launches, so a
whole pass can be captured in a CUDA graph (``capture`` / ``replay``).

W8A8 dataflow per layer (fp16 residual stream ``x``, int8 copies ``*_q``, one per-tensor
activation scale at each of the four GEMM inputs):

    x_q  --QKV GEMM s8 (dequant+bias -> fp16 [T,3H])--> q,k,v --attention (fp16, key-padding mask,
    int8 copy at s_ctx)--> ctx_q --out GEMM (dequant+bias -> fp16)--> +x, LayerNorm (fp16 + int8 copy
    at s_h1) --> h1_q --FFN1 GEMM (dequant+bias+GELU+requant at s_gelu)--> g_q --FFN2 GEMM (dequant+
    bias -> fp16)--> +h1, LayerNorm (fp16 + int8 copy at the next layer's s_x).

With hidden size 768 the two "GEMM, +residual, LayerNorm" pairs each run as ONE kernel
(``zen_linear_i8_add_layernorm``): 5 launches per layer.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from . import _capi, ops
from ._capi import ACT_GELU, ACT_NONE, DT_F16, DT_S8, GEMM_CONST_WEIGHTS, GEMM_NO_PAIR, GEMM_PAIR, ROUND_NEAREST_EVEN


@dataclass
class EncoderConfig:
    layers: int = 12
    hidden: int = 768
    heads: int = 12
    ffn: int = 3072
    vocab: int = 30522
    max_pos: int = 512
    type_vocab: int = 2
    eps: float = 1e-12

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


BERT_BASE = EncoderConfig()
BERT_LARGE = EncoderConfig(layers=24, hidden=1024, heads=16, ffn=4096)

LAYER_WEIGHTS = ("wqkv", "wo", "w1", "w2")
ACT_POINTS = ("x", "ctx", "h1", "gelu")


def init_params(cfg: EncoderConfig, seed: int = 1234, random_affine: bool = False) -> dict:
    """Random-init fp32 master weights: N(0, 0.02) matrices and embeddings, zero biases, unit
    LayerNorm — or, with ``random_affine``, small random biases and LayerNorm parameters."""
    rng = np.random.default_rng(seed)
    H, F = cfg.hidden, cfg.ffn

    def mat(*shape):
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)

    def bias(n):
        return (rng.standard_normal(n) * 0.02).astype(np.float32) if random_affine else np.zeros(n, np.float32)

    def gamma(n):
        return (1 + 0.1 * rng.standard_normal(n)).astype(np.float32) if random_affine else np.ones(n, np.float32)

    def beta(n):
        return (0.1 * rng.standard_normal(n)).astype(np.float32) if random_affine else np.zeros(n, np.float32)

    p = {"word": mat(cfg.vocab, H), "pos": mat(cfg.max_pos, H), "type": mat(cfg.type_vocab, H),
         "emb_ln_g": gamma(H), "emb_ln_b": beta(H), "layers": []}
    for _ in range(cfg.layers):
        p["layers"].append({
            "wqkv": mat(3 * H, H), "bqkv": bias(3 * H), "wo": mat(H, H), "bo": bias(H),
            "ln1_g": gamma(H), "ln1_b": beta(H), "w1": mat(F, H), "b1": bias(F), "w2": mat(H, F), "b2": bias(H),
            "ln2_g": gamma(H), "ln2_b": beta(H)})
    return p


def _row_ptr(t: torch.Tensor, row0: int) -> int:
    """Device address of row ``row0`` of a contiguous 1-D / 2-D tensor."""
    return t.data_ptr() + row0 * (t.stride(0) if t.dim() > 1 else 1) * t.element_size()


def _dev(a, dtype, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dtype)


class _EncoderBase:
    """Shared plumbing: embedding tables, per-shape buffers, the launch list, CUDA-graph capture."""


    def __init__(self, cfg: EncoderConfig, params: dict, device, micro_batches: int = 1, gemm_pair: bool | None = None):
        """``gemm_pair``: force the plain GEMMs onto the CTA-pair kernel (True) or the one-CTA kernel (False);
        None lets the library choose by shape."""
        self.gemm_flags = GEMM_CONST_WEIGHTS | (0 if gemm_pair is None else (GEMM_PAIR if gemm_pair else GEMM_NO_PAIR))
        if cfg.head_dim not in (64, 128):
            raise RuntimeError("head_dim must be 64 or 128")
        self.cfg = cfg
        self.micro_batches = max(1, int(micro_batches))
        self.device = torch.device(device)
        d = self.device
        self.word = _dev(params["word"], torch.float16, d)
        self.pos = _dev(params["pos"], torch.float16, d)
        self.type = _dev(params["type"], torch.float16, d)
        self.emb_g = _dev(params["emb_ln_g"], torch.float16, d)
        self.emb_b = _dev(params["emb_ln_b"], torch.float16, d)
        self._shape = None
        self._packed_rows = None  # row capacity of the packed (unpadded) form, None in the padded form
        self._launches: list = []
        self._graph = None
        self.launches_per_forward = 0

    # -- per-shape state --------------------------------------------------------------------
    def _prepare(self, B: int, S: int, packed_rows: int | None = None) -> None:
        if self._shape == (B, S, packed_rows):
            return
        if S > self.cfg.max_pos:
            raise RuntimeError("sequence longer than the position table")
        if packed_rows is not None:
            if self.micro_batches != 1:
                raise RuntimeError("unpadded batches need micro_batches == 1")
            if packed_rows <= 0 or packed_rows > B * S:
                raise RuntimeError("packed row capacity must lie in 1 .. B * S")
        self._shape = (B, S, packed_rows)
        self._packed_rows = packed_rows
        self._graph = None
        d = self.device
        # token ids and key lengths share one allocation, so that a host can feed both with one copy
        self.inputs = torch.zeros(B * S + B, dtype=torch.int32, device=d)
        self.ids = self.inputs[:B * S]
        self.kv_lens = self.inputs[B * S:]
        self.kv_lens.fill_(S)
        if packed_rows is not None:
            # offsets, then packed ids and positions: written by the first launch of every pass
            self.cu_seqlens = torch.zeros(B + 1, dtype=torch.int32, device=d)
            self.ids_packed = torch.zeros(packed_rows, dtype=torch.int32, device=d)
            self.pos_packed = torch.zeros(packed_rows, dtype=torch.int32, device=d)
        self._alloc(B, S)
        # Sequences are independent through the whole encoder, so the batch may be cut into micro-batches
        # whose launch sequences run side by side (separate streams / graph branches): the fill and
        # drain latency of one micro-batch's kernels then hides behind the other's work.  Every
        # micro-batch works on its own row range of the same buffers; results do not change.
        n = min(self.micro_batches, B)
        bounds = [(i * B // n, (i + 1) * B // n) for i in range(n)]
        self._micro = []
        for b0, b1 in bounds:
            self._launches = []
            self._build(b0, b1 - b0, S)
            self._micro.append(self._launches)
        self._launches = [l for m in self._micro for l in m]
        self.launches_per_forward = len(self._launches)
        self._streams = [torch.cuda.Stream(device=d) for _ in range(len(self._micro) - 1)]

    def _add(self, fn: str, *args) -> None:
        self._launches.append((getattr(_capi.lib(), fn), fn, args))

    @staticmethod
    def _issue(launches, stream) -> None:
        for f, name, args in launches:
            st = f(*args, stream)
            if st != 0:
                _capi.check(name, st)

    def _run(self) -> None:
        main = torch.cuda.current_stream()
        if len(self._micro) == 1:
            self._issue(self._micro[0], main.cuda_stream)
        else:
            for s in self._streams:
                s.wait_stream(main)
            self._issue(self._micro[0], main.cuda_stream)
            for s, launches in zip(self._streams, self._micro[1:]):
                with torch.cuda.stream(s):
                    self._issue(launches, s.cuda_stream)
            for s in self._streams:
                main.wait_stream(s)
        ops.launch_count += len(self._launches)

    # -- public ------------------------------------------------------------------------------
    def set_inputs(self, ids, kv_lens=None) -> None:
        """Copy token ids ([B,S] integer tensor, any device) and key lengths into the static buffers."""
        B, S = ids.shape
        same = self._shape is not None and self._shape[:2] == (B, S)
        self._prepare(B, S, self._packed_rows if same else None)
        self.ids.copy_(ids.reshape(-1), non_blocking=True)
        if kv_lens is not None:
            self.kv_lens.copy_(kv_lens, non_blocking=True)
        else:
            self.kv_lens.fill_(S)

    def set_inputs_packed(self, packed) -> None:
        """One copy for both inputs: ``packed`` is int32 ``[B*S + B]`` = token ids followed by key lengths, laid
        out like ``self.inputs`` (any device; a pinned host tensor makes the copy asynchronous)."""
        if self._shape is None or packed.numel() != self.inputs.numel() or packed.dtype != torch.int32:
            raise RuntimeError("packed inputs must be int32 [B*S + B] for the prepared shape")
        self.inputs.copy_(packed, non_blocking=True)

    def forward(self, ids, kv_lens=None) -> torch.Tensor:
        """Hidden states ``[B*S, hidden]`` fp16 (a static buffer, overwritten by the next call)."""
        self._prepare(*ids.shape, None)
        self.set_inputs(ids, kv_lens)
        self._run()
        return self.out

    # Unpadded form: the valid tokens of the batch are packed back to back (sequence b in rows cu_seqlens[b] ..),
    # the row-wise kernels and GEMMs run on ``capacity`` rows instead of B * S, attention takes its sequences
    # from the offsets, and the last launch spreads the rows back out (zeros at padding positions).  Every
    # valid token's result equals the padded pass's, bit for bit.
    @staticmethod
    def unpadded_capacity(kv_lens, S: int) -> int:
        """Rows needed for these key lengths (host values), rounded up to a whole 128-row tile."""
        total = int(sum(min(max(int(n), 0), S) for n in kv_lens))
        return max(128, -(-total // 128) * 128)

    def forward_unpadded(self, ids, kv_lens, capacity: int | None = None) -> torch.Tensor:
        """Padded-layout hidden states ``[B*S, hidden]`` fp16 computed on the packed rows (a static buffer);
        ``self.out`` holds the packed rows, ``self.cu_seqlens`` their offsets.  ``capacity`` defaults to what
        ``kv_lens`` needs (read on the host)."""
        B, S = ids.shape
        cap = min(B * S, self.unpadded_capacity(kv_lens.tolist(), S) if capacity is None else int(capacity))
        self._prepare(B, S, cap)
        self.set_inputs(ids, kv_lens)
        self._run()
        return self.out_padded

    def capture_unpadded(self, B: int, S: int, capacity: int, slots: int = 1) -> None:
        """``capture`` for the unpadded form with a fixed row capacity: batches whose valid tokens fit it replay the
        same graph (feed with ``set_inputs`` + ``replay``; the result is ``self.out_padded``)."""
        self._capture(B, S, min(B * S, int(capacity)), slots)

    def capture(self, B: int, S: int, slots: int = 1) -> None:
        """Capture one pass for shape (B, S) into a CUDA graph; feed it with ``set_inputs`` + ``replay``.
        ``slots`` > 1 captures that many graphs of the same pass, each with its own input block and its own result
        buffer (``inputs_of(k)``, ``result_of(k)``; slot 0 uses the object's own): a host loop can then fill the
        inputs of batch i + 1 and read the result of batch i - 1 while batch i computes, without a copy in
        between.  Intermediate buffers are shared: the graphs of one object run one after the other."""
        self._capture(B, S, None, slots)

    def _result(self) -> torch.Tensor:
        return self.out if self._packed_rows is None else self.out_padded

    def _capture(self, B: int, S: int, packed_rows, slots: int = 1) -> None:
        if slots < 1:
            raise ValueError("slots must be at least 1")
        self._prepare(B, S, packed_rows)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._run()  # warm-up: sets kernel attributes, loads modules
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        base_micro = self._micro
        res0 = self._result()
        self._slot_inputs = [self.inputs] + [torch.zeros_like(self.inputs) for _ in range(slots - 1)]
        self._slot_results = [res0] + [torch.empty_like(res0) for _ in range(slots - 1)]
        self._graphs = []
        for k in range(slots):
            if k:
                # the same launches with the slot's input block and result buffer in place of the object's own:
                # every pointer argument that falls inside one of the two is moved by the same offset
                spans = [(t0.data_ptr(), t0.numel() * t0.element_size(), t1.data_ptr())
                         for t0, t1 in ((self.inputs, self._slot_inputs[k]), (res0, self._slot_results[k]))]

                def move(a):
                    if isinstance(a, int) and not isinstance(a, bool):
                        for lo, n, new in spans:
                            if lo <= a < lo + n:
                                return a - lo + new
                    return a

                self._micro = [[(f, name, tuple(move(a) for a in args)) for f, name, args in m] for m in base_micro]
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._run()
            self._graphs.append(g)
        self._micro = base_micro
        self._graph = self._graphs[0]

    def inputs_of(self, slot: int) -> torch.Tensor:
        """int32 ``[B*S + B]`` input block of a captured slot: token ids, then key lengths."""
        return self._slot_inputs[slot]

    def result_of(self, slot: int) -> torch.Tensor:
        """Result buffer of a captured slot (written by ``replay(slot)``)."""
        return self._slot_results[slot]

    def replay(self, slot: int = 0) -> torch.Tensor:
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graphs[slot].replay()
        ops.launch_count += len(self._launches)
        return self._slot_results[slot]


class Fp16Encoder(_EncoderBase):
    """fp16 weights and activations, fp32 accumulation and statistics."""

    def __init__(self, cfg: EncoderConfig, params: dict, device="cuda:0", micro_batches: int = 1,
                 fuse_layernorm: bool | None = None, gemm_pair: bool | None = None):
        """``fuse_layernorm``: attention-output and FFN2 as one GEMM + residual + LayerNorm kernel each (5 launches
        per layer instead of 7); possible for hidden 768 and 1024, on by default for 768."""
        super().__init__(cfg, params, device, micro_batches, gemm_pair)
        self.fuse_layernorm = (cfg.hidden == 768) if fuse_layernorm is None else bool(fuse_layernorm)
        if self.fuse_layernorm and cfg.hidden not in (768, 1024):
            raise RuntimeError("the fused GEMM + LayerNorm kernel needs hidden == 768 or 1024")
        self.launches_per_layer = 5 if self.fuse_layernorm else 7
        d = self.device
        self.layers = []
        for lp in params["layers"]:
            L = {k: _dev(lp[k], torch.float16, d) for k in LAYER_WEIGHTS}
            L.update({k: _dev(lp[k], torch.float32, d) for k in ("bqkv", "bo", "b1", "b2")})
            L.update({k: _dev(lp[k], torch.float16, d) for k in ("ln1_g", "ln1_b", "ln2_g", "ln2_b")})
            self.layers.append(L)
        self.taps: dict | None = None  # filled by forward_with_taps

    def _alloc(self, B: int, S: int) -> None:
        cfg, d = self.cfg, self.device
        T, H, F = self._packed_rows or B * S, cfg.hidden, cfg.ffn
        f16 = dict(dtype=torch.float16, device=d)
        if self._packed_rows is not None:
            self.out_padded = torch.empty((B * S, H), **f16)
        self.x = [torch.empty((T, H), **f16) for _ in range(2)]
        self.qkv = torch.empty((T, 3 * H), **f16)
        self.ctx = torch.empty((T, H), **f16)
        self.ao = torch.empty((T, H), **f16)
        self.h1 = torch.empty((T, H), **f16)
        self.g = torch.empty((T, F), **f16)
        self.o = torch.empty((T, H), **f16)
        self.out = self.x[len(self.layers) & 1]

    def _build(self, b0: int, B: int, S: int) -> None:
        """Launch list for sequences [b0, b0 + B) of the batch (rows b0*S .. of every buffer)."""
        cfg = self.cfg
        packed = self._packed_rows is not None
        T, H, F, nh, hd = self._packed_rows or B * S, cfg.hidden, cfg.ffn, cfg.heads, cfg.head_dim
        r0 = b0 * S
        P = lambda t: _row_ptr(t, r0)
        # the weights of this object are written once, in __init__: every GEMM of the launch list carries the
        # constant-weights promise for its own call (nothing process-wide is switched)
        CW = GEMM_CONST_WEIGHTS
        GF = self.gemm_flags  # the plain GEMMs also carry the kernel choice
        self.lead_launches = 2 if packed else 1
        if packed:
            self._add("zen_pack_tokens_i32", self.ids.data_ptr(), None, self.kv_lens.data_ptr(), B, S, T,
                      self.cu_seqlens.data_ptr(), self.ids_packed.data_ptr(), self.pos_packed.data_ptr(), None)
            self._add("zen_embed_layernorm_unpadded_f16", self.ids_packed.data_ptr(), self.pos_packed.data_ptr(), None,
                      self.word.data_ptr(), self.pos.data_ptr(), self.type.data_ptr(), self.emb_g.data_ptr(),
                      self.emb_b.data_ptr(), P(self.x[0]), None, 1.0, ROUND_NEAREST_EVEN, T, cfg.max_pos, H, cfg.vocab, cfg.eps)
        else:
            self._add("zen_embed_layernorm_f16", P(self.ids), None, self.word.data_ptr(), self.pos.data_ptr(),
                      self.type.data_ptr(), self.emb_g.data_ptr(), self.emb_b.data_ptr(), P(self.x[0]), None, 1.0,
                      ROUND_NEAREST_EVEN, T, S, H, cfg.vocab, cfg.eps)
        qs = (S * 3 * H, hd, 3 * H)
        os_ = (S * H, hd, H)
        kv = self.kv_lens.data_ptr() + 4 * b0
        cur = 0
        for L in self.layers:
            x, xn = self.x[cur], self.x[cur ^ 1]
            self._add("zen_linear_f16_ex", P(x), H, L["wqkv"].data_ptr(), H, T, 3 * H, H, L["bqkv"].data_ptr(),
                      ACT_NONE, DT_F16, P(self.qkv), 3 * H, GF)
            if packed:
                self._add("zen_flash_attention_unpadded_f16", P(self.qkv), P(self.qkv) + 2 * H, P(self.qkv) + 4 * H,
                          P(self.ctx), None, 1.0, B, nh, S, hd, T, 3 * H, hd, 3 * H, hd, 3 * H, hd, H, hd,
                          self.cu_seqlens.data_ptr(), 0, 1.0 / math.sqrt(hd))
            else:
                self._add("zen_flash_attention_f16", P(self.qkv), P(self.qkv) + 2 * H, P(self.qkv) + 4 * H, P(self.ctx), None,
                          1.0, B, nh, S, hd, *qs, *qs, *qs, *os_, kv, 0, 1.0 / math.sqrt(hd))
            if self.fuse_layernorm:
                self._add("zen_linear_f16_add_layernorm_ex", P(self.ctx), H, L["wo"].data_ptr(), H, T, H, H,
                          L["bo"].data_ptr(), P(x), H, L["ln1_g"].data_ptr(), L["ln1_b"].data_ptr(), cfg.eps, P(self.h1),
                          None, 1.0, ROUND_NEAREST_EVEN, CW)
            else:
                self._add("zen_linear_f16_ex", P(self.ctx), H, L["wo"].data_ptr(), H, T, H, H, L["bo"].data_ptr(),
                          ACT_NONE, DT_F16, P(self.ao), H, GF)
                self._add("zen_add_layernorm_f16", P(self.ao), P(x), L["ln1_g"].data_ptr(), L["ln1_b"].data_ptr(),
                          P(self.h1), None, 1.0, ROUND_NEAREST_EVEN, T, H, cfg.eps)
            self._add("zen_linear_f16_ex", P(self.h1), H, L["w1"].data_ptr(), H, T, F, H, L["b1"].data_ptr(),
                      ACT_GELU, DT_F16, P(self.g), F, GF)
            if self.fuse_layernorm:
                self._add("zen_linear_f16_add_layernorm_ex", P(self.g), F, L["w2"].data_ptr(), F, T, H, F,
                          L["b2"].data_ptr(), P(self.h1), H, L["ln2_g"].data_ptr(), L["ln2_b"].data_ptr(), cfg.eps, P(xn),
                          None, 1.0, ROUND_NEAREST_EVEN, CW)
            else:
                self._add("zen_linear_f16_ex", P(self.g), F, L["w2"].data_ptr(), F, T, H, F, L["b2"].data_ptr(),
                          ACT_NONE, DT_F16, P(self.o), H, GF)
                self._add("zen_add_layernorm_f16", P(self.o), P(self.h1), L["ln2_g"].data_ptr(), L["ln2_b"].data_ptr(),
                          P(xn), None, 1.0, ROUND_NEAREST_EVEN, T, H, cfg.eps)
            cur ^= 1
        if packed:
            self._add("zen_unpad_rows_f16", self.x[cur].data_ptr(), self.cu_seqlens.data_ptr(), B, S, H, T,
                      self.out_padded.data_ptr())

    def forward_with_taps(self, ids, kv_lens=None, observers: dict | None = None) -> dict | None:
        """One pass that also observes, per layer, the range of the four tensors that feed a GEMM in the
        W8A8 dataflow: layer input ``x``, attention output ``ctx``, post-LN ``h1`` and GELU output ``gelu``.

        ``observers``: ``{point: [ops.RangeObserver per layer]}``; the ranges then accumulate on the device
        over any number of passes and nothing is read back here (returns None).  Without it the pass
        creates fresh observers and returns ``{point: [(min, max) per layer]}`` of this batch alone.
        Cold path used by calibration: runs layer by layer (padded form)."""
        self._prepare(*ids.shape, None)
        self.set_inputs(ids, kv_lens)
        if len(self._micro) != 1:
            raise RuntimeError("forward_with_taps needs micro_batches == 1")
        own = observers is None
        if own:
            observers = self.make_observers()
        stream = torch.cuda.current_stream().cuda_stream
        per_layer = self.launches_per_layer
        f, name, args = self._launches[0]
        _capi.check(name, f(*args, stream))
        cur = 0
        for li in range(len(self.layers)):
            observers["x"][li].observe(self.x[cur])
            for f, name, args in self._launches[1 + li * per_layer: 1 + (li + 1) * per_layer]:
                _capi.check(name, f(*args, stream))
            observers["ctx"][li].observe(self.ctx)
            observers["h1"][li].observe(self.h1)
            observers["gelu"][li].observe(self.g)
            cur ^= 1
        ops.launch_count += len(self._launches)
        if not own:
            return None
        return {p: [o.range() for o in v] for p, v in observers.items()}

    def make_observers(self, histogram: bool = False) -> dict:
        """``{point: [observer per layer]}`` for ``forward_with_taps``: running range only (``ops.RangeObserver``),
        or range + running histogram (``ops.HistogramObserver``) for the percentile / entropy calibrators."""
        make = ops.HistogramObserver if histogram else ops.RangeObserver
        return {p: [make(self.device) for _ in self.layers] for p in ACT_POINTS}


@dataclass
class Int8Scales:
    """Per-layer activation scales (one float per point) and the quantized weights."""

    act: list  # [{"x":..,"ctx":..,"h1":..,"gelu":..}] per layer
    weights: list  # [{"wqkv": (int8 [N,K], float32 [N]), ...}] per layer

    def save(self, path) -> None:
        """One ``.npz``: ``act`` float64 [layers, 4] in ``ACT_POINTS`` order, and per layer and weight the
        packed int8 matrix (``L{i}.{name}.q``) with its per-output-channel scales (``L{i}.{name}.s``)."""
        arrays = {"act": np.array([[a[p] for p in ACT_POINTS] for a in self.act], dtype=np.float64)}
        for li, layer in enumerate(self.weights):
            for name, (q, sc) in layer.items():
                arrays[f"L{li}.{name}.q"] = np.asarray(q, dtype=np.int8)
                arrays[f"L{li}.{name}.s"] = np.asarray(sc, dtype=np.float32)
        np.savez(path, **arrays)

    @classmethod
    def load(cls, path) -> "Int8Scales":
        with np.load(path) as z:
            act = [{p: float(v) for p, v in zip(ACT_POINTS, row)} for row in z["act"]]
            weights = []
            for li in range(len(act)):
                names = sorted({k.split(".")[1] for k in z.files if k.startswith(f"L{li}.")})
                weights.append({n: (z[f"L{li}.{n}.q"], z[f"L{li}.{n}.s"]) for n in names})
        return cls(act=act, weights=weights)


class Int8Encoder(_EncoderBase):
    """W8A8 encoder: int8 GEMM operands, int32 accumulation, fp16 residual stream / LayerNorm / softmax."""


    def __init__(self, cfg: EncoderConfig, params: dict, scales: Int8Scales, device="cuda:0", micro_batches: int = 1,
                 fuse_layernorm: bool | None = None, prefetch_weights: bool = True, gemm_pair: bool | None = None,
                 fuse_attention: bool | None = None, keep_qkv: bool = False):
        """``fuse_layernorm``: run attention-output and FFN2 as one GEMM + residual + LayerNorm kernel each
        (5 launches per layer instead of 7).  Possible for hidden 768 and 1024; on by default for 768 only (at
        BERT-large's 12k-token shards the separate kernels measured faster: 8.98 vs 10.26 ms per pass).  In the
        fused form the projection output is not rounded to fp16 before the residual add.
        ``fuse_attention``: QKV projection and attention as ONE kernel (``zen_qkv_attention_i8``), possible for
        sequences of at most 128 tokens with head size 64 and on by default there; same results bit for bit.
        ``keep_qkv``: the fused kernel also writes the fp16 projection to ``self.qkv`` (tests, inspection)."""
        super().__init__(cfg, params, device, micro_batches, gemm_pair)
        self.fuse_attention = fuse_attention
        self.keep_qkv = bool(keep_qkv)
        self.fuse_layernorm = (cfg.hidden == 768) if fuse_layernorm is None else bool(fuse_layernorm)
        if self.fuse_layernorm and cfg.hidden not in (768, 1024):
            raise RuntimeError("the fused GEMM + LayerNorm kernel needs hidden == 768 or 1024")
        self.launches_per_layer = 5 if self.fuse_layernorm else 7
        # The QKV GEMM hints the attention-output and FFN1 weights into L2 and the FFN1 GEMM the FFN2 and
        # next layer's QKV weights (zen_linear_i8_prefetch): a pass's weights do not stay in L2 beside
        # the activations, and a GEMM that starts on HBM-cold weights loses about a microsecond.
        self.prefetch_weights = bool(prefetch_weights)
        d = self.device
        self.act_scales = scales.act
        self.layers = []
        for lp, wq in zip(params["layers"], scales.weights):
            L = {}
            for k in LAYER_WEIGHTS:
                L[k] = _dev(wq[k][0], torch.int8, d)
                L[k + "_s"] = _dev(wq[k][1], torch.float32, d)
            L.update({k: _dev(lp[k], torch.float32, d) for k in ("bqkv", "bo", "b1", "b2")})
            L.update({k: _dev(lp[k], torch.float16, d) for k in ("ln1_g", "ln1_b", "ln2_g", "ln2_b")})
            self.layers.append(L)

    def _alloc(self, B: int, S: int) -> None:
        cfg, d = self.cfg, self.device
        T, H, F = self._packed_rows or B * S, cfg.hidden, cfg.ffn
        f16 = dict(dtype=torch.float16, device=d)
        s8 = dict(dtype=torch.int8, device=d)
        if self._packed_rows is not None:
            self.out_padded = torch.empty((B * S, H), **f16)
        self.x = [torch.empty((T, H), **f16) for _ in range(2)]
        self.xq = [torch.empty((T, H), **s8) for _ in range(2)]
        self.qkv = torch.empty((T, 3 * H), **f16)
        self.ctx = torch.empty((T, H), **f16)
        self.ctxq = torch.empty((T, H), **s8)
        self.ao = torch.empty((T, H), **f16)
        self.h1 = torch.empty((T, H), **f16)
        self.h1q = torch.empty((T, H), **s8)
        self.gq = torch.empty((T, F), **s8)
        self.o = torch.empty((T, H), **f16)
        self.out = self.x[len(self.layers) & 1]

    def _build(self, b0: int, B: int, S: int) -> None:
        """Launch list for sequences [b0, b0 + B) of the batch (rows b0*S .. of every buffer)."""
        cfg = self.cfg
        packed = self._packed_rows is not None
        T, H, F, nh, hd = self._packed_rows or B * S, cfg.hidden, cfg.ffn, cfg.heads, cfg.head_dim
        r0 = b0 * S
        P = lambda t: _row_ptr(t, r0)
        # the weights of this object are written once, in __init__: every GEMM of the launch list carries the
        # constant-weights promise for its own call (nothing process-wide is switched)
        CW = GEMM_CONST_WEIGHTS
        GF = self.gemm_flags  # the plain GEMMs also carry the kernel choice
        sc = self.act_scales
        can_fuse = S <= 128 and hd == 64
        if self.fuse_attention and not can_fuse:
            raise RuntimeError("the fused QKV + attention kernel needs seq <= 128 and head_dim == 64")
        fused_attn = can_fuse if self.fuse_attention is None else bool(self.fuse_attention)
        self.launches_per_layer = (5 if self.fuse_layernorm else 7) - (1 if fused_attn else 0)
        self.lead_launches = 2 if packed else 1
        if packed:
            self._add("zen_pack_tokens_i32", self.ids.data_ptr(), None, self.kv_lens.data_ptr(), B, S, T,
                      self.cu_seqlens.data_ptr(), self.ids_packed.data_ptr(), self.pos_packed.data_ptr(), None)
            self._add("zen_embed_layernorm_unpadded_f16", self.ids_packed.data_ptr(), self.pos_packed.data_ptr(), None,
                      self.word.data_ptr(), self.pos.data_ptr(), self.type.data_ptr(), self.emb_g.data_ptr(),
                      self.emb_b.data_ptr(), P(self.x[0]), P(self.xq[0]), sc[0]["x"], ROUND_NEAREST_EVEN, T, cfg.max_pos, H,
                      cfg.vocab, cfg.eps)
        else:
            self._add("zen_embed_layernorm_f16", P(self.ids), None, self.word.data_ptr(), self.pos.data_ptr(),
                      self.type.data_ptr(), self.emb_g.data_ptr(), self.emb_b.data_ptr(), P(self.x[0]), P(self.xq[0]),
                      sc[0]["x"], ROUND_NEAREST_EVEN, T, S, H, cfg.vocab, cfg.eps)
        qs = (S * 3 * H, hd, 3 * H)
        os_ = (S * H, hd, H)
        kv = self.kv_lens.data_ptr() + 4 * b0
        cur = 0
        n_layers = len(self.layers)
        for li, L in enumerate(self.layers):
            a = sc[li]
            x, xq, xn, xqn = self.x[cur], self.xq[cur], self.x[cur ^ 1], self.xq[cur ^ 1]
            last = li == n_layers - 1
            nbytes = lambda t: t.numel() * t.element_size()
            pf = lambda *ts: [v for t in ts for v in ((t.data_ptr(), nbytes(t)) if self.prefetch_weights and t is not None
                                                       else (None, 0))]
            if packed and not fused_attn:
                # longer sequences (or head size 128): projection, then attention on the packed rows from the offsets
                self._add("zen_linear_i8_ex", P(xq), H, L["wqkv"].data_ptr(), H, T, 3 * H, H, a["x"],
                          L["wqkv_s"].data_ptr(), L["bqkv"].data_ptr(), ACT_NONE, DT_F16, 1.0, ROUND_NEAREST_EVEN,
                          P(self.qkv), 3 * H, *pf(L["wo"], L["w1"]), GF)
                self._add("zen_flash_attention_unpadded_f16", P(self.qkv), P(self.qkv) + 2 * H, P(self.qkv) + 4 * H,
                          P(self.ctx), P(self.ctxq), a["ctx"], B, nh, S, hd, T, 3 * H, hd, 3 * H, hd, 3 * H, hd, H, hd,
                          self.cu_seqlens.data_ptr(), 0, 1.0 / math.sqrt(hd))
            elif packed:
                self._add("zen_qkv_attention_unpadded_i8", P(xq), H, L["wqkv"].data_ptr(), H, B, T,
                          self.cu_seqlens.data_ptr(), nh, H, a["x"], L["wqkv_s"].data_ptr(), L["bqkv"].data_ptr(),
                          1.0 / math.sqrt(hd), P(self.ctx), P(self.ctxq), a["ctx"], P(self.qkv) if self.keep_qkv else None,
                          *pf(L["wo"], L["w1"]), CW)
            elif fused_attn:
                self._add("zen_qkv_attention_i8", P(xq), H, L["wqkv"].data_ptr(), H, B, S, nh, H, a["x"],
                          L["wqkv_s"].data_ptr(), L["bqkv"].data_ptr(), kv, 1.0 / math.sqrt(hd), P(self.ctx), P(self.ctxq),
                          a["ctx"], P(self.qkv) if self.keep_qkv else None, *pf(L["wo"], L["w1"]), CW)
            else:
                self._add("zen_linear_i8_ex", P(xq), H, L["wqkv"].data_ptr(), H, T, 3 * H, H, a["x"],
                          L["wqkv_s"].data_ptr(), L["bqkv"].data_ptr(), ACT_NONE, DT_F16, 1.0, ROUND_NEAREST_EVEN,
                          P(self.qkv), 3 * H, *pf(L["wo"], L["w1"]), GF)
                self._add("zen_flash_attention_f16", P(self.qkv), P(self.qkv) + 2 * H, P(self.qkv) + 4 * H, P(self.ctx),
                          P(self.ctxq), a["ctx"], B, nh, S, hd, *qs, *qs, *qs, *os_, kv, 0, 1.0 / math.sqrt(hd))
            if self.fuse_layernorm:
                self._add("zen_linear_i8_add_layernorm_ex", P(self.ctxq), H, L["wo"].data_ptr(), H, T, H, H, a["ctx"],
                          L["wo_s"].data_ptr(), L["bo"].data_ptr(), P(x), H, L["ln1_g"].data_ptr(), L["ln1_b"].data_ptr(),
                          cfg.eps, P(self.h1), P(self.h1q), a["h1"], ROUND_NEAREST_EVEN, CW)
            else:
                self._add("zen_linear_i8_ex", P(self.ctxq), H, L["wo"].data_ptr(), H, T, H, H, a["ctx"],
                          L["wo_s"].data_ptr(), L["bo"].data_ptr(), ACT_NONE, DT_F16, 1.0, ROUND_NEAREST_EVEN,
                          P(self.ao), H, None, 0, None, 0, GF)
                self._add("zen_add_layernorm_f16", P(self.ao), P(x), L["ln1_g"].data_ptr(), L["ln1_b"].data_ptr(),
                          P(self.h1), P(self.h1q), a["h1"], ROUND_NEAREST_EVEN, T, H, cfg.eps)
            self._add("zen_linear_i8_ex", P(self.h1q), H, L["w1"].data_ptr(), H, T, F, H, a["h1"],
                      L["w1_s"].data_ptr(), L["b1"].data_ptr(), ACT_GELU, DT_S8, a["gelu"], ROUND_NEAREST_EVEN,
                      P(self.gq), F, *pf(L["w2"], None if last else self.layers[li + 1]["wqkv"]), GF)
            if self.fuse_layernorm:
                self._add("zen_linear_i8_add_layernorm_ex", P(self.gq), F, L["w2"].data_ptr(), F, T, H, F, a["gelu"],
                          L["w2_s"].data_ptr(), L["b2"].data_ptr(), P(self.h1), H, L["ln2_g"].data_ptr(),
                          L["ln2_b"].data_ptr(), cfg.eps, P(xn), None if last else P(xqn),
                          1.0 if last else sc[li + 1]["x"], ROUND_NEAREST_EVEN, CW)
            else:
                self._add("zen_linear_i8_ex", P(self.gq), F, L["w2"].data_ptr(), F, T, H, F, a["gelu"],
                          L["w2_s"].data_ptr(), L["b2"].data_ptr(), ACT_NONE, DT_F16, 1.0, ROUND_NEAREST_EVEN,
                          P(self.o), H, None, 0, None, 0, GF)
                self._add("zen_add_layernorm_f16", P(self.o), P(self.h1), L["ln2_g"].data_ptr(), L["ln2_b"].data_ptr(),
                          P(xn), None if last else P(xqn), 1.0 if last else sc[li + 1]["x"], ROUND_NEAREST_EVEN, T, H,
                          cfg.eps)
            cur ^= 1
        if packed:
            self._add("zen_unpad_rows_f16", self.x[cur].data_ptr(), self.cu_seqlens.data_ptr(), B, S, H, T,
                      self.out_padded.data_ptr())

    def forward_layerwise(self, ids, kv_lens=None):
        """Generator for tests: runs the pass one layer at a time and yields ``(layer, buffers)`` after
        each layer, where ``buffers`` are the live device tensors of that layer (inputs and outputs of
        every kernel), so that each kernel can be checked in isolation on the inputs it really saw."""
        self.set_inputs(ids, kv_lens)
        if len(self._micro) != 1:
            raise RuntimeError("forward_layerwise needs micro_batches == 1")
        stream = torch.cuda.current_stream().cuda_stream
        lead = self.lead_launches
        for f, name, args in self._launches[:lead]:
            _capi.check(name, f(*args, stream))
        cur = 0
        for li in range(len(self.layers)):
            n = self.launches_per_layer
            for f, name, args in self._launches[lead + li * n: lead + (li + 1) * n]:
                _capi.check(name, f(*args, stream))
            torch.cuda.synchronize()
            yield li, {"x": self.x[cur], "xq": self.xq[cur], "qkv": self.qkv, "ctx": self.ctx, "ctxq": self.ctxq,
                       "ao": self.ao, "h1": self.h1, "h1q": self.h1q, "gq": self.gq, "o": self.o,
                       "x_next": self.x[cur ^ 1], "xq_next": self.xq[cur ^ 1]}
            cur ^= 1
