"""numpy front-end of the CPU oracle — TEST INFRASTRUCTURE, NOT PRODUCT.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs may import this
module.  The arithmetic lives in ``oracle/zen_oracle.c`` (built by ``oracle/build.py``); every
function there cites the reference lines it restates.  Parity status: the quantization / QAT
arithmetic is pinned against the reference's own Python implementation and known-answer tests
(``tests/golden``); int32 GEMM, requantisation, masked / causal attention and the int8 encoder
dataflow have no test or golden vector in the reference ("parity unpinned" there) and are defined
by this restatement.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_SO = HERE / "_build" / "libzen_oracle.so"
_REF_SO = HERE / "_ref" / "libzenith_ref_cpu.so"

ACT = {"none": 0, None: 0, "gelu": 1, "relu": 2}
ROUND = {"nearest_even": 0, "trunc": 1}

_lib = None
_ref = None


def _load():
    global _lib
    if _lib is None:
        if not _SO.exists():
            import importlib.util

            spec = importlib.util.spec_from_file_location("_oracle_build", HERE / "build.py")
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        _lib = C.CDLL(str(_SO))
    return _lib


def ref_lib():
    """The reference's own CPU kernels (oracle/_ref), or None when they were not built."""
    global _ref
    if _ref is None and _REF_SO.exists():
        _ref = C.CDLL(str(_REF_SO))
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def gemm_s8(xq, wq):
    """int32 ``xq[M,K] @ wq[N,K].T`` (core/src/cuda_kernels.cu:963-978)."""
    xq, wq = _c(xq, np.int8), _c(wq, np.int8)
    M, K = xq.shape
    N = wq.shape[0]
    acc = np.empty((M, N), np.int32)
    _load().orc_gemm_s8s8_s32(_p(xq), _p(wq), _p(acc), M, N, K)
    return acc


def epilogue(acc, x_scale, w_scale=None, bias=None, act="none"):
    """fp32 ``act((acc * x_scale) * w_scale[n] + bias[n])`` (core/src/cuda_kernels.cu:1035-1036)."""
    acc = _c(acc, np.int32)
    M, N = acc.shape
    ws = _c(w_scale, np.float32) if w_scale is not None else None
    b = _c(bias, np.float32) if bias is not None else None
    y = np.empty((M, N), np.float32)
    _load().orc_epilogue_f32(_p(acc), _p(y), M, N, C.c_float(x_scale), _p(ws), _p(b), ACT[act])
    return y


def quantize(x, scale, zero_point=0, round="nearest_even"):
    """``clamp(round(x / scale + zp))`` as int8 (core/src/cuda_kernels.cu:918-929)."""
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.int8)
    _load().orc_quantize_f32(_p(x), _p(q), C.c_size_t(x.size), C.c_float(scale), int(zero_point), ROUND[round])
    return q


def dequantize(q, scale, zero_point=0):
    q = _c(q, np.int8)
    x = np.empty(q.shape, np.float32)
    _load().orc_dequantize_f32(_p(q), _p(x), C.c_size_t(q.size), C.c_float(scale), int(zero_point))
    return x


def linear_int8(xq, wq, x_scale, w_scale=None, bias=None, act="none", out_dtype="f32", out_scale=None,
                round="nearest_even"):
    """The pinned W8A8 Linear: int32 GEMM, fp32 epilogue, then s32 / f32 / f16 / requantised s8 output."""
    acc = gemm_s8(xq, wq)
    if out_dtype == "s32":
        return acc
    y = epilogue(acc, x_scale, w_scale, bias, act)
    if out_dtype == "f32":
        return y
    if out_dtype == "f16":
        return y.astype(np.float16)
    if out_dtype == "s8":
        return quantize(y, out_scale, 0, round)
    raise ValueError(out_dtype)


def gelu(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _load().orc_gelu_f32(_p(x), _p(y), C.c_size_t(x.size))
    return y


def gelu_libm(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    _load().orc_gelu_libm_f32(_p(x), _p(y), C.c_size_t(x.size))
    return y


def tanh(x, libm=False):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    (_load().orc_tanh_libm_f32 if libm else _load().orc_tanh_f32)(_p(x), _p(y), C.c_size_t(x.size))
    return y


def add_layernorm(x, residual, gamma, beta, eps=1e-5):
    """Two-pass fp32 ``LayerNorm(x + residual)`` (python/src/features_bindings.hpp:116-171)."""
    x = _c(x, np.float32)
    r = _c(residual, np.float32) if residual is not None else None
    g, b = _c(gamma, np.float32), _c(beta, np.float32)
    rows, hidden = x.shape
    y = np.empty_like(x)
    _load().orc_add_layernorm_f32(_p(x), _p(r), _p(g), _p(b), _p(y), rows, hidden, C.c_float(eps))
    return y


def layernorm(x, gamma, beta, eps=1e-5):
    return add_layernorm(x, None, gamma, beta, eps)


def attention(q, k, v, kv_lens=None, causal=False, scale=None):
    """fp32 attention over [B,H,S,D] with key-padding / causal masks (core/src/flash_attention.cu:194-321)."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    B, H, S, D = q.shape
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    kl = _c(kv_lens, np.int32) if kv_lens is not None else None
    o = np.empty_like(q)
    _load().orc_attention_f32(_p(q), _p(k), _p(v), _p(o), B, H, S, D, _p(kl), 1 if causal else 0, C.c_float(scale))
    return o


def attention_rows(q, k, v, rows, kv_lens=None, causal=False, scale=None):
    """Rows ``rows`` (query indices) of ``attention(q, k, v, ...)``: ``[B, H, len(rows), D]``."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    B, H, S, D = q.shape
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    kl = _c(kv_lens, np.int32) if kv_lens is not None else None
    rows = _c(rows, np.int32)
    o = np.empty((B, H, rows.size, D), np.float32)
    _load().orc_attention_rows_f32(_p(q), _p(k), _p(v), _p(o), B, H, S, D, _p(kl), 1 if causal else 0, C.c_float(scale),
                                   _p(rows), int(rows.size))
    return o


def gemm_f32_nt(a, w):
    """``a[M,K] @ w[N,K].T`` with double accumulation."""
    a, w = _c(a, np.float32), _c(w, np.float32)
    M, K = a.shape
    N = w.shape[0]
    c = np.empty((M, N), np.float32)
    _load().orc_gemm_f32_nt(_p(a), _p(w), _p(c), M, N, K)
    return c


def ref_matmul_avx2(a, b):
    """The reference's own AVX2 fp32 GEMM, ``a[M,K] @ b[K,N]`` (core/src/cpu_kernels.cpp:129-165)."""
    lib = ref_lib()
    if lib is None:
        raise RuntimeError("oracle/_ref was not built")
    a, b = _c(a, np.float32), _c(b, np.float32)
    M, K = a.shape
    N = b.shape[1]
    c = np.empty((M, N), np.float32)
    lib.ref_matmul_f32_avx2(_p(a), _p(b), _p(c), M, N, K)
    return c


# ---------------------------------------------------------------------------------------------
# FP8 e4m3 (the OCP 8-bit format: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinities, 0x7f / 0xff are NaN,
# largest finite value 448).  The reference has no FP8 kernel (docs/SPEEDUP_ROADMAP.md:201-210 sketches one), so this
# is the format's published definition restated: "parity unpinned" for this operator.
# ---------------------------------------------------------------------------------------------
def _e4m3_table():
    codes = np.arange(128, dtype=np.int64)
    e, m = codes >> 3, codes & 7
    v = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * 2.0 ** (e - 7.0))
    v[127] = np.nan
    return v


_E4M3 = _e4m3_table()


def e4m3_decode(bits):
    """float32 values of e4m3 bit patterns (uint8)."""
    b = np.asarray(bits, np.uint8)
    v = _E4M3[b & 0x7f]
    return np.where(b & 0x80, -v, v).astype(np.float32)


def e4m3_encode(x):
    """e4m3 bit patterns of float32 values: round to nearest, ties to the even code, saturating at +-448."""
    x = np.asarray(x, np.float32)
    a = np.minimum(np.abs(x.astype(np.float64)), 448.0)
    grid = _E4M3[:127]
    hi = np.clip(np.searchsorted(grid, a, side="left"), 0, 126)
    lo = np.maximum(hi - 1, 0)
    d_lo, d_hi = a - grid[lo], grid[hi] - a
    code = np.where(d_lo < d_hi, lo, np.where(d_hi < d_lo, hi, np.where(lo % 2 == 0, lo, hi)))
    code = np.where(grid[hi] == a, hi, code)
    code = np.where(np.isnan(x), 127, code).astype(np.uint8)
    return (code | np.where(np.signbit(x), 0x80, 0).astype(np.uint8)).astype(np.uint8)


def quantize_e4m3(x, scale):
    """e4m3(x / scale) with the division in float32."""
    return e4m3_encode(np.asarray(x, np.float32) / np.float32(scale))


def linear_fp8(xq, wq, x_scale, w_scale=None, bias=None, act="none"):
    """``act((xq . wq^T) * x_scale * w_scale + bias)`` for e4m3 operands, products summed in float64 (exact for any
    K of interest), scaled in float32 in the order of the int8 epilogue."""
    acc = (e4m3_decode(xq).astype(np.float64) @ e4m3_decode(wq).astype(np.float64).T).astype(np.float32)
    y = acc * np.float32(x_scale)
    if w_scale is not None:
        y = y * np.asarray(w_scale, np.float32)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, np.float32)[None, :]
    if act == "gelu":
        y = gelu(y)
    elif act == "relu":
        y = np.maximum(y, 0)
    return y.astype(np.float32)
