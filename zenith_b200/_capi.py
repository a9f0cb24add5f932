"""ctypes binding of ``libzenith_b200.so`` (the C ABI declared in ``include/zenith_b200.h``).

There is no fallback: if the shared library is missing, ``lib()`` raises and every operator of
this package fails.  Build it with ``python -m zenith_b200.build``.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libzenith_b200.so"

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_TIMEOUT, ERR_DRIVER, ERR_TOO_LARGE = range(7)
DT_S32, DT_F32, DT_F16, DT_S8 = range(4)
ACT_NONE, ACT_GELU, ACT_RELU = range(3)
ROUND_NEAREST_EVEN, ROUND_TRUNC = range(2)
GEMM_CONST_WEIGHTS, GEMM_NO_PAIR, GEMM_PAIR = 0x1, 0x2, 0x4


def gemm_tile_n(bn: int) -> int:
    """``ZEN_GEMM_TILE_N(bn)``: the flag bits that force a GEMM tile width (0 = automatic)."""
    return int(bn) << 8

_p, _i, _f, _i64, _u = C.c_void_p, C.c_int, C.c_float, C.c_int64, C.c_uint

# name -> argument types; every function returns int unless listed in _RESTYPES
SIGNATURES = {
    "zen_version": [],
    "zen_status_string": [_i],
    "zen_device_status_read": [C.POINTER(C.c_int)],
    "zen_device_status_clear": [],
    "zen_selftest_wait_limit": [_p, _p],
    "zen_memcpy_async": [_p, _p, C.c_size_t, _p],
    "zen_linear_i8": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _i, _i, _f, _i, _p, _i64, _p],
    "zen_linear_i8_prefetch": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _i, _i, _f, _i, _p, _i64, _p, C.c_size_t, _p,
                               C.c_size_t, _p],
    "zen_linear_i8_ex": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _i, _i, _f, _i, _p, _i64, _p, C.c_size_t, _p, C.c_size_t,
                         _u, _p],
    "zen_linear_i8_add_layernorm_ex": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _p, _i64, _p, _p, _f, _p, _p, _f, _i, _u,
                                       _p],
    "zen_linear_f16_add_layernorm_ex": [_p, _i64, _p, _i64, _i, _i, _i, _p, _p, _i64, _p, _p, _f, _p, _p, _f, _i, _u, _p],
    "zen_linear_f16_ex": [_p, _i64, _p, _i64, _i, _i, _i, _p, _i, _i, _p, _i64, _u, _p],
    "zen_linear_i8_add_layernorm": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _p, _i64, _p, _p, _f, _p, _p, _f, _i, _p],
    "zen_linear_f16_add_layernorm": [_p, _i64, _p, _i64, _i, _i, _i, _p, _p, _i64, _p, _p, _f, _p, _p, _f, _i, _p],
    "zen_linear_f16": [_p, _i64, _p, _i64, _i, _i, _i, _p, _i, _i, _p, _i64, _p],
    "zen_linear_f32": [_p, _i64, _p, _i64, _i, _i, _i, _p, _i, _p, _i64, _p],
    "zen_wmma_matmul_f16": [_p, _p, _p, _i, _i, _i, _p],
    "zen_matmul_f32_workspace_bytes": [_i, _i],
    "zen_matmul_f32": [_p, _p, _p, _i, _i, _i, _p, C.c_size_t, _p],
    "zen_matmul_f32_static": [_p, _p, _p, _i, _i, _i, _p],
    "zen_gelu_f32": [_p, _p, _i64, _p],
    "zen_gelu_f16": [_p, _p, _i64, _p],
    "zen_relu_f32": [_p, _p, _i64, _p],
    "zen_tanh_f32": [_p, _p, _i64, _p],
    "zen_tanh_f16": [_p, _p, _i64, _p],
    "zen_bias_gelu_f32": [_p, _p, _p, _i, _i, _p],
    "zen_layernorm_f32": [_p, _p, _p, _p, _i, _i, _f, _p],
    "zen_layernorm_f16": [_p, _p, _p, _p, _i, _i, _f, _p],
    "zen_add_layernorm_f32": [_p, _p, _p, _p, _p, _i, _i, _f, _p],
    "zen_add_layernorm_f16": [_p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _f, _p],
    "zen_quantize_f32": [_p, _p, _i64, _f, _i, _i, _p],
    "zen_quantize_f16": [_p, _p, _i64, _f, _i, _i, _p],
    "zen_dequantize_f32": [_p, _p, _i64, _f, _i, _p],
    "zen_flash_attention_f16": [_p, _p, _p, _p, _p, _f, _i, _i, _i, _i] + [_i64] * 12 + [_p, _i, _f, _p],
    "zen_qkv_attention_i8": [_p, _i64, _p, _i64, _i, _i, _i, _i, _f, _p, _p, _p, _f, _p, _p, _f, _p, _p, C.c_size_t, _p,
                             C.c_size_t, _u, _p],
    "zen_convert_f32_to_f16": [_p, _p, _i64, _p],
    "zen_convert_f16_to_f32": [_p, _p, _i64, _p],
    "zen_minmax_workspace_bytes": [],
    "zen_minmax_f32": [_p, _i64, _p, _p, C.c_size_t, _p],
    "zen_minmax_f16": [_p, _i64, _p, _p, C.c_size_t, _p],
    "zen_histogram_f32": [_p, _i64, _p, _i, _p, _p],
    "zen_histogram_f16": [_p, _i64, _p, _i, _p, _p],
    "zen_absmax_rows_f32": [_p, _i, _i, _i64, _p, _p],
    "zen_quantize_rows_f32": [_p, _p, _i, _i, _i64, _p, _i64, _i, _p],
    "zen_embed_layernorm_f16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _f, _p],
    "zen_linear_f8": [_p, _i64, _p, _i64, _i, _i, _i, _f, _p, _p, _i, _i, _p, _i64, _u, _p],
    "zen_quantize_e4m3_f32": [_p, _p, _i64, _f, _p],
    "zen_quantize_e4m3_f16": [_p, _p, _i64, _f, _p],
    "zen_flash_attention_unpadded_f16": [_p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i64,
                                         _i64, _i64, _p, _i, _f, _p],
    "zen_pack_tokens_i32": [_p, _p, _p, _i, _i, _i, _p, _p, _p, _p, _p],
    "zen_embed_layernorm_unpadded_f16": [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _f, _i, _i, _i, _i, _i, _f, _p],
    "zen_qkv_attention_unpadded_i8": [_p, _i64, _p, _i64, _i, _i64, _p, _i, _i, _f, _p, _p, _f, _p, _p, _f, _p, _p,
                                      C.c_size_t, _p, C.c_size_t, _u, _p],
    "zen_unpad_rows_f16": [_p, _p, _i, _i, _i, _i, _p, _p],
}
_RESTYPES = {"zen_status_string": C.c_char_p, "zen_matmul_f32_workspace_bytes": C.c_size_t,
             "zen_minmax_workspace_bytes": C.c_size_t}

_lib = None


class ZenithError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed: status {status} ({text})")
        self.status = status


def lib() -> C.CDLL:
    """Load the shared library once and declare every prototype."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build the CUDA extension with `python -m zenith_b200.build` "
                "(there is no CPU or PyTorch fallback)"
            )
        handle = C.CDLL(str(LIB_PATH))
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().zen_status_string(status).decode()


def check(fn: str, status: int) -> None:
    if status != OK:
        raise ZenithError(fn, status, status_string(status))


def call(fn: str, *args) -> None:
    """Call ``fn`` and raise ``ZenithError`` on a non-zero status."""
    check(fn, getattr(lib(), fn)(*args))


def device_status(clear: bool = False) -> int:
    """Synchronise the device and return the device status word (0 or a ZEN_ERR_* code)."""
    out = C.c_int(0)
    check("zen_device_status_read", lib().zen_device_status_read(C.byref(out)))
    if clear and out.value != 0:
        check("zen_device_status_clear", lib().zen_device_status_clear())
    return out.value
