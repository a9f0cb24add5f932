"""The C-ABI library loads without a GPU, exports every symbol the header declares, and validates
its arguments before touching the device."""
import ctypes
import re
from pathlib import Path

import pytest

from zenith_b200 import _capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "zenith_b200.h").read_text()


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(zen_[a-z0-9_]+)\s*\(", body)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _capi.lib()
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/zenith_b200.h but not exported"
        assert n in _capi.SIGNATURES, f"{n} has no ctypes prototype"
    assert set(_capi.SIGNATURES) <= set(names)


def test_version_and_status_strings():
    assert _capi.lib().zen_version() == 100
    assert _capi.status_string(0) == "ok"
    for s in range(1, 7):
        assert _capi.status_string(s) not in ("ok", "unknown status")
    assert _capi.status_string(99) == "unknown status"


def test_argument_validation_needs_no_device():
    lib = _capi.lib()
    z = None
    assert lib.zen_linear_i8(z, 16, z, 16, 1, 1, 16, 1.0, z, z, 0, 0, 1.0, 0, z, 1, z) == _capi.ERR_INVALID_ARG
    one = ctypes.c_void_p(16)  # never dereferenced: rejected before any launch
    assert lib.zen_linear_i8(one, 24, one, 24, 4, 4, 24, 1.0, z, z, 0, 0, 1.0, 0, one, 4, z) == _capi.ERR_UNSUPPORTED
    assert lib.zen_linear_i8(one, 16, one, 16, 4, 4, 16, 1.0, z, z, 9, 0, 1.0, 0, one, 4, z) == _capi.ERR_INVALID_ARG
    assert lib.zen_linear_i8(one, 16, one, 16, 4, 4, 16, 1.0, z, z, 0, 3, 0.0, 0, one, 4, z) == _capi.ERR_INVALID_ARG
    assert lib.zen_linear_f16(one, 12, one, 12, 4, 4, 12, z, 0, 2, one, 4, z) == _capi.ERR_UNSUPPORTED
    assert lib.zen_wmma_matmul_f16(one, one, one, 16, 12, 16, z) == _capi.ERR_UNSUPPORTED
    assert lib.zen_flash_attention_f16(one, one, one, one, z, 1.0, 1, 1, 8, 32, *([8] * 12), z, 0, 1.0, z) == _capi.ERR_UNSUPPORTED
    assert lib.zen_quantize_f32(one, one, 4, 0.0, 0, 0, z) == _capi.ERR_INVALID_ARG
    assert lib.zen_layernorm_f32(z, z, z, z, 4, 8, 1e-5, z) == _capi.ERR_INVALID_ARG
    # per-call options: an unknown flag bit or tile width is rejected
    ex = lambda flags: lib.zen_linear_i8_ex(one, 16, one, 16, 4, 4, 16, 1.0, z, z, 0, 0, 1.0, 0, one, 4, z, 0, z, 0, flags, z)
    assert ex(0x80) == _capi.ERR_INVALID_ARG and ex(_capi.gemm_tile_n(100)) == _capi.ERR_INVALID_ARG
    assert ex(_capi.GEMM_PAIR | _capi.GEMM_NO_PAIR) == _capi.ERR_INVALID_ARG
    # zero-sized work is a no-op, not an error
    assert lib.zen_gelu_f32(z, z, 0, z) == 0 and lib.zen_layernorm_f16(z, z, z, z, 0, 8, 1e-5, z) == 0


def test_operators_refuse_cpu_tensors():
    import torch

    from zenith_b200 import zenith_cuda

    x = torch.zeros(4, 8)
    for call in (lambda: zenith_cuda.gelu(x), lambda: zenith_cuda.relu(x), lambda: zenith_cuda.layernorm(x, x[0], x[0]),
                 lambda: zenith_cuda.matmul(x, x.T), lambda: zenith_cuda.wmma_matmul(x.half(), x.T.half()),
                 lambda: zenith_cuda.flash_attention(x[None, None], x[None, None], x[None, None])):
        with pytest.raises(RuntimeError):
            call()


def test_missing_extension_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _capi.lib()
