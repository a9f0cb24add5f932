"""zen_matmul_f32_static: the fp32 matmul for callers that cannot supply device memory.

Some users of this library cannot allocate: a plug-in invoked while a stream is being captured into a
CUDA graph must not call cudaMalloc, and a kernel called through a dispatcher that passes only inputs
and outputs has no channel for a workspace.  For them the library keeps the scratch (the transposed
right operand) in a fixed 4 MiB array of its own on each GPU.  This test calls that entry point through
the C ABI three times in a row, the largest shape first (the array is shared and still holds the earlier
calls' data, beyond the region a smaller call rewrites, during the later ones) and compares each result with the workspace-taking entry point, which must agree bit for bit.
The file name sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from zenith_b200 import _capi

pytestmark = pytest.mark.gpu


def _reference(lib, a, b, stream):
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N), dtype=torch.float32, device=a.device)
    nbytes = lib.zen_matmul_f32_workspace_bytes(N, K)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=a.device)
    assert lib.zen_matmul_f32(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ws.data_ptr(), nbytes, stream) == 0
    return c


def test_static_scratch_matmul_matches_workspace_matmul(cuda):
    lib = _capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cpu").manual_seed(5)
    # calls in a row on the shared array: a large shape, then a smaller one that rewrites only the head of
    # the scratch (stale data from the first call stays behind it), then a different one again
    for (M, N, K) in [(64, 1000, 512), (200, 328, 260), (96, 40, 24)]:
        a = torch.randn(M, K, generator=gen).to(cuda)
        b = (torch.randn(K, N, generator=gen) * 0.1).to(cuda)
        c = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
        st = lib.zen_matmul_f32_static(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, stream)
        assert st == 0, _capi.status_string(st)
        want = _reference(lib, a, b, stream)
        torch.cuda.synchronize()
        assert torch.equal(c, want)
        exact = a.double() @ b.double()
        assert ((c - exact).abs().max() / exact.abs().max()).item() < 1e-2  # TF32 tolerance used by the other tests
    assert _capi.device_status() == 0


def test_static_scratch_limits(cuda):
    lib = _capi.lib()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    assert lib.zen_matmul_f32_static(one, one, one, 16, 2048, 1024, None) == _capi.ERR_TOO_LARGE
    assert lib.zen_matmul_f32_static(one, one, one, 16, 16, 6, None) == _capi.ERR_UNSUPPORTED
    assert lib.zen_matmul_f32_static(None, one, one, 16, 16, 16, None) == _capi.ERR_INVALID_ARG
