"""The device-side wait limit, exercised the permitted way: a wait that nothing will ever satisfy runs out
after its (1 ms) limit, the kernel returns by itself, the host reads ZEN_ERR_TIMEOUT from the device status
word and clears it.  Nothing faults, traps or hangs; the context keeps working afterwards."""
import pytest
import torch

from zenith_b200 import _capi, ops

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_cleared(cuda):
    assert _capi.device_status() == 0
    res = torch.zeros(3, dtype=torch.int64, device=cuda)
    _capi.call("zen_selftest_wait_limit", res.data_ptr(), torch.cuda.current_stream().cuda_stream)
    try:
        assert _capi.device_status() == _capi.ERR_TIMEOUT  # synchronises: the kernel has returned on its own
        gave_up, saw_abort, ns = res.tolist()
        assert gave_up == 1, "the wait on a barrier nobody signals must give up"
        assert saw_abort == 1, "a second waiter of the CTA must leave once the abort flag is up"
        assert 0.9e6 < ns < 0.5e9, f"the limit is 1 ms; the waits took {ns} ns"
        assert _capi.device_status() == _capi.ERR_TIMEOUT  # reading does not clear
    finally:
        assert _capi.device_status(clear=True) in (0, _capi.ERR_TIMEOUT)
    assert _capi.device_status() == 0
    # the context is intact: a real kernel runs and is correct
    x = torch.linspace(-3, 3, 1000, device=cuda)
    assert (ops.gelu(x) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max().item() < 1e-5
    assert _capi.device_status() == 0
