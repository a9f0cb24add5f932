"""Registration into the REFERENCE's own kernel registry and dispatch through its own dispatcher
(zenith/runtime/kernel_registry.py:118-153, zenith/runtime/dispatcher.py:235-315).

Needs the reference tree: set the environment variable ``ZENITH_REFERENCE`` to its root (the directory that holds
the ``zenith`` package); without it these tests are skipped and tests/test_gpu_dropin.py covers the same contract
against a stand-in registry."""
import importlib
import inspect
import os
import sys

import pytest

REF = os.environ.get("ZENITH_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.isdir(os.path.join(REF or "", "zenith")),
                                reason="ZENITH_REFERENCE does not point at the reference tree")


@pytest.fixture(scope="module")
def ref():
    sys.dont_write_bytecode = True  # the reference tree may be read-only
    sys.path.insert(0, REF)
    try:
        kr = importlib.import_module("zenith.runtime.kernel_registry")
        disp = importlib.import_module("zenith.runtime.dispatcher")
        import zenith_b200.registry as plug

        plug = importlib.reload(plug)  # picks up the reference's KernelSpec / Precision types
        yield kr, disp, plug
    finally:
        sys.path.remove(REF)


OPS = {"Linear": 3, "MatMul": 2, "Gemm": 3, "Gelu": 1, "GELU": 1, "LayerNorm": 4, "LayerNormalization": 4, "Attention": 3,
       "MultiHeadAttention": 3, "FusedAddLayerNorm": 5, "FusedLinearGELU": 3, "FusedBiasGeLU": 2}


def test_specs_win_in_the_reference_registry(ref):
    kr, _, plug = ref
    assert plug.KernelSpec is kr.KernelSpec and plug.Precision is kr.Precision
    reg = kr.KernelRegistry()
    reg.initialize()  # the reference's own kernels first (PyTorch / numpy fallbacks on this host)
    before = {op: reg.get_kernel(op, kr.Precision.FP32) for op in OPS}
    n = plug.register(reg)
    assert n >= 13
    for op in OPS:
        for prec in (kr.Precision.FP32, kr.Precision.FP16):
            spec = reg.get_kernel(op, prec, [(32, 768)])
            assert spec is not None and spec.name.startswith("b200_") and spec.priority == plug.PRIORITY, (op, prec)
            assert spec.precision in (prec, kr.Precision.FP32)
        if before[op] is not None:
            assert before[op].priority < plug.PRIORITY
    assert reg.get_kernel("Linear", kr.Precision.INT8).name == "b200_linear_int8"
    assert reg.is_supported("FusedAddLayerNorm", kr.Precision.FP16)


def test_the_reference_dispatcher_calls_them_with_matching_signatures(ref):
    """KernelDispatcher._call_kernel builds the argument list per op type; every list must bind to the plug-in
    function's signature (the kernels themselves need a GPU, so the call is intercepted after binding)."""
    import dataclasses

    kr, disp, plug = ref
    reg = kr.KernelRegistry()
    plug.register(reg)
    d = disp.KernelDispatcher.__new__(disp.KernelDispatcher)  # _call_kernel uses no instance state
    x, w, b, g, r = "x", "w", "b", "gamma", "residual"
    cases = {"Linear": ([x], [w, b], {}), "MatMul": ([x, w], [], {}), "LayerNorm": ([x], [g, b], {"epsilon": 1e-12}),
             "Attention": (["q", "k", "v"], [], {}), "Gelu": ([x], [], {}), "FusedAddLayerNorm": ([x, r], [g, b], {"epsilon": 1e-12})}
    for op, (inputs, weights, attrs) in cases.items():
        spec = reg.get_kernel(op, kr.Precision.FP32)
        real = spec.kernel_fn
        got = {}

        def probe(*args, _real=real, _got=got):
            _got["bound"] = inspect.signature(_real).bind(*args)
            return "called"

        assert d._call_kernel(dataclasses.replace(spec, kernel_fn=probe), op, inputs, weights, attrs) == "called"
        assert len(got["bound"].args) == len(inputs) + len(weights) + (1 if "epsilon" in attrs else 0)
