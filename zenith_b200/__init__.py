"""zenith_b200: B200 (sm_100a) kernels behind the ``zenith_cuda`` operator surface and the
quantization / QAT API of the reference's transformer-encoder inference path."""
from __future__ import annotations

import sys

__version__ = "0.1.0"


def install_as_zenith_cuda() -> None:
    """Make ``import zenith_cuda`` resolve to this package's drop-in module."""
    from . import zenith_cuda

    sys.modules["zenith_cuda"] = zenith_cuda
