"""turbopi_b200: B200 (sm_100a) kernels behind TurboPi's quantized Pi0.5 inference plugins.

Python is the host side only: packing, module wrappers and the ctypes binding of the
C-ABI library (include/turbopi_b200.h).  All arithmetic on the hot path runs in the
CUDA kernels; there is no CPU or PyTorch fallback.
"""
from . import _lib  # noqa: F401
from ._lib import TurboPiError  # noqa: F401

__version__ = "0.1.0"
