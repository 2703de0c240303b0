"""gemq_b200: B200 (sm_100a) kernels and MoE blocks for GEMQ's real-quantized inference path.

Importing the package loads ``libgemq_b200.so``; there is no Triton or CPU fallback.
"""
from . import _capi  # noqa: F401  (fails loudly when the library is not built)

__version__ = "0.1"
