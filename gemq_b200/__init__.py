"""gemq_b200: B200 (sm_100a) kernels and MoE blocks for GEMQ's real-quantized inference path.

``gemq_b200.kernels`` and ``gemq_b200.inference`` load ``libgemq_b200.so`` on import and raise
when it is missing or stale; there is no Triton or CPU fallback.  The package itself stays
importable without the library so that ``python -m gemq_b200.csrc.build`` can (re)build it.
"""
__version__ = "0.1"
