"""B200-native fused per-token layer kernels: RMSNorm with optional residual add, per-head q/k norm + NeoX RoPE,
SwiGLU and Q8_0 / Q4_0 token-embedding gather, behind the C launcher surface of the reference engine's gpu_ops.h.

The product is the C-ABI shared library ``libb200_layer_ops.so`` (include/b200_layer_ops.h). ``ops`` mirrors its
launchers for callers that hold torch tensors; torch only provides device memory and streams.
"""
from . import _lib  # noqa: F401
from .ops import *  # noqa: F401,F403
