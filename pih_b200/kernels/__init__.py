"""The kernel pack: hand-written CUDA for sm_100a behind one ``ops`` object.

``get_ops(device)`` returns the object whose methods the parts call.  There
is no CPU path and no fallback: without a CUDA device, or if the library
cannot be built or loaded, it raises.
"""
from __future__ import annotations

_OPS = None


def get_ops(device=None):
    global _OPS
    if _OPS is None:
        from .ops import CudaOps
        _OPS = CudaOps(device)
    return _OPS


def set_ops_for_testing(ops) -> None:
    """Tests of host-side logic may install a stand-in; the product never does."""
    global _OPS
    _OPS = ops
