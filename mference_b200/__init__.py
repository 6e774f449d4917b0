"""mference_b200 — a B200-native (sm_100a) implementation of Mference's MoE feed-forward path.

The product is the C ABI in include/mfb200.h (mference_b200/lib/libmfb200.so, built from csrc/); this package
is the host-side mirror of the reference's kernel-call surface used by the tests and the benchmark.
"""
from . import _lib
from ._lib import (ACT_GELU_TANH, ACT_SILU, DT_BF16, DT_F16, DT_F32, ROUTER_SOFTMAX_TOPK, ROUTER_SQRTSOFTPLUS,
                   MfbError)

__all__ = ["_lib", "MfbError", "DT_BF16", "DT_F16", "DT_F32", "ACT_SILU", "ACT_GELU_TANH", "ROUTER_SOFTMAX_TOPK",
           "ROUTER_SQRTSOFTPLUS"]
