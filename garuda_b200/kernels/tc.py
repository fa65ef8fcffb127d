"""Tensor-core (tcgen05 / TMEM / TMA) kernels of the bfloat16 path.

Each method returns True when it ran, False when the shape is one it does not
take, in which case the caller uses the plain kernel instead.
"""
from __future__ import annotations


class TensorCoreKernels:
    def __init__(self, ops):
        self.ops = ops

    def linear(self, a, w, out, accumulate) -> bool:
        return False

    def linear_swiglu(self, h, w_gate_up, act) -> bool:
        return False

    def paged_attention(self, *args) -> bool:
        return False
