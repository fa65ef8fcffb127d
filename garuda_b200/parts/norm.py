"""RMS norm: ``x * 1/sqrt(mean(x^2) + eps) * weight``.

garuda/src/simd/mod.rs:166-173 (eps inside the root, added to the mean) and
garuda/src/llama/mod.rs:733-738 (scale, then a plain multiply by the weight).
The sum, the root and both multiplies are 32-bit in the kernel; only the result
is rounded to the compute dtype.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Norm, TensorSpec, register_norm


@register_norm("rms")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, weight_init=("ones",)):
        self.width = int(width)
        self.eps = float(eps)
        self.weight_init = tuple(weight_init)

    def tensors(self):
        return {"weight": TensorSpec((self.width,), role="vector", init=self.weight_init)}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.weight = tensors["weight"]

    def fold(self):
        """(weight in 32-bit, eps) for a product that folds this norm in, see
        ``CudaOps.linear``'s ``emit_norm``."""
        if getattr(self, "_weight32", None) is None:
            self._weight32 = self.weight.float().contiguous()
        return self._weight32, self.eps

    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                out_name: str = "normed") -> torch.Tensor:
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(out_name, (n, self.width), self.dtype)
        self.ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
