"""Dense SwiGLU feed-forward: ``down(silu(gate h) * (up h))``, no bias.

garuda/src/llama/mod.rs:1002-1020 (``expert_batch``; the dense model is the one
expert that every token goes through, :914-921) and garuda/src/simd/mod.rs:161-163
(``silu(x) = x / (1 + exp(-x))``). Gate and up are one matrix product against
their rows stacked; the activation is computed in 32-bit from the 32-bit
accumulators and rounded once.
"""
from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, width: int, inner: int, init_std: float = 0.02):
        self.width, self.inner = int(width), int(inner)
        self.init_std = float(init_std)

    def tensors(self):
        init = ("normal", self.init_std)
        return {"gate_proj.weight": TensorSpec((self.inner, self.width), init=init),
                "up_proj.weight": TensorSpec((self.inner, self.width), init=init),
                "down_proj.weight": TensorSpec((self.width, self.inner), init=init)}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.w_gate_up = ops.pack_gate_up(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.w_down = tensors["down_proj.weight"].contiguous()

    # ``h`` may be a norm that is half done (``CudaOps.linear_swiglu`` takes it), and the last product
    # may fold in the first half of the norm that follows (``emit_norm``)
    takes_pending_norm = True
    emits_norm = True

    def forward(self, ctx, h, residual=None, emit_norm=None):
        T = h.shape[0]
        act = ctx.ws.get("ffn_act", (T, self.inner), self.dtype)
        self.ops.linear_swiglu(ctx, h, self.w_gate_up, act)
        if residual is not None:
            if emit_norm is None:
                self.ops.linear(act, self.w_down, residual, accumulate=True)
            else:
                ctx.pending_norm = self.ops.linear(act, self.w_down, residual, accumulate=True, ctx=ctx,
                                                   emit_norm=emit_norm)
            return None
        y = ctx.ws.get("ffn_out", (T, self.width), torch.float32)
        self.ops.linear(act, self.w_down, y)
        return y
