"""Rotary position encoding.

garuda/src/simd/mod.rs:196-206: for ``i < head_dim/2`` the pair is rotated by
``pos * theta^(-2i/head_dim)``, frequency, angle, sine and cosine in 32-bit. The
reference pairs ``(2i, 2i+1)`` because GGUF Llama files carry permuted Q/K rows;
a safetensors folder keeps the original rows, for which the same rotation pairs
``(i, i + head_dim/2)``. ``layout`` names the pairing. It is applied to every
query and key head before the key is stored (garuda/src/llama/mod.rs:784-791),
which is why the engine's kernel rotates and stores in one pass.
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import PositionEncoding, register_position_encoding


@dataclass(frozen=True)
class RotaryParams:
    theta: float
    head_dim: int
    interleaved: bool


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    def __init__(self, theta: float, head_dim: int, layout: str = "half"):
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout must be 'half' or 'interleaved', got {layout!r}")
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {head_dim}")
        self.rotary = RotaryParams(float(theta), int(head_dim), layout == "interleaved")

    def apply(self, ctx, q, k, positions):
        r = self.rotary
        self.ops.rope_inplace(q, positions, r.theta, r.interleaved)
        if k is not None:
            self.ops.rope_inplace(k, positions, r.theta, r.interleaved)


@register_position_encoding("none")
class NoPositions(PositionEncoding):
    """Leaves queries and keys as they are."""
    changes_vectors = False

    def __init__(self):
        pass

    def apply(self, ctx, q, k, positions):
        return None
