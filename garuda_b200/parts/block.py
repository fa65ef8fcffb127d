"""How a mixer, a feed-forward and their norms are arranged in one layer.

``pre_norm`` is the reference's block (garuda/src/llama/mod.rs:851-893):
``x += mixer(norm1(x)); x += ffn(norm2(x))``, the residual stream ``x`` in
32-bit throughout. A part may add into the residual itself (fused into its
last matrix product); if it returns a tensor instead, the block adds it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

from .base import PartSpec, build_part, register_block


@dataclass(frozen=True)
class BlockSpec:
    """One layer as data: which parts, with which parameters and tensor prefixes."""
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: PartSpec
    feed_forward_norm: Optional[PartSpec]
    arrangement: str = "pre_norm"


@register_block("pre_norm")
class PreNormBlock:
    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.mixer = build_part("mixer", spec.mixer)
        self.mixer_norm = build_part("norm", spec.mixer_norm)
        self.feed_forward = build_part("feed_forward", spec.feed_forward) if spec.feed_forward else None
        self.feed_forward_norm = (build_part("norm", spec.feed_forward_norm)
                                  if spec.feed_forward_norm else None)

    def parts(self):
        """(part, tensor-name prefix) pairs, for the loader."""
        s = self.spec
        out = [(self.mixer_norm, s.mixer_norm.prefix), (self.mixer, s.mixer.prefix)]
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, s.feed_forward_norm.prefix),
                    (self.feed_forward, s.feed_forward.prefix)]
        return out

    def forward(self, ctx, x, cache):
        ops = ctx.ops
        h = self.mixer_norm.forward(ctx, x)
        y = self.mixer.forward(ctx, h, cache, residual=x)
        if y is not None:
            ops.residual_add(x, y)
        if self.feed_forward is not None:
            h2 = self.feed_forward_norm.forward(ctx, x)
            y2 = self.feed_forward.forward(ctx, h2, residual=x)
            if y2 is not None:
                ops.residual_add(x, y2)
        return x
