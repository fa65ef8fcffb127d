"""How a mixer, a feed-forward and their norms are arranged in one layer.

``pre_norm`` is the reference's block (garuda/src/llama/mod.rs:851-893):
``x += mixer(norm1(x)); x += ffn(norm2(x))``, the residual stream ``x`` in
32-bit throughout. A part may add into the residual itself (fused into its
last matrix product); if it returns a tensor instead, the block adds it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

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

    def takes_pending_norm(self, ops):
        """The norm part that the layer in front may fold into its last product (see
        ``forward``'s ``pending``), or None."""
        if getattr(ops, "folds_norms", False) and getattr(self.mixer, "takes_pending_norm", False) \
                and hasattr(self.mixer_norm, "fold"):
            return self.mixer_norm
        return None

    @property
    def graph_safe(self):
        return all(part.graph_safe for part, _ in self.parts())

    @staticmethod
    def _take_pending(ctx, x, added_in_place):
        """The one place where a folded norm changes hands: what the part that just ran left in
        ``ctx.pending_norm`` is taken out (the field is empty afterwards) and checked to be the
        norm of this block's residual stream. A part that returned its output instead of adding
        it in cannot have folded a norm of the sum; whatever it left is dropped."""
        p, ctx.pending_norm = ctx.pending_norm, None
        if p is None or not added_in_place:
            return None
        if p.x.data_ptr() != x.data_ptr() or tuple(p.x.shape) != tuple(x.shape):
            raise RuntimeError("a folded norm was left behind that is not of this block's residual stream")
        return p

    def forward(self, ctx, x, cache, pending=None, next_norm=None):
        """``pending``: this layer's first norm of ``x``, already half done by the layer in
        front (a ``PendingNorm``). ``next_norm``: the norm part that the next layer starts with,
        if that layer takes such a result. Returns the pending norm for the next layer, or None.
        Parts that know nothing of this are run with the plain norms."""
        ops = ctx.ops
        folds = getattr(ops, "folds_norms", False)
        h = pending if pending is not None else self.mixer_norm.forward(ctx, x)
        ff = self.feed_forward
        kw = {}
        if (folds and ff is not None and getattr(self.mixer, "emits_norm", False)
                and getattr(ff, "takes_pending_norm", False) and hasattr(self.feed_forward_norm, "fold")):
            kw["emit_norm"] = self.feed_forward_norm
        elif folds and ff is None and next_norm is not None and getattr(self.mixer, "emits_norm", False):
            kw["emit_norm"] = next_norm
        ctx.pending_norm = None
        y = self.mixer.forward(ctx, h, cache, residual=x, **kw)
        if y is not None:
            ops.residual_add(x, y)
        out = self._take_pending(ctx, x, y is None and "emit_norm" in kw)
        if ff is None:
            return out
        h2 = out if out is not None else self.feed_forward_norm.forward(ctx, x)
        kw = {}
        if folds and next_norm is not None and getattr(ff, "emits_norm", False):
            kw["emit_norm"] = next_norm
        y2 = ff.forward(ctx, h2, residual=x, **kw)
        if y2 is not None:
            ops.residual_add(x, y2)
        return self._take_pending(ctx, x, y2 is None and "emit_norm" in kw)
