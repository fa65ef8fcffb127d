"""Rotary position encoding.

garuda/src/simd/mod.rs:196-206: for ``i < head_dim/2`` the pair is rotated by
``pos * theta^(-2i/head_dim)``, frequency, angle, sine and cosine in 32-bit. The
reference pairs ``(2i, 2i+1)`` because GGUF Llama files carry permuted Q/K rows;
a safetensors folder keeps the original rows, for which the same rotation pairs
``(i, i + head_dim/2)``. ``layout`` names the pairing. It is applied to every
query and key head before the key is stored (garuda/src/llama/mod.rs:784-791),
which is why the engine's kernel rotates and stores in one pass.

The reference rotates the whole head at the frequencies above and nothing else.
The part takes two more parameters, so that an encoding with another frequency
schedule or a narrower rotation is this part with other numbers and still runs
in the fused kernel: ``inv_freq`` (one frequency per pair, in place of the
``theta`` formula; a frequency of zero leaves its pair alone) and
``rotary_dim`` (rotate the first ``rotary_dim`` channels only).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

from .base import PositionEncoding, register_position_encoding


@dataclass(frozen=True)
class RotaryParams:
    """What the rotating kernels need: the pairing, and one frequency per pair
    of the head (``inv_freq`` None: ``theta^(-2i/head_dim)`` in 32-bit, as the
    reference computes it)."""
    theta: float
    head_dim: int
    interleaved: bool
    inv_freq: Optional[Tuple[float, ...]] = None


def rotary_frequencies(r: RotaryParams):
    """float32 ``[head_dim / 2]``: the table of ``r``, or ``1 / theta^(2i/head_dim)`` with the
    power and the division in 32-bit (garuda/src/simd/mod.rs:199)."""
    import numpy as np
    if r.inv_freq is not None:
        return np.asarray(r.inv_freq, dtype=np.float32)
    i = np.arange(r.head_dim // 2, dtype=np.float32)
    return (np.float32(1.0) / np.power(np.float32(r.theta), np.float32(2.0) * i / np.float32(r.head_dim),
                                       dtype=np.float32)).astype(np.float32)


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, theta: float, head_dim: int, layout: str = "half",
                 inv_freq: Optional[Sequence[float]] = None, rotary_dim: Optional[int] = None):
        if layout not in ("half", "interleaved"):
            raise ValueError(f"rotary layout must be 'half' or 'interleaved', got {layout!r}")
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head_dim, got {head_dim}")
        head_dim = int(head_dim)
        rot = head_dim if rotary_dim is None else int(rotary_dim)
        if rot % 2 or not 0 < rot <= head_dim:
            raise ValueError(f"rotary_dim must be even and in (0, {head_dim}], got {rotary_dim}")
        if inv_freq is not None and len(inv_freq) != rot // 2:
            raise ValueError(f"inv_freq needs {rot // 2} entries (one per rotated pair), got {len(inv_freq)}")
        self.layout, self.head_dim, self.rotary_dim = layout, head_dim, rot
        interleaved = layout == "interleaved"
        if rot == head_dim:
            freqs = None if inv_freq is None else tuple(float(f) for f in inv_freq)
            self.rotary = RotaryParams(float(theta), head_dim, interleaved, freqs)
            self._narrow = None
        elif interleaved:
            # pairs (2i, 2i + 1): the pairs beyond the rotated width get frequency zero
            base = (tuple(float(f) for f in inv_freq) if inv_freq is not None
                    else tuple(float(f) for f in rotary_frequencies(RotaryParams(float(theta), rot, True))))
            self.rotary = RotaryParams(float(theta), head_dim, True, base + (0.0,) * ((head_dim - rot) // 2))
            self._narrow = None
        else:
            # pairs (i, i + rotary_dim/2) are not pairs of the whole head: rotate a narrower view in place
            self.rotary = None
            freqs = None if inv_freq is None else tuple(float(f) for f in inv_freq)
            self._narrow = RotaryParams(float(theta), rot, False, freqs)

    def apply(self, ctx, q, k, positions):
        r = self.rotary if self.rotary is not None else self._narrow
        width = r.head_dim
        self.ops.rope_inplace(q[..., :width], positions, r)
        if k is not None:
            self.ops.rope_inplace(k[..., :width], positions, r)


@register_position_encoding("none")
class NoPositions(PositionEncoding):
    """Leaves queries and keys as they are."""
    changes_vectors = False
    graph_safe = True

    def __init__(self):
        pass

    def apply(self, ctx, q, k, positions):
        return None
