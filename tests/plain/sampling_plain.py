"""Plain restatement of hanumanit/garuda's sampler and generator, for the tests.

Written from garuda/src/runtime/mod.rs; shares no code with ``garuda_b200``.
"""
from __future__ import annotations

import numpy as np

from .llama_plain import softmax, argmax_first

MASK = (1 << 64) - 1


class Rng:
    """splitmix64. garuda/src/runtime/mod.rs:64-84."""

    def __init__(self, seed: int):
        self.state = (seed ^ 0x9E3779B97F4A7C15) & MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
        return z ^ (z >> 31)

    def next_f32(self) -> np.float32:
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def candidates(logits: np.ndarray, temperature: float, top_k: int, top_p: float):
    """Temperature, softmax over the whole vocabulary, top-k, sort, top-p.

    garuda/src/runtime/mod.rs:133-175. Ties break on the lower token id; the
    survivors keep their softmax probabilities (no renormalisation).
    """
    scaled = (logits.astype(np.float32) / np.float32(temperature)).astype(np.float32)
    probs = softmax(scaled)
    order = sorted(range(len(probs)), key=lambda i: (-float(probs[i]), i))
    if 0 < top_k < len(order):
        order = order[:top_k]
    if top_p < 1.0:
        cumulative = np.float32(0.0)
        keep = 0
        for i, tok in enumerate(order):
            cumulative = np.float32(cumulative + probs[tok])
            keep = i + 1
            if cumulative >= np.float32(top_p):
                break
        order = order[:max(keep, 1)]
    return [(tok, probs[tok]) for tok in order]


def sample(logits: np.ndarray, temperature: float, top_k: int, top_p: float, rng: Rng) -> int:
    """garuda/src/runtime/mod.rs:87-125: greedy at temperature 0, else draw
    ``u * total`` and walk the sorted survivors, first ``<= 0`` wins."""
    if temperature == 0.0:
        return argmax_first(logits)
    cand = candidates(logits, temperature, top_k, top_p)
    total = np.float32(0.0)
    for _, p in cand:
        total = np.float32(total + p)
    if total <= 0:
        return cand[0][0]
    point = np.float32(rng.next_f32() * total)
    for tok, p in cand:
        point = np.float32(point - p)
        if point <= 0:
            return tok
    return cand[-1][0]
