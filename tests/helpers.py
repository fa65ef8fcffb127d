"""Shared by the tests: the tiny configurations, model folders, traces."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny configurations that differ in every size and option, and a third with
# a head size that is no power of two, q_dim != hidden_size and a window on every layer.
TINY_A = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=128)
TINY_B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=96, num_hidden_layers=3,
              num_attention_heads=3, num_key_value_heads=1, head_dim=32, intermediate_size=256,
              vocab_size=384, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=256, sliding_window=40,
              layer_types=["full_attention", "sliding_attention", "full_attention"],
              rope_layout="interleaved")
TINY_C = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=72, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=200,
              vocab_size=331, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=192, sliding_window=24)

# head size 64 (the size the tcgen05 prompt attention takes), groups of two, one windowed layer
TINY_D = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=128, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=320,
              vocab_size=500, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=512, sliding_window=160,
              layer_types=["full_attention", "sliding_attention"])

# head size 128 (two of the reference's published shapes have it), every query head with a kv head
# of its own (no groups), the reference's interleaved rotation pairs, tied embeddings
TINY_E = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=256, num_hidden_layers=2,
              num_attention_heads=2, num_key_value_heads=2, head_dim=128, intermediate_size=344,
              vocab_size=777, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=384, rope_layout="interleaved")

# (config.json, seed, how norm weights are drawn). "Ai" and "Bh" are A and B with the other pairing of
# the rotation (garuda/src/simd/mod.rs:196-206 pairs (2i, 2i + 1); a safetensors folder's rows want
# (i, i + head_dim / 2)): both tiny configurations run both ways.
TINY = {"A": (TINY_A, 0, None), "B": (TINY_B, 1, ("normal_about_one", 0.1)), "C": (TINY_C, 2, None),
        "D": (TINY_D, 3, None), "E": (TINY_E, 4, ("normal_about_one", 0.1)),
        "Ai": (dict(TINY_A, rope_layout="interleaved"), 0, None),
        "Bh": (dict(TINY_B, rope_layout="half"), 1, ("normal_about_one", 0.1))}

# Query and key projections eight times the usual N(0, 0.02): attention scores of the order of one,
# so that the keys do not all weigh the same and a wrong position, rotation, mask or page shows in
# the logits (with the plain scale a decode step that rotated by stale angles passed every test).
SHARPEN = {"q_proj": 8.0, "k_proj": 8.0}


def sharpen_for(hidden_size: int) -> dict:
    """The factor that gives scores a spread of about 1.6 at this width (8 at width 64: a score is a
    sum over ``hidden_size`` inputs per channel, so the factor falls with the root of the width).
    Much sharper than that and the softmax turns the bfloat16 rounding of a score into a large change
    of the result, which says nothing about the kernels."""
    f = min(8.0, max(1.0, 64.0 / float(hidden_size) ** 0.5))
    return {"q_proj": f, "k_proj": f}

_DIRS = {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    """A model folder for one of the tiny configurations, made once per session
    in a temporary folder."""
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed, norm_init = TINY[name]
        d = tempfile.mkdtemp(prefix=f"garuda_tiny_{name}_")
        scale = sharpen_for(cfg["hidden_size"])
        write_random_model(d, cfg, seed, norm_init=norm_init, store_dtype=store_dtype, scale=scale)
        _DIRS[key] = d
    return _DIRS[key]


def folder_weights(path: str) -> dict:
    """Every tensor of a folder as float32 numpy (bfloat16 is widened exactly)."""
    from garuda_b200.weights import SafetensorsFolder
    f = SafetensorsFolder(path)
    return {n: f.tensor(n).float().numpy() for n in f.names()}


_PLAIN = {}


def plain_logits(name: str, store_dtype, tokens) -> np.ndarray:
    """Logits at every position from the plain implementation (float32)."""
    from tests.plain import llama_plain
    key = (name, store_dtype, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = llama_plain.forward(TINY[name][0], folder_weights(model_dir(name, store_dtype)), tokens)
    return _PLAIN[key]


def random_tokens(name: str, n: int, seed: int):
    rng = np.random.default_rng(seed)
    return rng.integers(0, TINY[name][0]["vocab_size"], n).tolist()


# Tolerances against the plain implementation, as a fraction of the largest logit. 32-bit: rounding
# of sums taken in another order. bfloat16: per configuration, three times the largest difference
# seen on a B200 over every test that compares this configuration (weights, activations between
# products and the cache are rounded to 8 bits of mantissa; how much of that reaches the logits
# depends on depth and widths). A configuration without an entry takes the widest.
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}
# observed on a B200 (GARUDA_B200_RECORD_ERRORS, see tests/conftest.py), times three, at most the widest:
# A 0.0053, Ai 0.0064, B 0.0062, Bh 0.0057, C 0.0090, D 0.0092, E 0.0069, toy 0.0083; two layers at the
# TinyLlama, Llama-2-7B and Llama-3-8B widths 0.0147, 0.0137, 0.0115 (32-bit: at most 2.4e-6 and 7.9e-6)
TOL_BF16 = {"A": 0.016, "Ai": 0.02, "B": 0.019, "Bh": 0.017, "E": 0.021}

OBSERVED = {}        # (configuration, dtype) -> largest difference seen, as a fraction of the largest logit


def tolerance(dtype: str, config: str = None) -> float:
    if dtype == "bfloat16" and config in TOL_BF16:
        return TOL_BF16[config]
    return TOL[dtype]


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str = "", config: str = None):
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(got - want).max())
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    key = f"{config}/{dtype}"
    OBSERVED[key] = max(OBSERVED.get(key, 0.0), err / scale)
    limit = tolerance(dtype, config) * scale
    if err > limit:
        bad = np.unravel_index(np.argmax(np.abs(got - want)), got.shape)
        raise AssertionError(f"{what}: max difference {err:.3e} (limit {limit:.3e}) first at row {bad[0]}")


class TraceRunner:
    """Drives bin/trace_run as a child process, step by step."""

    def __init__(self, model: str, dtype: str, max_tokens: int, extra=()):
        self.out = tempfile.mkdtemp(prefix="garuda_trace_")
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", model, "--dtype", dtype, "--out", self.out,
             "--max-tokens", str(max_tokens), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0
        self.vocab = json.load(open(os.path.join(model, "config.json")))["vocab_size"]

    def step(self, entries, end=()):
        """entries: list of (id, tokens, want). Returns logits [wanted, vocab] or None."""
        rec = {"step": self.step_no, "entries": [{"id": i, "tokens": list(t), "want": list(w)}
                                                  for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_no} "
                               f"(exit code {self.proc.poll()})")
        path = os.path.join(self.out, f"{self.step_no}.f32")
        self.step_no += 1
        if any(len(w) for _, _, w in entries):
            return np.fromfile(path, dtype="<f4").reshape(-1, self.vocab)
        return None

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)


# ---------------------------------------------------------------------- sampling
def sampling_rows(few: bool = False):
    """(temperature, top_k, top_p, u) per row: greedy, top-k within and beyond the kernel's short
    list of 1,024 candidates, top-p alone, neither; each with draws at both ends and in between."""
    settings = [(0.8, 40, 0.95), (1.0, 0, 1.0), (0.5, 5, 1.0), (1.3, 0, 0.7), (0.0, 40, 0.95),
                (0.8, 1, 0.95), (2.0, 100, 0.5), (1.5, 1024, 0.9), (1.5, 1025, 0.9), (1.0, 64, 1.0)]
    draws = (0.0, 0.5, 0.999) if few else (0.0, 0.123, 0.5, 0.77, 0.999)
    if few:
        settings = settings[:5] + settings[7:9]
    return [(t, k, p, u) for t, k, p in settings for u in draws]


def assert_tokens_follow_the_plain_sampler(rows, logits, got):
    """``got[i]`` is the plain sampler's token for row i of ``logits`` (a CPU tensor) and ``rows[i]``
    = (temperature, top_k, top_p, u), or its neighbour when the draw falls within rounding of the
    boundary between two candidates.

    The reference walks the sorted candidates subtracting 32-bit probabilities one by one; a kernel
    sums in another order. Over tens of thousands of terms the two running sums differ in their last
    bits, and a draw that lands within that rounding of a boundary may fall on either side. Anything
    further from the boundary is a fault."""
    from tests.plain.sampling_plain import sample as plain_sample, candidates

    class FixedU:
        def __init__(self, u): self.u = u
        def next_f32(self): return np.float32(self.u)

    for i, (temp, k, p, u) in enumerate(rows):
        row = logits[i].numpy()
        want = plain_sample(row, temp, k, p, FixedU(u))
        if got[i] == want:
            continue
        assert temp > 0, f"row {i}: greedy gave {got[i]}, the plain sampler {want}"
        cand = candidates(row, temp, k, p)
        ids = [t for t, _ in cand]
        cum = np.cumsum(np.array([float(pr) for _, pr in cand], dtype=np.float64))
        point = float(u) * cum[-1]
        assert got[i] in ids, f"row {i}: token {got[i]} is not among the candidates"
        j = ids.index(got[i])
        lo = cum[j - 1] if j else 0.0
        slack = 16 * np.sqrt(len(cand)) * np.finfo(np.float32).eps * cum[-1]
        assert lo - slack <= point <= cum[j] + slack, (
            f"row {i}: temperature {temp}, top_k {k}, top_p {p}, u {u}: token {got[i]} covers "
            f"[{lo}, {cum[j]}], the draw is {point} (plain sampler: {want})")
