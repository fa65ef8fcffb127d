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

TINY = {"A": (TINY_A, 0, None), "B": (TINY_B, 1, ("normal_about_one", 0.1)), "C": (TINY_C, 2, None),
        "D": (TINY_D, 3, None)}

# Query and key projections eight times the usual N(0, 0.02): attention scores of the order of one,
# so that the keys do not all weigh the same and a wrong position, rotation, mask or page shows in
# the logits (with the plain scale a decode step that rotated by stale angles passed every test).
SHARPEN = {"q_proj": 8.0, "k_proj": 8.0}

_DIRS = {}


def model_dir(name: str, store_dtype=torch.float32) -> str:
    """A model folder for one of the tiny configurations, made once per session
    in a temporary folder."""
    from garuda_b200.weights import write_random_model
    key = (name, store_dtype)
    if key not in _DIRS:
        cfg, seed, norm_init = TINY[name]
        d = tempfile.mkdtemp(prefix=f"garuda_tiny_{name}_")
        write_random_model(d, cfg, seed, norm_init=norm_init, store_dtype=store_dtype, scale=SHARPEN)
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


# tolerances against the plain implementation, as a fraction of the largest logit
TOL = {"float32": 2e-5, "bfloat16": 2.5e-2}


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str = ""):
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(got - want).max())
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: not finite"
    if err > TOL[dtype] * scale:
        bad = np.unravel_index(np.argmax(np.abs(got - want)), got.shape)
        raise AssertionError(f"{what}: max difference {err:.3e} (limit {TOL[dtype] * scale:.3e}) "
                             f"first at row {bad[0]}")


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
