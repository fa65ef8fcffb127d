"""The scalar C++ restatement (llama_scalar.cpp) from Python: compiled with g++ into a temporary
folder the first time it is asked for, called through ctypes. Tests only."""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import tempfile

import numpy as np

_LIB = None


class _Sizes(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("layers", "width", "heads", "kv_heads", "head_dim", "inner", "vocab",
                                              "interleaved", "tied")] + [("eps", ctypes.c_float), ("theta", ctypes.c_float)]


def _lib():
    global _LIB
    if _LIB is None:
        src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama_scalar.cpp")
        out = os.path.join(tempfile.mkdtemp(prefix="garuda_scalar_"), "llama_scalar.so")
        cxx = shutil.which("g++") or "g++"
        # no fused multiply-adds and no reordering: the sums are the source's, one addition after another
        subprocess.run([cxx, "-O2", "-ffp-contract=off", "-fno-fast-math", "-std=c++17", "-shared", "-fPIC",
                        src, "-o", out], check=True)
        _LIB = ctypes.CDLL(out)
        _LIB.llama_scalar_forward.restype = ctypes.c_int
    return _LIB


def _with_defaults(cfg: dict) -> dict:
    """garuda/src/llama/mod.rs:428-461: kv heads default to the query heads, the head size to
    width / heads, eps to 1e-5, theta to 10000; untied; this engine's default pairing is "half"."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    for key, value in (("rms_norm_eps", 1e-5), ("rope_theta", 10000.0), ("rope_layout", "half"),
                       ("tie_word_embeddings", False)):
        c.setdefault(key, value)
    return c


def _window(c: dict, layer: int) -> int:
    """0 (everything) unless ``sliding_window`` is set and the layer's ``layer_types`` entry, if
    there is such a list, says ``sliding_attention`` (garuda/src/config/mod.rs:34-35, :390-392)."""
    w = c.get("sliding_window") or 0
    kinds = c.get("layer_types")
    return w if w and (kinds is None or kinds[layer] == "sliding_attention") else 0


def forward(cfg: dict, weights: dict, tokens) -> np.ndarray:
    """Logits ``[T, vocab]`` (float32) at every position of one whole sequence."""
    c = _with_defaults(cfg)
    L = c["num_hidden_layers"]
    names = ["model.embed_tokens.weight"]
    for l in range(L):
        p = f"model.layers.{l}."
        names += [p + n for n in ("input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                  "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                  "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                                  "mlp.down_proj.weight")]
    names.append("model.norm.weight")
    if not c["tie_word_embeddings"]:
        names.append("lm_head.weight")
    arrays = [np.ascontiguousarray(weights[n], dtype=np.float32) for n in names]
    if c["tie_word_embeddings"]:
        arrays.append(arrays[0])
    pointers = (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    sizes = _Sizes(L, c["hidden_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                   c["intermediate_size"], c["vocab_size"], int(c["rope_layout"] == "interleaved"),
                   int(bool(c["tie_word_embeddings"])), c["rms_norm_eps"], c["rope_theta"])
    windows = np.asarray([_window(c, l) for l in range(L)], dtype=np.int32)
    toks = np.ascontiguousarray(tokens, dtype=np.int32)
    logits = np.empty((toks.shape[0], c["vocab_size"]), dtype=np.float32)
    rc = _lib().llama_scalar_forward(ctypes.byref(sizes), pointers, windows.ctypes.data_as(ctypes.c_void_p),
                                     toks.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(toks.shape[0]),
                                     logits.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise ValueError("token id outside the vocabulary")
    return logits
