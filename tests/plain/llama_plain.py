"""Plain, slow Llama decoder: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite. It is written from the formulas of
hanumanit/garuda's CPU code and shares no code with ``garuda_b200``. The
reference is Rust and cannot be compiled on a machine without a Rust toolchain,
so nothing here was checked against a run of the reference: it rests on the
formulas, and every function cites the lines it restates.

Everything is numpy; ``dtype`` selects float32 (the reference's arithmetic) or
float64 (used by the tests to judge how much of a difference is rounding).
"""
from __future__ import annotations

import numpy as np


def embed(table: np.ndarray, tokens) -> np.ndarray:
    """Row copy of the embedding table, no scaling.

    garuda/src/llama/mod.rs:1078-1085 (gather, out-of-vocabulary refused before
    any layer runs) and :198-200 (``Weight::row``).
    """
    tokens = np.asarray(tokens, dtype=np.int64)
    if tokens.size and (tokens.min() < 0 or tokens.max() >= table.shape[0]):
        raise ValueError("token id outside the vocabulary")
    return table[tokens].copy()


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """``x * 1/sqrt(mean(x^2) + eps)`` then ``* weight``: scale first, weight second.

    garuda/src/simd/mod.rs:166-173 (eps inside the square root, added to the
    mean) and garuda/src/llama/mod.rs:733-738 (the weight is a plain multiplier).
    """
    dt = x.dtype
    mean_sq = (x * x).sum(axis=-1, keepdims=True, dtype=dt) / dt.type(x.shape[-1])
    scale = dt.type(1.0) / np.sqrt(mean_sq + dt.type(eps))
    return (x * scale) * weight.astype(dt)


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """``y = W x`` for a row-major ``[out, in]`` matrix, no bias.

    garuda/src/simd/mod.rs:72-86 (``matvec``) and :96-129 (``matmul``).
    """
    return x @ w.T


def rope(v: np.ndarray, positions: np.ndarray, theta: float, layout: str) -> np.ndarray:
    """Rotate pairs of one head vector by ``pos * theta^(-2i/head_dim)``.

    garuda/src/simd/mod.rs:196-206 rotates the interleaved pairs ``(2i, 2i+1)``:
    GGUF Llama files carry Q/K rows permuted for that pairing. A safetensors
    folder keeps the unpermuted rows, for which the same rotation pairs
    ``(i, i + head_dim/2)``; ``layout`` chooses between ``"interleaved"`` and
    ``"half"``. Frequency, angle and sin/cos are computed in ``v``'s precision,
    as the reference does in f32.

    ``v``: [T, heads, head_dim]; ``positions``: [T].
    """
    dt = v.dtype
    hd = v.shape[-1]
    i = np.arange(hd // 2, dtype=dt)
    freq = dt.type(1.0) / np.power(dt.type(theta), dt.type(2.0) * i / dt.type(hd), dtype=dt)
    ang = positions.astype(dt)[:, None] * freq[None, :]          # [T, hd/2]
    sin = np.sin(ang, dtype=dt)[:, None, :]
    cos = np.cos(ang, dtype=dt)[:, None, :]
    out = np.empty_like(v)
    if layout == "interleaved":
        a, b = v[..., 0::2], v[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    elif layout == "half":
        a, b = v[..., : hd // 2], v[..., hd // 2:]
        out[..., : hd // 2] = a * cos - b * sin
        out[..., hd // 2:] = a * sin + b * cos
    else:
        raise ValueError(f"unknown rope layout {layout!r}")
    return out


def softmax(s: np.ndarray) -> np.ndarray:
    """Max-subtracted softmax of a vector, with the reference's uniform fallbacks.

    garuda/src/simd/mod.rs:132-158.
    """
    dt = s.dtype
    if s.size == 0:
        return s.copy()
    m = s.max()
    if not np.isfinite(m):
        return np.full_like(s, dt.type(1.0) / dt.type(s.size))
    e = np.exp(s - m)
    total = e.sum(dtype=dt)
    if np.isfinite(total) and total > 0:
        return e * (dt.type(1.0) / total)
    return np.full_like(s, dt.type(1.0) / dt.type(s.size))


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int | None) -> np.ndarray:
    """Causal grouped-query attention over one whole sequence.

    garuda/src/llama/mod.rs:793-818: query head ``h`` reads kv head ``h // g``
    (``g = Hq / Hkv``, :781,799-801); ``s_j = dot(q, K_j) * (1/sqrt(hd))`` with
    the scale multiplied after the dot (:797,808); keys ``j`` in
    ``[start, pos]``; softmax; ``ctx = sum_j p_j V_j`` in key order (:812-818).
    ``start`` is 0, or with a sliding window ``pos + 1 - w`` clamped at 0
    (garuda/src/cache/mod.rs:333-338, evaluated after the append, so the window
    holds ``w`` positions including the current one).

    ``q``: [T, Hq, hd] (roped); ``k``: [T, Hkv, hd] (roped); ``v``: [T, Hkv, hd].
    Returns [T, Hq*hd], heads concatenated.
    """
    dt = q.dtype
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = dt.type(1.0) / np.sqrt(dt.type(hd))
    out = np.zeros((T, Hq, hd), dtype=dt)
    for pos in range(T):
        start = 0 if not window else max(0, pos + 1 - window)
        for h in range(Hq):
            kvh = h // g
            scores = (k[start:pos + 1, kvh, :] @ q[pos, h, :]) * scale
            p = softmax(scores)
            out[pos, h, :] = p @ v[start:pos + 1, kvh, :]
    return out.reshape(T, Hq * hd)


def silu(x: np.ndarray) -> np.ndarray:
    """``x / (1 + exp(-x))``. garuda/src/simd/mod.rs:161-163."""
    return x / (x.dtype.type(1.0) + np.exp(-x))


def swiglu(h: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray) -> np.ndarray:
    """``down(silu(gate h) * (up h))``. garuda/src/llama/mod.rs:1002-1020."""
    g = silu(linear(h, w_gate))
    u = linear(h, w_up)
    return linear(g * u, w_down)


def attention_block(x, lw, cfg, positions, window):
    """Norm, Q/K/V projections, rope on q and k, attention, output projection.

    garuda/src/llama/mod.rs:862-880 with ``attend_one`` :766-821 (rope is applied
    to all query and key heads before the key is stored, :784-791).
    """
    T = x.shape[0]
    Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    h = rmsnorm(x, lw["input_layernorm.weight"], cfg["rms_norm_eps"])
    q = linear(h, lw["self_attn.q_proj.weight"]).reshape(T, Hq, hd)
    k = linear(h, lw["self_attn.k_proj.weight"]).reshape(T, Hkv, hd)
    v = linear(h, lw["self_attn.v_proj.weight"]).reshape(T, Hkv, hd)
    q = rope(q, positions, cfg["rope_theta"], cfg["rope_layout"])
    k = rope(k, positions, cfg["rope_theta"], cfg["rope_layout"])
    ctx = attention(q, k, v, window)
    return linear(ctx, lw["self_attn.o_proj.weight"])


def decoder_layer(x, lw, cfg, positions, window):
    """Pre-norm block with two residuals. garuda/src/llama/mod.rs:851-893."""
    x = x + attention_block(x, lw, cfg, positions, window)
    h2 = rmsnorm(x, lw["post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    y = swiglu(h2, lw["mlp.gate_proj.weight"], lw["mlp.up_proj.weight"], lw["mlp.down_proj.weight"])
    return x + y


def layer_window(cfg: dict, layer: int) -> int | None:
    """The attention window of one layer: ``sliding_window`` where the layer's
    entry of ``layer_types`` says ``sliding_attention`` (every layer, when there
    is no such list), else none. garuda/src/config/mod.rs:34-35,390-392 (0 or
    absent attends to the whole context)."""
    w = cfg.get("sliding_window") or None
    types = cfg.get("layer_types")
    if w is None:
        return None
    if types is None:
        return w
    return w if types[layer] == "sliding_attention" else None


def normalise_config(cfg: dict) -> dict:
    """Fill the defaults the reference gives (garuda/src/llama/mod.rs:428-461)."""
    c = dict(cfg)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    c.setdefault("head_dim", c["hidden_size"] // c["num_attention_heads"])
    c.setdefault("rms_norm_eps", 1e-5)
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_layout", "half")
    c.setdefault("tie_word_embeddings", False)
    return c


def forward(cfg: dict, weights: dict, tokens, dtype=np.float32) -> np.ndarray:
    """Logits at every position of one whole sequence, ``[T, vocab]``.

    garuda/src/llama/mod.rs:1075-1113 (embed, the layers in order, final norm)
    and :1238-1240 (the head; the embedding table itself when tied, :563-572).
    """
    cfg = normalise_config(cfg)
    w = {k: np.asarray(v).astype(dtype) for k, v in weights.items()}
    tokens = np.asarray(tokens, dtype=np.int64)
    positions = np.arange(tokens.shape[0])
    x = embed(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["num_hidden_layers"]):
        prefix = f"model.layers.{l}."
        lw = {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}
        x = decoder_layer(x, lw, cfg, positions, layer_window(cfg, l))
    z = rmsnorm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(z, head)


def greedy_generate(cfg: dict, weights: dict, prompt, max_tokens: int, dtype=np.float32):
    """Greedy continuation by re-running the whole sequence for every token.

    garuda/src/runtime/mod.rs:698-740 with temperature 0 (:99-107).
    """
    seq = list(prompt)
    out = []
    for _ in range(max_tokens):
        logits = forward(cfg, weights, seq, dtype)[-1]
        tok = argmax_first(logits)
        out.append(tok)
        seq.append(tok)
    return out


def argmax_first(logits: np.ndarray) -> int:
    """First maximum wins (strict ``>`` scan from index 0).
    garuda/src/runtime/mod.rs:99-107."""
    best, best_v = 0, -np.inf
    for i, v in enumerate(logits):
        if v > best_v:
            best, best_v = i, v
    return int(best)
