"""A toy architecture that the framework knows nothing about, for the tests.

Importing this module registers, through the framework's public hooks only:
a mixer with state of its own (a running mean per request, in a fixed-size state
slot), a feed-forward with routing (every token goes through the one of a few
small experts that its router picks), a position encoding with a tensor of its
own (a learned vector per position, added to queries and keys), and the
architecture ``ToyForCausalLM`` that arranges them beside the built-in
attention (with frequencies of its own for the rotation, and without any
position encoding), names a layer twice in its run order and lets the second
call read the first call's cache. It is no model of anyone's: it exists to show
that the parts' interfaces are enough. ``plain_forward`` restates it in numpy
with the formulas of ``tests/plain/llama_plain.py``.

As a plugin: ``bin/garuda --plugin tests.toy_arch ...``.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from garuda_b200.config.model_config import ConfigError
from garuda_b200.config.registry import register_architecture
from garuda_b200.models.decoder import LayerCall, ModelSpec
from garuda_b200.parts import (BlockSpec, FeedForward, FixedState, Mixer, PartSpec, PositionEncoding,
                               TensorSpec, register_feed_forward, register_mixer, register_position_encoding)
from tests.plain import llama_plain


# ---------------------------------------------------------------------------- parts
@register_mixer("toy_running_mean")
class RunningMean(Mixer):
    """out_t = gain * mean(h_0 .. h_t) over the request's tokens so far: a running sum and a count
    in the request's state slot, carried across steps. Runs on the host's copies of the batch's
    arrays, so it says nothing about being safe to capture (the default: it is not)."""

    def __init__(self, width):
        self.width = int(width)

    def tensors(self):
        return {"gain": TensorSpec((self.width,), role="vector", init=("normal_about_one", 0.1))}

    def cache_need(self):
        return FixedState((self.width + 1,), torch.float32)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.gain = tensors["gain"].float()

    def forward(self, ctx, h, cache, residual=None):
        b = ctx.batch
        out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        cu = b.host["cu_q"]
        for r, slot in enumerate(b.host["slots"]):
            rows = h[cu[r]:cu[r + 1]].float()
            state = cache.state[slot]
            sums = state[:-1] + torch.cumsum(rows, 0)
            counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=h.device)
            out[cu[r]:cu[r + 1]] = sums / counts[:, None] * self.gain
            state[:-1] = sums[-1]
            state[-1] = counts[-1]
        return out


@register_feed_forward("toy_routed")
class RoutedExperts(FeedForward):
    """Router logits ``h W_r^T`` in 32-bit, the first largest picks the expert, and the token's
    output is that expert's ``W_2 relu(W_1 h)``. Computed for every expert and selected, which is
    all a toy needs; the products are the framework's."""

    def __init__(self, width, inner, experts):
        self.width, self.inner, self.experts = int(width), int(inner), int(experts)

    def tensors(self):
        t = {"router.weight": TensorSpec((self.experts, self.width), init=("normal", 0.5))}
        for e in range(self.experts):
            t[f"experts.{e}.w1"] = TensorSpec((self.inner, self.width), init=("normal", 0.1))
            t[f"experts.{e}.w2"] = TensorSpec((self.width, self.inner), init=("normal", 0.1))
        return t

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.router = tensors["router.weight"].float().contiguous()
        self.w1 = [tensors[f"experts.{e}.w1"].contiguous() for e in range(self.experts)]
        self.w2 = [tensors[f"experts.{e}.w2"].contiguous() for e in range(self.experts)]

    def forward(self, ctx, h, residual=None):
        ops, T = self.ops, h.shape[0]
        logits = torch.empty(T, self.experts, dtype=torch.float32, device=h.device)
        ops.linear(h.float().contiguous(), self.router, logits)         # the router stays 32-bit
        choice = torch.argmax(logits, dim=-1)
        out = torch.zeros(T, self.width, dtype=torch.float32, device=h.device)
        for e in range(self.experts):
            mid = torch.empty(T, self.inner, dtype=torch.float32, device=h.device)
            ops.linear(h, self.w1[e], mid)
            y = torch.empty(T, self.width, dtype=torch.float32, device=h.device)
            ops.linear(torch.relu(mid).to(h.dtype), self.w2[e], y)
            out = torch.where((choice == e)[:, None], y, out)
        return out


@register_position_encoding("toy_learned")
class LearnedPositions(PositionEncoding):
    """A learned vector per position, added to every query and key head. Has a tensor of its own,
    and no rotation that the fused kernel could apply: the attention part runs the product,
    calls ``apply`` on the 32-bit queries and keys, and stores."""

    def __init__(self, positions, head_dim):
        self.positions, self.head_dim = int(positions), int(head_dim)

    def tensors(self):
        return {"table": TensorSpec((self.positions, self.head_dim), role="vector", init=("normal", 0.3))}

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.table = tensors["table"].float()

    def apply(self, ctx, q, k, positions):
        add = self.table[positions.long()][:, None, :]
        q += add
        if k is not None:
            k += add


# ---------------------------------------------------------------------------- the architecture
@dataclass(frozen=True)
class ToyConfig:
    width: int
    vocab_size: int
    max_positions: int
    heads: int
    kv_heads: int
    head_dim: int
    inner: int
    experts: int
    eps: float
    window: int
    rotary_frequencies: tuple
    eos_token_ids: tuple = ()

    @classmethod
    def from_dict(cls, d):
        try:
            eos = d.get("eos_token_id", [])
            return cls(width=int(d["width"]), vocab_size=int(d["vocab_size"]), max_positions=int(d["max_positions"]),
                       heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), head_dim=int(d["head_dim"]),
                       inner=int(d["inner"]), experts=int(d["experts"]), eps=float(d["eps"]), window=int(d["window"]),
                       rotary_frequencies=tuple(float(f) for f in d["rotary_frequencies"]),
                       eos_token_ids=tuple(eos) if isinstance(eos, list) else (int(eos),))
        except KeyError as e:
            raise ConfigError(f"config.json is missing {e}") from None


TOY_CONFIG = dict(architectures=["ToyForCausalLM"], width=64, vocab_size=120, max_positions=96, heads=4, kv_heads=2,
                  head_dim=16, inner=80, experts=3, eps=1e-5, window=20,
                  rotary_frequencies=[0.9 ** i for i in range(8)])


def toy_spec(c: ToyConfig) -> ModelSpec:
    d = c.width

    def attention(l, position, window=None):
        return PartSpec("paged_attention", dict(width=d, heads=c.heads, kv_heads=c.kv_heads, head_dim=c.head_dim,
                                                position=position, window=window, init_std=0.15),
                        prefix=f"blocks.{l}.attention.")

    norm = lambda p: PartSpec("rms", dict(width=d, eps=c.eps, weight_init=("normal_about_one", 0.1)), prefix=p)
    learned = {"name": "toy_learned", "params": {"positions": c.max_positions, "head_dim": c.head_dim}}
    scaled = {"name": "rotary", "params": {"theta": 1.0, "head_dim": c.head_dim, "layout": "interleaved",
                                           "inv_freq": list(c.rotary_frequencies)}}
    layers = [
        BlockSpec(attention(0, learned), PartSpec("toy_routed", dict(width=d, inner=c.inner, experts=c.experts),
                                                  prefix="blocks.0.routed."),
                  norm("blocks.0.norm1."), norm("blocks.0.norm2.")),
        BlockSpec(PartSpec("toy_running_mean", dict(width=d), prefix="blocks.1.mean."),
                  PartSpec("swiglu", dict(width=d, inner=c.inner, init_std=0.1), prefix="blocks.1.mlp."),
                  norm("blocks.1.norm1."), norm("blocks.1.norm2.")),
        BlockSpec(attention(2, scaled, window=c.window), None, norm("blocks.2.norm1."), None),
        BlockSpec(attention(3, {"name": "none", "params": {}}),
                  PartSpec("swiglu", dict(width=d, inner=c.inner, init_std=0.1), prefix="blocks.3.mlp."),
                  norm("blocks.3.norm1."), norm("blocks.3.norm2.")),
    ]
    # layer 0 runs twice; its second call reads the keys and values that its first call stored
    order = [LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(3), LayerCall(0, reads_cache_of=0)]
    return ModelSpec(architecture="ToyForCausalLM", width=d, vocab_size=c.vocab_size, max_positions=c.max_positions,
                     embedding="tokens.weight", layers=layers, order=order, final_norm=norm("final_norm."),
                     head="out.weight", embedding_init=("normal", 0.5), eos_token_ids=c.eos_token_ids)


register_architecture("ToyForCausalLM", ToyConfig.from_dict, toy_spec)


# ---------------------------------------------------------------------------- the same in numpy
def plain_forward(cfg: dict, w: dict, tokens) -> np.ndarray:
    """Logits ``[T, vocab]`` of one whole sequence (float32 numpy), from the formulas alone."""
    c = ToyConfig.from_dict(cfg)
    lp = llama_plain
    T = len(tokens)
    pos = np.arange(T)
    x = lp.embed(w["tokens.weight"], tokens)
    g = c.heads // c.kv_heads

    def heads_of(h, prefix, which, n):
        return lp.linear(h, w[f"{prefix}{which}_proj.weight"]).reshape(T, n, c.head_dim)

    def attention_block(x, l, kind, window, stored=None):
        p = f"blocks.{l}.attention."
        h = lp.rmsnorm(x, w[f"blocks.{l}.norm1.weight"], c.eps)
        q = heads_of(h, p, "q", c.heads)
        if stored is None:
            k, v = heads_of(h, p, "k", c.kv_heads), heads_of(h, p, "v", c.kv_heads)
        if kind == "learned":
            add = w[p + "position.table"][pos][:, None, :]
            q = q + add
            if stored is None:
                k = k + add
        elif kind == "scaled":
            ang = pos[:, None].astype(np.float32) * np.asarray(c.rotary_frequencies, dtype=np.float32)[None, :]
            sin, cos = np.sin(ang)[:, None, :], np.cos(ang)[:, None, :]

            def rot(t):
                out = np.empty_like(t)
                a, b = t[..., 0::2], t[..., 1::2]
                out[..., 0::2] = a * cos - b * sin
                out[..., 1::2] = a * sin + b * cos
                return out
            q = rot(q)
            if stored is None:
                k = rot(k)
        if stored is not None:
            k, v = stored
        ctx = lp.attention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), window)
        return lp.linear(ctx, w[p + "o_proj.weight"]), (k, v)

    def routed(h):
        p = "blocks.0.routed."
        logits = lp.linear(h, w[p + "router.weight"])
        out = np.zeros_like(h)
        for t in range(T):
            e = lp.argmax_first(logits[t])
            mid = np.maximum(lp.linear(h[t], w[f"{p}experts.{e}.w1"]), 0)
            out[t] = lp.linear(mid, w[f"{p}experts.{e}.w2"])
        return out

    def mlp(h, l):
        p = f"blocks.{l}.mlp."
        return lp.swiglu(h, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])

    # layer 0: learned positions, routed feed-forward
    a, kv0 = attention_block(x, 0, "learned", None)
    x = x + a
    x = x + routed(lp.rmsnorm(x, w["blocks.0.norm2.weight"], c.eps))
    # layer 1: running mean, SwiGLU
    h = lp.rmsnorm(x, w["blocks.1.norm1.weight"], c.eps)
    x = x + np.cumsum(h, axis=0) / np.arange(1, T + 1, dtype=np.float32)[:, None] * w["blocks.1.mean.gain"]
    x = x + mlp(lp.rmsnorm(x, w["blocks.1.norm2.weight"], c.eps), 1)
    # layer 2: rotation at frequencies of its own, a window, no feed-forward
    a, _ = attention_block(x, 2, "scaled", c.window)
    x = x + a
    # layer 3: no position encoding
    a, _ = attention_block(x, 3, "none", None)
    x = x + a
    x = x + mlp(lp.rmsnorm(x, w["blocks.3.norm2.weight"], c.eps), 3)
    # layer 0 again, reading the first call's keys and values
    a, _ = attention_block(x, 0, "learned", None, stored=kv0)
    x = x + a
    x = x + routed(lp.rmsnorm(x, w["blocks.0.norm2.weight"], c.eps))
    return lp.linear(lp.rmsnorm(x, w["final_norm.weight"], c.eps), w["out.weight"])


def plain_greedy(cfg: dict, w: dict, prompt, max_tokens: int):
    seq, out = list(prompt), []
    for _ in range(max_tokens):
        tok = llama_plain.argmax_first(plain_forward(cfg, w, seq)[-1])
        out.append(tok)
        seq.append(tok)
    return out
