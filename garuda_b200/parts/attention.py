"""Causal grouped-query attention over the paged cache.

garuda/src/llama/mod.rs:743-757 (Q, K, V projections, no bias), :766-821
(``attend_one``: rotate q and k at the token's position, store the rotated key
and the raw value, then for every query head ``h`` read kv head ``h // g``:
``s_j = dot(q, K_j) / sqrt(head_dim)`` over ``j`` in ``[start, pos]``, softmax,
``sum_j p_j V_j``), :879-880 (output projection). A step's tokens are first all
stored and then all read, each query over keys up to its own position, which
is the same thing as the reference's token-by-token order.

The three projections are one matrix product against the rows of
``q_proj, k_proj, v_proj`` stacked (the reference runs three, :753-755); its
result stays 32-bit until after the rotation.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import (Mixer, PagedKV, TensorSpec, PartSpec, build_part, register_mixer)


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(self, width: int, heads: int, kv_heads: int, head_dim: int,
                 position: Optional[dict] = None, window: Optional[int] = None,
                 scale: Optional[float] = None, reads_shared_cache: bool = False,
                 init_std: float = 0.02):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads are not a multiple of {kv_heads} kv heads")
        self.width, self.heads, self.kv_heads, self.head_dim = int(width), int(heads), int(kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.reads_shared_cache = bool(reads_shared_cache)
        self.init_std = float(init_std)
        pos = position or {"name": "none", "params": {}}
        self.position = build_part("position_encoding", PartSpec(pos["name"], dict(pos.get("params", {}))))
        self.q_dim = self.heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim

    # ---- declarations ------------------------------------------------------
    def tensors(self):
        init = ("normal", self.init_std)
        t = {"q_proj.weight": TensorSpec((self.q_dim, self.width), init=init),
             "o_proj.weight": TensorSpec((self.width, self.q_dim), init=init)}
        if not self.reads_shared_cache:
            t["k_proj.weight"] = TensorSpec((self.kv_dim, self.width), init=init)
            t["v_proj.weight"] = TensorSpec((self.kv_dim, self.width), init=init)
        # a position encoding with tensors of its own (a learned table) keeps them under "position."
        for local, ts in self.position.tensors().items():
            t["position." + local] = ts
        return t

    @property
    def graph_safe(self):
        return self.position.graph_safe

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def load(self, tensors, ops, dtype):
        super().load(tensors, ops, dtype)
        self.position.load({local: tensors["position." + local] for local in self.position.tensors()}, ops, dtype)
        if self.reads_shared_cache:
            self.w_qkv = tensors["q_proj.weight"].contiguous()
        else:
            self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                    tensors["v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()

    # ---- one step ------------------------------------------------------------
    # ``h`` may be a norm that is half done (``CudaOps.qkv_rope_append`` takes it), and the output
    # product may fold in the first half of the norm that follows (``emit_norm``)
    takes_pending_norm = True
    emits_norm = True

    def forward(self, ctx, h, cache, residual=None, emit_norm=None):
        b, ops, ws = ctx.batch, self.ops, ctx.ws
        T = h.shape[0]
        writes = cache.writes and not self.reads_shared_cache
        cols = self.q_dim + (2 * self.kv_dim if writes else 0)
        # a call that reads another call's cache projects queries only (the first rows)
        w_qkv = self.w_qkv if self.w_qkv.shape[0] == cols else self.w_qkv[:cols]
        q = ws.get("q_heads", (T, self.heads, self.head_dim), self.dtype)
        rotary = self.position.rotary
        kv_heads = self.kv_heads if writes else 0
        if rotary is not None or not self.position.changes_vectors:
            # the product, the rotation and the write into the pages, fused where the kernels allow
            ops.qkv_rope_append(ctx, h, w_qkv, q, cache.k if writes else None, cache.v if writes else None,
                                b.positions, b.token_req, cache.block_table, self.heads, kv_heads,
                                self.head_dim, rotary, cache.page_size)
        else:
            # an encoding the fused kernel does not know: let the part change q and k in place
            qkv = ws.get("qkv", (T, cols), torch.float32)
            if hasattr(ops, "normed"):
                h = ops.normed(ctx, h)
            ops.linear(h, w_qkv, qkv)
            qv = qkv[:, :self.q_dim].unflatten(1, (self.heads, self.head_dim))
            kv = (qkv[:, self.q_dim:self.q_dim + self.kv_dim].unflatten(1, (self.kv_heads, self.head_dim))
                  if writes else None)
            self.position.apply(ctx, qv, kv, b.positions)
            ops.rope_kv_append(qkv, q, cache.k if writes else None, cache.v if writes else None,
                               b.positions, b.token_req, cache.block_table, self.heads, kv_heads,
                               self.head_dim, None, cache.page_size)
        out = ws.get("attn_ctx", (T, self.q_dim), self.dtype)
        ops.paged_attention(q, cache.k, cache.v, cache.block_table, b.cu_q, b.kv_lens, b.token_req, out,
                            self.scale, self.window or 0, cache.page_size,
                            b.num_requests, b.max_q_len, b.max_kv_len, ws=ws, min_q_len=b.min_q_len)
        if residual is not None:
            if emit_norm is None:
                ops.linear(out, self.w_o, residual, accumulate=True)
            else:
                ctx.pending_norm = ops.linear(out, self.w_o, residual, accumulate=True, ctx=ctx, emit_norm=emit_norm)
            return None
        y = ws.get("mixer_out", (T, self.width), torch.float32)
        ops.linear(out, self.w_o, y)
        return y
