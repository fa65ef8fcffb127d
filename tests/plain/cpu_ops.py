"""Plain references of the engine's kernels, one function per kernel, on the CPU.

Two uses. The ``-m gpu`` tests compare each CUDA kernel with the function of the
same name here. And because the functions take the same arguments as the
product's kernel set, an instance of ``CpuOps`` can stand in for it, so that
the step function, the cache and the batching logic can be exercised on a
machine without a GPU. It is never used outside the tests: the product path has
no CPU fallback.

Written from the reference's formulas (cited per function); shares no code with
``garuda_b200``.
"""
from __future__ import annotations


import numpy as np
import torch


class CpuOps:
    name = "cpu-reference"

    device = "cpu"

    def __init__(self):
        self.tc = None

    # garuda/src/llama/mod.rs:198-200, :1078-1085
    def embedding(self, table, ids, out):
        out[: ids.shape[0]] = table[ids.long()].float()

    # garuda/src/simd/mod.rs:166-173; garuda/src/llama/mod.rs:733-738
    def rmsnorm(self, x, weight, eps, out, rows=None):
        xs = x if rows is None else x[rows.long()]
        ms = (xs * xs).sum(-1, keepdim=True) / xs.shape[-1]
        out.copy_(((xs * (1.0 / torch.sqrt(ms + eps))) * weight.float()).to(out.dtype))

    # garuda/src/simd/mod.rs:96-129
    def linear(self, a, w, out, accumulate=False):
        y = a.float() @ w.float().t()
        if accumulate:
            out += y
        else:
            out.copy_(y.to(out.dtype))

    def pack_gate_up(self, gate, up):
        return torch.cat([gate, up], 0).contiguous()

    # garuda/src/llama/mod.rs:1002-1020; garuda/src/simd/mod.rs:161-163
    def linear_swiglu(self, ctx, h, w_gate_up, act):
        y = h.float() @ w_gate_up.float().t()
        self.silu_mul(y, act)

    def silu_mul(self, gate_up, out):
        F = out.shape[1]
        g, u = gate_up[:, :F].float(), gate_up[:, F:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    # garuda/src/simd/mod.rs:176-179
    def residual_add(self, x, y):
        x += y.float()

    # garuda/src/simd/mod.rs:196-206
    def _rotate(self, v, positions, rotary):
        """``rotary``: anything with ``theta``, ``interleaved`` and ``inv_freq`` (one frequency per
        pair in place of the formula, or None)."""
        hd = v.shape[-1]
        interleaved = rotary.interleaved
        if getattr(rotary, "inv_freq", None) is not None:
            inv = torch.tensor(list(rotary.inv_freq), dtype=torch.float32)
        else:
            i = np.arange(hd // 2, dtype=np.float32)
            inv = torch.from_numpy(np.float32(1.0) / np.power(np.float32(rotary.theta),
                                                              np.float32(2.0) * i / np.float32(hd), dtype=np.float32))
        ang = positions.float()[:, None] * inv[None, :]
        s, c = torch.sin(ang)[:, None, :], torch.cos(ang)[:, None, :]
        out = torch.empty_like(v)
        if interleaved:
            a, b = v[..., 0::2], v[..., 1::2]
            out[..., 0::2] = a * c - b * s
            out[..., 1::2] = a * s + b * c
        else:
            a, b = v[..., : hd // 2], v[..., hd // 2:]
            out[..., : hd // 2] = a * c - b * s
            out[..., hd // 2:] = a * s + b * c
        return out

    def rope_inplace(self, x, positions, rotary):
        x.copy_(self._rotate(x.clone(), positions, rotary))

    # garuda/src/llama/mod.rs:743-757 (the projections), then rotate and store
    def qkv_rope_append(self, ctx, h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                        heads, kv_heads, head_dim, rotary, page_size):
        qkv = h.float() @ w_qkv.float().t()
        self.rope_kv_append(qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            head_dim, rotary, page_size)

    # garuda/src/llama/mod.rs:784-791 (rotate, then store the rotated key and the raw value)
    def rope_kv_append(self, qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                       heads, kv_heads, head_dim, rotary, page_size):
        T = qkv.shape[0]
        x = qkv.float()
        q = x[:, : heads * head_dim].reshape(T, heads, head_dim)
        if rotary is not None:
            q = self._rotate(q, positions, rotary)
        q_out.copy_(q.to(q_out.dtype))
        if not kv_heads:
            return
        k = x[:, heads * head_dim: (heads + kv_heads) * head_dim].reshape(T, kv_heads, head_dim)
        v = x[:, (heads + kv_heads) * head_dim:].reshape(T, kv_heads, head_dim)
        if rotary is not None:
            k = self._rotate(k, positions, rotary)
        for t in range(T):
            pos = int(positions[t])
            page = int(block_table[int(token_req[t]), pos // page_size])
            assert page >= 0, "a position without a page"
            k_pool[page, :, pos % page_size, :] = k[t].to(k_pool.dtype)
            v_pool[page, :, pos % page_size, :] = v[t].to(v_pool.dtype)

    # garuda/src/llama/mod.rs:793-818; garuda/src/cache/mod.rs:333-338
    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out,
                        scale, window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1):
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        g = Hq // Hkv
        res = torch.zeros(T, Hq, hd)
        for t in range(T):
            r = int(token_req[t])
            q_len = int(cu_q[r + 1] - cu_q[r])
            pos = int(kv_lens[r]) - q_len + (t - int(cu_q[r]))
            start = max(0, pos + 1 - window) if window else 0
            js = torch.arange(start, pos + 1)
            pages = block_table[r, (js // page_size)].long()
            assert (pages >= 0).all(), "attention reads a position whose page was given back"
            K = k_pool[pages, :, (js % page_size), :].float()    # [n, Hkv, hd]
            V = v_pool[pages, :, (js % page_size), :].float()
            for h in range(Hq):
                s = (K[:, h // g, :] @ q[t, h].float()) * scale
                p = torch.softmax(s, 0)
                res[t, h] = p @ V[:, h // g, :]
        out.copy_(res.reshape(T, Hq * hd).to(out.dtype))

    # garuda/src/runtime/mod.rs:99-107
    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))

    # garuda/src/runtime/mod.rs:109-175
    def sample(self, logits, temperature, top_k, top_p, u, out, scratch):
        from .sampling_plain import candidates
        from .llama_plain import argmax_first
        for r in range(logits.shape[0]):
            row = logits[r].numpy()
            if float(temperature[r]) == 0.0:
                out[r] = argmax_first(row)
                continue
            cand = candidates(row, float(temperature[r]), int(top_k[r]), float(top_p[r]))
            total = np.float32(sum(np.float32(p) for _, p in cand))
            pick = cand[0][0]
            if total > 0:
                point = np.float32(np.float32(float(u[r])) * total)
                pick = cand[-1][0]
                for tok, p in cand:
                    point = np.float32(point - p)
                    if point <= 0:
                        pick = tok
                        break
            out[r] = pick
