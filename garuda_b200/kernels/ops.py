"""The kernel set of the product path: thin, checking wrappers around the CUDA
entry points. There is no other implementation behind them: without a CUDA
device or without the compiled library every call fails loudly.

Each method takes torch tensors that live on the device, checks dtypes, shapes
and contiguity, and launches on torch's current stream.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from ctypes import c_void_p, c_int, c_float, c_longlong
from typing import Optional

import numpy as np
import torch

from ..csrc.build import load_kernel_lib

GB_F32, GB_BF16 = 0, 1
_TAG = {torch.float32: GB_F32, torch.bfloat16: GB_BF16}


class KernelError(RuntimeError):
    pass


def _tag(t: torch.Tensor, what: str) -> int:
    try:
        return _TAG[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_ERROR_WORD = None


def _error_word() -> torch.Tensor:
    global _ERROR_WORD
    if _ERROR_WORD is None:
        _ERROR_WORD = torch.zeros(4, dtype=torch.int32).pin_memory()
    return _ERROR_WORD


class PendingNorm:
    """An RMS norm of which only the first half has run, folded into the product that wrote the
    residual stream ``x``: ``values`` is ``x * weight`` in bfloat16 and ``sums`` ``[tiles, T]``
    holds partial sums of ``x^2`` per token. A product that takes it as its tokens multiplies
    its results by ``1/sqrt(sum / width + eps)`` (32-bit); ``materialize`` runs the norm part
    on ``x`` the ordinary way instead, for a consumer that cannot."""

    def __init__(self, values, sums, weight, eps, norm, x):
        self.values, self.sums, self.weight, self.eps, self.norm, self.x = values, sums, weight, float(eps), norm, x

    @property
    def shape(self):
        return self.values.shape

    @property
    def dtype(self):
        return self.values.dtype

    def materialize(self, ctx):
        return self.norm.forward(ctx, self.x)


class CudaOps:
    """Hand-written sm_100a kernels. ``tensor_cores=False`` keeps every matrix
    product and the attention on the plain 32-bit-arithmetic kernels (the true
    32-bit path uses them in any case)."""

    name = "cuda"

    def __init__(self, device="cuda:0", tensor_cores: bool = True):
        if not torch.cuda.is_available():
            raise KernelError("garuda_b200 needs a CUDA device: there is no CPU path")
        self.device = torch.device(device)
        self.core = load_kernel_lib("garuda_core")
        self._declare_core()
        # A word of pinned host memory that a kernel whose bounded wait ran out writes its code to (the
        # device reaches pinned host memory directly); ``failed_wait`` reads it without a copy.
        # The kernel libraries are loaded once per process, so the word is one per process as well.
        self.error_word = _error_word()
        self.tc = None
        if tensor_cores:
            from .tc import TensorCoreKernels
            self.tc = TensorCoreKernels(self)
        # whether products fold the norms around them in (``linear``'s ``emit_norm``); a test flips
        # it to compare the two ways
        self.folds_norms = self.tc is not None
        self._inv_freq = {}
        self._held_stream = None
        self.launches = 0
        from ..engine.batch import Workspace
        self.private_ws = Workspace(self.device)   # scratch for calls made outside a step

    def failed_wait(self) -> int:
        """The code of a bounded wait that ran out in a kernel which has finished by now, or 0.
        Costs nothing: call it where the host has just waited for a step's results. The full check
        (``tc.check_errors``) synchronises and clears."""
        return int(self.error_word[0])

    # ------------------------------------------------------------------ plumbing
    def _declare_core(self):
        L = self.core
        L.gb_last_error.restype = ctypes.c_char_p
        sig = {
            "gb_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "gb_rmsnorm": [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
            "gb_rope_kv_append": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                  c_int, c_void_p],
            "gb_rope_inplace": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
            "gb_rope_table": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
            "gb_silu_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
            "gb_residual_add": [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
            "gb_gemm_simple": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
            "gb_attention_simple": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                    c_void_p],
            "gb_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p],
            "gb_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                          c_void_p],
            "gb_sample_small_k": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                  c_void_p],
        }
        for name, argtypes in sig.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = c_int

    def _stream(self):
        if self._held_stream is not None:
            return self._held_stream
        return torch.cuda.current_stream(self.device).cuda_stream

    @contextlib.contextmanager
    def on_current_stream(self):
        """Within the block every kernel is launched on the stream that is current now (asked
        for once, not per launch). The caller must not change the current stream inside."""
        outer = self._held_stream
        self._held_stream = torch.cuda.current_stream(self.device).cuda_stream
        try:
            yield
        finally:
            self._held_stream = outer

    def _check(self, lib, code: int, what: str, kernels: int = 1) -> None:
        if code != 0:
            raise KernelError(f"{what}: {lib.gb_last_error().decode()}")
        self.launches += kernels     # kernels of this library launched so far (not counting graph replays)

    def _on_device(self, *tensors):
        for t in tensors:
            if t is not None:
                _need(t.is_cuda, "kernel operands must live on the CUDA device")

    # ------------------------------------------------------------------ parts
    def inv_freq(self, rotary) -> torch.Tensor:
        """One frequency per pair of the head for a ``RotaryParams``: its own table if it has
        one, else ``1 / theta^(2i/head_dim)`` in 32-bit (garuda/src/simd/mod.rs:199). Made once
        per parameter set."""
        if rotary not in self._inv_freq:
            from ..parts.rotary import rotary_frequencies
            self._inv_freq[rotary] = torch.from_numpy(rotary_frequencies(rotary)).to(self.device)
        return self._inv_freq[rotary]

    def embedding(self, table, ids, out):
        self._on_device(table, ids, out)
        _need(out.dtype == torch.float32 and out.is_contiguous(), "embedding: out must be contiguous float32")
        _need(ids.dtype == torch.int32, "embedding: ids must be int32")
        _need(table.is_contiguous() and table.shape[1] == out.shape[1], "embedding: widths differ")
        T = ids.shape[0]
        _need(out.shape[0] >= T, "embedding: out has too few rows")
        self._check(self.core, self.core.gb_embedding(
            table.data_ptr(), _tag(table, "embedding table"), ids.data_ptr(), out.data_ptr(), T,
            table.shape[1], table.shape[0], self._stream()), "embedding")

    def rmsnorm(self, x, weight, eps, out, rows=None):
        self._on_device(x, weight, out, rows)
        _need(x.dtype == torch.float32 and x.is_contiguous(), "rmsnorm: x must be contiguous float32")
        d = x.shape[1]
        _need(weight.numel() == d and out.shape[1] == d and out.is_contiguous(), "rmsnorm: widths differ")
        n = x.shape[0] if rows is None else rows.shape[0]
        _need(out.shape[0] == n, "rmsnorm: out has the wrong number of rows")
        if rows is not None:
            _need(rows.dtype == torch.int32, "rmsnorm: rows must be int32")
        self._check(self.core, self.core.gb_rmsnorm(
            x.data_ptr(), weight.data_ptr(), _tag(weight, "norm weight"), float(eps), out.data_ptr(),
            _tag(out, "rmsnorm out"), _ptr(rows), n, d, self._stream()), "rmsnorm")

    def linear(self, a, w, out, accumulate: bool = False, ctx=None, emit_norm=None):
        """``out[M,N] (+)= a[M,K] @ w[N,K]^T``; accumulation is into a 32-bit ``out``.

        ``emit_norm`` (with ``ctx``): the norm part that will be applied to ``out`` next. Where
        the kernel can, it folds that norm's first half into this product and returns a
        ``PendingNorm`` to hand to ``qkv_rope_append`` or ``linear_swiglu`` in place of the
        normed tensor; else it returns None and the norm runs as usual."""
        self._on_device(a, w, out)
        _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "linear: operands must be matrices")
        M, K = a.shape
        N = w.shape[0]
        if not (w.shape[1] == K and out.shape == (M, N)):       # the message is made only when it is needed
            _need(False, f"linear: shapes {tuple(a.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
        _need(a.dtype == w.dtype, "linear: a and w must have one dtype")
        _need(a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "linear: operands must be contiguous")
        if self.tc is not None and a.dtype == torch.bfloat16:
            pending = self._pending_for(ctx, emit_norm, out, accumulate)
            if self.tc.linear(a, w, out, accumulate, emit=pending):
                return pending
        self._check(self.core, self.core.gb_gemm_simple(
            a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, _tag(a, "linear input"),
            _tag(out, "linear output"), int(accumulate), self._stream()), "linear")

    def _pending_for(self, ctx, norm, x, accumulate):
        """A ``PendingNorm`` with buffers for the product that adds into ``x``, or None."""
        if norm is None or ctx is None or not accumulate or x.dtype != torch.float32:
            return None
        fold = norm.fold() if hasattr(norm, "fold") else None
        T, d = x.shape
        tiles = self.tc.norm_tiles(T, d)
        if fold is None or not tiles:
            return None
        weight, eps = fold
        # two sets of buffers in turn: a block's second norm is pending while the first one's values are
        # still the operand of no kernel, but never more than two at a time
        turn = ctx.step_cache.get("pending_turn", 0) ^ 1
        ctx.step_cache["pending_turn"] = turn
        values = ctx.ws.get(f"pending_values_{turn}", (T, d), torch.bfloat16)
        sums = ctx.ws.get(f"pending_sums_{turn}", (tiles, T), torch.float32)
        return PendingNorm(values, sums, weight, eps, norm, x)

    def normed(self, ctx, h):
        """``h`` as a tensor: a ``PendingNorm`` is run as the ordinary norm."""
        return h.materialize(ctx) if isinstance(h, PendingNorm) else h

    def pack_gate_up(self, gate, up):
        """The layout ``linear_swiglu`` wants. With the tensor-core kernels: gate and
        up rows packed in groups of 64 (rows ``[128 g, 128 g + 64)`` are gate rows
        ``64 g ..``, the next 64 the matching up rows, zero rows padding the last
        group), so that a 128-row tile holds both values of 64 features. Without
        them: gate rows, then up rows."""
        F, K = gate.shape
        if self.tc is None or gate.dtype != torch.bfloat16:
            return torch.cat([gate, up], dim=0).contiguous()
        groups = (F + 63) // 64
        halves = []
        for m in (gate, up):
            padded = torch.zeros(groups * 64, K, dtype=m.dtype, device=m.device)
            padded[:F] = m
            halves.append(padded.view(groups, 64, K))
        packed = torch.stack(halves, dim=1).reshape(groups * 128, K).contiguous()
        packed.gb_group = 64
        return packed

    def linear_swiglu(self, ctx, h, w_gate_up, act):
        """``act[M,F] = silu(h @ gate^T) * (h @ up^T)``, the activation in 32-bit."""
        M, F = act.shape
        group = getattr(w_gate_up, "gb_group", 0)
        if isinstance(h, PendingNorm):
            if group == 64 and self.tc is not None and self.tc.linear_swiglu(h.values, w_gate_up, act, pending=h):
                return
            h = h.materialize(ctx)
        if (group == 64 and self.tc is not None and h.dtype == torch.bfloat16
                and self.tc.linear_swiglu(h, w_gate_up, act)):
            return
        tmp = ctx.ws.get("gate_up", (M, w_gate_up.shape[0]), torch.float32)
        self.linear(h, w_gate_up, tmp)
        self.silu_mul(tmp, act, group)

    def silu_mul(self, gate_up, out, group: int = 0):
        """``out[M,F] = silu(gate) * up``; ``gate_up`` rows are ``[gate | up]``, or with
        ``group`` 64 the packed layout of ``pack_gate_up``."""
        self._on_device(gate_up, out)
        M, F = out.shape
        width = 2 * group * ((F + group - 1) // group) if group else 2 * F
        _need(gate_up.shape == (M, width) and gate_up.is_contiguous() and out.is_contiguous(),
              f"silu_mul: gate_up must be [M, {width}] for out [M, {F}]")
        self._check(self.core, self.core.gb_silu_mul(
            gate_up.data_ptr(), _tag(gate_up, "silu_mul in"), out.data_ptr(), _tag(out, "silu_mul out"),
            M, F, group, width, self._stream()), "silu_mul")

    def residual_add(self, x, y):
        self._on_device(x, y)
        _need(x.dtype == torch.float32 and x.shape == y.shape and x.is_contiguous() and y.is_contiguous(),
              "residual_add: x must be contiguous float32 of y's shape")
        self._check(self.core, self.core.gb_residual_add(
            x.data_ptr(), y.data_ptr(), _tag(y, "residual_add y"), x.numel(), self._stream()), "residual_add")

    def qkv_rope_append(self, ctx, h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                        heads, kv_heads, head_dim, rotary, page_size):
        """``h @ w_qkv^T``, split into heads; queries and keys rotated (``rotary`` None:
        not), queries to ``q_out [T, heads, head_dim]``, keys and values into their
        pages. One kernel where the tensor-core product takes the shape, else the
        product in 32-bit followed by ``rope_kv_append``."""
        pending = h if isinstance(h, PendingNorm) else None
        if pending is not None:
            h = pending.values
            if self.tc is None or not self.tc.takes_qkv(h, w_qkv, q_out, head_dim):
                h, pending = pending.materialize(ctx), None
        self._on_device(h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table)
        T = h.shape[0]
        _need(w_qkv.shape == ((heads + 2 * kv_heads) * head_dim, h.shape[1]), "qkv_rope_append: weight shape")
        _need(q_out.is_contiguous() and q_out.shape == (T, heads, head_dim), "qkv_rope_append: q_out shape")
        if kv_heads:
            _need(k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.dtype == q_out.dtype
                  and tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), "qkv_rope_append: pool shape")
            _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "qkv_rope_append: block table")
        _need(positions.dtype == torch.int32 and token_req.dtype == torch.int32, "qkv_rope_append: int32 indices")
        if self.tc is not None and self.tc.takes_qkv(h, w_qkv, q_out, head_dim):
            table = None if rotary is None else self.rope_table(ctx, positions, rotary)
            self.tc.qkv_rope_append(h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads,
                                    kv_heads, head_dim, table, None if rotary is None else rotary.interleaved,
                                    page_size, pending=pending)
            return
        qkv = ctx.ws.get("qkv", (T, w_qkv.shape[0]), torch.float32)
        self.linear(h, w_qkv, qkv)
        self.rope_kv_append(qkv, q_out, k_pool, v_pool, positions, token_req, block_table, heads, kv_heads,
                            head_dim, rotary, page_size)

    def rope_table(self, ctx, positions, rotary):
        """``[T, head_dim / 2, 2]`` cosines and sines of every token's angles, made once per
        step (kept in the step's context) for every layer's fused projection to read."""
        half = rotary.head_dim // 2
        key = ("rope_table", rotary, positions.data_ptr(), positions.shape[0])
        cache = getattr(ctx, "step_cache", None)
        if cache is not None and key in cache:
            return cache[key]
        T = positions.shape[0]
        name = f"rope_table_{rotary.theta}_{rotary.head_dim}_{hash(rotary.inv_freq)}"
        out = ctx.ws.get(name, (T, half, 2), torch.float32)
        inv = self.inv_freq(rotary)
        code = self.core.gb_rope_table(positions.data_ptr(), inv.data_ptr(), out.data_ptr(), T, half, self._stream())
        self._check(self.core, code, "rope_table")
        if cache is not None:
            cache[key] = out
        return out

    def rope_kv_append(self, qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                       heads, kv_heads, head_dim, rotary, page_size):
        """Split ``qkv [T, (heads + 2 kv_heads) head_dim]``, rotate queries and keys
        (``rotary`` None: leave them), write queries to ``q_out [T, heads, head_dim]``
        and keys and values into their pages."""
        self._on_device(qkv, q_out, k_pool, v_pool, positions, token_req, block_table)
        T = qkv.shape[0]
        _need(qkv.stride(1) == 1 and qkv.shape[1] == (heads + 2 * kv_heads) * head_dim,
              "rope_kv_append: qkv has the wrong width")
        _need(q_out.is_contiguous() and q_out.shape == (T, heads, head_dim), "rope_kv_append: q_out shape")
        _need(positions.dtype == torch.int32 and token_req.dtype == torch.int32, "rope_kv_append: int32 indices")
        if kv_heads:
            _need(k_pool.dtype == q_out.dtype and v_pool.dtype == q_out.dtype, "rope_kv_append: cache dtype")
            _need(k_pool.is_contiguous() and v_pool.is_contiguous() and
                  tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), "rope_kv_append: pool shape")
            _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "rope_kv_append: block table")
        inv = None
        inter = 0
        if rotary is not None:
            _need(rotary.head_dim == head_dim, "rope_kv_append: rotary is for another head_dim")
            inv = self.inv_freq(rotary)
            inter = int(rotary.interleaved)
        self._check(self.core, self.core.gb_rope_kv_append(
            qkv.data_ptr(), _tag(qkv, "qkv"), qkv.stride(0), q_out.data_ptr(), _ptr(k_pool), _ptr(v_pool),
            _tag(q_out, "q_out"), positions.data_ptr(), token_req.data_ptr(), _ptr(block_table),
            block_table.shape[1] if block_table is not None else 0, T, heads, kv_heads, head_dim,
            _ptr(inv), inter, page_size, self._stream()), "rope_kv_append")

    def rope_inplace(self, x, positions, rotary):
        """Rotate ``x [T, H, rotary.head_dim]`` (float32; rows and heads may be strided, so a
        view of every head's first channels will do) in place."""
        self._on_device(x, positions)
        _need(x.dtype == torch.float32 and x.dim() == 3 and x.stride(2) == 1 and x.stride(1) >= x.shape[2],
              "rope_inplace: x must be float32 [T, H, width] with unit stride along the width")
        T, H, hd = x.shape
        _need(hd == rotary.head_dim, "rope_inplace: the view is not as wide as the rotation")
        self._check(self.core, self.core.gb_rope_inplace(
            x.data_ptr(), x.stride(0), x.stride(1), T, H, hd, positions.data_ptr(),
            self.inv_freq(rotary).data_ptr(), int(rotary.interleaved), self._stream()), "rope_inplace")

    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out,
                        scale, window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1):
        self._on_device(q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out)
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        _need(q.is_contiguous() and out.is_contiguous() and out.shape == (T, Hq * hd), "attention: q/out shape")
        _need(q.dtype == k_pool.dtype == v_pool.dtype == out.dtype, "attention: one dtype for q, cache and out")
        _need(tuple(k_pool.shape[1:]) == (Hkv, page_size, hd) and k_pool.shape == v_pool.shape,
              "attention: pool shape")
        _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: block table")
        if self.tc is not None and q.dtype == torch.bfloat16 and self.tc.paged_attention(
                q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale, window, page_size,
                num_requests, max_q_len, max_kv_len, ws, min_q_len):
            return
        self._check(self.core, self.core.gb_attention_simple(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _tag(q, "attention q"),
            block_table.data_ptr(), block_table.shape[1], cu_q.data_ptr(), kv_lens.data_ptr(),
            token_req.data_ptr(), out.data_ptr(), T, Hq, Hkv, hd, float(scale), int(window),
            int(page_size), self._stream()), "attention")

    # ------------------------------------------------------------------ sampling
    def argmax(self, logits, out):
        self._on_device(logits, out)
        _need(logits.dtype == torch.float32 and logits.is_contiguous() and out.dtype == torch.int32,
              "argmax: float32 logits, int32 out")
        R, V = logits.shape
        self._check(self.core, self.core.gb_argmax(logits.data_ptr(), out.data_ptr(), R, V, self._stream()),
                    "argmax")

    #: ``small_top_k`` may be said of rows that are greedy or have a top_k of 1 to this
    SMALL_TOP_K = 64

    def sample(self, logits, temperature, top_k, top_p, u, out, scratch, small_top_k: bool = False):
        """One token per row. ``temperature`` 0 is greedy; ``u`` is the row's uniform
        draw. ``scratch``: float32 ``[R, V]`` work space. ``small_top_k``: the caller knows
        that every row is greedy or has a top_k of 1 to ``SMALL_TOP_K`` (eight CTAs then share a
        row; the tokens are the same either way)."""
        self._on_device(logits, temperature, top_k, top_p, u, out, scratch)
        R, V = logits.shape
        _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: float32 logits")
        _need(temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and u.dtype == torch.float32
              and top_k.dtype == torch.int32 and out.dtype == torch.int32, "sample: parameter dtypes")
        _need(scratch.dtype == torch.float32 and scratch.numel() >= R * V, "sample: scratch too small")
        fn = self.core.gb_sample_small_k if small_top_k else self.core.gb_sample
        self._check(self.core, fn(
            logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(), u.data_ptr(),
            out.data_ptr(), scratch.data_ptr(), R, V, self._stream()), "sample")
