"""Tensor-core (tcgen05 / TMEM / TMA) kernels of the bfloat16 path.

Each method returns True when it ran, False when the shape is one it does not
take (a row pitch that is not a multiple of 16 bytes, for instance), in which
case the caller uses the plain kernel instead.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_float

import torch

from ..csrc.build import load_kernel_lib, attention_lib_name

_WAIT_NAMES = {1: "an operand tile never arrived (TMA)", 2: "a pipeline stage was never released",
               3: "the accumulator never completed", 4: "copies in flight did not land while winding down",
               5: "a decode attention cluster never delivered its partial results"}


class NormFold(ctypes.Structure):
    """GbNormFold of gemm_tcgen05.cu: an RMS norm folded into the products around it."""
    _fields_ = [("sums_in", c_void_p), ("tiles_in", c_int), ("eps", c_float), ("inv_width", c_float),
                ("h_out", c_void_p), ("weight", c_void_p), ("sums_out", c_void_p), ("sums_ld", c_int)]


class TensorCoreKernels:
    def __init__(self, ops):
        self.ops = ops
        self.lib = load_kernel_lib("garuda_tc")
        L = self.lib
        L.gb_last_error.restype = ctypes.c_char_p
        L.gb_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                 ctypes.POINTER(NormFold), c_void_p]
        L.gb_gemm_tc.restype = c_int
        L.gb_gemm_tc_norm_tiles.argtypes = [c_int, c_int]
        L.gb_gemm_tc_norm_tiles.restype = c_int
        L.gb_gemm_tc_supported.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int]
        L.gb_gemm_tc_supported.restype = c_int
        L.gb_tc_error_check.restype = c_int
        L.gb_tc_set_error_sink.argtypes = [c_void_p]
        L.gb_tc_set_error_sink.restype = c_int
        L.gb_tc_selftest_wait_runs_out.argtypes = [c_int, c_void_p]
        L.gb_tc_selftest_wait_runs_out.restype = c_int
        if L.gb_tc_set_error_sink(ops.error_word.data_ptr()):
            from .ops import KernelError
            raise KernelError("the tensor-core library could not be given the host's error word")
        L.gb_gemm_tc_qkv.argtypes = ([c_void_p, c_void_p, c_int, c_int] + [c_void_p] * 6 + [c_int] * 4 + [c_void_p]
                                     + [c_int, c_int, ctypes.POINTER(NormFold), c_void_p])
        L.gb_gemm_tc_qkv.restype = c_int
        self._attn = {}

    def check_errors(self) -> None:
        """Synchronises, and raises if a kernel gave up on a wait since the last check."""
        code = self.lib.gb_tc_error_check()
        for lib in self._attn.values():
            code = lib.gb_attention_error_check() or code
        seen, self.ops.error_word[0] = int(self.ops.error_word[0]), 0
        code = code or seen
        if code:
            from .ops import KernelError
            raise KernelError("a tensor-core kernel gave up waiting: " + _WAIT_NAMES.get(code, f"code {code}"))

    def selftest_wait_runs_out(self, limit_us: int = 1000) -> None:
        """Launches a kernel whose only wait runs out after ``limit_us`` microseconds and which
        then records its error code like any product kernel (for tests of the error path)."""
        self.ops._check(self.lib, self.lib.gb_tc_selftest_wait_runs_out(int(limit_us), self.ops._stream()),
                        "selftest_wait_runs_out")

    # ------------------------------------------------------------------ folded norms
    def norm_tiles(self, tokens: int, features: int) -> int:
        """Rows of partial sums that an accumulating product of this shape writes when the norm
        behind it is folded in; 0: it folds none."""
        return int(self.lib.gb_gemm_tc_norm_tiles(tokens, features))

    @staticmethod
    def _consume(pending):
        """The kernel's argument for a product whose tokens are a ``PendingNorm``."""
        if pending is None:
            return None
        return NormFold(sums_in=pending.sums.data_ptr(), tiles_in=pending.sums.shape[0], eps=pending.eps,
                        inv_width=1.0 / pending.values.shape[1], sums_ld=pending.sums.shape[1])

    def _gemm(self, x, w, out, n_out, epi, fold=None) -> bool:
        M, K = x.shape
        if not self.lib.gb_gemm_tc_supported(x.data_ptr(), w.data_ptr(), M, n_out, K):
            return False
        tag = 0 if out.dtype == torch.float32 else 1
        code = self.lib.gb_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, n_out, K, tag, epi,
                                   None if fold is None else ctypes.byref(fold), self.ops._stream())
        self.ops._check(self.lib, code, "gemm_tc")
        return True

    def linear(self, a, w, out, accumulate, emit=None) -> bool:
        """``emit``: a ``PendingNorm`` whose values and sums this accumulating product fills."""
        if w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
            return False
        fold = None
        if emit is not None:
            fold = NormFold(h_out=emit.values.data_ptr(), weight=emit.weight.data_ptr(),
                            sums_out=emit.sums.data_ptr(), sums_ld=emit.sums.shape[1])
        return self._gemm(a, w, out, w.shape[0], 1 if accumulate else 0, fold)

    def takes_qkv(self, h, w_qkv, q_out, head_dim) -> bool:
        """Whether the fused query/key/value product takes these operands (head sizes that
        divide 128, bfloat16, rows the TMA can address)."""
        M, K = h.shape
        return (h.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
                and head_dim % 16 == 0 and 128 % head_dim == 0
                and bool(self.lib.gb_gemm_tc_supported(h.data_ptr(), w_qkv.data_ptr(), M, w_qkv.shape[0], K)))

    def qkv_rope_append(self, h, w_qkv, q_out, k_pool, v_pool, positions, token_req, block_table,
                        heads, kv_heads, head_dim, cos_sin, interleaved, page_size, pending=None) -> None:
        """The query/key/value product with the rotation and the cache write in its
        epilogue. ``cos_sin``: ``CudaOps.rope_table`` of the step's positions, or None
        (no rotation). ``pending``: the ``PendingNorm`` whose values ``h`` is."""
        M, K = h.shape
        fold = self._consume(pending)
        code = self.lib.gb_gemm_tc_qkv(
            h.data_ptr(), w_qkv.data_ptr(), M, K, q_out.data_ptr(),
            None if k_pool is None else k_pool.data_ptr(), None if v_pool is None else v_pool.data_ptr(),
            positions.data_ptr(), token_req.data_ptr(), None if block_table is None else block_table.data_ptr(),
            0 if block_table is None else block_table.shape[1], heads, kv_heads, head_dim,
            None if cos_sin is None else cos_sin.data_ptr(), 0 if not interleaved else 1,
            int(page_size), None if fold is None else ctypes.byref(fold), self.ops._stream())
        self.ops._check(self.lib, code, "gemm_tc_qkv")

    def linear_swiglu(self, h, w_gate_up, act, pending=None) -> bool:
        """``w_gate_up``: the packed layout of ``CudaOps.pack_gate_up``. ``pending``: the
        ``PendingNorm`` whose values ``h`` is."""
        F = act.shape[1]
        if (w_gate_up.dtype != torch.bfloat16 or act.dtype != torch.bfloat16
                or w_gate_up.shape[0] != 128 * ((F + 63) // 64)):
            return False
        return self._gemm(h, w_gate_up, act, F, 2, self._consume(pending))

    # ------------------------------------------------------------------ attention
    def _attention_lib(self, head_dim: int):
        lib = self._attn.get(head_dim)
        if lib is None:
            lib = load_kernel_lib(attention_lib_name(head_dim))
            lib.gb_last_error.restype = ctypes.c_char_p
            lib.gb_attention_mma.argtypes = ([c_void_p] * 5 + [c_int] + [c_void_p] * 2 + [c_int] * 4 + [c_float]
                                             + [c_int] * 6 + [ctypes.c_longlong, c_void_p])
            lib.gb_attention_mma.restype = c_int
            lib.gb_attention_error_check.restype = c_int
            lib.gb_attention_set_error_sink.argtypes = [c_void_p]
            lib.gb_attention_set_error_sink.restype = c_int
            lib.gb_attention_set_error_sink(self.ops.error_word.data_ptr())
            self._attn[head_dim] = lib
        return lib

    @staticmethod
    def attention_plan(num_requests: int, kv_heads: int, max_kv_len: int):
        """(CTAs that share one decode request's keys, slots per warp), from timings
        at 1 to 64 requests: about two CTAs per SM; no warp without a tile where
        that can be avoided; clusters above four only while the whole grid stays
        under 64 CTAs (larger clusters are placed late and merge longer); a second
        slot per warp, so that the next tile is fetched while one is computed, only
        while every CTA has an SM to itself (two slots take most of its shared
        memory)."""
        tiles = max((max_kv_len + 63) // 64, 1)
        pairs = max(num_requests * kv_heads, 1)
        splits = max(1, min(2 * 148 // pairs, -(-tiles // 4), 8))
        if splits > 4 and pairs * 4 >= 64:
            splits = 4
        stages = 2 if tiles > 4 * splits and pairs * splits <= 148 else 1
        return splits, stages

    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale,
                        window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1) -> bool:
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        if hd % 16 or hd > 128 or Hq // Hkv > 64 or not scale > 0:
            return False
        lib = self._attention_lib(hd)
        g = Hq // Hkv
        has_decode = min_q_len * g <= 16
        splits, stages = self.attention_plan(num_requests, Hkv, max_kv_len) if has_decode else (1, 1)
        code = lib.gb_attention_mma(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], cu_q.data_ptr(), kv_lens.data_ptr(), T, num_requests, Hq, Hkv, float(scale),
            int(window), int(page_size), int(max_q_len), int(min_q_len), int(splits), int(stages),
            int(k_pool.shape[0]), self.ops._stream())
        self.ops._check(lib, code, "attention_mma", (1 if has_decode else 0) + (1 if max_q_len * g > 16 else 0))
        return True
