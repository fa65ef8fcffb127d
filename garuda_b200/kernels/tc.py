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
        L.gb_tc_hint_next_stream.argtypes = [c_void_p, ctypes.c_longlong]
        L.gb_tc_hint_next_stream.restype = c_int
        self._attn = {}
        # The weights that the products of a step stream, in launch order: recorded during one run
        # (``record_streams``) and replayed as hints during the next (``hint_streams``), so that every
        # few-token product asks for the weights of the product behind it to be brought into L2 while
        # it waits out its own latencies. Used when a decode step is captured into a graph.
        self._recording = None
        self._plan, self._plan_at = None, 0

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

    # ------------------------------------------------------------------ hints of the stream to come
    HINT_LIMIT = 48 << 20        # no more than L2 can keep beside what is in use

    def record_streams(self):
        """Start noting which weights the step's products stream, in order."""
        self._recording, self._plan = [], None

    def hint_streams(self):
        """The products of the next run of the same step are told what comes behind them."""
        self._plan, self._plan_at, self._recording = self._recording, 0, None

    def forget_streams(self):
        self._plan = self._recording = None

    def _stream(self, w):
        """Called once per product, before its launch."""
        if self._recording is not None:
            self._recording.append((w.data_ptr(), w.numel() * w.element_size()))
        elif self._plan is not None:
            i, self._plan_at = self._plan_at, self._plan_at + 1
            if i < len(self._plan) and self._plan[i][0] == w.data_ptr() and i + 1 < len(self._plan):
                ptr, nbytes = self._plan[i + 1]
                self.lib.gb_tc_hint_next_stream(ptr, min(nbytes, self.HINT_LIMIT) & ~15)
            elif i >= len(self._plan) or self._plan[i][0] != w.data_ptr():
                self._plan = None          # another step than the one that was recorded

    def _gemm(self, x, w, out, n_out, epi, fold=None) -> bool:
        M, K = x.shape
        if not self.lib.gb_gemm_tc_supported(x.data_ptr(), w.data_ptr(), M, n_out, K):
            return False
        self._stream(w)
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
        self._stream(w_qkv)
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
                                             + [c_int] * 6 + [ctypes.c_longlong, c_int, c_void_p, ctypes.c_longlong, c_void_p])
            lib.gb_attention_scratch_bytes.argtypes = [c_int, c_int, c_int]
            lib.gb_attention_scratch_bytes.restype = ctypes.c_longlong
            lib.gb_attention_mma.restype = c_int
            lib.gb_attention_error_check.restype = c_int
            lib.gb_attention_set_error_sink.argtypes = [c_void_p]
            lib.gb_attention_set_error_sink.restype = c_int
            lib.gb_attention_set_error_sink(self.ops.error_word.data_ptr())
            self._attn[head_dim] = lib
        return lib

    @staticmethod
    def attention_plan(num_requests: int, kv_heads: int, max_kv_len: int, head_dim: int = 0):
        """(CTAs that share one decode request's keys, slots per warp of the kernel with per-thread
        copies, whether those CTAs are a thread-block cluster), from timings at 1 to 64 requests and
        contexts of 512 to 8,192.

        The kernel that copies pages by TMA (head sizes 64 and 128). A few requests: a cluster per
        (request, kv head), as many CTAs as the SMs take one each, every CTA with at least 8 tiles
        of 32 keys, clusters of eight for up to 12 (request, kv head) pairs, of six for up to 20
        (more of them than that do not fit the GPU at once and run in two rounds). When that would leave clusters of under four (many requests, or many kv
        heads): independent CTAs that merge through scratch memory, about 256 in all, each with at
        least 16 tiles, at most 16 per request.

        The kernel with per-thread copies (other head sizes; clusters): about two CTAs per SM; no warp
        without a tile where that can be avoided; clusters above four only while the whole grid stays
        under 64 CTAs; a second slot per warp, so that the next tile is fetched while one is computed,
        only while every CTA has an SM to itself."""
        pairs = max(num_requests * kv_heads, 1)
        if head_dim in (64, 128):
            tiles = max((max_kv_len + 31) // 32, 1)
            c = min(148 // pairs, tiles // 8, 8 if head_dim == 64 else 4)
            # whole clusters have to find room in one GPC: the GPU holds 12 clusters of eight and 20
            # of six at once (16 and 24 ran in two rounds); clusters of four it holds 32 of
            if c > 6 and pairs > 12:
                c = 6
            if c > 4 and pairs > 20:
                c = 4
            independent = max(1, min(256 // pairs, tiles // 16, 16))
            # clusters, unless they would be under four CTAs or independent CTAs would put twice as many
            # SMs to work (one request with a context of thousands of keys and heads of 128)
            if c >= 4 and independent < 2 * c:
                return c, 1, True
            return independent, 1, False
        tiles = max((max_kv_len + 63) // 64, 1)
        splits = max(1, min(2 * 148 // pairs, -(-tiles // 4), 8))
        if splits > 4 and pairs * 4 >= 64:
            splits = 4
        stages = 2 if tiles > 4 * splits and pairs * splits <= 148 else 1
        return splits, stages, True

    def paged_attention(self, q, k_pool, v_pool, block_table, cu_q, kv_lens, token_req, out, scale,
                        window, page_size, num_requests, max_q_len, max_kv_len, ws=None, min_q_len=1) -> bool:
        T, Hq, hd = q.shape
        Hkv = k_pool.shape[1]
        if hd % 16 or hd > 128 or Hq // Hkv > 64 or not scale > 0:
            return False
        lib = self._attention_lib(hd)
        g = Hq // Hkv
        has_decode = min_q_len * g <= 16
        splits, stages, cluster = self.attention_plan(num_requests, Hkv, max_kv_len, hd) if has_decode else (1, 1, True)
        # work space for the partial results of CTAs that share a request's keys; zeroed when it is made
        # (its counters), and every launch leaves the counters at zero
        need = int(lib.gb_attention_scratch_bytes(num_requests, Hkv, splits)) if has_decode and not cluster else 0
        scratch = None
        if need:
            scratch = (ws if ws is not None else self.ops.private_ws).get("attention_partials", (need,), torch.uint8, zero=True)
        code = lib.gb_attention_mma(
            q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), out.data_ptr(), block_table.data_ptr(),
            block_table.shape[1], cu_q.data_ptr(), kv_lens.data_ptr(), T, num_requests, Hq, Hkv, float(scale),
            int(window), int(page_size), int(max_q_len), int(min_q_len), int(splits), int(stages),
            int(k_pool.shape[0]), int(cluster), None if scratch is None else scratch.data_ptr(), need,
            self.ops._stream())
        self.ops._check(lib, code, "attention_mma", (1 if has_decode else 0) + (1 if max_q_len * g > 16 else 0))
        return True
