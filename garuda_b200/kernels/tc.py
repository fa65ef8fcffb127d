"""Tensor-core (tcgen05 / TMEM / TMA) kernels of the bfloat16 path.

Each method returns True when it ran, False when the shape is one it does not
take (a row pitch that is not a multiple of 16 bytes, for instance), in which
case the caller uses the plain kernel instead.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int

import torch

from ..csrc.build import load_kernel_lib

_WAIT_NAMES = {1: "an operand tile never arrived (TMA)", 2: "a pipeline stage was never released",
               3: "the accumulator never completed", 4: "copies in flight did not land while winding down"}


class TensorCoreKernels:
    def __init__(self, ops):
        self.ops = ops
        self.lib = load_kernel_lib("garuda_tc")
        L = self.lib
        L.gb_last_error.restype = ctypes.c_char_p
        L.gb_gemm_tc.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        L.gb_gemm_tc.restype = c_int
        L.gb_gemm_tc_supported.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int]
        L.gb_gemm_tc_supported.restype = c_int
        L.gb_tc_error_check.restype = c_int

    def check_errors(self) -> None:
        """Synchronises, and raises if a kernel gave up on a wait since the last check."""
        code = self.lib.gb_tc_error_check()
        if code:
            from .ops import KernelError
            raise KernelError("a tensor-core kernel gave up waiting: " + _WAIT_NAMES.get(code, f"code {code}"))

    def _gemm(self, x, w, out, n_out, epi) -> bool:
        M, K = x.shape
        if not self.lib.gb_gemm_tc_supported(x.data_ptr(), w.data_ptr(), M, n_out, K):
            return False
        tag = 0 if out.dtype == torch.float32 else 1
        code = self.lib.gb_gemm_tc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, n_out, K, tag, epi,
                                   self.ops._stream())
        self.ops._check(self.lib, code, "gemm_tc")
        return True

    def linear(self, a, w, out, accumulate) -> bool:
        if w.dtype != torch.bfloat16 or out.dtype not in (torch.float32, torch.bfloat16):
            return False
        return self._gemm(a, w, out, w.shape[0], 1 if accumulate else 0)

    def linear_swiglu(self, h, w_gate_up, act) -> bool:
        if w_gate_up.dtype != torch.bfloat16 or act.dtype != torch.bfloat16:
            return False
        return self._gemm(h, w_gate_up, act, act.shape[1], 2)

    def paged_attention(self, *args) -> bool:
        return False
