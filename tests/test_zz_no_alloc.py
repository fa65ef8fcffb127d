"""gb_sample_noalloc, the sampling entry point for callers that cannot allocate
device memory (a host that has given the whole device to its own pool, or a
loop that cannot afford cudaMalloc's device-wide synchronisation): called
through its exported C symbol, it must give the same tokens as gb_sample does
with the caller's scratch, on two calls in a row that share the built-in work
space, and refuse what does not fit. Collected last on purpose."""
import ctypes
from ctypes import c_void_p, c_int

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from garuda_b200.csrc.build import load_kernel_lib
    lib = load_kernel_lib("garuda_core")
    lib.gb_last_error.restype = ctypes.c_char_p
    lib.gb_sample.argtypes = [c_void_p] * 7 + [c_int, c_int, c_void_p]
    lib.gb_sample.restype = c_int
    lib.gb_sample_noalloc.argtypes = [c_void_p] * 6 + [c_int, c_int, c_void_p]
    lib.gb_sample_noalloc.restype = c_int
    return lib


def _problem(R, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = (torch.randn(R, V, generator=g) * 2).cuda()
    temperature = torch.tensor([0.0, 0.7, 1.0, 1.5] * (R // 4 + 1))[:R].float().cuda()
    top_k = torch.tensor([0, 40, 5, 0] * (R // 4 + 1))[:R].int().cuda()
    top_p = torch.tensor([1.0, 0.95, 1.0, 0.6] * (R // 4 + 1))[:R].float().cuda()
    u = torch.rand(R, generator=g).cuda()
    return logits, temperature, top_k, top_p, u


def test_no_alloc_sampling_matches_the_entry_point_with_caller_scratch():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, of different shapes, sharing the built-in work space
    for R, V, seed in ((9, 32000, 1), (16, 331, 2)):
        logits, temperature, top_k, top_p, u = _problem(R, V, seed)
        want = torch.full((R,), -1, dtype=torch.int32, device="cuda")
        scratch = torch.empty(R * V, dtype=torch.float32, device="cuda")
        rc = lib.gb_sample(logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                           u.data_ptr(), want.data_ptr(), scratch.data_ptr(), R, V, stream)
        assert rc == 0, lib.gb_last_error().decode()
        got = torch.full((R,), -2, dtype=torch.int32, device="cuda")
        rc = lib.gb_sample_noalloc(logits.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                                   u.data_ptr(), got.data_ptr(), R, V, stream)
        assert rc == 0, lib.gb_last_error().decode()
        torch.cuda.synchronize()
        # the same kernel on the same inputs: the tokens are identical, not merely close
        assert got.tolist() == want.tolist()
        assert all(0 <= t < V for t in got.tolist())


def test_no_alloc_sampling_refuses_what_does_not_fit():
    lib = _lib()
    R, V = 70, 32000                      # 2,240,000 floats: more than the built-in 2,097,152
    out = torch.full((R,), -5, dtype=torch.int32, device="cuda")
    rc = lib.gb_sample_noalloc(None, None, None, None, None, out.data_ptr(), R, V,
                               torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "work space" in lib.gb_last_error().decode()
    torch.cuda.synchronize()
    assert out.tolist() == [-5] * R       # nothing was launched
