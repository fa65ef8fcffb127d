"""gb_sample_noalloc, the sampling entry point for callers that cannot allocate
device memory (a host that has given the whole device to its own pool, or a
loop that cannot afford cudaMalloc's device-wide synchronisation): called
through its exported C symbol, it must give the same tokens as gb_sample does
with the caller's scratch and as the plain sampler, on calls in a row that
share the built-in work space, and refuse what does not fit. The vocabularies
of the first cases are too large for a row to stay in shared memory, so that
the built-in array is what the kernel really works in. Collected last on
purpose."""
import ctypes
from ctypes import c_void_p, c_int

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 2 * 1024 * 1024          # GB_SAMPLE_NOALLOC_MAX_FLOATS of no_alloc.h
IN_SHARED_UP_TO = 200 * 1024 // 4     # a row of more floats than this lives in the work space


def _lib():
    from garuda_b200.csrc.build import load_kernel_lib
    lib = load_kernel_lib("garuda_core")
    lib.gb_last_error.restype = ctypes.c_char_p
    lib.gb_sample.argtypes = [c_void_p] * 7 + [c_int, c_int, c_void_p]
    lib.gb_sample.restype = c_int
    lib.gb_sample_noalloc.argtypes = [c_void_p] * 6 + [c_int, c_int, c_void_p]
    lib.gb_sample_noalloc.restype = c_int
    return lib


def _problem(rows, V, seed):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(len(rows), V, generator=g) * 2
    col = lambda i, dt: torch.tensor([r[i] for r in rows], dtype=dt).cuda()
    return logits, (col(0, torch.float32), col(1, torch.int32), col(2, torch.float32), col(3, torch.float32))


def _both(lib, logits, params):
    """(tokens of gb_sample with the caller's scratch, tokens of gb_sample_noalloc)."""
    R, V = logits.shape
    dev = logits.cuda()
    temperature, top_k, top_p, u = params
    stream = torch.cuda.current_stream().cuda_stream
    want = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    scratch = torch.empty(R * V, dtype=torch.float32, device="cuda")
    rc = lib.gb_sample(dev.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                       u.data_ptr(), want.data_ptr(), scratch.data_ptr(), R, V, stream)
    assert rc == 0, lib.gb_last_error().decode()
    got = torch.full((R,), -2, dtype=torch.int32, device="cuda")
    rc = lib.gb_sample_noalloc(dev.data_ptr(), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                               u.data_ptr(), got.data_ptr(), R, V, stream)
    assert rc == 0, lib.gb_last_error().decode()
    torch.cuda.synchronize()
    return want.tolist(), got.tolist()


def test_no_alloc_sampling_works_in_its_own_array_and_matches_both_references():
    """Rows too long for shared memory: every pass over the probabilities goes through the built-in
    array at the address looked up with cudaGetSymbolAddress. Greedy, top-k, top-p alone and plain
    rows; then a second call of another shape, which finds the first call's values in the array and
    must not be misled by them; then shapes that fit in shared memory."""
    from tests.helpers import assert_tokens_follow_the_plain_sampler
    lib = _lib()
    base = [(0.0, 40, 0.95), (0.7, 40, 0.95), (1.0, 5, 1.0), (1.5, 0, 0.6), (1.0, 0, 1.0), (1.2, 1024, 0.9)]
    for V, draws, seed in ((65536, (0.0, 0.37, 0.999), 1), (128256, (0.61,), 2), (32000, (0.25, 0.9), 3), (331, (0.5,), 4)):
        rows = [(t, k, p, u) for t, k, p in base for u in draws]
        assert (V > IN_SHARED_UP_TO) == (V >= 65536) and len(rows) * V <= MAX_FLOATS
        logits, params = _problem(rows, V, seed)
        want, got = _both(lib, logits, params)
        # the same kernel on the same inputs: the tokens are identical, not merely close
        assert got == want, (V, got, want)
        assert all(0 <= t < V for t in got)
        assert_tokens_follow_the_plain_sampler(rows, logits, got)


def test_no_alloc_sampling_takes_exactly_what_fits_and_refuses_one_more():
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    R, V = 32, 65536                      # exactly the 2,097,152 floats of the built-in array
    assert R * V == MAX_FLOATS
    rows = [(1.0, 0, 1.0, (i + 0.5) / R) for i in range(R)]
    logits, params = _problem(rows, V, 9)
    want, got = _both(lib, logits, params)
    assert got == want and len(set(got)) > 1
    for R, V in ((70, 32000), (MAX_FLOATS + 1, 1), (1, MAX_FLOATS + 1)):
        out = torch.full((min(R, 128),), -5, dtype=torch.int32, device="cuda")
        rc = lib.gb_sample_noalloc(None, None, None, None, None, out.data_ptr(), R, V, stream)
        assert rc != 0 and "work space" in lib.gb_last_error().decode()
        torch.cuda.synchronize()
        assert set(out.tolist()) == {-5}       # nothing was launched
