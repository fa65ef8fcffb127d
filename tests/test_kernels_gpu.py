"""Each CUDA kernel alone against its plain reference (tests/plain/cpu_ops.py),
at sizes other than the tiny models': widths and vocabularies that are no power
of two, head sizes in steps of 16, odd numbers of heads and groups."""
import ctypes

import numpy as np
import pytest
import torch

from tests.plain.cpu_ops import CpuOps
from tests.plain.sampling_plain import Rng

pytestmark = pytest.mark.gpu
cpu = CpuOps()


@pytest.fixture(scope="module")
def ops():
    from garuda_b200.kernels import CudaOps
    return CudaOps("cuda:0", tensor_cores=True)


def dev(t):
    return t.cuda()


def close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    scale = max(float(want.abs().max()), 1e-6)
    err = float((got - want).abs().max())
    assert torch.isfinite(got).all(), what
    assert err <= tol * scale, f"{what}: {err:.3e} > {tol * scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(ops, dtype):
    table = torch.randn(331, 72).to(dtype)
    ids = torch.tensor([0, 330, 5, 5, 17], dtype=torch.int32)
    out = torch.zeros(5, 72, device="cuda")
    ops.embedding(dev(table), dev(ids), out)
    assert torch.equal(out.cpu(), table[ids.long()].float())


@pytest.mark.parametrize("d,eps", [(72, 1e-5), (2048, 1e-6), (100, 1e-3)])
@pytest.mark.parametrize("wdt,odt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.bfloat16)])
def test_rmsnorm(ops, d, eps, wdt, odt):
    x = torch.randn(9, d) * 3
    w = (1 + 0.1 * torch.randn(d)).to(wdt)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    for r in (None, rows):
        n = 9 if r is None else 3
        ref = torch.zeros(n, d)
        cpu.rmsnorm(x, w, eps, ref, r)
        out = torch.zeros(n, d, dtype=odt, device="cuda")
        ops.rmsnorm(dev(x), dev(w), eps, out, None if r is None else dev(r))
        close(out, ref, 1e-6 if odt == torch.float32 else 8e-3, "rmsnorm")


@pytest.mark.parametrize("M,N,K", [(1, 130, 72), (7, 331, 200), (70, 96, 176), (130, 250, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_plain_matrix_product(ops, M, N, K, dtype):
    from garuda_b200.kernels import CudaOps
    plain = CudaOps("cuda:0", tensor_cores=False)
    a, w = torch.randn(M, K).to(dtype), (torch.randn(N, K) * 0.1).to(dtype)
    ref = a.float() @ w.float().t()
    out = torch.zeros(M, N, device="cuda")
    plain.linear(dev(a), dev(w), out)
    close(out, ref, 2e-6, "store")
    base = torch.randn(M, N)
    acc = dev(base.clone())
    plain.linear(dev(a), dev(w), acc, accumulate=True)
    close(acc, base + ref, 2e-6, "accumulate")


def test_plain_product_does_not_depend_on_the_batch(ops):
    from garuda_b200.kernels import CudaOps
    plain = CudaOps("cuda:0", tensor_cores=False)
    a, w = torch.randn(77, 200), torch.randn(130, 200)
    whole = torch.zeros(77, 130, device="cuda")
    plain.linear(dev(a), dev(w), whole)
    one = torch.zeros(1, 130, device="cuda")
    plain.linear(dev(a[40:41].contiguous()), dev(w), one)
    assert torch.equal(whole[40:41], one)


@pytest.mark.parametrize("M", [1, 8, 16, 17, 40, 64, 65, 130, 300])
@pytest.mark.parametrize("N,K", [(250, 72), (331, 200), (1000, 1024)])
def test_tensor_core_product(ops, M, N, K):
    a, w = (torch.randn(M, K) * 0.5).bfloat16(), (torch.randn(N, K) * 0.1).bfloat16()
    ref = a.float() @ w.float().t()
    for odt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        out = torch.full((M, N), 5.0, dtype=odt, device="cuda")
        assert ops.tc.linear(dev(a), dev(w), out, False)
        close(out, ref, tol, f"store {odt}")
    base = torch.randn(M, N)
    acc = dev(base.clone())
    assert ops.tc.linear(dev(a), dev(w), acc, True)
    close(acc, base + ref, 1e-5, "accumulate")
    ops.tc.check_errors()


@pytest.mark.parametrize("M", [1, 5, 16, 33, 64, 100, 256])
@pytest.mark.parametrize("N,K", [(2048, 2048), (2560, 2048), (2048, 5632), (640, 4096)])
def test_few_token_products_at_layer_sizes_give_the_same_bits_every_time(ops, M, N, K):
    """Layer-sized shapes, so that clusters of several CTAs split K (the leading CTA adds up the partial
    sums in rank order); twice in a row, which must give the same bits."""
    g = torch.Generator().manual_seed(M + N + K)
    a = (torch.randn(M, K, generator=g) * 0.5).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    ref = a.float() @ w.float().t()
    base = torch.randn(M, N, generator=g)
    outs = []
    for again in range(2):
        out = torch.full((M, N), 5.0, dtype=torch.float32, device="cuda")
        assert ops.tc.linear(dev(a), dev(w), out, False)
        acc = dev(base.clone())
        assert ops.tc.linear(dev(a), dev(w), acc, True)
        torch.cuda.synchronize()
        outs.append((out.cpu(), acc.cpu()))
    close(outs[0][0], ref, 2e-5, "store")
    close(outs[0][1], base + ref, 2e-5, "accumulate")
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    ops.tc.check_errors()


# the last case: so many packed rows that CTA pairs take the product below a thousand tokens
@pytest.mark.parametrize("M,F,K", [(M, F, K) for F, K in [(176, 64), (200, 72), (1000, 256)]
                                   for M in [1, 9, 33, 64, 100, 257]] + [(520, 5632, 64)])
def test_tensor_core_gate_up(ops, M, F, K):
    h = (torch.randn(M, K) * 0.5).bfloat16()
    w = (torch.randn(2 * F, K) * 0.2).bfloat16()
    ref = torch.zeros(M, F)
    cpu.linear_swiglu(None, h, w, ref)
    out = torch.full((M, F), 9.0, dtype=torch.bfloat16, device="cuda")
    packed = ops.pack_gate_up(dev(w[:F]), dev(w[F:]))
    assert packed.shape == (128 * ((F + 63) // 64), K)
    assert ops.tc.linear_swiglu(dev(h), packed, out)
    close(out, ref, 8e-3, "swiglu")
    ops.tc.check_errors()
    # the same packed weights through the plain product and the separate SiLU-gate kernel
    tmp = torch.zeros(M, packed.shape[0], device="cuda")
    out2 = torch.zeros(M, F, dtype=torch.bfloat16, device="cuda")
    from garuda_b200.kernels import CudaOps
    CudaOps("cuda:0", tensor_cores=False).linear(dev(h), packed, tmp)
    ops.silu_mul(tmp, out2, 64)
    close(out2, ref, 8e-3, "swiglu, unfused")


@pytest.mark.parametrize("M", [1, 8, 17, 40, 64, 100, 300, 1100])
@pytest.mark.parametrize("d,K,F", [(200, 72, 176), (1024, 256, 1000), (2560, 192, 300)])
def test_norm_folded_into_the_products_around_it(ops, M, d, K, F):
    """The product that adds into the residual stream writes x * weight and partial sums of x^2;
    the products behind it (gate/up; queries, keys and values) scale their results by 1/rms."""
    from garuda_b200.engine.batch import StepContext, Workspace
    from garuda_b200.parts.norm import RMSNorm
    from garuda_b200.parts.rotary import RotaryParams
    g = torch.Generator().manual_seed(M + d)
    eps = 1e-3
    a, w_o = (torch.randn(M, K, generator=g) * 0.5).bfloat16(), (torch.randn(d, K, generator=g) * 0.1).bfloat16()
    # every token at a scale of its own, so that a 1/rms taken from another token's sums shows
    x = torch.randn(M, d, generator=g) * (1 + torch.arange(M) % 5).float()[:, None]
    gamma = (1 + 0.3 * torch.randn(d, generator=g)).bfloat16()
    norm = RMSNorm(d, eps)
    norm.load({"weight": dev(gamma)}, ops, torch.bfloat16)
    ctx = StepContext(batch=None, ws=Workspace("cuda:0"), ops=ops, dtype=torch.bfloat16)
    res = dev(x.clone())
    pending = ops.linear(dev(a), dev(w_o), res, accumulate=True, ctx=ctx, emit_norm=norm)
    assert pending is not None, "this shape folds the norm in"
    x_new = x + a.float() @ w_o.float().t()
    close(res, x_new, 1e-5, "residual")
    close(pending.values, x_new * gamma.float(), 4e-3, "x * weight")
    torch.testing.assert_close(pending.sums.sum(0).cpu(), (x_new ** 2).sum(1), rtol=1e-4, atol=1e-6)
    # what the consumers must compute, from the rounded values they read
    inv = torch.rsqrt((x_new ** 2).mean(1, keepdim=True) + eps)
    h_ref = pending.values.float().cpu() * inv
    close(pending.materialize(ctx), x_new * inv * gamma.float(), 8e-3, "the norm run the ordinary way")
    w = (torch.randn(2 * F, d, generator=g) * 0.2).bfloat16()
    ref = torch.zeros(M, F)
    cpu.linear_swiglu(None, h_ref, w.float(), ref)
    out = torch.full((M, F), 9.0, dtype=torch.bfloat16, device="cuda")
    ops.linear_swiglu(ctx, pending, ops.pack_gate_up(dev(w[:F]), dev(w[F:])), out)
    close(out, ref, 8e-3, "gate/up behind a folded norm")
    Hq, Hkv, hd, page = 4, 2, 32, 8
    wq = (torch.randn((Hq + 2 * Hkv) * hd, d, generator=g) * 0.2).bfloat16()
    req = torch.arange(M, dtype=torch.int32)
    positions = (torch.arange(M, dtype=torch.int32) * 3) % 29
    table = torch.randperm(M * 4, generator=g).int().view(M, 4)
    rot = RotaryParams(10000.0, hd, False)
    k_ref, v_ref = torch.zeros(M * 4, Hkv, page, hd), torch.zeros(M * 4, Hkv, page, hd)
    q_ref = torch.zeros(M, Hq, hd)
    cpu.qkv_rope_append(None, h_ref, wq.float(), q_ref, k_ref, v_ref, positions, req, table, Hq, Hkv, hd, rot, page)
    k = torch.zeros(M * 4, Hkv, page, hd, dtype=torch.bfloat16, device="cuda")
    v, q = torch.zeros_like(k), torch.zeros(M, Hq, hd, dtype=torch.bfloat16, device="cuda")
    ops.qkv_rope_append(ctx, pending, dev(wq), q, k, v, dev(positions), dev(req), dev(table), Hq, Hkv, hd, rot, page)
    close(q, q_ref, 1e-2, "q"), close(k, k_ref, 1e-2, "k"), close(v, v_ref, 1e-2, "v")
    ops.tc.check_errors()


def test_products_with_more_tiles_than_cta_pairs(ops):
    """2,048 tokens times 2,560 features are 80 tiles of 256 x 256 for 74 CTA pairs: some pairs take
    a second tile (the other accumulator stage, the persistent loop). Every epilogue at that shape."""
    M, N, K = 2048, 2560, 192
    a, w = (torch.randn(M, K) * 0.5).bfloat16(), (torch.randn(N, K) * 0.1).bfloat16()
    ref = a.float() @ w.float().t()
    for odt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 8e-3)):
        out = torch.full((M, N), 5.0, dtype=odt, device="cuda")
        assert ops.tc.linear(dev(a), dev(w), out, False)
        close(out, ref, tol, f"store {odt}")
    base = torch.randn(M, N)
    acc = dev(base.clone())
    assert ops.tc.linear(dev(a), dev(w), acc, True)
    close(acc, base + ref, 1e-5, "accumulate")
    F = N // 2
    refs = torch.zeros(M, F)
    cpu.linear_swiglu(None, a, w, refs)
    outs = torch.full((M, F), 9.0, dtype=torch.bfloat16, device="cuda")
    assert ops.tc.linear_swiglu(dev(a), ops.pack_gate_up(dev(w[:F]), dev(w[F:])), outs)
    close(outs, refs, 8e-3, "swiglu")
    ops.tc.check_errors()


def test_row_pitch_that_tma_cannot_take_uses_the_plain_kernel(ops):
    a, w = torch.randn(5, 20).bfloat16(), torch.randn(12, 20).bfloat16()     # K = 20: 40-byte rows
    out = torch.zeros(5, 12, device="cuda")
    assert not ops.tc.linear(dev(a), dev(w), out, False)
    ops.linear(dev(a), dev(w), out)
    close(out, a.float() @ w.float().t(), 2e-6)


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotate_and_store(ops, interleaved, dtype):
    from garuda_b200.parts.rotary import RotaryParams
    Hq, Hkv, hd, page, T = 6, 3, 48, 8, 11
    rot = RotaryParams(500000.0, hd, interleaved)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd)
    positions = torch.tensor([0, 1, 2, 3, 40, 41, 7, 100, 101, 102, 103], dtype=torch.int32)
    token_req = torch.tensor([0, 0, 0, 0, 1, 1, 2, 3, 3, 3, 3], dtype=torch.int32)
    bt = torch.full((4, 14), -1, dtype=torch.int32)
    bt[0, 0], bt[1, 5], bt[2, 0], bt[3, 12] = 3, 0, 5, 1
    k_ref, v_ref = torch.zeros(6, Hkv, page, hd), torch.zeros(6, Hkv, page, hd)
    q_ref = torch.zeros(T, Hq, hd)
    cpu.rope_kv_append(qkv, q_ref, k_ref, v_ref, positions, token_req, bt, Hq, Hkv, hd, rot, page)
    k, v = torch.zeros(6, Hkv, page, hd, dtype=dtype, device="cuda"), torch.zeros(6, Hkv, page, hd, dtype=dtype, device="cuda")
    q = torch.zeros(T, Hq, hd, dtype=dtype, device="cuda")
    ops.rope_kv_append(dev(qkv), q, k, v, dev(positions), dev(token_req), dev(bt), Hq, Hkv, hd, rot, page)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(q, q_ref, tol, "q"), close(k, k_ref, tol, "k"), close(v, v_ref, tol, "v")
    # rotation in place, for position encodings that are applied outside the fused kernel
    x = torch.randn(T, Hq, hd)
    ref = x.clone()
    cpu.rope_inplace(ref, positions, rot)
    xd = dev(x)
    ops.rope_inplace(xd, dev(positions), rot)
    close(xd, ref, 2e-6, "in place")
    # the first 32 channels of every head only, at frequencies of its own
    narrow = RotaryParams(1.0, 32, interleaved, tuple(0.5 ** i for i in range(16)))
    ref = x.clone()
    cpu.rope_inplace(ref[..., :32], positions, narrow)
    xd = dev(x)
    ops.rope_inplace(xd[..., :32], dev(positions), narrow)
    close(xd, ref, 2e-6, "in place, narrow")
    assert torch.equal(xd[..., 32:].cpu(), x[..., 32:])


@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("Hq,Hkv,hd,d", [(4, 2, 16, 64), (3, 1, 32, 96), (32, 4, 64, 256), (2, 2, 128, 72), (6, 3, 48, 72)])
@pytest.mark.parametrize("T", [1, 11, 70, 200, 300, 2048])
def test_fused_projection_rotation_and_cache_write(ops, interleaved, Hq, Hkv, hd, d, T):
    """The query/key/value product with rotation and page write in its epilogue
    against the plain product followed by the plain rotate-and-store."""
    from garuda_b200.parts.rotary import RotaryParams
    from garuda_b200.engine.batch import Workspace
    if T == 2048 and (Hq, hd) != (32, 64):
        pytest.skip("the 2,048-token case is for the 2,560-feature shape (more tiles than CTA pairs)")

    class Ctx:
        ws = Workspace("cuda:0")

    g = torch.Generator().manual_seed(T + hd)
    rot = RotaryParams(10000.0, hd, interleaved)
    page = 8
    h = (torch.randn(T, d, generator=g) * 0.5).bfloat16()
    w = (torch.randn((Hq + 2 * Hkv) * hd, d, generator=g) * 0.2).bfloat16()
    # three requests share the tokens; positions start at different offsets
    starts = [0, 37, 100]
    req = torch.tensor([i % 3 for i in range(T)], dtype=torch.int32).sort().values
    positions = torch.zeros(T, dtype=torch.int32)
    seen = [0, 0, 0]
    for t in range(T):
        r = int(req[t])
        positions[t] = starts[r] + seen[r]
        seen[r] += 1
    width = (max(int(positions.max()) + 1, 1) + page - 1) // page + 1
    perm = torch.randperm(3 * width, generator=g).int().view(3, width)
    npages = 3 * width
    for rotary in (rot, None):
        k_ref, v_ref = torch.zeros(npages, Hkv, page, hd), torch.zeros(npages, Hkv, page, hd)
        q_ref = torch.zeros(T, Hq, hd)
        cpu.qkv_rope_append(None, h, w, q_ref, k_ref, v_ref, positions, req, perm, Hq, Hkv, hd, rotary, page)
        k = torch.zeros(npages, Hkv, page, hd, dtype=torch.bfloat16, device="cuda")
        v = torch.zeros_like(k)
        q = torch.zeros(T, Hq, hd, dtype=torch.bfloat16, device="cuda")
        ops.qkv_rope_append(Ctx, dev(h), dev(w), q, k, v, dev(positions), dev(req), dev(perm), Hq, Hkv, hd, rotary, page)
        close(q, q_ref, 1e-2, "q"), close(k, k_ref, 1e-2, "k"), close(v, v_ref, 1e-2, "v")
    ops.tc.check_errors()


def _attention_case(Hq, Hkv, hd, page, reqs, window, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    R, T = len(reqs), sum(q for _, q in reqs)
    npages = sum((kv + page - 1) // page for kv, _ in reqs) + 2
    perm = torch.randperm(npages, generator=g)
    width = max((kv + page - 1) // page for kv, _ in reqs) + 1
    bt = torch.full((R, width), -1, dtype=torch.int32)
    c = 0
    for i, (kv, _) in enumerate(reqs):
        n = (kv + page - 1) // page
        bt[i, :n] = perm[c:c + n].int()
        c += n
    k = torch.randn(npages, Hkv, page, hd, generator=g).to(dtype)
    v = torch.randn(npages, Hkv, page, hd, generator=g).to(dtype)
    q = torch.randn(T, Hq, hd, generator=g).to(dtype)
    cu = torch.tensor([0] + list(np.cumsum([ql for _, ql in reqs])), dtype=torch.int32)
    kvl = torch.tensor([kv for kv, _ in reqs], dtype=torch.int32)
    treq = torch.cat([torch.full((ql,), i, dtype=torch.int32) for i, (_, ql) in enumerate(reqs)])
    ref = torch.zeros(T, Hq * hd)
    cpu.paged_attention(q.float(), k.float(), v.float(), bt, cu, kvl, treq, ref, hd ** -0.5, window, page, R, 0, 0)
    return q, k, v, bt, cu, kvl, treq, ref


ATTENTION_CASES = [
    (4, 2, 16, 8, [(70, 70)], 0), (4, 2, 16, 8, [(70, 1)], 0),
    (3, 1, 32, 16, [(96, 30), (50, 1), (33, 2), (200, 1)], 0),
    (3, 1, 32, 16, [(96, 30), (50, 1), (33, 2), (200, 1)], 20),
    (6, 3, 48, 16, [(130, 65), (64, 64), (65, 1)], 16),
    (32, 4, 64, 32, [(700, 1)] * 5, 0), (32, 4, 64, 32, [(1500, 1), (300, 3)], 100),
    (8, 8, 128, 64, [(257, 129), (300, 1)], 0), (5, 5, 80, 8, [(77, 77), (13, 1)], 0),
    (7, 1, 112, 4, [(40, 9), (41, 1)], 0),
]


@pytest.mark.parametrize("Hq,Hkv,hd,page,reqs,window", ATTENTION_CASES)
def test_attention_plain_kernel(ops, Hq, Hkv, hd, page, reqs, window):
    from garuda_b200.kernels import CudaOps
    plain = CudaOps("cuda:0", tensor_cores=False)
    for dtype, tol in ((torch.float32, 3e-6), (torch.bfloat16, 8e-3)):
        q, k, v, bt, cu, kvl, treq, ref = _attention_case(Hq, Hkv, hd, page, reqs, window, dtype)
        out = torch.zeros(ref.shape, dtype=dtype, device="cuda")
        plain.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5,
                              window, page, len(reqs), max(x for _, x in reqs), max(x for x, _ in reqs))
        close(out, ref, tol, f"plain attention {dtype}")


@pytest.mark.parametrize("Hq,Hkv,hd,page,reqs,window", ATTENTION_CASES)
def test_attention_tensor_core_kernel(ops, Hq, Hkv, hd, page, reqs, window):
    q, k, v, bt, cu, kvl, treq, ref = _attention_case(Hq, Hkv, hd, page, reqs, window, torch.bfloat16)
    out = torch.zeros(ref.shape, dtype=torch.bfloat16, device="cuda")
    assert ops.tc.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5,
                                  window, page, len(reqs), max(x for _, x in reqs), max(x for x, _ in reqs))
    close(out, ref, 1e-2, "tensor-core attention")


TCGEN05_ATTENTION_CASES = [
    (32, 4, 64, 32, [(700, 700)], 0),                          # a whole prompt, groups of 8
    (8, 8, 64, 16, [(300, 300), (520, 130), (64, 1)], 0),      # no grouping; a portion, a decode token beside it
    (16, 2, 64, 64, [(1000, 257)], 0),                         # the end of a long context, pages of 64
    (32, 4, 64, 32, [(900, 400)], 200),                        # a window shorter than the context
    (4, 1, 64, 8, [(500, 500), (129, 129)], 50),               # groups of 4, pages of 8, a short window
    (2, 1, 64, 128, [(3, 3), (131, 131), (256, 128)], 0),      # pages as long as a key tile
    (8, 8, 128, 32, [(700, 700), (130, 130)], 0),              # heads of 128, each with its own kv head
    (32, 8, 128, 64, [(1000, 300), (64, 1), (257, 257)], 0),   # heads of 128 in groups of 4; a portion; pages of 64
    (16, 2, 128, 16, [(900, 500)], 150),                       # heads of 128 in groups of 8, a window
    (4, 4, 128, 128, [(5, 5), (400, 272)], 0),                 # heads of 128, pages as long as a key tile
]


@pytest.mark.parametrize("Hq,Hkv,hd,page,reqs,window", TCGEN05_ATTENTION_CASES)
def test_attention_tcgen05_prompt_portions(ops, Hq, Hkv, hd, page, reqs, window):
    """Prompt portions on the tcgen05 kernel. Every cache slot that no query may read holds NaN:
    a key or value fetched from beyond a request's length, or from another request's page, shows."""
    q, k, v, bt, cu, kvl, treq, ref = _attention_case(Hq, Hkv, hd, page, reqs, window, torch.bfloat16)
    used = torch.zeros(k.shape[0], page, dtype=torch.bool)
    for i, (kv, _) in enumerate(reqs):
        for j in range(kv):
            used[int(bt[i, j // page]), j % page] = True
    k = k.clone(); v = v.clone()
    k.transpose(1, 2)[~used] = float("nan")
    v.transpose(1, 2)[~used] = float("nan")
    lib = ops.tc._attention_lib(hd)
    lib.gb_attention_tc_tile_launches.restype = ctypes.c_longlong
    before = lib.gb_attention_tc_tile_launches()
    out = torch.zeros(ref.shape, dtype=torch.bfloat16, device="cuda")
    assert ops.tc.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5,
                                  window, page, len(reqs), max(x for _, x in reqs), max(x for x, _ in reqs),
                                  min_q_len=min(x for _, x in reqs))
    ops.tc.check_errors()
    assert lib.gb_attention_tc_tile_launches() == before + 1, "the tcgen05 kernel did not take the shape"
    close(out, ref, 1e-2, "tcgen05 attention")


DECODE_TMA_CASES = [
    # Hq, Hkv, hd, page, [(keys, new tokens)], window
    (32, 4, 64, 32, [(2048, 1), (1, 1), (64, 1), (65, 1), (700, 2), (1333, 1)], 0),     # groups of 8; tile edges; two tokens
    (32, 4, 64, 16, [(900, 1), (130, 1), (511, 1)], 200),                               # a window; pages of 16
    (8, 8, 64, 8, [(300, 1), (77, 3), (1000, 1)], 0),                                   # no groups; pages of 8
    (32, 32, 128, 32, [(1500, 1), (200, 1)], 0),                                        # heads of 128, each with its own kv head
    (32, 8, 128, 64, [(4000, 1), (129, 2), (640, 1)], 0),                               # heads of 128 in groups of 4; pages of 64
    (16, 4, 128, 16, [(777, 1), (33, 4)], 96),                                          # heads of 128, a window
]


@pytest.mark.parametrize("ranks,cluster", [(1, 0), (2, 0), (3, 0), (4, 0), (8, 0), (16, 0), (2, 1), (3, 1), (4, 1), (6, 1), (8, 1)])
@pytest.mark.parametrize("Hq,Hkv,hd,page,reqs,window", DECODE_TMA_CASES)
def test_attention_decode_with_tma_page_copies(ops, Hq, Hkv, hd, page, reqs, window, ranks, cluster):
    """The decode kernel that fetches pages by TMA, with every way of splitting a request's keys
    over several CTAs, independent ones that merge through scratch memory and thread-block clusters
    that merge through shared memory. Every cache slot that no query may read holds NaN (beyond a
    request's length, another request's page, before a window's start), pages that a window has
    passed are given back (-1 in the block table), and the table's tail is -1 as well."""
    q, k, v, bt, cu, kvl, treq, ref = _attention_case(Hq, Hkv, hd, page, reqs, window, torch.bfloat16, seed=ranks + 20 * cluster)
    used = torch.zeros(k.shape[0], page, dtype=torch.bool)
    bt = bt.clone()
    for i, (kv, ql) in enumerate(reqs):
        first = max(0, kv - ql + 1 - window) if window else 0          # the first key that the first new token reads
        for j in range(first, kv):
            used[int(bt[i, j // page]), j % page] = True
        bt[i, :first // page] = -1                                      # pages wholly before it were given back
    k = k.clone(); v = v.clone()
    k.transpose(1, 2)[~used] = float("nan")
    v.transpose(1, 2)[~used] = float("nan")
    lib = ops.tc._attention_lib(hd)
    T = q.shape[0]
    out = torch.full(ref.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    qd, kd, vd, btd, cud, kvd = dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl)
    if cluster and ranks > (8 if hd == 64 else 4):
        pytest.skip("more CTAs than a cluster of this head size holds")
    need = 0 if cluster else lib.gb_attention_scratch_bytes(len(reqs), Hkv, ranks)
    assert (need == 0) == (ranks == 1 or cluster == 1)
    scratch = torch.zeros(max(need, 16), dtype=torch.uint8, device="cuda")
    for again in range(2):      # a second launch finds the counters as the first one left them
        out.fill_(float("nan"))
        rc = lib.gb_attention_mma(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr(), btd.data_ptr(), bt.shape[1],
                                  cud.data_ptr(), kvd.data_ptr(), T, len(reqs), Hq, Hkv, hd ** -0.5, window, page,
                                  max(x for _, x in reqs), min(x for _, x in reqs), ranks, 1, k.shape[0], cluster,
                                  scratch.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.gb_last_error().decode()
        torch.cuda.synchronize()
        assert int(scratch[:65536].view(torch.int32).abs().sum()) == 0 or need == 0
    ops.tc.check_errors()
    lib.gb_attention_decode_tma_launches.restype = ctypes.c_longlong
    assert lib.gb_attention_decode_tma_launches() > 0, "the TMA kernel did not take the shape"
    close(out, ref, 1e-2, f"decode attention by TMA, {ranks} CTAs per request")
    assert lib.gb_attention_scratch_bytes(len(reqs), Hkv, 1) == 0


def test_attention_decode_with_tma_far_key(ops):
    """One early key stands out among two thousand: whichever CTA and warp of the cluster holds its
    tile, its weight must survive both merges."""
    Hq, Hkv, hd, page = 32, 4, 64, 32
    for far in (3, 700, 2046):
        q, k, v, bt, cu, kvl, treq, _ = _attention_case(Hq, Hkv, hd, page, [(2047, 1), (500, 1)], 0, torch.bfloat16, seed=far)
        head = 13                                            # reads kv head 1
        pg = int(bt[0, far // page])
        k[pg, 1, far % page] = (q[0, head].float() * 4).bfloat16()
        v[pg, 1, far % page] = 50.0
        ref = torch.zeros(2, Hq * hd)
        cpu.paged_attention(q.float(), k.float(), v.float(), bt, cu, kvl, treq, ref, hd ** -0.5, 0, page, 2, 0, 0)
        assert ref[0, head * hd:(head + 1) * hd].mean() > 40
        out = torch.zeros(ref.shape, dtype=torch.bfloat16, device="cuda")
        ops.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5, 0, page, 2,
                            1, 2047, min_q_len=1)
        close(out, ref, 1e-2, f"far key at {far}, decode by TMA")


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("far", [5, 720, 1050])
def test_attention_tcgen05_one_key_stands_out(ops, hd, far):
    """One key stands out for one late query row of a long portion: an early one (its weight must
    survive every later tile), or a late one after hundreds of ordinary keys (the running maximum
    jumps, and what has been accumulated is rescaled), in either half of a key tile."""
    Hq, Hkv, page = 8, 2, 32
    q, k, v, bt, cu, kvl, treq, _ = _attention_case(Hq, Hkv, hd, page, [(1100, 600)], 0, torch.bfloat16, seed=far)
    tok, head = 577, 6                                       # head 6 reads kv head 1; the token stands at position 1077
    pg = int(bt[0, far // page])
    k[pg, 1, far % page] = (q[tok, head].float() * 4).bfloat16()
    v[pg, 1, far % page] = 50.0
    ref = torch.zeros(600, Hq * hd)
    cpu.paged_attention(q.float(), k.float(), v.float(), bt, cu, kvl, treq, ref, hd ** -0.5, 0, page, 1, 0, 0)
    assert ref[tok, head * hd:(head + 1) * hd].mean() > 40
    lib = ops.tc._attention_lib(hd)
    lib.gb_attention_tc_tile_launches.restype = ctypes.c_longlong
    before = lib.gb_attention_tc_tile_launches()
    out = torch.zeros(ref.shape, dtype=torch.bfloat16, device="cuda")
    ops.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5, 0, page, 1,
                        600, 1100, min_q_len=600)
    ops.tc.check_errors()
    assert lib.gb_attention_tc_tile_launches() == before + 1, "the tcgen05 kernel did not take the shape"
    close(out, ref, 1e-2, f"key {far} stands out, tcgen05, head size {hd}")


def test_attention_finds_one_far_key_among_hundreds(ops):
    # random values hide a missed key: make one early key's score stand out for one query head
    Hq, Hkv, hd, page = 4, 2, 64, 16
    for dtype in (torch.float32, torch.bfloat16):
        q, k, v, bt, cu, kvl, treq, _ = _attention_case(Hq, Hkv, hd, page, [(900, 1), (333, 5)], 0, dtype)
        far = 3                                   # position 3 of request 0, in its first page
        pg = int(bt[0, far // page])
        k[pg, 1, far % page] = (q[0, 2].float() * 4).to(dtype)      # head 2 reads kv head 1
        v[pg, 1, far % page] = 50.0
        ref = torch.zeros(6, Hq * hd)
        cpu.paged_attention(q.float(), k.float(), v.float(), bt, cu, kvl, treq, ref, hd ** -0.5, 0, page, 2, 0, 0)
        assert ref[0, 2 * hd:3 * hd].mean() > 40              # the far key dominates that head
        out = torch.zeros(ref.shape, dtype=dtype, device="cuda")
        ops.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5, 0,
                            page, 2, 5, 900)
        close(out, ref, 3e-6 if dtype == torch.float32 else 1e-2, f"far key {dtype}")


def test_attention_window_edge(ops):
    # the key just outside the window must not be read, the one just inside must
    Hq, Hkv, hd, page, window = 2, 1, 32, 8, 24
    for dtype in (torch.float32, torch.bfloat16):
        q, k, v, bt, cu, kvl, treq, _ = _attention_case(Hq, Hkv, hd, page, [(100, 1)], window, dtype)
        pos = 99
        inside, outside = pos + 1 - window, pos - window
        for j, val in ((inside, 30.0), (outside, -70.0)):
            pg = int(bt[0, j // page])
            k[pg, 0, j % page] = (q[0, 0].float() * 4).to(dtype)
            v[pg, 0, j % page] = val
        out = torch.zeros(1, Hq * hd, dtype=dtype, device="cuda")
        ops.paged_attention(dev(q), dev(k), dev(v), dev(bt), dev(cu), dev(kvl), dev(treq), out, hd ** -0.5,
                            window, page, 1, 1, 100)
        head0 = out[0, :hd].float().cpu()
        assert head0.mean() > 25, "the key at the window's edge was not read"
        ref = torch.zeros(1, Hq * hd)
        cpu.paged_attention(q.float(), k.float(), v.float(), bt, cu, kvl, treq, ref, hd ** -0.5, window, page, 1, 0, 0)
        close(out, ref, 3e-6 if dtype == torch.float32 else 1e-2, "window edge")


def test_silu_gate_and_residual(ops):
    gu = torch.randn(7, 2 * 200) * 3
    ref = torch.zeros(7, 200)
    cpu.silu_mul(gu, ref)
    for odt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        out = torch.zeros(7, 200, dtype=odt, device="cuda")
        ops.silu_mul(dev(gu), out)
        close(out, ref, tol, "silu_mul")
    x, y = torch.randn(5, 72), torch.randn(5, 72)
    xd = dev(x.clone())
    ops.residual_add(xd, dev(y.bfloat16()))
    close(xd, x + y.bfloat16().float(), 1e-7, "residual")


def test_argmax_first_maximum_wins(ops):
    logits = torch.randn(6, 32003)
    logits[1, 100] = logits[1, 31000] = 50.0          # a tie: the lower index
    logits[2, :] = -float("inf")
    logits[3, 0] = float("nan")
    logits[3, 77] = 60.0
    out = torch.zeros(6, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), out)
    want = [int(torch.argmax(logits[0])), 100, 0, 77, int(torch.argmax(logits[4])), int(torch.argmax(logits[5]))]
    assert out.tolist() == want


def test_sampling_among_equal_probabilities_goes_by_token_id(ops):
    """All logits equal: the top k are the k lowest token ids (ties go by id), each with the same
    probability, and the draw walks them in that order. With far more ties than the kernel's short
    list of candidates holds."""
    from tests.plain.sampling_plain import sample as plain_sample

    class FixedU:
        def __init__(self, u): self.u = u
        def next_f32(self): return np.float32(self.u)

    V = 5000
    # top-p alone: reached within the short list (0.1 of 5,000 equal tokens are 500) or far beyond it (2,500)
    rows = [(1.0, k, p, u) for k, p in ((40, 1.0), (7, 0.5), (1024, 1.0), (300, 0.02), (0, 0.1), (0, 0.5), (2000, 0.3))
            for u in (0.0, 0.26, 0.5, 0.99)]
    R = len(rows)
    logits = torch.full((R, V), 0.25)
    out = torch.zeros(R, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(R * V, device="cuda")
    f = lambda i, dt: dev(torch.tensor([r[i] for r in rows], dtype=dt))
    ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32),
               out, scratch)
    got = out.tolist()
    for i, (temp, k, p, u) in enumerate(rows):
        want = plain_sample(logits[i].numpy(), temp, k, p, FixedU(u))
        assert abs(got[i] - want) <= 1 and (k == 0 or got[i] < k), (rows[i], got[i], want)    # a draw on a boundary may round either way


def test_sampling_with_ties_at_the_last_place_of_top_k(ops):
    """Several tokens share the k-th largest logit: the ones with the lowest ids are the candidates,
    whichever thread met them. Few enough ties for the short list of candidates, and (second half of
    the rows) so many that the kernel falls back on its passes over the whole vocabulary."""
    from tests.helpers import assert_tokens_follow_the_plain_sampler
    V, k = 32000, 6
    g = torch.Generator().manual_seed(3)
    base = torch.randn(V, generator=g)
    top = torch.topk(base, 4).indices.tolist()                 # four clear leaders
    rows, logits = [], []
    for ties in ([31000, 17, 9000, 1024, 2047], list(range(3000, 3000 + 1500, 1))):     # all at one value below the leaders
        row = base.clone()
        row[row > 2.5] = 2.0
        for i, t in enumerate(top):
            row[t] = 6.0 - 0.5 * i
        row[torch.tensor(ties)] = 3.0                           # places 5 and 6 go to the two lowest ids among these
        for u in (0.0, 0.3, 0.6, 0.9, 0.97, 0.999):
            rows.append((1.0, k, 1.0, u))
            logits.append(row)
    R = len(rows)
    logits = torch.stack(logits)
    out = torch.zeros(R, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(R * V, device="cuda")
    f = lambda i, dt: dev(torch.tensor([r[i] for r in rows], dtype=dt))
    ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32), out, scratch)
    got = out.tolist()
    assert_tokens_follow_the_plain_sampler(rows, logits, got)
    shared = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32), shared, scratch,
               small_top_k=True)
    assert_tokens_follow_the_plain_sampler(rows, logits, shared.tolist())
    seen = set(got)
    for i in range(R):
        assert got[i] in set(top) | ({17, 1024} if i < 6 else {3000, 3001}), (i, got[i])
    assert {17, 1024} & seen and {3000, 3001} & seen, "the tied candidates are reached by the later draws"


@pytest.mark.parametrize("V", [50, 331, 32000, 128256])
def test_sampling_rows_shared_by_clusters(ops, V):
    """Few enough rows for a cluster of eight CTAs each: rows with a small top_k go the shared way
    (each CTA an eighth of the vocabulary, also where an eighth is less than top_k), the others
    (greedy, top-p alone, a large top_k) are done by the cluster's first CTA alone."""
    from tests.helpers import assert_tokens_follow_the_plain_sampler
    settings = [(0.8, 40, 0.95), (1.0, 64, 1.0), (0.5, 5, 1.0), (0.0, 40, 0.95), (0.8, 1, 0.95), (2.0, 30, 0.5),
                (1.3, 0, 0.7), (1.5, 100, 0.9)]
    for u in (0.0, 0.37, 0.999):
        rows = [(t, k, p, u) for t, k, p in settings]
        R = len(rows)
        g = torch.Generator().manual_seed(V + int(u * 100))
        logits = torch.randn(R, V, generator=g) * 2
        logits[1, 5] = logits[1, V - 2] = logits[1].max() + 1          # ties among the most likely, in two CTAs' parts
        out = torch.full((R,), -1, dtype=torch.int32, device="cuda")
        scratch = torch.full((R * V,), float("nan"), device="cuda")
        f = lambda i, dt: dev(torch.tensor([r[i] for r in rows], dtype=dt))
        ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32),
                   out, scratch, small_top_k=True)
        assert_tokens_follow_the_plain_sampler(rows, logits, out.tolist())


@pytest.mark.parametrize("V", [50, 331, 32000, 128256])
def test_sampling_follows_the_plain_sampler(ops, V):
    """At 128,256 entries a row's probabilities no longer fit in shared memory: the kernel keeps
    them in the caller's scratch instead (another branch of it, and the one a Llama-3 vocabulary takes)."""
    from tests.helpers import sampling_rows, assert_tokens_follow_the_plain_sampler
    rows = sampling_rows(few=V > 50000)
    R = len(rows)
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(R, V, generator=g) * 2
    logits[3, 5] = logits[3, 9] = logits[3].max() + 1          # ties among the most likely
    out = torch.zeros(R, dtype=torch.int32, device="cuda")
    scratch = torch.full((R * V,), float("nan"), device="cuda")   # nothing in it may be read before it is written
    f = lambda i, dt: dev(torch.tensor([r[i] for r in rows], dtype=dt))
    ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32),
               out, scratch)
    assert_tokens_follow_the_plain_sampler(rows, logits, out.tolist())
    # the kernel in which eight CTAs share a row (meant for rows with a small top_k; it does the others the
    # general way): the same tokens
    shared = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    scratch.fill_(float("nan"))
    ops.sample(dev(logits), f(0, torch.float32), f(1, torch.int32), f(2, torch.float32), f(3, torch.float32),
               shared, scratch, small_top_k=True)
    assert_tokens_follow_the_plain_sampler(rows, logits, shared.tolist())
