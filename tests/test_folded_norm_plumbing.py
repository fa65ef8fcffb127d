"""How blocks and the decoder hand a half-done norm from one part to the next, on the CPU.

The kernels that fold a norm into the products around it are tested on the GPU
(test_kernels_gpu.py, test_shapes_gpu.py). Here a stand-in kernel set does the same
arithmetic with torch, so that what is tested is the pairing: which product is asked to
fold which norm in, who gets the result, and that parts which know nothing of it still
get plain tensors."""
import torch

from garuda_b200 import Engine, StepEntry
from garuda_b200.kernels.ops import PendingNorm
from garuda_b200.parts.attention import PagedAttention
from garuda_b200.parts.mlp import SwiGLU
from tests.helpers import model_dir, plain_logits, random_tokens, assert_close
from tests.plain.cpu_ops import CpuOps


class FoldingCpuOps(CpuOps):
    """CpuOps that folds norms the way the tensor-core kernels do, and keeps a record."""
    folds_norms = True

    def __init__(self):
        super().__init__()
        self.emitted, self.consumed, self.norm_kernels = [], [], 0

    def rmsnorm(self, *a, **kw):
        self.norm_kernels += 1
        return super().rmsnorm(*a, **kw)

    def linear(self, a, w, out, accumulate=False, ctx=None, emit_norm=None):
        super().linear(a, w, out, accumulate)
        if emit_norm is None or not accumulate:
            return None
        weight, eps = emit_norm.fold()
        self.emitted.append(emit_norm)
        return PendingNorm(out * weight.float(), (out * out).sum(1)[None], weight, eps, emit_norm, out)

    def _scaled(self, h, who):
        if not isinstance(h, PendingNorm):
            return h
        self.consumed.append((who, h.norm))
        inv = torch.rsqrt(h.sums.sum(0) / h.values.shape[1] + h.eps)
        return h.values * inv[:, None]

    def normed(self, ctx, h):
        return h.materialize(ctx) if isinstance(h, PendingNorm) else h

    def linear_swiglu(self, ctx, h, w_gate_up, act):
        return super().linear_swiglu(ctx, self._scaled(h, "feed_forward"), w_gate_up, act)

    def qkv_rope_append(self, ctx, h, *a, **kw):
        return super().qkv_rope_append(ctx, self._scaled(h, "mixer"), *a, **kw)


def _engine(name, ops):
    return Engine(model_dir(name), dtype="float32", ops=ops, cuda_graphs=False, page_size=8, kv_tokens=512)


def test_every_norm_between_two_products_is_folded_and_the_logits_stay():
    name = "A"
    ops = FoldingCpuOps()
    e = _engine(name, ops)
    blocks = e.model.blocks
    toks = random_tokens(name, 40, 3)
    out = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(out, plain_logits(name, torch.float32, toks), "float32", "folded norms")
    L = len(blocks)
    # each block's mixer folds its own second norm in; each feed-forward but the last the next block's first
    want = []
    for i, b in enumerate(blocks):
        want.append(b.feed_forward_norm)
        if i + 1 < L:
            want.append(blocks[i + 1].mixer_norm)
    assert ops.emitted == want
    assert [n for _, n in ops.consumed] == want
    assert [w for w, _ in ops.consumed] == (["feed_forward", "mixer"] * L)[:2 * L - 1]
    assert ops.norm_kernels == 2            # the first block's first norm and the last norm


def test_a_part_that_knows_nothing_of_it_gets_the_plain_norm(monkeypatch):
    name = "A"
    toks = random_tokens(name, 25, 4)
    ref = plain_logits(name, torch.float32, toks)
    # a feed-forward that neither takes a half-done norm nor folds one in
    monkeypatch.setattr(SwiGLU, "takes_pending_norm", False)
    monkeypatch.setattr(SwiGLU, "emits_norm", False)
    ops = FoldingCpuOps()
    e = _engine(name, ops)
    out = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(out, ref, "float32", "feed-forward without folding")
    assert ops.emitted == [] and ops.consumed == []
    assert ops.norm_kernels == 2 * len(e.model.blocks) + 1
    # a mixer that does not take one: its block's first norm runs as a kernel, the second is still folded
    monkeypatch.undo()
    monkeypatch.setattr(PagedAttention, "takes_pending_norm", False)
    ops = FoldingCpuOps()
    e = _engine(name, ops)
    out = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(out, ref, "float32", "mixer that takes no half-done norm")
    L = len(e.model.blocks)
    assert ops.emitted == [b.feed_forward_norm for b in e.model.blocks]
    assert ops.norm_kernels == L + 1


def test_kernels_that_cannot_fold_leave_the_norms_alone():
    """The plain kernel set (as in 32-bit) says nothing about folding: no part is asked to."""
    name = "A"
    calls = []

    class Plain(CpuOps):
        def linear(self, a, w, out, accumulate=False, **kw):
            calls.append(kw)
            return super().linear(a, w, out, accumulate)

    e = _engine(name, Plain())
    toks = random_tokens(name, 12, 5)
    out = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(out, plain_logits(name, torch.float32, toks), "float32", "no folding")
    assert all(kw == {} for kw in calls)
