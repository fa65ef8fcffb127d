"""The layer sizes of the benchmarked model (TinyLlama-1.1B: hidden 2048, 32 query and 4 kv heads of
64, intermediate 5632), two layers of it with random weights: the bfloat16 engine's ways through
its kernels (a whole prompt: CTA-pair products and tcgen05 attention; portions; token by token:
cluster products and decode attention; several requests in a batch) against the 32-bit engine,
which the other tests tie to the plain implementation on the tiny configurations."""
import tempfile

import numpy as np
import pytest
import torch

from tests.helpers import TOL

pytestmark = pytest.mark.gpu

SHAPE = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048, num_hidden_layers=2,
             num_attention_heads=32, num_key_value_heads=4, head_dim=64, intermediate_size=5632,
             vocab_size=4096, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
             max_position_embeddings=1024)


@pytest.fixture(scope="module")
def engines():
    from garuda_b200 import Engine
    from garuda_b200.weights import write_random_model
    d = tempfile.mkdtemp(prefix="garuda_shape_")
    # 32-bit on disk: the 32-bit engine reads it as it is, the bfloat16 engine rounds it once
    write_random_model(d, SHAPE, seed=5, store_dtype=torch.float32)
    kw = dict(context=1024, page_size=32, kv_tokens=8192, max_concurrent=64)
    return Engine(d, dtype="float32", **kw), Engine(d, dtype="bfloat16", **kw)


def close(got, want, what):
    got, want = got.float().cpu().numpy(), want.float().cpu().numpy()
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(got - want).max())
    assert np.isfinite(got).all(), f"{what}: not finite"
    assert err <= TOL["bfloat16"] * scale, f"{what}: max difference {err:.3e} (limit {TOL['bfloat16'] * scale:.3e})"


def test_whole_portions_and_decoding_agree_with_32_bit(engines):
    from garuda_b200 import StepEntry
    e32, e16 = engines
    rng = np.random.default_rng(3)
    toks = rng.integers(0, SHAPE["vocab_size"], 600).tolist()
    want = list(range(0, 600, 7)) + [599]
    ref = e32.step([StepEntry(1, toks, want)]).clone()
    e32.runner.end(1)
    # whole
    out = e16.step([StepEntry(1, toks, want)])
    e16.runner.end(1)
    close(out, ref, "whole prompt")
    # portions that end inside, at and after the edges of 128-key and 256-token tiles, then single tokens
    cuts = [255, 1, 2, 130, 128, 44]
    pos, rows = 0, []
    for c in cuts:
        w = [i - pos for i in want if pos <= i < pos + c]
        o = e16.step([StepEntry(2, toks[pos:pos + c], w)])
        if w:
            rows.append(o.clone())      # a step's logits are valid until the next step
        pos += c
    for i in range(pos, 600):
        o = e16.step([StepEntry(2, [toks[i]], [0] if i in want else [])])
        if i in want:
            rows.append(o.clone())
    e16.runner.end(2)
    close(torch.cat(rows), ref, "portions, then token by token")


def test_batched_requests_agree_with_32_bit(engines):
    from garuda_b200 import StepEntry
    e32, e16 = engines
    rng = np.random.default_rng(4)
    lens = [300, 17, 129, 64]
    toks = [rng.integers(0, SHAPE["vocab_size"], n).tolist() for n in lens]
    ref = torch.cat([e32.step([StepEntry(10 + i, t, [len(t) - 1])]).clone() for i, t in enumerate(toks)])
    for i in range(len(lens)):
        e32.runner.end(10 + i)
    # all four prompts in one step, then eight decode steps of the four together
    out = e16.step([StepEntry(10 + i, t, [len(t) - 1]) for i, t in enumerate(toks)])
    close(out, ref, "four prompts in one step")
    nxt = [int(x) for x in rng.integers(0, SHAPE["vocab_size"], 4)]
    for i in range(4):
        e32.step([StepEntry(20 + i, toks[i], [])])
    for step in range(8):
        r = e32.step([StepEntry(20 + i, [nxt[i]], [0]) for i in range(4)])
        o = e16.step([StepEntry(10 + i, [nxt[i]], [0]) for i in range(4)])
        close(o, r, f"decode step {step} of four requests")
        nxt = [int(x) for x in r.argmax(-1).cpu()]
    for i in range(4):
        e32.runner.end(20 + i)
        e16.runner.end(10 + i)
    e16.ops.tc.check_errors()


def test_forty_requests_decoding_together(engines):
    """Batches of 17 to 64 tokens take the wider tiles of the few-token product and another plan of
    the decode attention than batches of a few."""
    from garuda_b200 import StepEntry
    e32, e16 = engines
    rng = np.random.default_rng(6)
    n = 40
    lens = [int(x) for x in rng.integers(3, 90, n)]
    toks = [rng.integers(0, SHAPE["vocab_size"], m).tolist() for m in lens]
    for eng in (e32, e16):
        for lo in range(0, n, 8):       # prompts eight at a time
            eng.step([StepEntry(100 + i, toks[i], []) for i in range(lo, lo + 8)])
    nxt = [int(x) for x in rng.integers(0, SHAPE["vocab_size"], n)]
    for step in range(3):
        r = e32.step([StepEntry(100 + i, [nxt[i]], [0]) for i in range(n)]).clone()
        o = e16.step([StepEntry(100 + i, [nxt[i]], [0]) for i in range(n)])
        close(o, r, f"decode step {step} of forty requests")
        nxt = [int(x) for x in r.argmax(-1).cpu()]
    for i in range(n):
        e32.runner.end(100 + i)
        e16.runner.end(100 + i)
    e16.ops.tc.check_errors()


def test_norms_between_products_run_inside_the_products(engines):
    """With the tensor-core kernels a layer is five launches: the norms between the products are
    folded into them (only the first layer's first norm and the last norm run as kernels). With the
    folding switched off the same step launches two more per layer and gives the same logits within
    rounding. Few tokens (cluster kernel), 65 to 255 (one CTA per tile) and more (CTA pairs)."""
    from garuda_b200 import StepEntry
    e32, e16 = engines
    rng = np.random.default_rng(8)
    layers = SHAPE["num_hidden_layers"]
    ops = e16.ops
    assert ops.folds_norms
    for n in (5, 64, 150, 400):
        toks = rng.integers(0, SHAPE["vocab_size"], n).tolist()
        ref = e32.step([StepEntry(50, toks, [0, n - 1])]).clone()
        e32.runner.end(50)
        counts, outs = [], []
        for fold in (True, False):
            ops.folds_norms = fold
            try:
                before = ops.launches
                outs.append(e16.step([StepEntry(51, toks, [0, n - 1])]).clone())
                counts.append(ops.launches - before)
            finally:
                ops.folds_norms = True
                e16.runner.end(51)
        assert counts[1] - counts[0] == 2 * layers - 1, (n, counts)
        close(outs[0], ref, f"{n} tokens, norms folded in")
        close(outs[1], ref, f"{n} tokens, norm kernels")
    e16.ops.tc.check_errors()
