"""Real layer sizes against the plain implementation.

Two layers, with random weights, of three of the shapes the reference publishes figures for:
TinyLlama-1.1B (hidden 2048, 32 query and 4 kv heads of 64, intermediate 5632), Llama-2-7B (hidden
4096, 32 heads of 128 each with a kv head of its own, intermediate 11008) and Llama-3-8B (hidden
4096, 32 query and 8 kv heads of 128, intermediate 14336, a vocabulary of 128,256). Both engines, the
32-bit one and the bfloat16 one, are driven through ``bin/trace_run`` the four ways (whole; most in
one step and the last 32 tokens one by one; portions of changing size; mixed with other requests in
a pool so small that pages are used again) and compared with ``tests/plain/llama_plain.py`` at the
same positions. The tiny configurations cannot show a fault that needs 32 heads, more than 2,048
columns, a second tile of keys or a thousand tiles of the vocabulary product; these can.
(The reference's model for this: garuda/src/llama/mod.rs:1556-1612, :1640-1715, :1750-1772.)

A few tests below use the engines in-process for what a trace cannot express (launch counts, forty
requests in a batch)."""
import tempfile

import numpy as np
import pytest
import torch

from tests.helpers import TraceRunner, assert_close, folder_weights, sharpen_for
from tests.plain import llama_plain

pytestmark = pytest.mark.gpu

TINYLLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048, num_hidden_layers=2,
                 num_attention_heads=32, num_key_value_heads=4, head_dim=64, intermediate_size=5632,
                 vocab_size=4096, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                 max_position_embeddings=1024)
LLAMA2_7B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=2,
                 num_attention_heads=32, num_key_value_heads=32, head_dim=128, intermediate_size=11008,
                 vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                 max_position_embeddings=512)
LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=4096, num_hidden_layers=2,
                 num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                 vocab_size=128256, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                 max_position_embeddings=512)
SHAPE = TINYLLAMA


def up64(n):
    return (n + 63) // 64 * 64


class Shape:
    """A model folder of one shape (bfloat16 on disk, so that both engines and the plain model start
    from the same numbers), the plain model's hidden states and logits for sequences of it."""

    def __init__(self, name, cfg, seed):
        from garuda_b200.weights import write_random_model
        self.name, self.cfg = name, cfg
        self.dir = tempfile.mkdtemp(prefix=f"garuda_shape_{name}_")
        # attention scores of the order of one instead of all but equal (tests/helpers.py, SHARPEN)
        write_random_model(self.dir, cfg, seed=seed, store_dtype=torch.bfloat16, scale=sharpen_for(cfg["hidden_size"]))
        self._weights = None
        self._plain = {}

    @property
    def weights(self):
        if self._weights is None:
            self._weights = folder_weights(self.dir)
        return self._weights

    def tokens(self, n, seed):
        return np.random.default_rng(seed).integers(0, self.cfg["vocab_size"], n).tolist()

    def plain(self, toks, rows):
        """Plain logits at ``rows`` of the sequence: the layers over everything, the final norm and
        the head at the wanted rows only (the head of a 128,256-entry vocabulary over hundreds of
        rows would take the CPU longer than all the rest)."""
        key = tuple(toks)
        if key not in self._plain:
            c = llama_plain.normalise_config(self.cfg)
            w = self.weights
            x = llama_plain.embed(w["model.embed_tokens.weight"], toks)
            pos = np.arange(len(toks))
            for l in range(c["num_hidden_layers"]):
                p = f"model.layers.{l}."
                lw = {k[len(p):]: v for k, v in w.items() if k.startswith(p)}
                x = llama_plain.decoder_layer(x, lw, c, pos, llama_plain.layer_window(c, l))
            self._plain[key] = x
        x = self._plain[key][list(rows)]
        z = llama_plain.rmsnorm(x, self.weights["model.norm.weight"], self.cfg["rms_norm_eps"])
        return llama_plain.linear(z, self.weights["lm_head.weight"])


@pytest.fixture(scope="module")
def tinyllama():
    return Shape("tinyllama", TINYLLAMA, 5)


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def tiny_run(request, tinyllama):
    tr = TraceRunner(tinyllama.dir, request.param, max_tokens=4 * up64(700), extra=["--page-size", "32"])
    yield tinyllama, request.param, tr
    assert tr.close() == 0


def test_tinyllama_whole(tiny_run):
    shape, dtype, tr = tiny_run
    toks = shape.tokens(600, 3)
    rows = list(range(0, 600, 7)) + [599]
    out = tr.step([("w", toks, rows)], end=["w"])
    assert_close(out, shape.plain(toks, rows), dtype, "whole, 600 tokens", config=shape.name)


def test_tinyllama_last_32_tokens_one_by_one(tiny_run):
    shape, dtype, tr = tiny_run
    toks = shape.tokens(600, 3)
    outs = [tr.step([("d", toks[:568], [567])])]
    for i in range(568, 600):
        outs.append(tr.step([("d", [toks[i]], [0])], end=["d"] if i == 599 else []))
    assert_close(np.concatenate(outs), shape.plain(toks, range(567, 600)), dtype, "decode after a prompt",
                 config=shape.name)


def test_tinyllama_portions_of_changing_size(tiny_run):
    """Portions that end inside, at and just after the edges of 128-key tiles and 256-token tiles,
    down to two tokens, then single tokens."""
    shape, dtype, tr = tiny_run
    toks = shape.tokens(600, 3)
    cuts = [255, 1, 2, 130, 128, 44, 2, 17, 3]
    cuts += [1] * (600 - sum(cuts))
    pos, outs, rows = 0, [], []
    for i, c in enumerate(cuts):
        want = [j for j in range(c) if (pos + j) % 5 == 0 or j == c - 1]
        out = tr.step([("p", toks[pos:pos + c], want)], end=["p"] if i == len(cuts) - 1 else [])
        outs.append(out)
        rows += [pos + j for j in want]
        pos += c
    assert_close(np.concatenate(outs), shape.plain(toks, rows), dtype, "portions", config=shape.name)


def test_tinyllama_mixed_requests_reusing_pages(tiny_run):
    shape, dtype, tr = tiny_run
    lens = [300, 90, 640, 21, 170, 64, 210]
    toks = [shape.tokens(n, 20 + i) for i, n in enumerate(lens)]
    pool = 4 * up64(700) - 256
    fed, got, rows = [0] * len(lens), [[] for _ in lens], [[] for _ in lens]
    live, waiting = [], list(range(len(lens)))
    rng = np.random.default_rng(1)
    most_live = 0
    while live or waiting:
        while waiting and len(live) < 4 and sum(up64(lens[i]) for i in live) + up64(lens[waiting[0]]) <= pool:
            live.append(waiting.pop(0))
        most_live = max(most_live, len(live))
        entries, ended = [], []
        active = [i for i in live if rng.random() > 0.15] or live[:1]
        for i in active:
            left = lens[i] - fed[i]
            n = 1 if left <= 12 else int(min(left - 12, rng.integers(2, 150)))
            want = [j for j in range(n) if j % 9 == 0 or j == n - 1]
            entries.append((f"m{i}", toks[i][fed[i]:fed[i] + n], want))
            if fed[i] + n == lens[i]:
                ended.append(f"m{i}")
        out = tr.step(entries, end=ended)
        row = 0
        for (rid, t, want), i in zip(entries, active):
            got[i].append(out[row:row + len(want)])
            rows[i] += [fed[i] + j for j in want]
            row += len(want)
            fed[i] += len(t)
            if fed[i] == lens[i]:
                live.remove(i)
    assert most_live == 4
    for i in range(len(lens)):
        assert_close(np.concatenate(got[i]), shape.plain(toks[i], rows[i]), dtype, f"mixed, request {i}",
                     config=shape.name)


@pytest.mark.parametrize("which", ["llama2-7b", "llama3-8b"])
def test_head_size_128_shapes_whole_and_decoded(which):
    """Two layers of the Llama-2-7B shape (every query head with a kv head of its own) and of the
    Llama-3-8B shape (groups of four, 128,256-entry vocabulary: a thousand tiles of the vocabulary
    product): a prompt in one step, the same prompt in two portions, then decoding, in both precisions."""
    cfg = {"llama2-7b": LLAMA2_7B, "llama3-8b": LLAMA3_8B}[which]
    shape = Shape(which, cfg, 11)
    toks = shape.tokens(200, 13)
    rows = [0, 1, 63, 64, 127, 128, 150, 167]
    ref_rows = rows + list(range(168, 200))
    ref = shape.plain(toks, ref_rows)
    for dtype in ("float32", "bfloat16"):
        tr = TraceRunner(shape.dir, dtype, max_tokens=2 * up64(200), extra=["--page-size", "32"])
        out = tr.step([("w", toks[:168], rows)], end=["w"])
        assert_close(out, ref[:len(rows)], dtype, f"{which}: whole prompt", config=which)
        outs = [tr.step([("d", toks[:130], [r for r in rows if r < 130])]),
                tr.step([("d", toks[130:168], [r - 130 for r in rows if r >= 130])])]
        for i in range(168, 200):
            outs.append(tr.step([("d", [toks[i]], [0])], end=["d"] if i == 199 else []))
        assert_close(np.concatenate(outs), ref, dtype, f"{which}: two portions, then decoded", config=which)
        assert tr.close() == 0


# ---------------------------------------------------------------------- in-process
@pytest.fixture(scope="module")
def engines(tinyllama):
    from garuda_b200 import Engine
    kw = dict(context=1024, page_size=32, kv_tokens=8192, max_concurrent=64)
    return Engine(tinyllama.dir, dtype="float32", **kw), Engine(tinyllama.dir, dtype="bfloat16", **kw)


def test_forty_requests_decoding_together(engines, tinyllama):
    """Batches of 17 to 64 tokens take the wider tiles of the few-token product and another plan of
    the decode attention than batches of a few."""
    from garuda_b200 import StepEntry
    shape = tinyllama
    rng = np.random.default_rng(6)
    n = 40
    lens = [int(x) for x in rng.integers(3, 90, n)]
    toks = [shape.tokens(m, 200 + i) for i, m in enumerate(lens)]
    nxt = [shape.tokens(3, 300 + i) for i in range(n)]
    ref = [np.concatenate([shape.plain(toks[i] + nxt[i], [lens[i] + s]) for i in range(n)]) for s in range(3)]
    for eng, dtype in zip(engines, ("float32", "bfloat16")):
        for lo in range(0, n, 8):       # prompts eight at a time
            eng.step([StepEntry(100 + i, toks[i], []) for i in range(lo, lo + 8)])
        for step in range(3):
            o = eng.step([StepEntry(100 + i, [nxt[i][step]], [0]) for i in range(n)]).float().cpu().numpy()
            assert_close(o, ref[step], dtype, f"decode step {step} of forty requests", config=shape.name)
        for i in range(n):
            eng.runner.end(100 + i)
    engines[1].check_errors()
    engines[1].ops.tc.check_errors()


def test_norms_between_products_run_inside_the_products(engines, tinyllama):
    """With the tensor-core kernels a layer is five launches: the norms between the products are
    folded into them (only the first layer's first norm and the last norm run as kernels). With the
    folding switched off the same step launches two more per layer and gives the same logits within
    rounding. Few tokens (cluster kernel), 65 to 255 (one CTA per tile) and more (CTA pairs)."""
    from garuda_b200 import StepEntry
    e32, e16 = engines
    layers = SHAPE["num_hidden_layers"]
    ops = e16.ops
    assert ops.folds_norms
    for n in (5, 64, 150, 400):
        toks = tinyllama.tokens(n, 400 + n)
        ref = tinyllama.plain(toks, [0, n - 1])
        counts, outs = [], []
        for fold in (True, False):
            ops.folds_norms = fold
            try:
                before = ops.launches
                outs.append(e16.step([StepEntry(51, toks, [0, n - 1])]).float().cpu().numpy())
                counts.append(ops.launches - before)
            finally:
                ops.folds_norms = True
                e16.runner.end(51)
        assert counts[1] - counts[0] == 2 * layers - 1, (n, counts)
        assert_close(outs[0], ref, "bfloat16", f"{n} tokens, norms folded in", config=tinyllama.name)
        assert_close(outs[1], ref, "bfloat16", f"{n} tokens, norm kernels", config=tinyllama.name)
    e16.ops.tc.check_errors()
