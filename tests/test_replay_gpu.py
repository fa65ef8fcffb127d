"""bin/trace_run replays the same requests whole, with the last 32 tokens decoded
one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again, in 32-bit and in bfloat16, and every
way agrees with the plain implementation at every position.
(The reference asserts the same self-consistency: garuda/src/llama/mod.rs:1556-1612,
:1640-1715, :1750-1772.)"""
import numpy as np
import pytest
import torch

from tests.helpers import (TINY, TraceRunner, model_dir, plain_logits, random_tokens, assert_close)

pytestmark = pytest.mark.gpu

STORE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def up64(n):
    return (n + 63) // 64 * 64


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "C", "D", "E", "Ai", "Bh") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def run(request):
    name, dtype = request.param
    ctx = TINY[name][0]["max_position_embeddings"]
    # the mixed phase holds the most: four live requests
    tr = TraceRunner(model_dir(name, STORE[dtype]), dtype, max_tokens=4 * up64(min(ctx, 120)),
                     extra=["--page-size", "16"])
    yield name, dtype, tr
    assert tr.close() == 0


def test_whole(run):
    name, dtype, tr = run
    for n, seed in ((1, 1), (2, 2), (17, 3), (100, 4)):
        toks = random_tokens(name, n, seed)
        out = tr.step([("w", toks, range(n))], end=["w"])
        assert_close(out, plain_logits(name, STORE[dtype], toks), dtype, f"whole, {n} tokens", config=name)


def test_last_32_tokens_one_by_one(run):
    name, dtype, tr = run
    toks = random_tokens(name, 110, 7)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = [tr.step([("d", toks[:78], [77])])]
    for i in range(78, 110):
        outs.append(tr.step([("d", [toks[i]], [0])], end=["d"] if i == 109 else []))
    assert_close(np.concatenate(outs), ref[77:], dtype, "decode after a prompt", config=name)


def test_first_tokens_and_long_decoding(run):
    # a request that starts from a single token and is decoded token by token across many pages
    name, dtype, tr = run
    toks = random_tokens(name, 100, 9)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = []
    for i, t in enumerate(toks):
        outs.append(tr.step([("l", [t], [0])], end=["l"] if i == 99 else []))
    got = np.concatenate(outs)
    assert_close(got[:4], ref[:4], dtype, "first tokens", config=name)
    assert_close(got, ref, dtype, "long decoding", config=name)


def test_portions_of_changing_size(run):
    name, dtype, tr = run
    toks = random_tokens(name, 118, 11)
    ref = plain_logits(name, STORE[dtype], toks)
    cuts = [7, 2, 19, 3, 2, 16, 2, 31, 1, 15, 2, 18]
    assert sum(cuts) == 118
    pos, outs = 0, []
    for i, c in enumerate(cuts):
        outs.append(tr.step([("p", toks[pos:pos + c], range(c))], end=["p"] if i == len(cuts) - 1 else []))
        pos += c
    assert_close(np.concatenate(outs), ref, dtype, "portions", config=name)


def test_mixed_requests_reusing_pages(run):
    name, dtype, tr = run
    lens = [90, 33, 120, 21, 64, 47, 75]
    toks = [random_tokens(name, n, 20 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(name, STORE[dtype], t) for t in toks]
    pool = 4 * up64(120) - 128          # the other tests have ended their requests; leave a margin unused
    fed = [0] * len(lens)
    got = [[] for _ in lens]
    live, waiting = [], list(range(len(lens)))
    rng = np.random.default_rng(1)
    most_live = 0
    while live or waiting:
        while waiting and len(live) < 4 and sum(up64(lens[i]) for i in live) + up64(lens[waiting[0]]) <= pool:
            live.append(waiting.pop(0))
        most_live = max(most_live, len(live))
        entries, ended = [], []
        # now and then a request sits a step out and goes on later
        active = [i for i in live if rng.random() > 0.15] or live[:1]
        for i in active:
            left = lens[i] - fed[i]
            n = 1 if left <= 12 else int(min(left - 12, rng.integers(2, 24)))
            entries.append((f"m{i}", toks[i][fed[i]:fed[i] + n], range(n)))
            if fed[i] + n == lens[i]:
                ended.append(f"m{i}")
        out = tr.step(entries, end=ended)
        row = 0
        for (rid, t, _), i in zip(entries, active):
            got[i].append(out[row:row + len(t)])
            row += len(t)
            fed[i] += len(t)
            if fed[i] == lens[i]:
                live.remove(i)
    assert most_live == 4
    for i in range(len(lens)):
        assert_close(np.concatenate(got[i]), refs[i], dtype, f"mixed, request {i}", config=name)


def test_long_prompt_across_key_tiles(run):
    """Prompts longer than one 128-key tile of the prompt attention, whole and in portions that end
    inside, at and just after a tile's edge, then decoded; a window shorter than the prompt."""
    name, dtype, tr = run
    if name != "D":
        pytest.skip("the configuration with room for 300 tokens")
    toks = random_tokens(name, 300, 41)
    ref = plain_logits(name, STORE[dtype], toks)
    out = tr.step([("t", toks, range(300))], end=["t"])
    assert_close(out, ref, dtype, "whole, 300 tokens", config=name)
    cuts = [127, 1, 2, 126, 33]
    pos, outs = 0, []
    for c in cuts:
        outs.append(tr.step([("u", toks[pos:pos + c], range(c))]))
        pos += c
    for i in range(pos, 300):
        outs.append(tr.step([("u", [toks[i]], [0])], end=["u"] if i == 299 else []))
    assert_close(np.concatenate(outs), ref, dtype, "portions across tiles, then decoded", config=name)


def test_every_way_of_cutting_gives_the_same_logits_in_32_bit(run):
    # beyond agreeing with the plain model: whole, decoded and cut runs agree with each other
    name, dtype, tr = run
    if dtype != "float32":
        pytest.skip("compared against the plain model in bfloat16")
    toks = random_tokens(name, 80, 31)
    whole = tr.step([("x", toks, range(80))], end=["x"])
    parts = [tr.step([("y", toks[:50], range(50))])]
    parts += [tr.step([("y", [t], [0])]) for t in toks[50:79]]
    parts.append(tr.step([("y", [toks[79]], [0])], end=["y"]))
    cut = np.concatenate(parts)
    assert np.abs(cut - whole).max() <= 1e-6 * max(1.0, np.abs(whole).max())


def test_decode_without_graphs_matches():
    name, dtype = "A", "bfloat16"
    tr = TraceRunner(model_dir(name, STORE[dtype]), dtype, max_tokens=256, extra=["--no-graphs"])
    toks = random_tokens(name, 70, 41)
    ref = plain_logits(name, STORE[dtype], toks)
    outs = [tr.step([("d", toks[:40], [39])])]
    outs += [tr.step([("d", [t], [0])]) for t in toks[40:]]
    assert_close(np.concatenate(outs), ref[39:], dtype, "decode, kernel by kernel", config=name)
    assert tr.close() == 0
