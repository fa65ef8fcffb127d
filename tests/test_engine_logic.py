"""The step function, the cache and the scheduler working together, on the CPU:
the kernels are replaced by their plain references (tests/plain/cpu_ops.py), so
what is tested here is everything around them. The same comparisons run on the
GPU with the real kernels in test_replay_gpu.py."""
import numpy as np
import pytest
import torch

from garuda_b200 import Engine, SamplingParams, StepEntry, StepError
from garuda_b200.csrc.build import load_host_module
from tests.helpers import TINY, model_dir, plain_logits, random_tokens, assert_close, folder_weights
from tests.plain.cpu_ops import CpuOps
from tests.plain import llama_plain
from tests.plain.sampling_plain import Rng, sample as plain_sample

host = load_host_module()


def engine(name, **kw):
    kw.setdefault("page_size", 8)
    kw.setdefault("kv_tokens", 512)
    return Engine(model_dir(name), dtype="float32", ops=CpuOps(), cuda_graphs=False, **kw)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_decode_and_portions_agree_with_the_plain_model(name):
    e = engine(name)
    toks = random_tokens(name, 90, 5)
    ref = plain_logits(name, torch.float32, toks)
    whole = e.step([StepEntry(1, toks, range(len(toks)))]).numpy().copy()
    assert_close(whole, ref, "float32", "whole")
    e.runner.end(1)
    outs = [e.step([StepEntry(2, toks[:58], [57])]).numpy().copy()]
    for t in toks[58:]:
        outs.append(e.step([StepEntry(2, [t], [0])]).numpy().copy())
    assert_close(np.concatenate(outs), ref[57:], "float32", "decode")
    e.runner.end(2)
    pos, outs = 0, []
    for c in [7, 2, 19, 3, 2, 11, 2, 30, 14]:
        outs.append(e.step([StepEntry(3, toks[pos:pos + c], range(c))]).numpy().copy())
        pos += c
    assert pos == 90
    assert_close(np.concatenate(outs), ref, "float32", "portions")
    e.runner.end(3)
    e.cache.manager.check_invariants()
    assert e.cache.manager.pages_reused > 0


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_few_pages(name):
    # four requests of different lengths, portions of some beside decoded tokens of others,
    # in a pool so small that pages are given back and used again
    e = engine(name, kv_tokens=160, max_concurrent=4)
    lens = [70, 33, 50, 21, 44]
    toks = [random_tokens(name, n, 10 + i) for i, n in enumerate(lens)]
    refs = [plain_logits(name, torch.float32, t) for t in toks]
    fed = [0] * 5
    got = [[] for _ in range(5)]
    live, waiting = [], list(range(5))
    rng = np.random.default_rng(0)
    pool = 160

    def held(i):
        return (lens[i] + 7) // 8 * 8

    most_live = 0
    while live or waiting:
        # a request comes in when the pool can hold all of it beside the live ones
        while waiting and len(live) < 4 and sum(held(i) for i in live) + held(waiting[0]) <= pool:
            live.append(waiting.pop(0))
        most_live = max(most_live, len(live))
        entries = []
        for i in list(live):
            left = lens[i] - fed[i]
            n = 1 if left <= 8 else int(min(left - 8, rng.integers(2, 12)))
            entries.append((i, n))
        out = e.step([StepEntry(100 + i, toks[i][fed[i]:fed[i] + n], range(n)) for i, n in entries]).numpy().copy()
        row = 0
        for i, n in entries:
            got[i].append(out[row:row + n])
            row += n
            fed[i] += n
            if fed[i] == lens[i]:
                e.runner.end(100 + i)
                live.remove(i)
        e.cache.manager.check_invariants()
    assert most_live >= 3
    for i in range(5):
        assert_close(np.concatenate(got[i]), refs[i], "float32", f"request {i}")
    assert e.cache.manager.pages_reused > 0 and e.cache.manager.live_requests == 0


def test_a_refused_step_changes_nothing():
    e = engine("A", kv_tokens=64)
    toks = random_tokens("A", 40, 1)
    e.step([StepEntry(1, toks[:10], [9])])
    free = e.cache.manager.free_pages(0)
    for bad in ([StepEntry(1, [300], [0])],                              # outside the vocabulary
                [StepEntry(1, [1], [0]), StepEntry(1, [2], [0])],        # the same request twice
                [StepEntry(1, [1], [3])],                                # a place that does not exist
                [StepEntry(1, [], [])],
                [StepEntry(1, [1] * 200, [])]):                          # beyond the context
        with pytest.raises(StepError):
            e.step(bad)
    with pytest.raises(host.OutOfPages):
        e.step([StepEntry(1, toks[10:12], []), StepEntry(2, random_tokens("A", 60, 2), [])])
    assert e.cache.manager.free_pages(0) == free and e.cache.manager.length(1) == 10
    assert not e.cache.manager.known(2)
    ref = plain_logits("A", torch.float32, toks)
    out = e.step([StepEntry(1, toks[10:], [29])]).numpy()
    assert_close(out, ref[39:40], "float32", "after refusals")


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_the_plain_model(name):
    cfg = TINY[name][0]
    e = engine(name, max_concurrent=3, max_batch_tokens=24, prefill_chunk=7)
    prompts = [random_tokens(name, n, 40 + n) for n in (5, 23, 1, 37)]
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=6))
    w = folder_weights(model_dir(name))
    for p, r in zip(prompts, res):
        assert r.finish_reason == "length"
        assert r.tokens == llama_plain.greedy_generate(cfg, w, p, 6)
    st = e.stats()
    assert st["completed"] == 4 and st["running"] == 0 and st["pages_free"] == st["pages_total"]
    # one request alone gives the same tokens as in the batch (garuda/src/scheduler/mod.rs:982-1029)
    solo = engine(name).generate([prompts[1]], SamplingParams.greedy(max_tokens=6))
    assert solo[0].tokens == res[1].tokens


def test_generation_survives_preemption():
    cfg = TINY["A"][0]
    prompts = [random_tokens("A", 20, 70 + i) for i in range(3)]
    roomy = engine("A", max_concurrent=3).generate(prompts, SamplingParams.greedy(max_tokens=24))
    tight = engine("A", kv_tokens=96, max_concurrent=3)      # 12 pages of 8: not enough for three at 44
    res = tight.generate(prompts, SamplingParams.greedy(max_tokens=24))
    assert tight.stats()["preemptions"] > 0
    assert [r.tokens for r in res] == [r.tokens for r in roomy]
    assert all(r.finish_reason == "length" for r in res)
    tight.cache.manager.check_invariants()


def test_sampled_generation_follows_the_plain_sampler_draw_for_draw():
    cfg = TINY["A"][0]
    e = engine("A")
    prompt = random_tokens("A", 12, 3)
    params = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, max_tokens=8, seed=1234)
    res = e.generate([prompt], params)[0]
    w = folder_weights(model_dir("A"))
    rng, seq, want = Rng(1234), list(prompt), []
    for _ in range(8):
        logits = llama_plain.forward(cfg, w, seq)[-1]
        tok = plain_sample(logits, 0.9, 20, 0.9, rng)
        want.append(tok)
        seq.append(tok)
    assert res.tokens == want
    again = engine("A").generate([prompt], params)[0]
    assert again.tokens == res.tokens                    # the same seed reproduces


def test_eos_and_errors_in_generate():
    e = engine("A")
    prompt = random_tokens("A", 9, 8)
    first = e.generate([prompt], SamplingParams.greedy(max_tokens=5))[0].tokens
    stop = Engine(model_dir("A"), dtype="float32", ops=CpuOps(), cuda_graphs=False, page_size=8,
                  kv_tokens=256, eos_token_id=first[2])
    r = stop.generate([prompt], SamplingParams.greedy(max_tokens=5))[0]
    assert r.finish_reason == "eos" and r.tokens == first[:first.index(first[2])]
    res = e.generate([[], [999], prompt], SamplingParams.greedy(max_tokens=2))
    assert res[0].finish_reason == "error" and "empty" in res[0].error
    assert res[1].finish_reason == "error" and "vocabulary" in res[1].error
    assert res[2].finish_reason == "length" and len(res[2].tokens) == 2


def test_generation_with_a_timeout_ends_the_request_and_frees_what_it_held():
    e = engine("A", max_concurrent=2)
    prompts = [random_tokens("A", 9, 1), random_tokens("A", 5, 2)]
    e.scheduler.set_time(10.0)
    seen = []

    def on_token(i, tok):
        seen.append(i)
        if len(seen) == 6:                       # three tokens each: now the clock jumps past the deadline
            e.scheduler.set_time(20.0)

    res = e.generate(prompts, SamplingParams.greedy(max_tokens=40), on_token=on_token, timeout=5.0)
    assert [r.finish_reason for r in res] == ["error", "error"] and [r.error for r in res] == ["timeout", "timeout"]
    assert [len(r.tokens) for r in res] == [3, 3]
    st = e.stats()
    assert st["timed_out"] == 2 and st["running"] == 0 and st["pages_free"] == st["pages_total"]
    # the tokens that came before the deadline are those of an unlimited run
    e.scheduler.set_time(30.0)
    free = e.generate(prompts, SamplingParams.greedy(max_tokens=3))
    assert [r.tokens for r in free] == [r.tokens for r in res] and all(r.finish_reason == "length" for r in free)
    with pytest.raises(Exception):
        e.generate(prompts, timeout=0)


def test_trace_replay_loop_writes_the_plain_models_logits(tmp_path):
    """The loop behind bin/trace_run, `garuda replay` and Engine.replay, over the reference kernels:
    requests named by strings or numbers, one left out of a step and going on later, blank lines, a
    step that only ends requests, an unknown name in `end`, pages used again."""
    import json
    from garuda_b200.engine.replay import replay
    e = engine("B", kv_tokens=96, max_concurrent=3)           # 12 pages of 8 for 40 + 30 + 33 tokens in turn
    a, b, c = (random_tokens("B", n, 60 + n) for n in (40, 30, 33))
    refs = {k: plain_logits("B", torch.float32, t) for k, t in (("a", a), ("b", b), ("c", c))}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}, {"id": 7, "tokens": b[:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[17:39], "want": [21]}], "end": []},          # 7 sits this one out
        {"step": 2, "entries": [{"id": 7, "tokens": b[2:], "want": [0, 27]}, {"id": "a", "tokens": a[39:], "want": [0]}], "end": ["a", "nobody"]},
        {"step": 3, "entries": [], "end": [7]},
        {"step": 5, "entries": [{"id": "c", "tokens": c, "want": [32]}], "end": ["c"]},
    ]
    lines = [json.dumps(s) for s in steps]
    lines.insert(2, "   ")
    seen = []
    n = replay(e, lines, str(tmp_path / "out"), report=seen.append)
    assert n == 5 and seen == [0, 1, 2, 3, 5]
    vocab = refs["a"].shape[1]

    def got(step):
        return np.fromfile(tmp_path / "out" / f"{step}.f32", dtype="<f4").reshape(-1, vocab)

    assert_close(got(0), refs["a"][[0, 16]], "float32", "step 0")
    assert_close(got(1), refs["a"][[38]], "float32", "step 1")
    assert_close(got(2), np.concatenate([refs["b"][[2, 29]], refs["a"][[39]]]), "float32", "step 2")
    assert not (tmp_path / "out" / "3.f32").exists()
    assert_close(got(5), refs["c"][[32]], "float32", "step 5")
    m = e.cache.manager
    assert m.live_requests == 0 and m.pages_reused > 0
    m.check_invariants()


def test_paced_prompt_portions_change_the_steps_and_not_the_tokens():
    cfg = TINY["A"][0]
    prompts = [random_tokens("A", n, 90 + n) for n in (3, 60, 45, 2, 70)]
    plain = engine("A", max_concurrent=3).generate(prompts, SamplingParams.greedy(max_tokens=10))
    paced = engine("A", max_concurrent=3, paced_prefill=True)
    res = paced.generate(prompts, SamplingParams.greedy(max_tokens=10))
    assert [r.tokens for r in res] == [r.tokens for r in plain]
    p = paced.scheduler.pacing
    assert p.decode_step > 0 and p.prefill_token > 0 and 1 <= p.chunk <= 512      # both costs were measured
    unpaced = engine("A", max_concurrent=3)
    unpaced.generate(prompts, SamplingParams.greedy(max_tokens=10))
    assert unpaced.scheduler.pacing.decode_step == -1.0                             # nothing is timed without it
    w = folder_weights(model_dir("A"))
    assert res[1].tokens == llama_plain.greedy_generate(cfg, w, prompts[1], 10)


def test_a_callback_that_answers_false_cancels_its_request():
    prompts = [random_tokens("A", 9, 1), random_tokens("A", 5, 2)]
    free = engine("A").generate(prompts, SamplingParams.greedy(max_tokens=8))
    e = engine("A")
    got = {0: 0, 1: 0}

    def on_token(i, tok):
        got[i] += 1
        return not (i == 0 and got[0] == 3)          # the first request's reader leaves after three tokens

    res = e.generate(prompts, SamplingParams.greedy(max_tokens=8), on_token=on_token)
    assert (res[0].finish_reason, res[0].error, res[0].tokens) == ("error", "cancelled", free[0].tokens[:3])
    assert (res[1].finish_reason, res[1].tokens) == ("length", free[1].tokens)
    st = e.stats()
    assert st["cancelled"] == 1 and st["completed"] == 1 and st["pages_free"] == st["pages_total"]


def test_events_stream_as_they_happen_and_leaving_early_cancels():
    """garuda/src/scheduler/mod.rs:67-71 (tokens, then one Done or Error per request) and :92-109 (a
    dropped handle cancels)."""
    prompts = [random_tokens("A", 9, 1), random_tokens("A", 5, 2), []]
    free = engine("A").generate(prompts[:2], SamplingParams.greedy(max_tokens=6))
    e = engine("A")
    events = list(e.stream(prompts, SamplingParams.greedy(max_tokens=6)))
    assert (events[0].index, events[0].kind) == (2, "error") and "empty" in events[0].detail     # refused at once
    for i in (0, 1):
        mine = [ev for ev in events if ev.index == i]
        assert [ev.kind for ev in mine] == ["token"] * 6 + ["done"] and mine[-1].detail == "length"
        assert [ev.token for ev in mine[:-1]] == free[i].tokens
        assert len({ev.request for ev in mine}) == 1
    # the two requests run together: their tokens alternate
    assert [ev.index for ev in events[1:5]] == [0, 1, 0, 1]
    # leaving after a few events cancels what is running, and everything goes back
    it = e.stream(prompts[:2], SamplingParams.greedy(max_tokens=50))
    seen = [next(it) for _ in range(5)]
    assert all(ev.kind == "token" for ev in seen)
    it.close()
    st = e.stats()
    assert st["running"] == 0 and st["queued"] == 0 and st["cancelled"] == 2
    assert st["pages_free"] == st["pages_total"]
    e.cache.manager.check_invariants()
    again = e.generate(prompts[:2], SamplingParams.greedy(max_tokens=6))          # and the engine goes on
    assert [r.tokens for r in again] == [r.tokens for r in free]
    with pytest.raises(Exception):
        e.stream(prompts[:2], [SamplingParams.greedy()])                          # refused when called, not later


def test_priorities_decide_who_waits():
    # one request runs at a time and all four wait when the first plan is made: the higher priority goes
    # first, equal ones keep their order (garuda/src/scheduler/mod.rs:138-148, :1052-1112)
    prompts = [random_tokens("A", 4, i) for i in range(4)]
    e = engine("A", max_concurrent=1)
    order = []
    for ev in e.stream(prompts, SamplingParams.greedy(max_tokens=2), priority=[0, 0, 5, 0]):
        if ev.kind == "done":
            order.append(ev.index)
    assert order == [2, 0, 1, 3]
    solo = engine("A").generate(prompts, SamplingParams.greedy(max_tokens=2))
    res = e.generate(prompts, SamplingParams.greedy(max_tokens=2), priority=[0, 1, 2, 3])
    assert [r.tokens for r in res] == [r.tokens for r in solo]
    with pytest.raises(Exception):
        e.generate(prompts, priority=[1, 2])
