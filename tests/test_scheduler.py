"""The scheduler's decisions, without a model: what goes into a step, when a
request finishes, and what happens when pages run out.
(The reference's scheduler tests: garuda/src/scheduler/mod.rs:760-1112.)"""
import pytest

from garuda_b200.csrc.build import load_host_module

host = load_host_module()
Token, Done, Error = host.EventKind.Token, host.EventKind.Done, host.EventKind.Error


def make(pages=64, page_size=4, max_concurrent=4, max_batch_tokens=32, prefill_chunk=16, max_context=64,
         queue_capacity=8, eos=-1, windows=(0,), vocab=100, paced=False):
    cache = host.CacheManager([host.GroupConfig(pages, w) for w in windows], page_size, max_concurrent, max_context)
    c = host.SchedulerConfig()
    c.max_concurrent, c.queue_capacity, c.max_batch_tokens = max_concurrent, queue_capacity, max_batch_tokens
    c.prefill_chunk, c.max_context, c.eos_token_id, c.vocab_size = prefill_chunk, max_context, eos, vocab
    c.paced_prefill = paced
    return host.Scheduler(c, cache), cache


def greedy(max_tokens=4, seed=None, temperature=0.0):
    return host.SamplingParams(temperature=temperature, top_p=1.0, top_k=0, max_tokens=max_tokens, seed=seed)


def run_step(s, cache, token=7):
    plan = s.plan()
    sampled = [token] * sum(1 for e in plan.entries if e.sample)
    return plan, s.complete(plan, sampled)


def test_prompt_is_cut_into_portions_under_the_budget():
    s, cache = make(max_batch_tokens=32, prefill_chunk=16)
    a = s.submit(list(range(40)), greedy())
    plan, ev = run_step(s, cache)
    assert [(e.id, e.start, len(e.tokens), e.sample) for e in plan.entries] == [(a, 0, 16, False)] and not ev
    plan, ev = run_step(s, cache)
    assert [(e.start, len(e.tokens), e.sample) for e in plan.entries] == [(16, 16, False)]
    plan, ev = run_step(s, cache)
    assert [(e.start, len(e.tokens), e.sample) for e in plan.entries] == [(32, 8, True)]
    assert plan.entries[0].tokens == list(range(32, 40))
    assert [(e.kind, e.token) for e in ev] == [(Token, 7)]
    plan, ev = run_step(s, cache)                       # now decoding: one token
    assert [(e.start, e.tokens, e.sample) for e in plan.entries] == [(40, [7], True)]


def test_decode_tokens_come_first_and_share_the_step_with_prompt_portions():
    s, cache = make(max_batch_tokens=10, prefill_chunk=16)
    a = s.submit([1, 2, 3], greedy(max_tokens=8))
    run_step(s, cache)                                  # a's prompt; a is decoding from now on
    b = s.submit(list(range(30)), greedy(max_tokens=8))
    plan, _ = run_step(s, cache)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 1), (b, 9)]   # 10 tokens in all
    assert plan.num_tokens == 10
    plan, _ = run_step(s, cache)
    assert [(e.id, e.start, len(e.tokens)) for e in plan.entries] == [(a, 4, 1), (b, 9, 9)]


def test_admission_stops_at_max_concurrent_and_goes_on_when_one_finishes():
    s, cache = make(max_concurrent=2)
    ids = [s.submit([1, 2], greedy(max_tokens=2)) for _ in range(3)]
    plan, ev = run_step(s, cache)
    assert [e.id for e in plan.entries] == ids[:2] and s.stats().queued == 1
    plan, ev = run_step(s, cache)                       # second token: both reach max_tokens
    assert [(e.kind, e.detail) for e in ev if e.kind == Done] == [(Done, "length")] * 2
    assert cache.live_requests == 0
    plan, ev = run_step(s, cache)
    assert [e.id for e in plan.entries] == ids[2:]
    cache.check_invariants()


def test_finish_reasons():
    s, cache = make(eos=9, max_context=8)
    a = s.submit([1, 2, 3], greedy(max_tokens=10))
    plan = s.plan()
    ev = s.complete(plan, [9])                          # the end-of-sequence token is not emitted
    assert [(e.kind, e.detail) for e in ev] == [(Done, "eos")] and not cache.known(a)
    b = s.submit([1, 2, 3, 4, 5, 6], greedy(max_tokens=10))
    _, ev = run_step(s, cache)                          # 7 tokens in the context
    assert [e.kind for e in ev] == [Token]
    _, ev = run_step(s, cache)                          # 8 = max_context: full
    assert [(e.kind, e.detail) for e in ev] == [(Token, ""), (Done, "context_full")]
    c = s.submit([1], greedy(max_tokens=1))
    _, ev = run_step(s, cache)
    assert [(e.kind, e.detail) for e in ev] == [(Token, ""), (Done, "length")]
    assert s.idle() and s.stats().completed == 3
    cache.check_invariants()


def test_submit_refuses_what_cannot_run():
    s, cache = make(max_context=8, queue_capacity=2, vocab=50)
    with pytest.raises(host.SchedulerError, match="empty"):
        s.submit([], greedy())
    with pytest.raises(host.SchedulerError, match="does not fit"):
        s.submit(list(range(8)), greedy())
    with pytest.raises(host.SchedulerError, match="vocabulary"):
        s.submit([1, 50], greedy())
    with pytest.raises(host.SchedulerError, match="temperature"):
        s.submit([1], host.SamplingParams(temperature=-1.0))
    with pytest.raises(host.SchedulerError, match="top_p"):
        s.submit([1], host.SamplingParams(top_p=0.0))
    with pytest.raises(host.SchedulerError, match="max_tokens"):
        s.submit([1], host.SamplingParams(max_tokens=0))
    s.submit([1], greedy())
    s.submit([1], greedy())
    with pytest.raises(host.Busy):
        s.submit([1], greedy())
    assert s.stats().rejected_busy == 1


def test_priority_overtakes_and_fifo_within():
    s, cache = make(max_concurrent=1)
    low = s.submit([1], greedy(max_tokens=1), 0)
    low2 = s.submit([1], greedy(max_tokens=1), 0)
    high = s.submit([1], greedy(max_tokens=1), 5)
    order = []
    while not s.idle():
        plan, _ = run_step(s, cache)
        order += [e.id for e in plan.entries]
    assert order == [high, low, low2]


def test_cancel_frees_pages_between_steps():
    s, cache = make()
    a = s.submit(list(range(20)), greedy(max_tokens=50))
    b = s.submit([1, 2], greedy(max_tokens=50))
    run_step(s, cache)
    s.cancel(a)
    plan = s.plan()
    assert [(e.id, e.kind, e.detail) for e in plan.events] == [(a, Error, "cancelled")]
    assert [e.id for e in plan.entries] == [b] and not cache.known(a)
    s.complete(plan, [3])
    assert s.stats().cancelled == 1
    cache.check_invariants()


def test_when_pages_run_out_the_most_recent_request_goes_back_to_the_queue():
    # 6 pages of 4 positions; two requests of 8 tokens fill 4 pages, then both decode
    s, cache = make(pages=6, page_size=4, max_concurrent=2, prefill_chunk=8, max_batch_tokens=16)
    a = s.submit(list(range(8)), greedy(max_tokens=12))
    b = s.submit(list(range(10, 18)), greedy(max_tokens=12))
    plan, _ = run_step(s, cache, token=1)
    assert [e.id for e in plan.entries] == [a, b]
    preempted_at = None
    for step in range(12):
        plan, ev = run_step(s, cache, token=1)
        cache.check_invariants()
        if plan.preempted:
            preempted_at = step
            assert plan.preempted == [b]                # the most recently admitted one
            assert [e.id for e in plan.entries] == [a]
            assert not cache.known(b) and s.stats().queued == 1
            break
    assert preempted_at is not None
    assert s.stats().preemptions == 1
    # a runs on to its limit; b comes back with its prompt and what it had generated, and finishes
    done = {}
    refed = []
    for _ in range(200):
        if s.idle():
            break
        plan, ev = run_step(s, cache, token=1)
        for e in plan.entries:
            if e.id == b:
                assert e.start == len(refed)
                refed += e.tokens
        for e in ev:
            if e.kind == Done:
                done[e.id] = e.detail
        cache.check_invariants()
    assert done == {a: "length", b: "length"}
    # b was recomputed from its prompt and the tokens it had generated before it was sent back
    assert refed[:8] == list(range(10, 18)) and refed[8:12] == [1, 1, 1, 1] and len(refed) == 8 + 11
    assert cache.live_requests == 0 and cache.free_pages(0) == 6


def test_a_request_that_cannot_fit_alone_ends_with_an_error():
    s, cache = make(pages=2, page_size=4, max_concurrent=2, max_context=64)
    a = s.submit(list(range(6)), greedy(max_tokens=30))
    errors = []
    for _ in range(20):
        if s.idle():
            break
        plan, ev = run_step(s, cache)
        errors += [e for e in list(plan.events) + list(ev) if e.kind == Error]
    assert len(errors) == 1 and errors[0].id == a and "more pages" in errors[0].detail
    assert cache.free_pages(0) == 2 and s.stats().failed == 1
    # and a prompt longer than the whole pool
    b = s.submit(list(range(20)), greedy())
    for _ in range(5):
        plan, ev = run_step(s, cache)
        errors += [e for e in list(plan.events) + list(ev) if e.kind == Error]
        if s.idle():
            break
    assert errors[-1].id == b and s.idle()
    cache.check_invariants()


def test_admission_waits_for_the_pages_of_a_first_portion():
    s, cache = make(pages=5, page_size=4, max_concurrent=2, prefill_chunk=16, max_batch_tokens=32)
    a = s.submit(list(range(12)), greedy(max_tokens=2))     # 3 pages, a 4th with its first decoded token
    run_step(s, cache)
    b = s.submit(list(range(16)), greedy(max_tokens=2))     # wants 4 pages, 1 is free
    plan, ev = run_step(s, cache)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 1)]      # b is not admitted yet
    assert [e.detail for e in ev if e.kind == Done] == ["length"]         # a has its 2 tokens
    plan, _ = run_step(s, cache)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(b, 16)]
    cache.check_invariants()


def test_prefill_portion_is_cut_to_the_pages_there_are():
    s, cache = make(pages=5, page_size=4, max_concurrent=2, prefill_chunk=8, max_batch_tokens=32)
    a = s.submit([1, 2, 3, 4], greedy(max_tokens=20))        # 1 page, a 2nd as soon as it decodes
    b = s.submit(list(range(16)), greedy(max_tokens=2))
    plan, _ = run_step(s, cache)
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 4), (b, 8)]     # 1 + 2 pages
    plan, _ = run_step(s, cache)
    # a takes its 2nd page; one page is left, so b's second portion is 4 tokens instead of 8
    assert [(e.id, e.start, len(e.tokens)) for e in plan.entries] == [(a, 4, 1), (b, 8, 4)]
    assert cache.free_pages(0) == 0
    cache.check_invariants()


def test_seeded_draws_are_reproducible_and_default_to_the_request_id():
    s, cache = make()
    a = s.submit([1], greedy(max_tokens=3, seed=42, temperature=0.8))
    us = []
    for _ in range(3):
        plan = s.plan()
        us.append(plan.entries[0].u)
        s.complete(plan, [5])
    r = host.Rng(42)
    assert us == [r.next_f32() for _ in range(3)]
    b = s.submit([1], greedy(max_tokens=1, temperature=0.8))
    plan = s.plan()
    assert plan.entries[0].u == host.Rng(b).next_f32()      # garuda/src/runtime/mod.rs:612
    c = s.submit([1], greedy(max_tokens=1))
    s.complete(plan, [5])
    plan = s.plan()
    assert plan.entries[0].u == 0.0                          # greedy draws nothing


def test_windowed_group_lets_a_long_request_run_in_few_pages():
    s, cache = make(pages=4, page_size=4, windows=(6,), max_context=64, prefill_chunk=4)
    a = s.submit(list(range(30)), greedy(max_tokens=20))
    done = None
    for _ in range(100):
        plan, ev = run_step(s, cache)
        cache.check_invariants()
        for e in ev:
            if e.kind in (Done, Error):
                done = e
        if s.idle():
            break
    assert done is not None and done.kind == Done and done.detail == "length"
    assert s.stats().preemptions == 0


def test_the_next_draw_can_be_looked_at_without_taking_it():
    """A decode step launched before its plan is made needs the uniform that the plan will bring."""
    s, cache = make()
    a = s.submit([1], greedy(max_tokens=4, seed=9, temperature=0.8))
    plan = s.plan()
    for _ in range(3):
        ahead = s.peek_uniform(a)
        assert s.peek_uniform(a) == ahead                   # looking twice takes nothing
        s.complete(plan, [5])
        plan = s.plan()
        assert plan.entries[0].u == ahead
    with pytest.raises(host.SchedulerError, match="not running"):
        s.peek_uniform(12345)


def test_any_of_several_end_tokens_finishes_a_request():
    """config.json may list several end-of-sequence ids (current Llama checkpoints list three):
    each of them ends a request, joins the context and is not emitted
    (garuda/src/runtime/mod.rs:733-738)."""
    s, cache = make()
    s_cfg = host.SchedulerConfig()
    assert s_cfg.eos_token_id == -1 and s_cfg.eos_token_ids == []
    s_cfg.eos_token_id = 5
    assert s_cfg.eos_token_ids == [5]
    cache = host.CacheManager([host.GroupConfig(64, 0)], 4, 4, 64)
    c = host.SchedulerConfig()
    c.max_concurrent, c.queue_capacity, c.max_batch_tokens, c.prefill_chunk = 4, 8, 32, 16
    c.max_context, c.vocab_size = 64, 100
    c.eos_token_ids = [90, 91, 92]
    s = host.Scheduler(c, cache)
    ids = [s.submit([1, 2, 3], greedy(max_tokens=6)) for _ in range(3)]
    plan = s.plan()
    s.complete(plan, [7, 7, 7])
    plan = s.plan()
    ev = s.complete(plan, [92, 7, 91])
    done = {e.id: e.detail for e in ev if e.kind == Done}
    assert done == {ids[0]: "eos", ids[2]: "eos"}
    assert [e.token for e in ev if e.kind == Token] == [7]        # the end tokens are not emitted
    plan = s.plan()
    ev = s.complete(plan, [90])
    assert [(e.id, e.detail) for e in ev if e.kind == Done] == [(ids[1], "eos")]
    assert s.idle() and cache.free_pages(0) == 64


def test_a_request_that_outruns_its_timeout_is_stopped_between_steps():
    # garuda/src/scheduler/mod.rs:1032-1049; here on a clock that the test sets
    s, cache = make(max_concurrent=2, pages=16)
    s.set_time(100.0)
    a = s.submit([1, 2, 3], greedy(max_tokens=50), 0, 5.0)     # running when its time runs out
    b = s.submit([4, 5], greedy(max_tokens=50))                 # no limit
    c = s.submit([6, 7], greedy(max_tokens=50), 0, 2.0)        # still waiting when its time runs out
    with pytest.raises(host.SchedulerError):
        s.submit([1], greedy(), 0, -1.0)
    plan, _ = run_step(s, cache)
    assert sorted(e.id for e in plan.entries) == [a, b] and s.stats().queued == 1
    s.set_time(101.9)
    plan, _ = run_step(s, cache)
    assert not plan.events and s.stats().queued == 1
    s.set_time(102.0)                                           # c's deadline: submission + 2 s
    plan, _ = run_step(s, cache)
    assert [(e.id, e.kind, e.detail) for e in plan.events] == [(c, Error, "timeout")]
    assert sorted(e.id for e in plan.entries) == [a, b]
    held = cache.free_pages(0)
    s.set_time(105.0)
    plan, _ = run_step(s, cache)
    assert [(e.id, e.kind, e.detail) for e in plan.events] == [(a, Error, "timeout")]
    assert [e.id for e in plan.entries] == [b]
    assert not cache.known(a) and cache.free_pages(0) > held    # what it held went back
    st = s.stats()
    assert (st.timed_out, st.cancelled, st.failed, st.running, st.queued) == (2, 0, 0, 1, 0)
    s.set_time(1e9)                                             # b has no deadline
    plan, _ = run_step(s, cache)
    assert [e.id for e in plan.entries] == [b] and not plan.events
    cache.check_invariants()


def test_the_scheduler_clock_runs_by_itself_unless_it_is_set():
    s, _ = make()
    t0 = s.now()
    assert 0.0 <= t0 < 5.0
    import time
    time.sleep(0.02)
    assert s.now() >= t0 + 0.015
    s.set_time(42.0)
    assert s.now() == 42.0


def _next_token(history, vocab):
    """A stand-in for the model: the next token as a function of everything before it."""
    h = 0
    for t in history:
        h = (h * 131 + t + 7) % 1000003
    return h % vocab


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_keep_every_promise(seed):
    """Random arrivals, lengths, priorities, cancellations and limits of time in a pool so small
    that requests are sent back and recomputed. Every step keeps the budget and the portion size,
    feeds each request exactly the positions it has not fed, and loses no page; every request that
    ends normally has the tokens of a run alone, whatever happened to it on the way."""
    import random
    rng = random.Random(seed)
    vocab, eos = 50, 49
    page_size = rng.choice([2, 4, 8])
    max_context = 48
    pages = rng.randint(max_context // page_size + 1, 3 * max_context // page_size)
    max_concurrent = rng.randint(2, 4)
    budget = rng.randint(6, 24)
    chunk = rng.choice([0, 3, 8, 16])
    s, cache = make(pages=pages, page_size=page_size, max_concurrent=max_concurrent, max_batch_tokens=budget,
                    prefill_chunk=chunk, max_context=max_context, queue_capacity=6, eos=eos, vocab=vocab)
    clock = 0.0
    s.set_time(clock)
    prompts, limits, deadline, emitted, ended, fed_history = {}, {}, {}, {}, {}, {}
    cancelled = set()
    to_submit = 25
    for _ in range(4000):
        if to_submit and rng.random() < 0.3:
            prompt = [rng.randrange(vocab - 1) for _ in range(rng.randint(1, 30))]
            limit = rng.randint(1, 25)
            timeout = rng.choice([0.0, 0.0, 0.0, rng.uniform(1.0, 40.0)])
            try:
                rid = s.submit(prompt, greedy(max_tokens=limit), rng.randint(0, 2), timeout)
            except host.Busy:
                pass
            else:
                to_submit -= 1
                prompts[rid], limits[rid], emitted[rid], fed_history[rid] = prompt, limit, [], []
                deadline[rid] = clock + timeout if timeout else None
        live = [r for r in prompts if r not in ended]
        if live and rng.random() < 0.03:
            victim = rng.choice(live)
            s.cancel(victim)
            cancelled.add(victim)
        if s.idle():
            if not to_submit:
                break
            continue
        clock += rng.uniform(0.0, 0.5)
        s.set_time(clock)
        plan = s.plan()
        for ev in plan.events:
            assert ev.kind == Error and ev.id not in ended
            ended[ev.id] = ev.detail
            if ev.detail == "timeout":
                assert deadline[ev.id] is not None and clock >= deadline[ev.id]
            if ev.detail == "cancelled":
                assert ev.id in cancelled
        for rid in plan.preempted:
            fed_history[rid] = []                         # it will be fed again from its first token
        assert plan.num_tokens <= budget and len(plan.entries) <= max_concurrent
        assert len({e.id for e in plan.entries}) == len(plan.entries)
        sampled = []
        for e in plan.entries:
            assert e.id not in ended
            assert deadline[e.id] is None or clock < deadline[e.id]
            assert e.start == len(fed_history[e.id])       # exactly the positions not fed yet
            assert 1 <= len(e.tokens) <= (chunk or budget) or len(e.tokens) == 1
            assert cache.reserved_length(e.id) >= e.start + len(e.tokens) and cache.slot(e.id) == e.slot
            fed_history[e.id] += e.tokens
            whole = prompts[e.id] + emitted[e.id]
            assert fed_history[e.id] == whole[:len(fed_history[e.id])]
            assert e.sample == (len(fed_history[e.id]) == len(whole))
            if e.sample:
                sampled.append(_next_token(fed_history[e.id], vocab))
        for ev in s.complete(plan, sampled):
            assert ev.id not in ended
            if ev.kind == Token:
                emitted[ev.id].append(ev.token)
            else:
                ended[ev.id] = ev.detail
        cache.check_invariants()
        assert s.stats().running <= max_concurrent
    assert s.idle() and not to_submit and set(ended) == set(prompts)
    assert cache.live_requests == 0 and all(cache.free_pages(g) == pages for g in range(cache.num_groups))
    reasons = set(ended.values())
    for rid, prompt in prompts.items():
        # alone: token by token until the limit, the end token or a full context
        seq, want, why = list(prompt), [], None
        while why is None:
            t = _next_token(seq, vocab)
            seq.append(t)
            if t == eos:
                why = "eos"
                break
            want.append(t)
            if len(want) >= limits[rid]:
                why = "length"
            elif len(seq) >= max_context:
                why = "context_full"
        if ended[rid] in ("length", "eos", "context_full"):
            assert (emitted[rid], ended[rid]) == (want, why), rid
        else:
            assert ended[rid] in ("cancelled", "timeout") or "more pages" in ended[rid], ended[rid]
            assert emitted[rid] == want[:len(emitted[rid])]
    st = s.stats()
    assert st.submitted == 25 and st.completed + st.cancelled + st.timed_out + st.failed == 25
    assert reasons & {"length", "eos", "context_full"}


def test_paced_prompt_portions_cost_about_one_decode_step():
    """garuda/src/scheduler/mod.rs:305-370 and :473-491: nothing decoding, a prompt goes in as fast as
    the budget lets it; beside decoding requests it goes in by portions of decode step / prompt token
    tokens (32 until both are measured), moving averages with weight 0.25 on the newest sample."""
    s, cache = make(pages=600, page_size=4, max_batch_tokens=700, prefill_chunk=600, max_context=1000, paced=True)
    p = s.pacing
    assert (p.decode_step, p.prefill_token, p.chunk) == (-1.0, -1.0, 32)
    a = s.submit(list(range(50)), greedy(max_tokens=100))
    plan = s.plan()
    assert [(e.id, len(e.tokens), e.decode) for e in plan.entries] == [(a, 50, False)]    # nobody to stall
    s.complete(plan, [1], 0.050)                            # 1 ms a prompt token
    assert s.pacing.prefill_token == pytest.approx(0.001) and s.pacing.chunk == 32         # no decode step seen yet
    b = s.submit([3] * 99, greedy(max_tokens=100))
    plan = s.plan()
    assert [(e.id, len(e.tokens), e.decode) for e in plan.entries] == [(a, 1, True), (b, 32, False)]
    s.complete(plan, [1], 0.040)                            # a mixed step before any decode step was timed: no sample
    assert s.pacing.decode_step == -1.0 and s.pacing.prefill_token == pytest.approx(0.001)
    s.cancel(b)
    plan = s.plan()
    assert [(e.id, e.decode) for e in plan.entries] == [(a, True)]
    s.complete(plan, [1], 0.010)                            # a decode step: 10 ms
    assert s.pacing.decode_step == pytest.approx(0.010) and s.pacing.chunk == 10
    plan = s.plan()
    s.complete(plan, [1], 0.020)
    assert s.pacing.decode_step == pytest.approx(0.0125) and s.pacing.chunk == 12          # 0.75 * 10 + 0.25 * 20
    c = s.submit([5] * 100, greedy(max_tokens=100))
    plan = s.plan()
    assert [(e.id, len(e.tokens)) for e in plan.entries] == [(a, 1), (c, 12)]
    s.complete(plan, [1], 0.0125 + 12 * 0.003)              # the time beyond a decode step is the prompt tokens'
    assert s.pacing.prefill_token == pytest.approx(0.75 * 0.001 + 0.25 * 0.003)
    assert s.pacing.chunk == 8                              # 12.5 ms / 1.5 ms
    plan = s.plan()
    assert [(e.id, e.start, len(e.tokens)) for e in plan.entries] == [(a, 54, 1), (c, 12, 8)]
    # the estimate is held to [1, 512], and to the configured portion
    s.complete(plan, [1], 100.0)
    assert s.pacing.chunk == 1
    for _ in range(40):
        plan = s.plan()
        if len(plan.entries) == 1:
            break
        assert len(plan.entries[1].tokens) == 1
        s.complete(plan, [1] * sum(e.sample for e in plan.entries))
    s2, _ = make(pages=600, page_size=4, max_batch_tokens=700, prefill_chunk=20, max_context=1000, paced=True)
    x = s2.submit([1, 2], greedy(max_tokens=100))
    s2.complete(s2.plan(), [1], 0.001)
    s2.complete(s2.plan(), [1], 1.0)                        # a decode step of a second
    y = s2.submit([7] * 300, greedy())
    plan = s2.plan()
    assert s2.pacing.chunk == 512 and [(e.id, len(e.tokens)) for e in plan.entries] == [(x, 1), (y, 20)]
    # without pacing the portion is the configured one
    s3, _ = make(pages=600, page_size=4, max_batch_tokens=700, prefill_chunk=600, max_context=1000)
    x = s3.submit([1, 2], greedy(max_tokens=100))
    s3.complete(s3.plan(), [1], 0.5)
    y = s3.submit([7] * 300, greedy())
    assert [(e.id, len(e.tokens)) for e in s3.plan().entries] == [(x, 1), (y, 300)]
