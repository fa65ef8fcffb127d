"""The C++ step builder (csrc/host/step_batch.hpp) alone: what it refuses, what it reserves, and
the arrays it writes for the kernels, against a restatement in numpy."""
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import pytest

from garuda_b200.csrc.build import load_host_module

host = load_host_module()


@dataclass
class Entry:
    request: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


def manager(pages=(64, 64), windows=(0, 24), page_size=8, max_requests=4, max_positions=128):
    return host.CacheManager([host.GroupConfig(p, w) for p, w in zip(pages, windows)], page_size,
                             max_requests, max_positions)


def run_step(mgr, b, entries):
    """Checks, reserves, fills, commits; returns (layout, the buffer, new_lens)."""
    reqs = host.StepRequests(entries)
    res = b.check_and_reserve(reqs)
    lay = b.layout(reqs)
    buf = np.full(lay.words + 5, -7, dtype=np.int32)
    b.fill(reqs, res.new_lens, lay, buf)
    b.commit(res.new_lens)
    return lay, buf, res


def test_the_arrays_of_a_mixed_step():
    mgr = manager()
    b = host.StepBuilder(mgr, 1000)
    # request 5 has 37 positions already; 9 comes new with a portion of 19 tokens; 7 new with one token
    _, _, first = run_step(mgr, b, [Entry(5, list(range(37)), [36])])
    assert first.new_lens == [(5, 37)] and first.starting_slots == [mgr.slot(5)]
    entries = [Entry(5, [11], [0]), Entry(9, list(range(100, 119)), [0, 18]), Entry(7, np.array([3]), [])]
    lay, buf, res = run_step(mgr, b, entries)
    assert res.new_lens == [(5, 38), (9, 19), (7, 1)]
    assert sorted(res.starting_slots) == sorted([mgr.slot(9), mgr.slot(7)])
    assert (lay.tokens, lay.rows, lay.wanted, lay.groups, lay.table_width) == (21, 3, 3, 2, 16)
    assert (lay.max_q, lay.min_q, lay.max_kv) == (19, 1, 38)
    starts = [lay.token_ids, lay.positions, lay.token_req, lay.cu_q, lay.kv_lens, lay.slots, lay.logit_rows, lay.tables]
    assert all(s % 4 == 0 for s in starts) and starts == sorted(starts)
    assert lay.words == lay.tables + 2 * 3 * 16 and (buf[lay.words:] == -7).all()

    def arr(at, n):
        return buf[at:at + n].tolist()

    assert arr(lay.token_ids, 21) == [11] + list(range(100, 119)) + [3]
    assert arr(lay.positions, 21) == [37] + list(range(19)) + [0]
    assert arr(lay.token_req, 21) == [0] + [1] * 19 + [2]
    assert arr(lay.cu_q, 4) == [0, 1, 20, 21]
    assert arr(lay.kv_lens, 3) == [38, 19, 1]
    assert arr(lay.slots, 3) == [mgr.slot(5), mgr.slot(9), mgr.slot(7)]
    assert arr(lay.logit_rows, 3) == [0, 1, 19]
    tables = buf[lay.tables:lay.words].reshape(2, 3, 16)
    for g in range(2):
        for i, r in enumerate((5, 9, 7)):
            assert tables[g, i].tolist() == mgr.block_table_row(r, g).tolist()
    # the windowed group has given request 5's first page back (positions 0-7 lie behind 38 + 1 - 24)
    assert tables[0, 0, 0] >= 0 and tables[1, 0, 0] == -1 and tables[1, 0, 4] >= 0
    mgr.check_invariants()


def test_a_step_of_single_tokens_padded_to_a_fixed_number_of_rows():
    mgr = manager()
    b = host.StepBuilder(mgr, 50)
    run_step(mgr, b, [Entry(1, [1] * 9), Entry(2, [2] * 20)])
    entries = [Entry(2, [7], [0]), Entry(1, [8], [0]), Entry(3, [9], [0])]
    reqs = host.StepRequests(entries)
    res = b.check_and_reserve(reqs)
    lay = b.decode_layout(4)
    buf = np.zeros(lay.words, dtype=np.int32)
    b.fill_decode(reqs, res.new_lens, lay, buf)
    b.commit(res.new_lens)

    def arr(at, n):
        return buf[at:at + n].tolist()

    assert arr(lay.token_ids, 4) == [7, 8, 9, 0]
    assert arr(lay.positions, 4) == [20, 9, 0, 0]
    assert arr(lay.token_req, 4) == [0, 1, 2, 3] and arr(lay.cu_q, 5) == [0, 1, 2, 3, 4]
    assert arr(lay.kv_lens, 4) == [21, 10, 1, 1]
    assert arr(lay.slots, 4) == [mgr.slot(2), mgr.slot(1), mgr.slot(3), -1]
    assert arr(lay.logit_rows, 4) == [0, 1, 2, 3]
    tables = buf[lay.tables:lay.words].reshape(2, 4, 16)
    assert (tables[:, 3] == -1).all()                       # the padding row holds no page
    assert tables[0, 0].tolist() == mgr.block_table_row(2, 0).tolist()
    with pytest.raises(host.StepError):                     # more requests than rows
        b.fill_decode(reqs, res.new_lens, b.decode_layout(2), buf)
    with pytest.raises(host.StepError):                     # a portion is no decode step
        two = host.StepRequests([Entry(1, [1, 2])])
        b.fill_decode(two, [(1, 12)], lay, buf)


def test_what_is_refused_and_that_nothing_changes_then():
    mgr = manager(pages=(6, 6), windows=(0, 0), max_requests=2, max_positions=40)
    b = host.StepBuilder(mgr, 100)
    run_step(mgr, b, [Entry(1, [1] * 10)])
    free, slots = mgr.free_pages(0), mgr.free_slots
    for bad, words in (
            ([], "at least one entry"),
            ([Entry(1, [100])], "token 100 of request 1 is outside the vocabulary of 100"),
            ([Entry(1, [-1])], "outside the vocabulary"),
            ([Entry(1, [1]), Entry(1, [2])], "request 1 appears twice"),
            ([Entry(1, [1], [1])], "request 1 wants logits at place 1 of 1 tokens"),
            ([Entry(1, [1], [-1])], "wants logits at place -1"),
            ([Entry(1, [])], "request 1 brings no tokens"),
            ([Entry(1, [1] * 31)], "31 tokens do not fit the 40-position context (10 used) of request 1"),
            ([Entry(1, [1]), Entry(2, [1]), Entry(3, [1])], "2 new requests but only 1 request slots are free"),
            ([Entry(1, [1.5])], "must be integers"),
            ([Entry("one", [1])], "must be integers")):
        with pytest.raises(host.StepError) as info:
            b.check_and_reserve(host.StepRequests(bad))
        assert words in str(info.value)
        assert isinstance(info.value, ValueError)
    # pages: request 1 holds 2 of 6; 1 more token for it and 40 for a new one need 0 + 5 > 4
    with pytest.raises(host.OutOfPages) as info:
        b.check_and_reserve(host.StepRequests([Entry(1, [1]), Entry(2, [1] * 40)]))
    assert "needs [5, 5] pages per group but only [4, 4] are free" in str(info.value)
    assert mgr.free_pages(0) == free and mgr.free_slots == slots and not mgr.known(2) and mgr.length(1) == 10
    mgr.check_invariants()
    # a buffer that is too small is refused before anything is written
    reqs = host.StepRequests([Entry(1, [1, 2, 3])])
    res = b.check_and_reserve(reqs)
    lay = b.layout(reqs)
    small = np.zeros(lay.words - 1, dtype=np.int32)
    with pytest.raises(host.StepError):
        b.fill(reqs, res.new_lens, lay, small)
    assert not small.any()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_batches_against_a_restatement(seed):
    rng = np.random.default_rng(seed)
    mgr = manager(pages=(200, 200), windows=(0, 16), max_requests=4, max_positions=96)
    b = host.StepBuilder(mgr, 500)
    lens = {}
    next_id = 0
    for _ in range(60):
        live = list(lens)
        while len(live) < 4 and rng.random() < 0.5:
            live.append(next_id)
            lens[next_id] = 0
            next_id += 1
        if not live:
            continue
        rng.shuffle(live)
        entries = []
        for r in live[:int(rng.integers(1, len(live) + 1))]:
            room = 96 - lens[r]
            n = int(min(room, rng.integers(1, 20))) if rng.random() < 0.6 else 1
            toks = rng.integers(0, 500, n).tolist()
            want = sorted(set(rng.integers(0, n, int(rng.integers(0, 3))).tolist()))
            entries.append(Entry(r, toks, want))
        lay, buf, res = run_step(mgr, b, entries)
        t = 0
        rows = []
        for i, e in enumerate(entries):
            n = len(e.tokens)
            assert buf[lay.token_ids + t:lay.token_ids + t + n].tolist() == list(e.tokens)
            assert buf[lay.positions + t:lay.positions + t + n].tolist() == list(range(lens[e.request], lens[e.request] + n))
            assert (buf[lay.token_req + t:lay.token_req + t + n] == i).all()
            rows += [t + w for w in e.want]
            t += n
            lens[e.request] += n
            assert buf[lay.cu_q + i + 1] == t and buf[lay.kv_lens + i] == lens[e.request]
            assert mgr.length(e.request) == lens[e.request]
        assert buf[lay.logit_rows:lay.logit_rows + lay.wanted].tolist() == rows
        for r in list(lens):
            if lens[r] >= 96 or rng.random() < 0.1:
                if mgr.known(r):              # it may not have been in a step yet
                    mgr.release(r)
                del lens[r]
        mgr.check_invariants()
