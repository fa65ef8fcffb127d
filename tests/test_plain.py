"""The plain implementation checks itself where a property is known
(the reference tests the same ones: garuda/src/simd/mod.rs:251-298,
garuda/src/attention/mod.rs:161-238, garuda/src/runtime/mod.rs:1112-1224)."""
import numpy as np
import pytest

from tests.plain import llama_plain as P
from tests.plain.sampling_plain import Rng, sample, candidates
from tests.helpers import TINY, model_dir, folder_weights, random_tokens


def test_rope_keeps_norm_and_is_identity_at_zero():
    v = np.random.default_rng(0).standard_normal((3, 2, 8)).astype(np.float32)
    for layout in ("half", "interleaved"):
        out = P.rope(v, np.array([5, 0, 77]), 10000.0, layout)
        assert np.allclose(np.linalg.norm(out, axis=-1), np.linalg.norm(v, axis=-1), atol=1e-5)
        assert np.allclose(out[1], v[1], atol=1e-6)


def test_rope_layouts_agree_after_permuting_rows():
    # rotating interleaved pairs of permuted vectors equals rotating half-split pairs
    v = np.random.default_rng(1).standard_normal((4, 1, 16)).astype(np.float32)
    pos = np.array([3, 9, 0, 40])
    perm = np.concatenate([np.arange(0, 16, 2), np.arange(1, 16, 2)])   # interleaved -> half order
    a = P.rope(v, pos, 500000.0, "interleaved")[..., perm]
    b = P.rope(v[..., perm], pos, 500000.0, "half")
    assert np.allclose(a, b, atol=1e-6)


def test_softmax_fallbacks():
    assert np.allclose(P.softmax(np.array([1000.0, 1000.5, 999.0], dtype=np.float32)).sum(), 1, atol=1e-5)
    assert np.allclose(P.softmax(np.full(3, -np.inf, dtype=np.float32)), 1 / 3)
    out = P.softmax(np.array([1.0, np.nan, 2.0], dtype=np.float32))
    assert np.isfinite(out).all() and abs(out.sum() - 1) < 1e-5


def test_first_token_attends_only_to_itself_and_window_cuts():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((6, 2, 4)).astype(np.float32)
    k = rng.standard_normal((6, 1, 4)).astype(np.float32)
    v = rng.standard_normal((6, 1, 4)).astype(np.float32)
    out = P.attention(q, k, v, None).reshape(6, 2, 4)
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 1], v[0, 0])
    # causality: changing a later key leaves earlier outputs alone
    k2, v2 = k.copy(), v.copy()
    k2[4] += 1.0
    v2[4] -= 2.0
    out2 = P.attention(q, k2, v2, None).reshape(6, 2, 4)
    assert np.array_equal(out[:4], out2[:4]) and not np.allclose(out[4:], out2[4:])
    # window of 2: position 5 reads keys 4 and 5 only
    w = P.attention(q, k, v, 2).reshape(6, 2, 4)
    s = (k[4:6, 0] @ q[5, 0]) * 0.5
    p = np.exp(s - s.max()); p /= p.sum()
    assert np.allclose(w[5, 0], p @ v[4:6, 0], atol=1e-6)


def test_forward_float32_against_float64():
    cfg, _, _ = TINY["A"]
    w = folder_weights(model_dir("A"))
    toks = random_tokens("A", 40, 0)
    a = P.forward(cfg, w, toks, np.float32)
    b = P.forward(cfg, w, toks, np.float64)
    assert np.abs(a - b).max() < 1e-5 * max(1.0, np.abs(b).max())


def test_sampler_properties():
    rng = np.random.default_rng(3)
    logits = rng.standard_normal(50).astype(np.float32)
    assert sample(logits, 0.0, 40, 0.95, Rng(1)) == int(np.argmax(logits))
    assert sample(logits, 0.8, 1, 1.0, Rng(7)) == int(np.argmax(logits))
    a = [sample(logits, 0.8, 40, 0.95, Rng(11)) for _ in range(3)]
    assert a[0] == a[1] == a[2] and 0 <= a[0] < 50
    c = candidates(logits, 1.0, 5, 1.0)
    assert [t for t, _ in c] == list(np.argsort(-logits, kind="stable")[:5])
    # ties break on the lower token id
    tied = np.zeros(6, dtype=np.float32)
    assert [t for t, _ in candidates(tied, 1.0, 3, 1.0)] == [0, 1, 2]
    # first maximum wins
    assert P.argmax_first(np.array([1.0, 3.0, 3.0, 2.0])) == 1


def test_generator_matches_the_host_runtime():
    from garuda_b200.csrc.build import load_host_module
    host = load_host_module()
    for seed in (0, 1, 0xBEEF, 2**63 + 5):
        a, b = Rng(seed), host.Rng(seed)
        for _ in range(5):
            assert a.next_u64() == b.next_u64()
        assert float(a.next_f32()) == b.next_f32()


@pytest.mark.parametrize("name", sorted(TINY))
def test_the_two_restatements_agree(name):
    """The numpy restatement (whole sequences, numpy's sums) and the scalar C++ one (token by token
    over a growing cache, every sum in the reference's order), written apart from the same lines of
    the reference, give the same logits to 32-bit rounding, in every tiny configuration: both
    pairings of the rotation, windows, tied and untied heads, groups of one, two and three. Each is
    as far from the 64-bit result as the other."""
    from tests.plain import llama_scalar
    cfg = TINY[name][0]
    w = folder_weights(model_dir(name))
    toks = random_tokens(name, min(cfg["max_position_embeddings"], 200), 17)     # beyond every window
    a = P.forward(cfg, w, toks, np.float32)
    b = llama_scalar.forward(cfg, w, toks)
    exact = P.forward(cfg, w, toks, np.float64)
    top = np.abs(exact).max()
    assert np.abs(a - b).max() <= 5e-6 * top
    assert np.abs(a - exact).max() <= 5e-6 * top and np.abs(b - exact).max() <= 5e-6 * top
    # the same first maximum at every position: greedy decoding agrees token for token
    assert [P.argmax_first(r) for r in a] == [P.argmax_first(r) for r in b]
    with pytest.raises(ValueError):
        llama_scalar.forward(cfg, w, [0, cfg["vocab_size"]])
