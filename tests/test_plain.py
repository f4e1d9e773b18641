"""The plain implementation checked against itself and against hand-made cases (CPU)."""
import numpy as np
import pytest

from plain import qwen2_moe_plain as P
from conftest import TINY


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_a_prefix_gives_the_same_logits(plain_models, name):
    m = plain_models[name]
    toks = np.random.default_rng(0).integers(0, TINY[name][0]["vocab_size"], size=50).tolist()
    full = P.forward(m, toks)
    assert np.isfinite(full).all()
    assert np.abs(full[:20] - P.forward(m, toks[:20])).max() < 1e-12      # causal


def test_rmsnorm_and_softmax_by_hand():
    x = np.array([[3.0, 4.0]])
    assert np.allclose(P.rmsnorm(x, np.array([1.0, 2.0]), 0.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    assert np.allclose(P.softmax(np.array([1000.0, 1000.0])), [0.5, 0.5])


def test_rotary_pairings():
    x = np.arange(8, dtype=float).reshape(1, 1, 8)
    assert np.allclose(P.rotary(x, np.array([0]), 1e4, "half"), x)         # position 0 is the identity
    h = P.rotary(x, np.array([3]), 1e4, "half")
    i = P.rotary(x, np.array([3]), 1e4, "interleaved")
    assert np.allclose(np.linalg.norm(h), np.linalg.norm(x)) and np.allclose(np.linalg.norm(i), np.linalg.norm(x))
    perm = [0, 4, 1, 5, 2, 6, 3, 7]                                        # interleaved = half on permuted dims
    assert np.allclose(P.rotary(x[..., perm], np.array([3]), 1e4, "interleaved")[..., [0, 2, 4, 6, 1, 3, 5, 7]],
                       P.rotary(x, np.array([3]), 1e4, "half"))


def test_attention_window_and_groups():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(9, 4, 8)), rng.normal(size=(9, 2, 8)), rng.normal(size=(9, 2, 8))
    full = P.attention(q, k, v, 0)
    assert np.allclose(full[0], np.concatenate([v[0, 0], v[0, 0], v[0, 1], v[0, 1]]))    # position 0 sees itself only
    assert np.allclose(P.attention(q, k, v, 100), full)
    one = P.attention(q, k, v, 1)
    assert np.allclose(one[5], np.concatenate([v[5, 0], v[5, 0], v[5, 1], v[5, 1]]))
    w3 = P.attention(q, k, v, 3)
    assert np.allclose(w3[:3], full[:3]) and not np.allclose(w3[5], full[5])


def test_router_norm_and_ties():
    x = np.eye(3)
    wr = np.array([[1.0, 0, 0], [0.5, 0, 0], [1.0, 0, 0], [0, 0, 0]])
    ids, w, margin = P.router(x[:1], wr, 2, False)
    assert ids.tolist() == [[0, 2]]                                         # equal logits: the lower index first
    p = np.exp([1, .5, 1, 0]) / np.exp([1, .5, 1, 0]).sum()
    assert np.allclose(w, [[p[0], p[2]]]) and np.allclose(margin, [0.5 / np.std([1, .5, 1, 0])])
    _, wn, _ = P.router(x[:1], wr, 2, True)
    assert np.allclose(wn.sum(), 1.0) and np.allclose(wn, [[0.5, 0.5]])


def test_sampling_rules():
    l = np.array([0.0, 5.0, 5.0, 1.0])
    assert P.sample_argmax(l) == 1
    assert P.sample_top_p(l, 0.0, 0.9, 0.3) == 1 and P.sample_top_p(l, 1.0, 0.0, 0.3) == 1
    assert P.sample_top_p(l, 1.0, 1.0, 0.0) == 1 and P.sample_top_p(l, 1.0, 1.0, 0.6) == 2
    assert P.sample_top_p(l, 1.0, 0.4, 0.99) == 1                           # the nucleus holds the first maximum only
    assert P.sample_top_p(np.array([0.0, 100.0]), 1.0, 1.0, 0.999999) == 1  # the prefilter drops the other
    draws = [P.sample_top_p(np.zeros(4), 1.0, 1.0, P.uniform_for(1, 0, s)) for s in range(4000)]
    assert all(abs(draws.count(t) / 4000 - 0.25) < 0.03 for t in range(4))


def test_bf16_rounding():
    a = np.array([1.0, 1.00390625, 1.001953125, 1.005859375, -3.1415926])
    r = P.round_bf16(a)
    assert r.tolist()[:4] == [1.0, 1.0, 1.0, 1.0078125]                      # ties to even
    assert abs(r[4] + 3.140625) < 1e-9


def test_repetition_penalty_of_the_plain_loop():
    """Once per occurrence among the last `window` tokens; positive logits are divided, the others multiplied
    (src/engine/tq_generate.c:586-600); ids outside the vocabulary are skipped (:592)."""
    l = np.array([2.0, -1.0, 0.0, 4.0, 0.5], dtype=np.float32)
    out = P.repetition_penalty(l, [0, 1, 3, 3, 7, -1], 2.0)
    assert np.allclose(out, [1.0, -2.0, 0.0, 1.0, 0.5]) and out.dtype == np.float32
    assert np.array_equal(l, np.array([2.0, -1.0, 0.0, 4.0, 0.5], dtype=np.float32))       # the input is left alone
    assert P.recent_tokens([1, 2, 3, 4], [5, 6], 3) == [4, 5, 6]
    assert P.recent_tokens([1, 2], [], 32) == [1, 2] and P.recent_tokens([1], [2], 0) == []
    assert len(P.recent_tokens(list(range(300)), [], 1000)) == 128
