"""The plain implementation's parts against closed forms (as the reference's own unit tests do,
test/test_transformer.c:427-624)."""
import numpy as np

import plain_llama as P


def test_rmsnorm_closed_form():
    x = np.array([[3.0, 4.0]])
    out = P.rmsnorm(x, np.array([2.0, 0.5]), 1e-5)
    s = 1 / np.sqrt(12.5 + 1e-5)
    assert np.allclose(out, [[3 * s * 2, 4 * s * 0.5]])


def test_rope_identity_at_zero_and_norm_preserved():
    x = np.random.default_rng(0).normal(size=(3, 2, 16))
    assert np.array_equal(P.apply_rope(x, [0, 0, 0], 10000.0), x)
    y = P.apply_rope(x, [5, 77, 1000], 500000.0)
    assert np.allclose(np.linalg.norm(x, axis=-1), np.linalg.norm(y, axis=-1))
    # pairs are (i, i + half): rotating by pos 1 turns (1, 0) in the first pair by one radian
    e = np.zeros((1, 1, 4))
    e[0, 0, 0] = 1
    r = P.apply_rope(e, [1], 10000.0)
    assert np.allclose(r[0, 0], [np.cos(1), 0, np.sin(1), 0], atol=1e-7)


def test_softmax_and_attention_causal_and_window():
    p = P.softmax(np.array([1.0, 2.0, 3.0]))
    assert abs(p.sum() - 1) < 1e-12 and p[2] > p[1] > p[0]
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(6, 4, 8)), rng.normal(size=(6, 2, 8)), rng.normal(size=(6, 2, 8))
    out = P.attention(q, k, v, 8 ** -0.5)
    assert np.allclose(out[0, 0], v[0, 0]) and np.allclose(out[0, 3], v[0, 1])  # token 0 sees itself; heads 2,3 share kv head 1
    k2 = k.copy()
    k2[5] += 10
    assert np.allclose(P.attention(q, k2, v, 8 ** -0.5)[:5], out[:5])  # later keys do not reach earlier tokens
    w = P.attention(q, k, v, 8 ** -0.5, window=2)
    assert np.allclose(w[:2], out[:2]) and not np.allclose(w[5], out[5])


def test_sampler_generator_and_walk():
    r = P.Xorshift64Star(0)
    assert r.state == 42
    a = [r.next_float() for _ in range(3)]
    assert all(0 <= x < 1 for x in a) and len(set(a)) == 3
    logits = np.array([0.0, 5.0, 1.0], dtype=np.float32)
    assert P.sample(logits, 0.0, 0.9, P.Xorshift64Star(1)) == 1
    picks = [P.sample(logits, 1.0, 1.0, P.Xorshift64Star(s)) for s in range(1, 200)]
    assert set(picks) <= {0, 1, 2} and picks.count(1) > 150
    assert all(P.sample(logits, 1.0, 0.5, P.Xorshift64Star(s)) == 1 for s in range(1, 50))  # nucleus of one
    pen = P.apply_repeat_penalty(np.array([2.0, -2.0, 1.0]), [0, 1, 0], 2.0)
    assert pen.tolist() == [1.0, -4.0, 1.0]
