"""The plain implementation's parts against hand-made cases and against each other."""
import math

import numpy as np

import plain_llama as plain
import tiny


def test_rmsnorm_by_hand():
    x = np.array([[3.0, 4.0]])
    got = plain.rmsnorm(x, np.array([2.0, 0.5]), 0.5)
    inv = 1 / math.sqrt((9 + 16) / 2 + 0.5)
    assert np.allclose(got, [[3 * inv * 2, 4 * inv * 0.5]])


def test_rope_pairings_by_hand():
    x = np.arange(1.0, 9.0).reshape(1, 8)       # one head of 8 dims
    inv = plain.rope_inv_freq(4, 100.0)          # rotate 4 of 8 dims
    assert np.allclose(inv, [1.0, 0.1])
    pos = [3]
    c, s = np.cos(3 * inv), np.sin(3 * inv)
    ll = plain.rope(x, pos, 1, 8, 4, inv, "llama")[0, 0]
    assert np.allclose(ll[:4], [1 * c[0] - 2 * s[0], 1 * s[0] + 2 * c[0], 3 * c[1] - 4 * s[1], 3 * s[1] + 4 * c[1]])
    assert np.allclose(ll[4:], [5, 6, 7, 8])
    nx = plain.rope(x, pos, 1, 8, 4, inv, "neox")[0, 0]
    assert np.allclose(nx[:4], [1 * c[0] - 3 * s[0], 2 * c[1] - 4 * s[1], 1 * s[0] + 3 * c[0], 2 * s[1] + 4 * c[1]])
    assert np.allclose(nx[4:], [5, 6, 7, 8])
    assert np.allclose(plain.rope(x, [0], 1, 8, 4, inv, "neox")[0, 0], x[0])


def test_llama3_scaling_hits_all_three_branches():
    sc = tiny.TINY_B["rope_scaling"]
    inv = plain.rope_inv_freq(32, 500000.0)
    out = plain.scale_inv_freq(inv, sc)
    lam = 2 * math.pi / inv
    L = sc["original_max_position_embeddings"]
    kept, blended, divided = lam < L / 4, (lam >= L / 4) & (lam <= L / 1), lam > L
    assert kept.any() and blended.any() and divided.any()
    assert np.allclose(out[kept], inv[kept])
    assert np.allclose(out[divided], inv[divided] / 4)
    assert ((out[blended] <= inv[blended]) & (out[blended] >= inv[blended] / 4)).all()
    assert np.allclose(plain.scale_inv_freq(inv, {"rope_type": "linear", "factor": 2.0}), inv / 2)
    assert plain.scale_inv_freq(inv, None) is inv


def test_attention_grouped_equals_per_head_einsum():
    """The reference's grouped form (alpacca/model.py:457-467) against the per-head loop."""
    rng = np.random.default_rng(0)
    T, H, K, D = 5, 4, 2, 3
    q, k, v = rng.standard_normal((T, H, D)), rng.standard_normal((T, K, D)), rng.standard_normal((T, K, D))
    got = plain.attention(q, k, v)
    qg = q.reshape(T, K, H // K, D)
    sc = np.einsum("tkgh,skh->tkgs", qg, k) / math.sqrt(D)
    sc = np.where(np.arange(T)[None, :] <= np.arange(T)[:, None], 0, -1e30)[:, None, None, :] + sc
    w = np.exp(sc - sc.max(-1, keepdims=True))
    w /= w.sum(-1, keepdims=True)
    want = np.einsum("tkgs,skh->tkgh", w, v).reshape(T, H, D)
    assert np.abs(got - want).max() < 1e-12
    # a window of 2 keeps the token itself and one before
    win = plain.attention(q, k, v, window=2)
    assert np.allclose(win[0], got[0]) and np.allclose(win[1], got[1]) and not np.allclose(win[4], got[4])


def test_swiglu_by_hand():
    assert np.allclose(plain.swiglu([0.0, 2.0], [5.0, 3.0]), [0.0, 2 / (1 + math.exp(-2)) * 3])


def test_philox_known_answer():
    # Random123's known-answer vectors for philox4x32-10
    assert plain.philox4x32([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert plain.philox4x32([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert plain.philox4x32([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]
    us = [plain.uniform(7, 3, s) for s in range(1000)]
    assert all(0 <= u < 1 for u in us) and 0.45 < sum(us) / 1000 < 0.55


def test_sampler_rules():
    l = np.array([1.0, 3.0, 3.0, 0.5, 2.0])
    assert plain.sample(l, 0.0, 40, 0.95, 0.3) == 1            # greedy: first index of the maximum
    assert plain.sample(l, 1.0, 1, 1.0, 0.99) == 1             # top_k 1, tie to the lower index
    # top_k 2 keeps indices 1 and 2, equal weights: u below a half -> 1, above -> 2
    assert plain.sample(l, 1.0, 2, 1.0, 0.49) == 1 and plain.sample(l, 1.0, 2, 1.0, 0.51) == 2
    # top_p: probabilities of (1, 2, 4) are about (.40, .40, .15): 0.5 keeps the two threes
    assert {plain.sample(l, 1.0, 0, 0.5, u) for u in np.linspace(0, 0.999, 50)} == {1, 2}
    assert {plain.sample(l, 1.0, 0, 0.85, u) for u in np.linspace(0, 0.999, 200)} == {1, 2, 4}
    # all kept: every index can come, in index order of the running sum
    assert plain.sample(l, 1.0, 0, 1.0, 0.0) == 0 and plain.sample(l, 1.0, 0, 1.0, 0.9999) == 4
    # penalty: positive logits divided, others multiplied, each distinct token once
    assert np.allclose(plain.penalize([2.0, -2.0, 1.0], [0, 1, 0], 2.0), [1.0, -4.0, 1.0])


def test_plain_generate_stop_and_budget():
    cfg = tiny.TINY_A
    m = plain.PlainLlama(cfg, tiny.make_weights(cfg, 0))
    toks, rows = plain.generate(m, [5, 6, 7], 4)
    assert len(toks) == 4 and len(rows) == 4
    toks2, _ = plain.generate(m, [5, 6, 7], 4, stop=(toks[1],))
    assert toks2 == toks[:2]          # the stop token is counted and ends the sequence
