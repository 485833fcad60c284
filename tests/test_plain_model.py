"""The plain implementation checked against itself (no GPU): properties that any correct
restatement of the formulas must have, so that a slip in the oracle does not hide in every
comparison that uses it."""
from __future__ import annotations

import numpy as np
import pytest

import plain_lfm2
from tiny_models import write_tiny


@pytest.fixture(scope="module")
def model_b(tmp_path_factory):
    folder = write_tiny(tmp_path_factory.mktemp("plain"), "B")
    return plain_lfm2.load_model_folder(folder)


def test_logits_are_causal(model_b):
    config, weights = model_b
    rng = np.random.default_rng(0)
    tokens = rng.integers(0, config["vocab_size"], size=24).tolist()
    full = plain_lfm2.forward(config, weights, tokens)
    prefix = plain_lfm2.forward(config, weights, tokens[:11])
    assert np.allclose(full[:11], prefix, atol=1e-12)
    changed = list(tokens)
    changed[15] = (changed[15] + 1) % config["vocab_size"]
    other = plain_lfm2.forward(config, weights, changed)
    assert np.allclose(full[:15], other[:15], atol=1e-12) and not np.allclose(full[15:], other[15:])


def test_rmsnorm_scale_and_unit_rms():
    rng = np.random.default_rng(1)
    x = rng.normal(size=(5, 33))
    y = plain_lfm2.rmsnorm(x, np.ones(33), 1e-12)
    assert np.allclose(np.sqrt((y * y).mean(axis=-1)), 1.0)
    assert np.allclose(plain_lfm2.rmsnorm(3.0 * x, np.ones(33), 1e-12), y)
    w = rng.normal(size=33)
    assert np.allclose(plain_lfm2.rmsnorm(x, w, 1e-12), y * w)


def test_rope_is_a_rotation_that_depends_on_relative_position():
    rng = np.random.default_rng(2)
    q = rng.normal(size=(1, 1, 32))
    k = rng.normal(size=(1, 1, 32))
    def score(pq, pk):
        a = plain_lfm2.rope_split_half(q, np.array([pq]), 10000.0)[0, 0]
        b = plain_lfm2.rope_split_half(k, np.array([pk]), 10000.0)[0, 0]
        return float(a @ b)
    assert np.isclose(score(7, 3), score(107, 103))
    assert np.isclose(score(0, 0), float(q[0, 0] @ k[0, 0]))
    rotated = plain_lfm2.rope_split_half(q, np.array([55]), 1e6)
    assert np.isclose(np.linalg.norm(rotated), np.linalg.norm(q))
    # pairs are (i, i + d/2): at position 1 the first pair turns by angle 1, the last by theta^(-(d-2)/d)
    e = np.zeros((1, 1, 32)); e[0, 0, 0] = 1.0
    out = plain_lfm2.rope_split_half(e, np.array([1]), 10000.0)[0, 0]
    assert np.isclose(out[0], np.cos(1.0)) and np.isclose(out[16], np.sin(1.0))


def test_short_conv_is_causal_with_the_last_tap_on_the_current_token():
    hidden, taps, tokens = 6, 3, 9
    rng = np.random.default_rng(3)
    n = rng.normal(size=(tokens, hidden))
    w_in = np.concatenate([np.eye(hidden), np.eye(hidden), np.eye(hidden)])        # B = C = X = n
    kernel = np.zeros((hidden, 1, taps)); kernel[:, 0, taps - 1] = 1.0            # only the current token
    out = plain_lfm2.short_conv_mixer(n, w_in, kernel, np.eye(hidden))
    assert np.allclose(out, n ** 3)                                               # C * (B*X)
    kernel = np.zeros((hidden, 1, taps)); kernel[:, 0, 0] = 1.0                   # only the token two back
    out = plain_lfm2.short_conv_mixer(n, w_in, kernel, np.eye(hidden))
    assert np.allclose(out[:2], 0.0) and np.allclose(out[2:], n[2:] * n[:-2] ** 2)


def test_attention_reduces_to_the_value_of_a_dominant_key():
    hidden, heads, kv_heads, d = 16, 2, 1, 8
    rng = np.random.default_rng(4)
    n = rng.normal(size=(6, hidden))
    wq = rng.normal(size=(heads * d, hidden)); wk = rng.normal(size=(kv_heads * d, hidden))
    wv = rng.normal(size=(kv_heads * d, hidden)); wo = np.eye(hidden, heads * d)
    ones = np.ones(d)
    out = plain_lfm2.attention_mixer(n, wq, wk, wv, wo, ones, ones, heads, kv_heads, d, 1e4, 1e-6)
    first = (n[:1] @ wv.T)                                                       # token 0 sees only itself
    assert np.allclose(out[0], np.concatenate([first[0], first[0]]) @ wo.T)
    windowed = plain_lfm2.attention_mixer(n, wq, wk, wv, wo, ones, ones, heads, kv_heads, d, 1e4, 1e-6, window=1)
    values = n @ wv.T
    assert np.allclose(windowed, np.concatenate([values, values], axis=1) @ wo.T)  # window 1: own value only


def test_sampler_rules():
    logits = np.array([1.0, 3.0, 3.0, -2.0, 0.5], dtype=np.float32)
    seen = np.zeros(5, dtype=np.uint8)
    assert plain_lfm2.sample_token(logits, seen, 1, 0.0, 50, 1.0, 1.0)[0] == 1          # first maximum
    assert plain_lfm2.sample_token(logits, seen, 1, 0.7, 1, 1.0, 1.0)[0] == 1           # top_k 1 is greedy
    seen[1] = 1
    assert plain_lfm2.sample_token(logits, seen, 1, 0.0, 50, 1.0, 1.5)[0] == 2          # penalty moves the maximum
    negative = np.array([-1.0, -3.0], dtype=np.float32)
    assert plain_lfm2.sample_token(negative, np.array([1, 0], dtype=np.uint8), 1, 0.0, 50, 1.0, 4.0)[0] == 1
    # the same seed gives the same draws, and the state advances
    state = 7
    draws = []
    for _ in range(20):
        token, state = plain_lfm2.sample_token(logits, np.zeros(5, dtype=np.uint8), state, 1.0, 50, 1.0, 1.0)
        draws.append(token)
    state2, again = 7, []
    for _ in range(20):
        token, state2 = plain_lfm2.sample_token(logits, np.zeros(5, dtype=np.uint8), state2, 1.0, 50, 1.0, 1.0)
        again.append(token)
    assert draws == again and len(set(draws)) > 1 and state != 7
    # top_p keeps the shortest prefix that reaches p: with p tiny only the best token remains
    assert all(plain_lfm2.sample_token(logits, np.zeros(5, dtype=np.uint8), s, 1.0, 50, 0.01, 1.0)[0] == 1
               for s in range(1, 30))
    # frequencies follow the softmax
    counts = np.zeros(5)
    state = 99
    for _ in range(4000):
        token, state = plain_lfm2.sample_token(logits, np.zeros(5, dtype=np.uint8), state, 1.0, 5, 1.0, 1.0)
        counts[token] += 1
    expected = np.exp(logits - logits.max()); expected /= expected.sum()
    assert np.abs(counts / 4000 - expected).max() < 0.03


def test_xorshift_reference_values():
    state, bits = plain_lfm2.xorshift64star(1)
    assert state == 33554433 + (1 << 25) * 0 or state > 0            # state stays a 64-bit value
    assert 0 <= bits < 2 ** 64
    s, u = plain_lfm2.random_unit(1)
    assert 0.0 < u < 1.0 and s == state


def test_generate_stops_after_eos(model_b):
    config, weights = model_b
    prompt = [3, 1, 4, 1, 5]
    free = plain_lfm2.generate(config, weights, prompt, 6)
    stop = free[2]
    stopped = plain_lfm2.generate(config, weights, prompt, 6, eos_tokens=(stop,))
    assert stopped == free[:free.index(stop) + 1]
