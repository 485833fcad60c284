"""Each CUDA kernel alone against a plain float64 reference of the same operation, at sizes
other than the engine's tiny models (odd widths, head sizes in steps of 16, ragged spans)."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_lfm2

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def rounded(x: np.ndarray, dtype) -> np.ndarray:
    """The values a tensor of ``dtype`` holds, as float64."""
    return torch.as_tensor(x).to(dtype).to(torch.float64).numpy()


def close(got: torch.Tensor, want: np.ndarray, dtype, scale=1.0):
    got = got.detach().to(torch.float64).cpu().numpy()
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    err = np.abs(got - want)
    bound = tol * scale + tol * np.abs(want)
    assert (err <= bound).all(), f"max err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(40, 33), (1536, 100)])
def test_embedding(dtype, hidden, vocab):
    from celeg_b200 import kernels
    rng = np.random.default_rng(0)
    table = rounded(rng.normal(size=(vocab, hidden)), dtype)
    tokens = rng.integers(0, vocab, size=19)
    out = torch.zeros((19, hidden), dtype=torch.float32, device="cuda")
    kernels.embedding(dev(table, dtype), dev(tokens, torch.int32), out, 1.0)
    close(out, table[tokens], torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,eps", [(40, 1e-5), (1000, 1e-6), (2048, 1e-5), (4100, 1e-3)])
def test_add_rmsnorm(dtype, width, eps):
    from celeg_b200 import kernels
    rng = np.random.default_rng(1)
    rows = 7
    residual = rng.normal(size=(rows, width)).astype(np.float32).astype(np.float64)
    delta = rounded(rng.normal(size=(rows, width)), dtype)
    weight = (1 + 0.05 * rng.normal(size=width)).astype(np.float32).astype(np.float64)
    res_dev = dev(residual, torch.float32)
    out = torch.zeros((rows, width), dtype=dtype, device="cuda")
    kernels.add_rmsnorm(res_dev, dev(delta, dtype), dev(weight, torch.float32), out, eps)
    summed = (residual + delta).astype(np.float32).astype(np.float64)
    close(res_dev, summed, torch.float32)
    close(out, plain_lfm2.rmsnorm(summed, weight, eps), dtype)
    # gathered, without delta, residual untouched
    pick = np.array([5, 0, 5], dtype=np.int32)
    out2 = torch.zeros((3, width), dtype=dtype, device="cuda")
    before = res_dev.clone()
    kernels.add_rmsnorm(res_dev, None, dev(weight, torch.float32), out2, eps, rows=dev(pick))
    assert torch.equal(before, res_dev)
    close(out2, plain_lfm2.rmsnorm(summed[pick], weight, eps), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,inner", [(5, 136), (33, 1000)])
def test_swiglu(dtype, tokens, inner):
    from celeg_b200 import kernels
    rng = np.random.default_rng(2)
    gate_up = rounded(rng.normal(size=(tokens, 2 * inner)) * 2, dtype)
    out = torch.zeros((tokens, inner), dtype=dtype, device="cuda")
    kernels.swiglu(dev(gate_up, dtype), out, tokens, inner)
    g, u = gate_up[:, :inner], gate_up[:, inner:]
    close(out, g / (1 + np.exp(-g)) * u, dtype)


@pytest.mark.parametrize("m,n,k", [(1, 70, 33), (5, 64, 64), (67, 130, 100), (130, 257, 513)])
def test_gemm_f32(m, n, k):
    from celeg_b200 import kernels
    rng = np.random.default_rng(3)
    x = rng.normal(size=(m, k)).astype(np.float32)
    w = rng.normal(size=(n, k)).astype(np.float32)
    y = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    kernels.gemm_f32(dev(x), dev(w), y, m)
    close(y, x.astype(np.float64) @ w.astype(np.float64).T, torch.float32, scale=math.sqrt(k))
    # a row's result does not depend on the other rows of the batch
    y1 = torch.zeros((1, n), dtype=torch.float32, device="cuda")
    kernels.gemm_f32(dev(x[m - 1:m]), dev(w), y1, 1)
    assert torch.equal(y1[0], y[m - 1])


def conv_reference(proj, kernel, history, spans):
    """Per span: bx history (taps-1 values before the span) ++ span; returns out and new history."""
    hidden = kernel.shape[0]
    taps = kernel.shape[1]
    out = np.zeros((proj.shape[0], hidden))
    new_history = []
    for (begin, end), hist in zip(spans, history):
        b, c, x = (proj[begin:end, i * hidden:(i + 1) * hidden] for i in range(3))
        bx = np.concatenate([hist, b * x], axis=0)
        for j in range(end - begin):
            conv = sum(kernel[:, tap] * bx[j + tap] for tap in range(taps))
            out[begin + j] = c[j] * conv
        new_history.append(bx[bx.shape[0] - (taps - 1):] if taps > 1 else bx[:0])
    return out, new_history


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,taps", [(40, 3), (300, 4), (64, 2), (48, 1), (96, 7)])
def test_short_conv_spans_and_state(dtype, hidden, taps):
    """Spans shorter and longer than the kernel, two steps in a row so the carried state is used,
    slots out of order."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(4)
    keep = taps - 1
    slots = 5
    slot_stride = keep * hidden + 12
    state = torch.zeros((slots, slot_stride), dtype=torch.float32, device="cuda")
    offset = 4
    kernel = rng.normal(size=(hidden, taps)).astype(np.float32).astype(np.float64)
    span_slots = [3, 0, 4, 1]
    history = [np.zeros((keep, hidden)) for _ in span_slots]
    for lengths in ([1, 2, 9, 3], [2, 1, 1, 12], [5, 1, 2, 1]):
        tokens = sum(lengths)
        begins = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
        spans = [(int(begins[i]), int(begins[i + 1])) for i in range(len(lengths))]
        token_span = np.concatenate([np.full(n, i) for i, n in enumerate(lengths)]).astype(np.int32)
        proj = rounded(rng.normal(size=(tokens, 3 * hidden)), dtype)
        out = torch.zeros((tokens, hidden), dtype=dtype, device="cuda")
        kernels.short_conv(dev(proj, dtype), dev(kernel, torch.float32), state[:, offset:], slot_stride, out,
                           dev(token_span), dev(begins), dev(np.array(span_slots, dtype=np.int32)), tokens,
                           len(lengths), hidden, taps)
        want, history = conv_reference(proj, kernel, history, spans)
        close(out, want, dtype, scale=3.0)
        for slot, hist in zip(span_slots, history):
            got = state[slot, offset:offset + keep * hidden].reshape(keep, hidden)
            close(got, hist.astype(np.float32).astype(np.float64), torch.float32)
    assert float(state[2].abs().sum()) == 0.0          # a slot no span named stays untouched


def paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages):
    """Random K/V for several requests scattered over shuffled pages."""
    order = rng.permutation(pages)
    k_cache = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    max_pages = max((n + page_tokens - 1) // page_tokens for n in lengths)
    table = np.full((len(lengths), max_pages), -1, dtype=np.int32)
    ks, vs, used = [], [], 0
    for r, n in enumerate(lengths):
        k = rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype)
        v = rounded(rng.normal(size=(n, kv_heads, head_dim)), dtype)
        for p in range((n + page_tokens - 1) // page_tokens):
            page = int(order[used])
            used += 1
            table[r, p] = page
            lo, hi = p * page_tokens, min(n, (p + 1) * page_tokens)
            k_cache[page, :, :hi - lo] = dev(k[lo:hi], dtype).transpose(0, 1)
            v_cache[page, :, :hi - lo] = dev(v[lo:hi], dtype).transpose(0, 1)
        ks.append(k)
        vs.append(v)
    return k_cache, v_cache, table, ks, vs


def attention_reference(q, k, v, pos, scale, window):
    """q [heads, d] at absolute position pos over keys k,v [n, kv_heads, d]."""
    heads, kv_heads = q.shape[0], k.shape[1]
    out = np.zeros_like(q)
    first = max(0, pos - window + 1) if window else 0
    for h in range(heads):
        kh = h // (heads // kv_heads)
        s = (k[first:pos + 1, kh] @ q[h]) * scale
        w = np.exp(s - s.max())
        w /= w.sum()
        out[h] = w @ v[first:pos + 1, kh]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 16, None), (8, 2, 64, 64, None),
    (6, 3, 80, 16, 37), (2, 1, 128, 32, None), (4, 4, 24, 16, 5),
])
def test_attention_generic(dtype, heads, kv_heads, head_dim, page_tokens, window):
    """Mixed batch: a long portion, a decoded token far into a sequence, a two-token portion, a
    first token; with one key made to stand out so a missed far key shows."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(5)
    lengths = [150, 301, 40, 1]                  # keys each request has AFTER this step
    span_len = [70, 1, 2, 1]                     # tokens it brings to this step
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, 64)
    # request 1: key 3 is far from the query at position 300 and dominates its scores
    tokens = sum(span_len)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    positions, token_span = [], []
    for r, (n, m) in enumerate(zip(lengths, span_len)):
        positions += list(range(n - m, n))
        token_span += [r] * m
    far_row = span_len[0]
    if not window:
        q[far_row] = rounded(ks[1][3, 0][None, :].repeat(heads, 0) * 3.0, dtype)
    scale = head_dim ** -0.5
    out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.attention_generic(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                              dev(np.array(positions, dtype=np.int32)), dev(np.array(token_span, dtype=np.int32)),
                              dev(table), tokens, heads, kv_heads, head_dim, page_tokens, window, scale, flag)
    assert int(flag.item()) == 0
    want = np.stack([attention_reference(q[t], ks[token_span[t]], vs[token_span[t]], positions[t], scale, window)
                     for t in range(tokens)]).reshape(tokens, -1)
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,theta,eps,count", [
    (4, 2, 16, 16, 1e4, 1e-5, (9, 5, 1)), (3, 1, 32, 8, 1e6, 1e-6, (9, 5, 1)), (5, 5, 48, 16, 5e4, 3e-6, (9, 5, 1)),
    (2, 2, 80, 32, 1e6, 1e-5, (9, 5, 1)),
    # head sizes of 64, 128 and 256: the one-pass form per head (few tokens) and the kernel that takes a
    # token and a run of eight heads per warp (64 tokens and more, bfloat16), heads that do not fill the runs
    (4, 2, 64, 16, 1e6, 1e-5, (9, 5, 1)), (5, 1, 64, 16, 1e6, 1e-5, (70, 40, 1)), (9, 3, 128, 16, 1e4, 1e-6, (33, 64, 2)),
    (2, 2, 256, 32, 5e4, 1e-5, (60, 10, 1)), (32, 8, 64, 16, 1e6, 1e-5, (100, 3, 1)),
])
def test_qk_norm_rope_store(dtype, heads, kv_heads, head_dim, page_tokens, theta, eps, count):
    from celeg_b200 import kernels
    rng = np.random.default_rng(6)
    start = [37, 0, 255]
    count = list(count)
    tokens = sum(count)
    pages = 60
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rounded(rng.normal(size=(tokens, width)), dtype)
    q_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    k_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    positions, token_span = [], []
    for r, (s, n) in enumerate(zip(start, count)):
        positions += list(range(s, s + n))
        token_span += [r] * n
    positions = np.array(positions)
    max_pages = max((s + n + page_tokens - 1) // page_tokens for s, n in zip(start, count))
    order = rng.permutation(pages)
    table = np.full((3, max_pages), -1, dtype=np.int32)
    used = 0
    for r, (s, n) in enumerate(zip(start, count)):
        for p in range((s + n + page_tokens - 1) // page_tokens):
            table[r, p] = order[used]
            used += 1
    k_cache = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    half = head_dim // 2
    inv_freq = (theta ** (-2.0 * np.arange(half) / head_dim)).astype(np.float32)
    qkv_dev = dev(qkv, dtype)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.qk_norm_rope_store(qkv_dev, dev(q_w, torch.float32), dev(k_w, torch.float32), dev(inv_freq),
                               dev(positions.astype(np.int32)), dev(np.array(token_span, dtype=np.int32)),
                               dev(table), k_cache, v_cache, tokens, heads, kv_heads, head_dim, head_dim,
                               page_tokens, eps, True, flag)
    assert int(flag.item()) == 0
    q = qkv[:, :heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].reshape(tokens, kv_heads, head_dim)
    q_want = plain_lfm2.rope_split_half(plain_lfm2.rmsnorm(q, q_w, eps), positions, theta)
    k_want = plain_lfm2.rope_split_half(plain_lfm2.rmsnorm(k, k_w, eps), positions, theta)
    close(qkv_dev[:, :heads * head_dim], q_want.reshape(tokens, -1), dtype, scale=3.0)
    for t in range(tokens):
        page = table[token_span[t], positions[t] // page_tokens]
        inside = positions[t] % page_tokens
        close(k_cache[page, :, inside], k_want[t], dtype, scale=3.0)
        close(v_cache[page, :, inside], v[t], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim,rotary,tokens", [(64, 32, 7), (64, 32, 80), (48, 20, 5), (128, 64, 66), (16, 2, 3)])
def test_qk_norm_rope_over_a_part_of_the_head(dtype, head_dim, rotary, tokens):
    """rotary_dim < head_dim: elements [0, rotary) rotate in pairs (i, i + rotary/2) with angles
    position * theta^(-2i/rotary), the others are normalised and pass; k and v land in the cache."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(17)
    heads, kv_heads, eps, theta, page_tokens = 3, 1, 1e-5, 10000.0, 16
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rounded(rng.normal(size=(tokens, width)), dtype)
    q_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    k_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    positions = np.arange(3, 3 + tokens)
    pages = (3 + tokens + page_tokens - 1) // page_tokens
    table = dev(np.arange(pages, dtype=np.int32)[::-1].copy().reshape(1, pages))
    k_cache = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    inv_freq = (theta ** (-2.0 * np.arange(rotary // 2) / rotary)).astype(np.float32)
    qkv_dev = dev(qkv, dtype)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.qk_norm_rope_store(qkv_dev, dev(q_w, torch.float32), dev(k_w, torch.float32), dev(inv_freq),
                               dev(positions.astype(np.int32)), torch.zeros(tokens, dtype=torch.int32, device="cuda"),
                               table, k_cache, v_cache, tokens, heads, kv_heads, head_dim, rotary, page_tokens, eps,
                               True, flag)
    assert int(flag.item()) == 0

    def want_of(x, weight):
        n = plain_lfm2.rmsnorm(x, weight, eps)
        n[..., :rotary] = plain_lfm2.rope_split_half(n[..., :rotary].copy(), positions, theta)
        return n

    q = qkv[:, :heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    v = qkv[:, (heads + kv_heads) * head_dim:].reshape(tokens, kv_heads, head_dim)
    close(qkv_dev[:, :heads * head_dim], want_of(q, q_w).reshape(tokens, -1), dtype, scale=3.0)
    k_want = want_of(k, k_w)
    for t in range(tokens):
        page = pages - 1 - positions[t] // page_tokens
        close(k_cache[page, :, positions[t] % page_tokens], k_want[t], dtype, scale=3.0)
        close(v_cache[page, :, positions[t] % page_tokens], v[t], dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,with_rotation", [(5, False), (70, True), (3, True)])
def test_qk_norm_rope_in_place_for_a_position_part_of_its_own(dtype, tokens, with_rotation):
    """store_kv = 2: the k heads are normalised (and rotated, if tables are given) in place like the q heads;
    v heads and the cache stay as they are. The step before a position encoding that has no tables."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(16)
    heads, kv_heads, head_dim, eps, theta = 6, 2, 64, 1e-5, 20000.0
    width = (heads + 2 * kv_heads) * head_dim
    qkv = rounded(rng.normal(size=(tokens, width)), dtype)
    q_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    k_w = (1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32).astype(np.float64)
    positions = np.arange(11, 11 + tokens)
    inv_freq = (theta ** (-2.0 * np.arange(head_dim // 2) / head_dim)).astype(np.float32)
    cache = torch.full((4, kv_heads, 16, head_dim), 7.0, dtype=dtype, device="cuda")
    table = torch.zeros((1, 8), dtype=torch.int32, device="cuda")
    qkv_dev = dev(qkv, dtype)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.qk_norm_rope_store(qkv_dev, dev(q_w, torch.float32), dev(k_w, torch.float32),
                               dev(inv_freq) if with_rotation else None, dev(positions.astype(np.int32)),
                               torch.zeros(tokens, dtype=torch.int32, device="cuda"), table, cache, cache, tokens,
                               heads, kv_heads, head_dim, head_dim if with_rotation else 0, 16, eps, 2, flag)
    assert int(flag.item()) == 0
    q = qkv[:, :heads * head_dim].reshape(tokens, heads, head_dim)
    k = qkv[:, heads * head_dim:(heads + kv_heads) * head_dim].reshape(tokens, kv_heads, head_dim)
    q_want, k_want = plain_lfm2.rmsnorm(q, q_w, eps), plain_lfm2.rmsnorm(k, k_w, eps)
    if with_rotation:
        q_want = plain_lfm2.rope_split_half(q_want, positions, theta)
        k_want = plain_lfm2.rope_split_half(k_want, positions, theta)
    close(qkv_dev[:, :heads * head_dim], q_want.reshape(tokens, -1), dtype, scale=3.0)
    close(qkv_dev[:, heads * head_dim:(heads + kv_heads) * head_dim], k_want.reshape(tokens, -1), dtype, scale=3.0)
    assert torch.equal(qkv_dev[:, (heads + kv_heads) * head_dim:].cpu(),
                       torch.tensor(qkv[:, (heads + kv_heads) * head_dim:]).to(dtype))
    assert float((cache.float() - 7.0).abs().max()) == 0.0


@pytest.mark.parametrize("pieces", [False, True])
def test_sampling_greedy_and_seeded(pieces):
    from celeg_b200 import kernels
    rng = np.random.default_rng(7)
    vocab, rows = 1000, 6
    logits = rng.normal(size=(rows, vocab)).astype(np.float32) * 3
    logits[0, 17] = logits[0, 400] = logits[0].max() + 1        # a tie: the first maximum wins
    seen = np.zeros((8, vocab), dtype=np.uint8)
    seen[:, rng.integers(0, vocab, size=200)] = 1
    slots = np.array([5, 2, 7, 0, 1, 3], dtype=np.int32)
    temperature = np.array([0.0, 0.8, 1.0, 0.7, 1.3, 0.1], dtype=np.float32)
    top_k = np.array([50, 50, 128, 1, 5, 40], dtype=np.int32)
    top_p = np.array([1.0, 1.0, 0.9, 1.0, 0.5, 1.0], dtype=np.float32)
    penalty = np.array([1.0, 1.05, 1.3, 1.0, 1.0, 2.0], dtype=np.float32)
    rng_state = np.array([1, 7, 99, 12345, 2**40 + 3, 5, 6, 8], dtype=np.uint64)
    seen_dev, rng_dev = dev(seen), dev(rng_state.view(np.int64)).view(torch.int64)
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    states = rng_state.copy()
    seen_host = seen.copy()
    for _ in range(4):                                          # several draws advance the generators
        kernels.sample(dev(logits), rows, dev(slots), seen_dev, rng_dev, dev(temperature), dev(top_k), dev(top_p),
                       dev(penalty), out, scratch=kernels.sample_scratch("cuda") if pieces else None)
        got = out.cpu().numpy()
        for r in range(rows):
            slot = slots[r]
            token, new_state = plain_lfm2.sample_token(logits[r], seen_host[slot], int(states[slot]),
                                                       float(temperature[r]), int(top_k[r]), float(top_p[r]),
                                                       float(penalty[r]))
            assert got[r] == token, f"row {r}: kernel {got[r]}, plain {token}"
            states[slot] = new_state
            seen_host[slot, token] = 1
    assert np.array_equal(seen_dev.cpu().numpy(), seen_host)


@pytest.mark.parametrize("pieces", [False, True])
@pytest.mark.parametrize("vocab", [65536, 20000, 1000, 40])
def test_sampling_with_equal_scores_and_small_vocabularies(vocab, pieces):
    """The selection of the k best has to order equal scores by token id: rows made of a few distinct values
    (thousands of ties at the k-th place), of one value only, with -0.0 beside 0.0, with a k larger than the
    vocabulary, and with the penalty moving seen tokens across the k-th place; every draw against the plain
    sampler, several draws in a row."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(19)
    rows = 6
    logits = np.zeros((rows, vocab), dtype=np.float32)
    logits[0] = rng.integers(0, 3, size=vocab).astype(np.float32)                 # three values only
    logits[1] = 1.25                                                              # one value only
    logits[2] = np.where(rng.random(vocab) < 0.5, -0.0, 0.0).astype(np.float32)   # signed zeros
    logits[2, 7 % vocab] = 0.5
    logits[3] = rng.normal(size=vocab).astype(np.float32)
    logits[4] = np.round(rng.normal(size=vocab) * 2).astype(np.float32) / 2       # a grid of values: many ties
    logits[5] = -np.abs(rng.normal(size=vocab)).astype(np.float32)                # all negative
    seen = (rng.random((rows, vocab)) < 0.3).astype(np.uint8)
    slots = np.arange(rows, dtype=np.int32)
    temperature = np.array([0.9, 1.0, 0.8, 1.1, 1.0, 0.0], dtype=np.float32)
    top_k = np.array([50, 128, 20, 128, 64, 50], dtype=np.int32)
    top_p = np.array([1.0, 0.7, 1.0, 0.95, 1.0, 1.0], dtype=np.float32)
    penalty = np.array([1.0, 1.0, 1.0, 1.3, 1.5, 1.2], dtype=np.float32)
    states = np.array([3, 5, 7, 11, 13, 17], dtype=np.uint64)
    seen_dev, rng_dev = dev(seen), dev(states.view(np.int64)).view(torch.int64)
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    seen_host = seen.copy()
    for draw in range(5):
        kernels.sample(dev(logits), rows, dev(slots), seen_dev, rng_dev, dev(temperature), dev(top_k), dev(top_p),
                       dev(penalty), out, scratch=kernels.sample_scratch("cuda") if pieces else None)
        got = out.cpu().numpy()
        for r in range(rows):
            token, new_state = plain_lfm2.sample_token(logits[r], seen_host[r], int(states[r]), float(temperature[r]),
                                                       int(top_k[r]), float(top_p[r]), float(penalty[r]))
            assert got[r] == token, f"draw {draw} row {r}: kernel {got[r]}, plain {token}"
            states[r] = new_state
            seen_host[r, token] = 1
    assert np.array_equal(seen_dev.cpu().numpy(), seen_host)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window,chunk", [
    (4, 2, 16, 16, None, 64), (3, 1, 32, 8, None, 64), (5, 5, 48, 16, None, 128), (32, 8, 64, 16, None, 64),
    (6, 3, 80, 32, 37, 64), (16, 1, 128, 64, None, 256), (4, 4, 24, 16, 5, 64),
])
def test_attention_decode_split_keys(heads, kv_heads, head_dim, page_tokens, window, chunk):
    """One query token per request at very different context lengths (one key, a page edge,
    hundreds), twice in a row so the counters' reset is used; a far key made to dominate."""
    from celeg_b200 import kernels
    dtype = torch.bfloat16
    rng = np.random.default_rng(8)
    lengths = [1, 16, 17, 300, 511, 64]
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 7
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
    tokens = len(lengths)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    if not window:
        q[3] = rounded(ks[3][2, 0][None, :].repeat(heads, 0) * 3.0, dtype)      # key 2 of 300 stands out
    positions = np.array([n - 1 for n in lengths], dtype=np.int32)
    token_span = np.arange(tokens, dtype=np.int32)
    scale = head_dim ** -0.5
    max_splits = (512 + chunk - 1) // chunk
    partial_o = torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = np.stack([attention_reference(q[t], ks[t], vs[t], int(positions[t]), scale, window)
                     for t in range(tokens)]).reshape(tokens, -1)
    for _ in range(2):
        out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
        kernels.attention_decode(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                                 dev(positions), dev(token_span), dev(table), tokens, heads, kv_heads, head_dim,
                                 page_tokens, window, scale, chunk, max_splits, partial_o, partial_ml, counters,
                                 flag)
        assert int(flag.item()) == 0
        assert int(counters.abs().sum().item()) == 0
        close(out, want, dtype)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window,normed,rotary", [
    (4, 2, 16, 16, None, True, 16), (32, 8, 64, 16, None, True, 64), (5, 5, 48, 8, None, True, 48),
    (6, 3, 80, 16, 37, True, 80), (16, 1, 128, 64, None, False, 128), (3, 1, 48, 16, 5, True, 20),
])
def test_attention_decode_one_warp_an_item(heads, kv_heads, head_dim, page_tokens, window, normed, rotary):
    """The form for very many requests with short contexts, where one warp serves a (token, kv head) item over
    all of its keys and nothing is exchanged between warps: forced here for a handful of requests (contexts of
    one key, a page edge, a tile edge, several tiles; a far key made to dominate), against the formula, and with
    the q/k step inside against the separate kernels (same output, same cache), twice in a row."""
    from celeg_b200 import kernels
    library = kernels.library()
    dtype = torch.bfloat16
    rng = np.random.default_rng(28)
    lengths = [1, 16, 17, 32, 33, 200, 256, 64, 129]
    chunk, max_splits = 256, 1
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 7
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
    tokens = len(lengths)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    if not window:
        q[5] = rounded(ks[5][2, 0][None, :].repeat(heads, 0) * 3.0, dtype)      # key 2 of 200 stands out
    positions = np.array([n - 1 for n in lengths], dtype=np.int32)
    token_span = np.arange(tokens, dtype=np.int32)
    scale, eps = head_dim ** -0.5, 1e-5
    partial_o = torch.empty(tokens * heads * head_dim, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(tokens * heads * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = np.stack([attention_reference(q[t], ks[t], vs[t], int(positions[t]), scale, window)
                     for t in range(tokens)]).reshape(tokens, -1)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = dev(rounded(rng.normal(size=(tokens, width)), dtype), dtype)
    q_w = dev((1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32)) if normed else None
    k_w = dev((1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32)) if normed else None
    inv_freq = dev((1e6 ** (-2.0 * np.arange(rotary // 2) / rotary)).astype(np.float32))
    library.celeg_attention_decode_solo_items(1)
    try:
        out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
        kernels.attention_decode(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                                 dev(positions), dev(token_span), dev(table), tokens, heads, kv_heads, head_dim,
                                 page_tokens, window, scale, chunk, max_splits, partial_o, partial_ml, counters, flag)
        assert int(flag.item()) == 0
        close(out, want, dtype)
        # the q/k step inside, against the separate kernels (which run in the four-warp form)
        library.celeg_attention_decode_solo_items(1 << 40)
        qkv_a, k_a, v_a = qkv.clone(), k_cache.clone(), v_cache.clone()
        kernels.qk_norm_rope_store(qkv_a, q_w, k_w, inv_freq, dev(positions), dev(token_span), dev(table), k_a, v_a,
                                   tokens, heads, kv_heads, head_dim, rotary, page_tokens, eps, True, flag)
        out_a = torch.zeros_like(out)
        kernels.attention_decode(qkv_a, width, out_a, k_a, v_a, dev(positions), dev(token_span), dev(table), tokens,
                                 heads, kv_heads, head_dim, page_tokens, window, scale, chunk, max_splits, partial_o,
                                 partial_ml, counters, flag)
        library.celeg_attention_decode_solo_items(1)
        k_b, v_b = k_cache.clone(), v_cache.clone()
        for _ in range(2):
            out_b = torch.zeros_like(out)
            kernels.attention_decode_fused(qkv.clone(), width, out_b, k_b, v_b, dev(positions), dev(token_span),
                                           dev(table), tokens, heads, kv_heads, head_dim, page_tokens, window, scale,
                                           chunk, max_splits, partial_o, partial_ml, counters, flag, q_w, k_w,
                                           inv_freq, rotary, eps)
            assert int(flag.item()) == 0
            assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
            # one warp sums a row's tiles in another order than four warps and a merge do: equal to rounding
            assert float((out_a.float() - out_b.float()).abs().max()) <= 2e-2 * max(1.0, float(out_a.float().abs().max()))
    finally:
        library.celeg_attention_decode_solo_items(1536)
    # a context beyond what the launch was laid out for: code 3, nothing written for that token
    library.celeg_attention_decode_solo_items(1)
    try:
        out = torch.full((tokens, heads * head_dim), 7.0, dtype=dtype, device="cuda")
        kernels.attention_decode(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                                 dev(positions), dev(token_span), dev(table), tokens, heads, kv_heads, head_dim,
                                 page_tokens, None, scale, 128, 1, partial_o, partial_ml, counters, flag)
        assert int(flag.item()) == 3
        flag.zero_()
        assert bool((out[5].float() == 7.0).all()) and bool((out[6].float() == 7.0).all())
    finally:
        library.celeg_attention_decode_solo_items(1536)


def test_attention_decode_reports_too_few_splits():
    """A launch with fewer key splits than a token's context needs cannot merge that token's output: the
    kernel says so through the error flag (code 3), writes nothing for the token, leaves its counters at
    zero and serves the other tokens as usual."""
    from celeg_b200 import kernels
    dtype = torch.bfloat16
    rng = np.random.default_rng(18)
    heads, kv_heads, head_dim, page_tokens, chunk = 4, 2, 64, 16, 64
    lengths = [40, 300]
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, 40)
    tokens = len(lengths)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    positions = np.array([n - 1 for n in lengths], dtype=np.int32)
    max_splits = 2                                   # 300 keys in chunks of 64 need five
    partial_o = torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((tokens, heads * head_dim), 7.0, dtype=dtype, device="cuda")
    scale = head_dim ** -0.5
    kernels.attention_decode(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                             dev(positions), dev(np.arange(tokens, dtype=np.int32)), dev(table), tokens, heads,
                             kv_heads, head_dim, page_tokens, None, scale, chunk, max_splits, partial_o, partial_ml,
                             counters, flag)
    assert int(flag.item()) == 3
    assert int(counters.abs().sum().item()) == 0
    assert bool((out[1].float() == 7.0).all())
    close(out[:1], attention_reference(q[0], ks[0], vs[0], 39, scale, None).reshape(1, -1), dtype)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window,chunk,normed,rotary", [
    (4, 2, 16, 16, None, 64, True, 16), (8, 2, 64, 16, None, 128, True, 64), (6, 3, 80, 16, 37, 64, True, 80),
    (2, 1, 128, 32, None, 512, False, 128), (5, 5, 48, 8, None, 64, True, 48), (32, 8, 64, 16, None, 256, True, 64),
    # a rotation over the first elements of a head only; the rest is normalised and passes
    (8, 2, 64, 16, None, 128, True, 32), (3, 1, 48, 16, None, 64, True, 20),
])
def test_attention_decode_with_the_qk_step_inside(heads, kv_heads, head_dim, page_tokens, window, chunk, normed, rotary):
    """The decode kernel fed with the raw q|k|v projection (it normalises and rotates q and the token's own
    key, writes key and value into the cache, attends) against the separate kernels: same output, same cache."""
    from celeg_b200 import kernels
    dtype = torch.bfloat16
    rng = np.random.default_rng(19)
    lengths = [1, 16, 17, 300, 511, 64]                    # keys of each request including the step's token
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 7
    k_cache, v_cache, table, _, _ = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
    tokens = len(lengths)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = dev(rounded(rng.normal(size=(tokens, width)), dtype), dtype)
    q_w = dev((1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32)) if normed else None
    k_w = dev((1 + 0.05 * rng.normal(size=head_dim)).astype(np.float32)) if normed else None
    inv_freq = dev((1e6 ** (-2.0 * np.arange(rotary // 2) / rotary)).astype(np.float32))
    positions = dev(np.array([n - 1 for n in lengths], dtype=np.int32))
    token_span = dev(np.arange(tokens, dtype=np.int32))
    table_dev = dev(table)
    scale, eps = head_dim ** -0.5, 1e-5
    max_splits = (512 + chunk - 1) // chunk
    partial_o = torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    # separate kernels on copies
    qkv_a, k_a, v_a = qkv.clone(), k_cache.clone(), v_cache.clone()
    kernels.qk_norm_rope_store(qkv_a, q_w, k_w, inv_freq, positions, token_span, table_dev, k_a, v_a, tokens, heads,
                               kv_heads, head_dim, rotary, page_tokens, eps, True, flag)
    out_a = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
    kernels.attention_decode(qkv_a, width, out_a, k_a, v_a, positions, token_span, table_dev, tokens, heads, kv_heads,
                             head_dim, page_tokens, window, scale, chunk, max_splits, partial_o, partial_ml, counters, flag)
    # one kernel, twice in a row (the second time the cache already holds the token's key: same result)
    k_b, v_b = k_cache.clone(), v_cache.clone()
    for _ in range(2):
        out_b = torch.zeros_like(out_a)
        kernels.attention_decode_fused(qkv.clone(), width, out_b, k_b, v_b, positions, token_span, table_dev, tokens,
                                       heads, kv_heads, head_dim, page_tokens, window, scale, chunk, max_splits,
                                       partial_o, partial_ml, counters, flag, q_w, k_w, inv_freq, rotary, eps)
        assert int(flag.item()) == 0 and int(counters.abs().sum().item()) == 0
        assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
        assert torch.equal(out_a, out_b)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_tokens,window", [
    (4, 2, 16, 16, None), (3, 1, 32, 8, None), (5, 5, 48, 16, None), (8, 2, 64, 64, None),
    (6, 3, 80, 16, 37), (2, 1, 128, 32, None), (4, 4, 24, 16, 5), (2, 1, 256, 16, None), (4, 1, 112, 16, 100),
])
def test_attention_prefill_tensor_cores(heads, kv_heads, head_dim, page_tokens, window):
    """The same mixed batch as the general kernel's test plus a portion that spans three query
    tiles and starts in the middle of a page."""
    from celeg_b200 import kernels
    dtype = torch.bfloat16
    rng = np.random.default_rng(9)
    lengths = [150, 301, 40, 1, 333]             # keys each request has AFTER this step
    span_len = [70, 1, 2, 1, 150]                # tokens it brings to this step
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 5
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
    tokens = sum(span_len)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    positions, token_span, begins = [], [], [0]
    for r, (n, m) in enumerate(zip(lengths, span_len)):
        positions += list(range(n - m, n))
        token_span += [r] * m
        begins.append(begins[-1] + m)
    if not window:
        q[span_len[0]] = rounded(ks[1][3, 0][None, :].repeat(heads, 0) * 3.0, dtype)   # far key 3 dominates
    scale = head_dim ** -0.5
    out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    kernels.attention_prefill(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                              dev(np.array(positions, dtype=np.int32)), dev(np.array(begins, dtype=np.int32)),
                              dev(table), tokens, len(lengths), heads, kv_heads, head_dim, page_tokens, window,
                              scale, flag)
    assert int(flag.item()) == 0
    want = np.stack([attention_reference(q[t], ks[token_span[t]], vs[token_span[t]], positions[t], scale, window)
                     for t in range(tokens)]).reshape(tokens, -1)
    close(out, want, dtype, scale=1.5)


@pytest.mark.parametrize("heads,kv_heads,page_tokens,window,lengths,starts", [
    (1, 1, 16, None, (128,), (0,)), (2, 1, 16, None, (200,), (0,)), (8, 2, 16, None, (130, 5, 77), (37, 0, 255)),
    (6, 2, 8, 150, (300,), (100,)), (4, 4, 32, None, (100, 260), (0, 40)), (3, 1, 64, 70, (1, 129, 2), (500, 3, 64)),
])
def test_attention_prefill_tcgen05(heads, kv_heads, page_tokens, window, lengths, starts):
    """Prompt-portion attention of head size 64 on tcgen05 (S and O' in tensor memory, Q/K/V by TMA through the
    block table) against the formula, with tiles that end inside a block of keys, a window, several spans."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(18)
    dtype, head_dim = torch.bfloat16, 64
    assert kernels.attention_prefill_tcgen05_supported(heads, kv_heads, head_dim, page_tokens, dtype)
    spans, tokens = len(lengths), sum(lengths)
    pages_per = (max(s + n for s, n in zip(starts, lengths)) + page_tokens - 1) // page_tokens
    pages = spans * pages_per + 3
    order = rng.permutation(pages)
    table = order[:spans * pages_per].reshape(spans, pages_per).astype(np.int32)
    k_cache = np.zeros((pages, kv_heads, page_tokens, head_dim))
    v_cache = np.zeros_like(k_cache)
    ks, vs = [], []
    for r, (start, n) in enumerate(zip(starts, lengths)):
        k = rounded(rng.normal(size=(start + n, kv_heads, head_dim)), dtype)
        v = rounded(rng.normal(size=(start + n, kv_heads, head_dim)), dtype)
        ks.append(k)
        vs.append(v)
        for position in range(start + n):
            k_cache[table[r, position // page_tokens], :, position % page_tokens] = k[position]
            v_cache[table[r, position // page_tokens], :, position % page_tokens] = v[position]
    # what lies in unused pages must never matter, whatever it is
    k_cache[order[spans * pages_per:]] = 1e4
    v_cache[order[spans * pages_per:]] = -1e4
    positions = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lengths)])
    token_span = np.concatenate([np.full(n, r) for r, n in enumerate(lengths)])
    begins = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    width = (heads + 2 * kv_heads) * head_dim
    qkv = np.zeros((tokens + 3, width))
    qkv[:tokens, :heads * head_dim] = q.reshape(tokens, -1)
    out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = head_dim ** -0.5
    tiles = sum((n + 127) // 128 for n in lengths)
    kernels.attention_prefill_tcgen05(dev(qkv, dtype), width, out, dev(k_cache, dtype), dev(v_cache, dtype),
                                      dev(positions.astype(np.int32)), dev(begins), dev(table), tokens, spans, tiles,
                                      heads, kv_heads, head_dim, page_tokens, window, scale, flag)
    assert int(flag.item()) == 0
    want = np.stack([attention_reference(q[t], ks[token_span[t]], vs[token_span[t]], positions[t], scale, window)
                     for t in range(tokens)]).reshape(tokens, -1)
    close(out, want, dtype, scale=1.5)


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (8, 2048, 2048), (3, 70, 136), (8, 100, 8200), (16, 48, 520),
                                   (11, 1000, 96), (5, 33, 24), (2, 16, 8)])
def test_gemv_bf16_modes(m, n, k):
    from celeg_b200 import kernels
    rng = np.random.default_rng(10)
    x = rounded(rng.normal(size=(m, k)), torch.bfloat16)
    w = rounded(rng.normal(size=(n, k)) * 0.1, torch.bfloat16)
    want = x @ w.T
    x_dev, w_dev = dev(x, torch.bfloat16), dev(w, torch.bfloat16)
    assert kernels.gemv_supported(m, x_dev, w_dev)
    y = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemv_bf16(x_dev, w_dev, y, m, kernels.GEMV_STORE)
    close(y, want, torch.bfloat16)
    y32 = torch.full((m, n), 7.0, dtype=torch.float32, device="cuda")
    kernels.gemv_bf16(x_dev, w_dev, y32, m, kernels.GEMV_STORE_F32)
    close(y32, want, torch.float32, scale=50 * math.sqrt(k))       # products are exact, sums are float32
    before = rng.normal(size=(m, n)).astype(np.float32)
    res = dev(before)
    kernels.gemv_bf16(x_dev, w_dev, res, m, kernels.GEMV_ADD_RESIDUAL)
    # the product is rounded to bfloat16 as a stored product would be, then added in float32
    err = np.abs(res.cpu().numpy() - (before.astype(np.float64) + want))
    assert (err <= 2.0 ** -8 * np.abs(want) + 1e-5).all(), err.max()
    if n % 2 == 0:
        inner = n // 2
        act = torch.zeros((m, inner), dtype=torch.bfloat16, device="cuda")
        kernels.gemv_bf16(x_dev, w_dev, act, m, kernels.GEMV_SWIGLU)
        gate = rounded(want[:, :inner], torch.bfloat16)
        up = rounded(want[:, inner:], torch.bfloat16)
        close(act, gate / (1 + np.exp(-gate)) * up, torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("m,n,k,ahead_bytes", [(8, 2048, 256, 1 << 20), (3, 70, 136, 4096 + 48), (16, 4800, 64, 200),
                                               (1, 16, 8, 16)])
def test_gemv_bf16_with_a_prefetch_hint(m, n, k, ahead_bytes):
    """A product that asks the next product's weights into the L2 gives the same bits as one that does not,
    whatever the size of the hint (more blocks than askers, fewer, bytes that are no multiple of a slice);
    the hint holds for one call."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(12)
    x_dev = dev(rounded(rng.normal(size=(m, k)), torch.bfloat16), torch.bfloat16)
    w_dev = dev(rounded(rng.normal(size=(n, k)) * 0.1, torch.bfloat16), torch.bfloat16)
    later = torch.zeros(ahead_bytes + 64, dtype=torch.uint8, device="cuda")
    plain = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    hinted = torch.zeros_like(plain)
    kernels.gemv_bf16(x_dev, w_dev, plain, m, kernels.GEMV_STORE)
    before = kernels.LAUNCHES
    kernels.gemv_bf16(x_dev, w_dev, hinted, m, kernels.GEMV_STORE, ahead=(later.data_ptr(), ahead_bytes))
    assert kernels.LAUNCHES == before + 1                  # the hint is no launch
    torch.cuda.synchronize()
    assert torch.equal(plain, hinted)
    again = torch.zeros_like(plain)
    kernels.gemv_bf16(x_dev, w_dev, again, m, kernels.GEMV_STORE)      # no hint left over
    torch.cuda.synchronize()
    assert torch.equal(plain, again)
    with pytest.raises(kernels.KernelLibraryError):
        kernels.gemv_bf16(x_dev, w_dev, again, m, kernels.GEMV_STORE, ahead=(later.data_ptr() + 4, 64))


def test_runtime_learns_the_order_of_streamed_weights():
    """The successor of a weight is what was streamed after it the last time; the hint is capped."""
    from celeg_b200.parts.runtime import Runtime
    rt = Runtime(torch.device("cuda:0"), torch.bfloat16, 16, max_requests=4, max_context=64)
    rt.prefetch_bytes = 1024
    a = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    assert rt._ahead(a) is None and rt._ahead(b) is None and rt._ahead(c) is None
    assert rt._ahead(a) == (b.data_ptr(), 1024)            # second round: a was followed by b, ...
    assert rt._ahead(b) == (c.data_ptr(), 1024)
    assert rt._ahead(c) == (a.data_ptr(), 1024)            # ... and the last one by the first of the next step
    rt.prefetch_bytes = 0
    assert rt._ahead(a) is None


@pytest.mark.parametrize("m,width,inner", [(1, 64, 192), (8, 2048, 1024), (5, 80, 136), (16, 96, 256), (3, 40, 72)])
def test_split_norm_over_two_products(m, width, inner):
    """residual += x w_down^T; y = rmsnorm(residual) w_next^T, with the norm split over the two products
    (no kernel of its own), against the formulas; also from the embedding as the first half."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(14)
    eps = 1e-5
    x = rounded(rng.normal(size=(m, inner)), torch.bfloat16)
    w_down = rounded(rng.normal(size=(width, inner)) * 0.1, torch.bfloat16)
    w_next = rounded(rng.normal(size=(48, width)) * 0.1, torch.bfloat16)
    norm_w = (1.0 + 0.1 * rng.normal(size=width)).astype(np.float32)
    before = rng.normal(size=(m, width)).astype(np.float32)
    residual = dev(before)
    pieces = (width + 15) // 16
    split = kernels.SplitNorm(torch.zeros((m, width), dtype=torch.bfloat16, device="cuda"),
                              torch.full((16, pieces + 3), 9.0, dtype=torch.float32, device="cuda"), pieces, eps, width)
    kernels.gemv_bf16(dev(x, torch.bfloat16), dev(w_down, torch.bfloat16), residual, m, kernels.GEMV_ADD_RESIDUAL,
                      prepare=split, next_weight=dev(norm_w))
    delta = rounded(x @ w_down.T, torch.bfloat16)
    want_residual = before.astype(np.float64) + delta
    got_residual = residual.cpu().numpy().astype(np.float64)
    assert np.abs(got_residual - want_residual).max() <= 2.0 ** -7 * np.abs(delta).max() + 1e-5
    # judged against the residual the kernel really holds: the halves of the norm
    sums = split.sumsq[:m, :pieces].sum(dim=1).cpu().numpy()
    assert np.allclose(sums, (got_residual ** 2).sum(axis=1), rtol=1e-5)
    close(split.xw, got_residual * norm_w, torch.bfloat16)
    y = torch.zeros((m, 48), dtype=torch.float32, device="cuda")
    kernels.gemv_bf16(split, dev(w_next, torch.bfloat16), y, m, kernels.GEMV_STORE_F32)
    inv = 1.0 / np.sqrt((got_residual ** 2).mean(axis=1, keepdims=True) + eps)
    want_y = (rounded(got_residual * norm_w, torch.bfloat16) * inv) @ w_next.T
    close(y, want_y, torch.float32, scale=50 * math.sqrt(width))
    # the whole norm, loosely: rounding before and after the scale differ
    full = (rounded(got_residual * inv * norm_w, torch.bfloat16)) @ w_next.T
    assert np.abs(y.cpu().numpy() - full).max() <= 0.02 * np.abs(full).max() + 1e-3

    # the embedding as the first half
    vocab = 50
    table = rounded(rng.normal(size=(vocab, width)), torch.bfloat16)
    tokens = rng.integers(0, vocab, size=m).astype(np.int32)
    out = torch.zeros((m, width), dtype=torch.float32, device="cuda")
    first = kernels.SplitNorm(torch.zeros((m, width), dtype=torch.bfloat16, device="cuda"),
                              torch.zeros((16, pieces), dtype=torch.float32, device="cuda"), 1, eps, width)
    kernels.embedding(dev(table, torch.bfloat16), dev(tokens, torch.int32), out, 2.0, prepare=first, next_weight=dev(norm_w))
    rows = table[tokens] * 2.0
    close(out, rows, torch.float32)
    close(first.xw, rows * norm_w, torch.bfloat16)
    assert np.allclose(first.sumsq[:m, 0].cpu().numpy(), (rows ** 2).sum(axis=1), rtol=1e-5)


@pytest.mark.parametrize("m,hidden,k,taps", [(1, 64, 64, 3), (8, 2048, 2048, 3), (5, 40, 136, 4), (16, 48, 520, 2),
                                             (3, 33, 64, 1), (7, 96, 96, 7), (8, 2048, 512, 3)])
def test_gemv_conv_epilogue_matches_the_separate_kernels(m, hidden, k, taps):
    """Input projection + gate + taps over the carried state + state shift in one kernel, against the
    projection followed by the span kernel, three decode steps in a row: same bits, same state."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(13)
    w = dev(rounded(rng.normal(size=(3 * hidden, k)) * 0.1, torch.bfloat16), torch.bfloat16)
    conv_w = dev(rng.normal(size=(hidden, taps)).astype(np.float32))
    keep = taps - 1
    slot_stride = keep * hidden + 8
    slots = [5, 0, 9, 3, 1, 2, 4, 6, 7, 8, 10, 11, 12, 13, 14, 15][:m]
    state_a = torch.zeros((16, slot_stride), dtype=torch.float32, device="cuda")
    state_a[:] = dev(rng.normal(size=(16, slot_stride)).astype(np.float32))
    state_b = state_a.clone()
    span_slot = dev(np.array(slots, dtype=np.int32))
    token_span = dev(np.arange(m, dtype=np.int32))
    span_begin = dev(np.arange(m + 1, dtype=np.int32))
    kernels.library().celeg_gemv_set_warps(8)        # the same summation order on both sides
    for _ in range(3):
        x = dev(rounded(rng.normal(size=(m, k)), torch.bfloat16), torch.bfloat16)
        fused = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
        kernels.gemv_bf16(x, w, fused, m, kernels.GEMV_CONV, conv_w=conv_w, taps=taps, state=state_a[:, 4:],
                          slot_stride=slot_stride, span_slot=span_slot)
        proj = torch.zeros((m, 3 * hidden), dtype=torch.bfloat16, device="cuda")
        kernels.gemv_bf16(x, w, proj, m)
        separate = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
        kernels.short_conv(proj, conv_w, state_b[:, 4:], slot_stride, separate, token_span, span_begin, span_slot, m,
                           m, hidden, taps)
        assert torch.equal(fused, separate)
        assert torch.equal(state_a, state_b)
    kernels.library().celeg_gemv_set_warps(0)
    # with the block size the host would pick, the result agrees to rounding
    x = dev(rounded(rng.normal(size=(m, k)), torch.bfloat16), torch.bfloat16)
    auto = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
    kernels.gemv_bf16(x, w, auto, m, kernels.GEMV_CONV, conv_w=conv_w, taps=taps, state=state_a[:, 4:],
                      slot_stride=slot_stride, span_slot=span_slot)
    kernels.library().celeg_gemv_set_warps(8)
    forced = torch.zeros((m, hidden), dtype=torch.bfloat16, device="cuda")
    kernels.gemv_bf16(x, w, forced, m, kernels.GEMV_CONV, conv_w=conv_w, taps=taps, state=state_b[:, 4:],
                      slot_stride=slot_stride, span_slot=span_slot)
    kernels.library().celeg_gemv_set_warps(0)
    close(auto, forced.double().cpu().numpy(), torch.bfloat16, scale=2.0)


@pytest.mark.parametrize("warps", [8, 16, 32])
def test_gemv_bf16_with_every_block_size(warps):
    """The host picks 8, 16 or 32 warps per block from the shape; here each is forced in turn."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(15)
    lib = kernels.library()
    try:
        lib.celeg_gemv_set_warps(warps)
        for m, n, k in ((8, 100, 8200), (13, 48, 520), (1, 64, 2048)):
            x = rounded(rng.normal(size=(m, k)), torch.bfloat16)
            w = rounded(rng.normal(size=(n, k)) * 0.1, torch.bfloat16)
            y = torch.zeros((m, n), dtype=torch.float32, device="cuda")
            kernels.gemv_bf16(dev(x, torch.bfloat16), dev(w, torch.bfloat16), y, m, kernels.GEMV_STORE_F32)
            close(y, x @ w.T, torch.float32, scale=50 * math.sqrt(k))
    finally:
        lib.celeg_gemv_set_warps(0)


@pytest.mark.parametrize("vocab", [1000, 65536, 3000])
def test_greedy_sampling_fast_path(vocab):
    """Arg-max in two kernels equals the general kernel's greedy rows, ties and penalty included."""
    from celeg_b200 import kernels
    rng = np.random.default_rng(16)
    rows = 5
    logits = rng.normal(size=(rows, vocab)).astype(np.float32) * 3
    logits[0, 17] = logits[0, vocab - 3] = logits[0].max() + 1          # a tie across two pieces
    logits[1, vocab - 1] = logits[1].max() + 2                          # the very last token
    seen = np.zeros((8, vocab), dtype=np.uint8)
    seen[:, rng.integers(0, vocab, size=vocab // 5)] = 1
    best2 = int(np.argmax(logits[2]))
    seen[3, best2] = 1                                                  # row 2 uses slot 3: its best is penalised
    slots = np.array([5, 2, 3, 0, 1], dtype=np.int32)
    penalty = np.array([1.0, 1.05, 50.0, 1.0, 1.3], dtype=np.float32)
    seen_dev = dev(seen)
    out = torch.zeros(rows, dtype=torch.int32, device="cuda")
    kernels.sample_greedy(dev(logits), rows, dev(slots), seen_dev, dev(penalty), out,
                          torch.zeros(rows * 64, device="cuda"), torch.zeros(rows * 64, dtype=torch.int32, device="cuda"))
    got = out.cpu().numpy()
    for r in range(rows):
        want, _ = plain_lfm2.sample_token(logits[r], seen[slots[r]], 1, 0.0, 1, 1.0, float(penalty[r]))
        assert got[r] == want, (r, got[r], want)
        seen[slots[r], want] = 1
    assert got[0] == 17 and got[1] == vocab - 1 and got[2] != best2
    assert np.array_equal(seen_dev.cpu().numpy(), seen)


@pytest.mark.parametrize("variant", [1, 2, 3, -1])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 264, 520), (17, 1000, 96), (640, 512, 2048), (2048, 384, 1024)])
def test_gemm_tcgen05_store_and_swiglu(m, n, k, variant):
    """The TMA + tcgen05 product against float64, every kernel variant (128x128 tiles with 3 stages,
    128x256 with 4, persistent with two accumulators, and the library's own choice), sizes that are no
    multiple of the tiles, K with a tail, and the fused SwiGLU epilogue. The error flag stays clear."""
    import math
    from celeg_b200 import kernels
    torch.manual_seed(1)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * n, k, device="cuda") * 0.1).to(torch.bfloat16)
    ref = x.double() @ w.double().t()
    y32 = torch.full((m, n), 7.0, dtype=torch.float32, device="cuda")
    kernels.gemm_tcgen05(x, w[:n], y32, m, kernels.TC_STORE_F32, flag, variant)
    err = (y32.double() - ref[:, :n]).abs().max().item()
    assert err < 1e-3 * math.sqrt(k), ("f32", err)
    y = torch.zeros((m, n + 8), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05(x, w[:n], y, m, kernels.TC_STORE, flag, variant)
    want = ref[:, :n]
    bad = ((y[:, :n].double() - want).abs() > 1.2e-2 * (1 + want.abs())).sum().item()
    assert bad == 0, ("bf16", bad)
    assert float(y[:, n:].abs().sum()) == 0.0
    act = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05(x, w, act, m, kernels.TC_SWIGLU, flag, variant)
    g = ref[:, :n].to(torch.bfloat16).double()
    u = ref[:, n:].to(torch.bfloat16).double()
    want = g / (1 + torch.exp(-g)) * u
    bad = ((act.double() - want).abs() > 2.5e-2 * (1 + want.abs())).sum().item()
    assert bad <= m * n // 2000, ("swiglu", bad)          # a gate on a rounding edge may flip
    assert int(flag.item()) == 0


@pytest.mark.parametrize("chunk", [1472, 2880, 4096])
def test_attention_decode_long_contexts_in_large_chunks(chunk):
    """Contexts of thousands of keys in the chunks that long contexts get (up to 4,096 keys, any multiple of 64):
    a context that ends on a chunk's last key, one key into the next chunk, one key in all; more than eight
    splits for one request and one split for another in the same launch; a far key made to dominate."""
    from celeg_b200 import kernels
    dtype = torch.bfloat16
    rng = np.random.default_rng(41)
    heads, kv_heads, head_dim, page_tokens = 8, 2, 64, 16
    lengths = [9 * chunk - 5, chunk, chunk + 1, 1, 3000]
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 3
    k_cache, v_cache, table, ks, vs = paged_setup(rng, dtype, lengths, kv_heads, head_dim, page_tokens, pages)
    tokens = len(lengths)
    q = rounded(rng.normal(size=(tokens, heads, head_dim)), dtype)
    q[0] = rounded(ks[0][chunk + 2, 0][None, :].repeat(heads, 0) * 3.0, dtype)      # a key of the second chunk stands out
    positions = np.array([n - 1 for n in lengths], dtype=np.int32)
    token_span = np.arange(tokens, dtype=np.int32)
    scale = head_dim ** -0.5
    max_splits = (max(lengths) + chunk - 1) // chunk
    partial_o = torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda")
    partial_ml = torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = np.stack([attention_reference(q[t], ks[t], vs[t], int(positions[t]), scale, None)
                     for t in range(tokens)]).reshape(tokens, -1)
    for _ in range(2):
        out = torch.zeros((tokens, heads * head_dim), dtype=dtype, device="cuda")
        kernels.attention_decode(dev(q.reshape(tokens, -1), dtype), heads * head_dim, out, k_cache, v_cache,
                                 dev(positions), dev(token_span), dev(table), tokens, heads, kv_heads, head_dim,
                                 page_tokens, None, scale, chunk, max_splits, partial_o, partial_ml, counters, flag)
        assert int(flag.item()) == 0
        assert int(counters.abs().sum().item()) == 0
        close(out, want, dtype)
