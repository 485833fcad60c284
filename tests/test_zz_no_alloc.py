"""The entry point of the kernel library that allocates nothing, celeg_attention_decode_static.

It serves callers that cannot call cudaMalloc when they need decode attention (all device memory
already given to their own pool, or no tolerance for the synchronisation an allocation causes):
its scratch is a fixed array inside the library. Here it is called through its exported C symbol,
twice in a row with different inputs, and compared

* with the ordinary entry point, which takes scratch from the caller: both run the same kernel on the
  same inputs, so the outputs must be equal bit for bit;
* with a float64 restatement of attention written here, with one far key made to dominate one query,
  so that a fault of the layout inside the array that both entry points shared would still show.

The second call is smaller than the first and finds the array as the first one left it, so it also
shows that nothing stale (partial results, counters) is used. Cases: eight splits and fewer, more
than eight splits (the merge then runs in several batches), a window. Sizes up to the array's
capacity are taken, one step beyond it is refused with a message.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from celeg_b200 import kernels
    lib = kernels.library()
    fn = lib.celeg_attention_decode_static
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    lib.celeg_attention_decode_static_capacity.restype = c_longlong
    return lib, fn


def _bf16(values: np.ndarray) -> torch.Tensor:
    return torch.tensor(values).to(torch.bfloat16)


def _case(seed, lengths, heads, kv_heads, head_dim, page_tokens, dominant=None):
    """Random queries, keys and values (bfloat16 values, kept as float64 too) over shuffled pages.
    ``dominant`` = (request, key index): that request's query is made three times that key, so the key
    takes nearly all of the softmax."""
    rng = np.random.default_rng(seed)
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 3
    order = rng.permutation(pages)
    k_cache = torch.zeros((pages, kv_heads, page_tokens, head_dim), dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    max_pages = max((n + page_tokens - 1) // page_tokens for n in lengths)
    table = np.full((len(lengths), max_pages), -1, dtype=np.int32)
    keys, values, used = [], [], 0
    for r, n in enumerate(lengths):
        k = _bf16(rng.normal(size=(n, kv_heads, head_dim)))
        v = _bf16(rng.normal(size=(n, kv_heads, head_dim)))
        for p in range((n + page_tokens - 1) // page_tokens):
            page = int(order[used])
            used += 1
            table[r, p] = page
            lo, hi = p * page_tokens, min(n, (p + 1) * page_tokens)
            k_cache[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_cache[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
        keys.append(k.double().numpy())
        values.append(v.double().numpy())
    tokens = len(lengths)
    q = _bf16(rng.normal(size=(tokens, heads, head_dim)))
    if dominant is not None:
        request, key = dominant
        q[request] = _bf16(np.repeat(keys[request][key, 0][None, :], heads, axis=0) * 3.0)
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    token_span = torch.arange(tokens, dtype=torch.int32).cuda()
    return (q.reshape(tokens, heads * head_dim).cuda(), k_cache.cuda(), v_cache.cuda(), positions, token_span,
            torch.tensor(table).cuda(), q.double().numpy(), keys, values)


def _attention_float64(q, k, v, pos, scale, window):
    """softmax(q k^T * scale) v for one token in float64: q [heads, d] at position ``pos`` over keys and
    values [n, kv_heads, d]; query head h reads kv head h // (heads / kv_heads); with a window only the
    last ``window`` positions (the query's own included) are read."""
    heads, kv_heads = q.shape[0], k.shape[1]
    out = np.zeros_like(q)
    first = max(0, pos - window + 1) if window else 0
    for h in range(heads):
        kh = h // (heads // kv_heads)
        scores = (k[first:pos + 1, kh] @ q[h]) * scale
        weights = np.exp(scores - scores.max())
        weights /= weights.sum()
        out[h] = weights @ v[first:pos + 1, kh]
    return out


# (seed, lengths, heads, kv_heads, head_dim, page_tokens, chunk, window, dominant): run in this order, the
# second of each pair is the smaller call
CALLS = {
    "up to eight splits": [
        (40, [300, 17, 1, 511], 8, 2, 64, 16, 64, 0, (3, 5)),
        (41, [64, 129, 2], 8, 2, 64, 16, 64, 0, (1, 3)),
    ],
    "more than eight splits, then a window": [
        (42, [1500, 1031, 77], 6, 3, 64, 16, 64, 0, (0, 9)),          # 24 splits: three batches of the merge
        (43, [700, 90], 6, 3, 64, 16, 64, 200, None),
    ],
    "other head size and page size": [
        (44, [260, 33, 513], 4, 4, 128, 32, 128, 0, (2, 1)),
        (45, [100, 5], 4, 4, 128, 32, 128, 37, None),
    ],
}


@pytest.mark.parametrize("name", list(CALLS))
def test_static_scratch_entry_point_twice_in_a_row(name):
    from celeg_b200 import kernels
    lib, fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lengths, heads, kv_heads, head_dim, page_tokens, chunk, window, dominant in CALLS[name]:
        (q, k_cache, v_cache, positions, token_span, table, q64, keys, values) = _case(
            seed, lengths, heads, kv_heads, head_dim, page_tokens, dominant)
        tokens = len(lengths)
        longest = min(max(lengths), window) if window else max(lengths)
        max_splits = (longest + chunk - 1) // chunk
        scale = head_dim ** -0.5
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        ordinary = torch.zeros((tokens, heads * head_dim), dtype=torch.bfloat16, device="cuda")
        kernels.attention_decode(
            q, heads * head_dim, ordinary, k_cache, v_cache, positions, token_span, table, tokens, heads, kv_heads,
            head_dim, page_tokens, window or None, scale, chunk, max_splits,
            torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda"),
            torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda"),
            torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda"), flag)
        got = torch.zeros_like(ordinary)
        code = fn(q.data_ptr(), heads * head_dim, got.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                  k_cache.stride(0), positions.data_ptr(), token_span.data_ptr(), table.data_ptr(),
                  table.stride(0), tokens, heads, kv_heads, head_dim, page_tokens, window, scale, chunk, max_splits,
                  flag.data_ptr(), stream)
        assert code == 0, lib.celeg_last_error().decode()
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        # the same kernel on the same inputs, only the scratch lives elsewhere: equal bit for bit
        assert torch.equal(got.view(torch.int16), ordinary.view(torch.int16))
        # and right: against float64, at the tolerance of the kernel tests for bfloat16
        want = np.stack([_attention_float64(q64[t], keys[t], values[t], lengths[t] - 1, scale, window)
                         for t in range(tokens)]).reshape(tokens, -1)
        assert float(np.abs(want).max()) > 0.1
        err = np.abs(got.float().cpu().numpy().astype(np.float64) - want)
        bound = 1.2e-2 + 1.2e-2 * np.abs(want)
        assert bool((err <= bound).all()), float(err.max())


def _scratch_bytes(tokens, heads, kv_heads, head_dim, max_splits):
    """What a call needs of the array: counters, maxima and sums, partial outputs, the first two rounded up
    to 256 bytes (the layout the entry point's header gives)."""
    def up(n):
        return (n + 255) // 256 * 256
    return (up(tokens * kv_heads * 4) + up(tokens * heads * max_splits * 2 * 4)
            + tokens * heads * max_splits * head_dim * 4)


def test_static_scratch_entry_point_takes_what_fits_and_refuses_the_next_size():
    lib, fn = _symbol()
    capacity = lib.celeg_attention_decode_static_capacity()
    assert capacity == 8 * 1024 * 1024
    heads, kv_heads, head_dim, page_tokens, chunk = 16, 1, 64, 16, 64
    # one token, one kv head: 256 B of counters + 128 B * splits rounded up + 4,096 B * splits of partials
    fits = max(s for s in range(1, 4096) if _scratch_bytes(1, heads, kv_heads, head_dim, s) <= capacity)
    assert _scratch_bytes(1, heads, kv_heads, head_dim, fits) <= capacity < _scratch_bytes(1, heads, kv_heads,
                                                                                           head_dim, fits + 1)
    (q, k_cache, v_cache, positions, token_span, table, q64, keys, values) = _case(
        46, [200], heads, kv_heads, head_dim, page_tokens, (0, 7))
    scale = head_dim ** -0.5
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = torch.zeros((1, heads * head_dim), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call(max_splits):
        return fn(q.data_ptr(), heads * head_dim, got.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                  k_cache.stride(0), positions.data_ptr(), token_span.data_ptr(), table.data_ptr(), table.stride(0),
                  1, heads, kv_heads, head_dim, page_tokens, 0, scale, chunk, max_splits, flag.data_ptr(), stream)

    assert call(fits) == 0, lib.celeg_last_error().decode()          # the whole array is in use: still right
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    want = _attention_float64(q64[0], keys[0], values[0], 199, scale, 0).reshape(1, -1)
    err = np.abs(got.float().cpu().numpy().astype(np.float64) - want)
    assert bool((err <= 1.2e-2 + 1.2e-2 * np.abs(want)).all()), float(err.max())
    assert call(fits + 1) != 0                                         # one split more: refused, nothing launched
    message = lib.celeg_last_error().decode()
    assert "bytes of scratch" in message and str(capacity) in message
    torch.cuda.synchronize()


def test_static_scratch_entry_point_refuses_a_large_batch():
    lib, fn = _symbol()
    capacity = lib.celeg_attention_decode_static_capacity()
    tokens, heads, kv_heads, head_dim, max_splits = 64, 32, 8, 128, 32       # 33.5 MB of partial outputs
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    code = fn(dummy.data_ptr(), heads * head_dim, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 1,
              dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 1, tokens, heads, kv_heads, head_dim, 16, 0,
              1.0, 64, max_splits, dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code != 0
    message = lib.celeg_last_error().decode()
    assert "bytes of scratch" in message and str(capacity) in message
    torch.cuda.synchronize()
