"""The entry point of the kernel library that allocates nothing, celeg_attention_decode_static.

It serves callers that cannot call cudaMalloc when they need decode attention (all device memory
already given to their own pool, or no tolerance for the synchronisation an allocation causes):
its scratch is a fixed array inside the library. Here it is called through its exported C symbol,
twice in a row with different inputs, and compared with the ordinary entry point, which takes
scratch from the caller. The second call finds the array as the first one left it, so it also
shows that nothing stale is used. Sizes beyond the array are refused with a message.
"""
from __future__ import annotations

import ctypes
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


def _case(seed, lengths, heads, kv_heads, head_dim, page_tokens):
    rng = np.random.default_rng(seed)
    pages = sum((n + page_tokens - 1) // page_tokens for n in lengths) + 3
    order = rng.permutation(pages)
    k_cache = torch.tensor(rng.normal(size=(pages, kv_heads, page_tokens, head_dim))).to(torch.bfloat16).cuda()
    v_cache = torch.tensor(rng.normal(size=(pages, kv_heads, page_tokens, head_dim))).to(torch.bfloat16).cuda()
    max_pages = max((n + page_tokens - 1) // page_tokens for n in lengths)
    table = np.full((len(lengths), max_pages), -1, dtype=np.int32)
    used = 0
    for r, n in enumerate(lengths):
        for p in range((n + page_tokens - 1) // page_tokens):
            table[r, p] = order[used]
            used += 1
    tokens = len(lengths)
    q = torch.tensor(rng.normal(size=(tokens, heads * head_dim))).to(torch.bfloat16).cuda()
    positions = torch.tensor([n - 1 for n in lengths], dtype=torch.int32).cuda()
    token_span = torch.arange(tokens, dtype=torch.int32).cuda()
    return q, k_cache, v_cache, positions, token_span, torch.tensor(table).cuda()


def test_static_scratch_entry_point_matches_the_ordinary_one_twice():
    from celeg_b200 import kernels
    lib, fn = _symbol()
    heads, kv_heads, head_dim, page_tokens, chunk = 8, 2, 64, 16, 64
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lengths in ((40, [300, 17, 1, 511]), (41, [64, 129, 500, 2])):
        q, k_cache, v_cache, positions, token_span, table = _case(seed, lengths, heads, kv_heads, head_dim,
                                                                  page_tokens)
        tokens = len(lengths)
        max_splits = (512 + chunk - 1) // chunk
        scale = head_dim ** -0.5
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        want = torch.zeros((tokens, heads * head_dim), dtype=torch.bfloat16, device="cuda")
        kernels.attention_decode(
            q, heads * head_dim, want, k_cache, v_cache, positions, token_span, table, tokens, heads, kv_heads,
            head_dim, page_tokens, None, scale, chunk, max_splits,
            torch.empty(tokens * heads * max_splits * head_dim, dtype=torch.float32, device="cuda"),
            torch.empty(tokens * heads * max_splits * 2, dtype=torch.float32, device="cuda"),
            torch.zeros(tokens * kv_heads, dtype=torch.int32, device="cuda"), flag)
        got = torch.zeros_like(want)
        code = fn(q.data_ptr(), heads * head_dim, got.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                  k_cache.stride(0), positions.data_ptr(), token_span.data_ptr(), table.data_ptr(),
                  table.stride(0), tokens, heads, kv_heads, head_dim, page_tokens, 0, scale, chunk, max_splits,
                  flag.data_ptr(), stream)
        assert code == 0, lib.celeg_last_error().decode()
        torch.cuda.synchronize()
        assert int(flag.item()) == 0
        assert float(want.float().abs().max()) > 0.1
        err = (got.float() - want.float()).abs()
        bound = 1.2e-2 + 1.2e-2 * want.float().abs()          # the tolerance of the kernel tests for bfloat16
        assert bool((err <= bound).all()), float(err.max())


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib, fn = _symbol()
    capacity = lib.celeg_attention_decode_static_capacity()
    assert capacity == 8 * 1024 * 1024
    tokens, heads, kv_heads, head_dim, max_splits = 64, 32, 8, 128, 32       # 33.5 MB of partial outputs
    dummy = torch.zeros(16, dtype=torch.int32, device="cuda")
    code = fn(dummy.data_ptr(), heads * head_dim, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 1,
              dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 1, tokens, heads, kv_heads, head_dim, 16, 0,
              1.0, 64, max_splits, dummy.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code != 0
    message = lib.celeg_last_error().decode()
    assert "bytes of scratch" in message and str(capacity) in message
    torch.cuda.synchronize()
