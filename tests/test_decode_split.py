"""How the decode attention's keys are split (``parts.mixers.decode_split``), over the sizes a configuration
allows: the splits cover the context bucket, fit the scratch that was sized from the longest context alone, and
are chunks the kernel takes (multiples of 64 keys, at most 4,096)."""
from __future__ import annotations

import itertools

import pytest

from celeg_b200.parts.mixers import DECODE_RESIDENT_BLOCKS, decode_split


def test_splits_cover_the_bucket_and_fit_the_scratch():
    checked = 0
    for max_context, window, resident in itertools.product((256, 4096, 131072, 1 << 20), (None, 5, 37, 1000, 5000),
                                                           (148, 444, DECODE_RESIDENT_BLOCKS)):
        bucket = 256
        while bucket <= max(256, 1 << (max_context - 1).bit_length()):
            for tokens, kv_heads in itertools.product((1, 2, 3, 8, 17, 64, 256), (1, 2, 4, 8)):
                chunk, max_splits, cap_splits = decode_split(tokens, kv_heads, bucket, window, max_context, resident)
                effective = bucket if not window else min(bucket, 1 << max(8, (window - 1).bit_length()))
                assert chunk % 64 == 0 and 64 <= chunk <= 4096, (tokens, kv_heads, bucket, window, chunk)
                assert chunk * max_splits >= effective, (tokens, kv_heads, bucket, window, chunk, max_splits)
                assert 1 <= max_splits <= cap_splits, (tokens, kv_heads, bucket, window, max_splits, cap_splits)
                # the scratch depends on the longest context alone, never on the step
                assert cap_splits == decode_split(1, 1, 256, window, max_context, resident)[2]
                checked += 1
            bucket *= 2
    assert checked > 5000


def test_a_bucket_beyond_the_longest_context_is_refused():
    with pytest.raises(ValueError, match="splits"):
        decode_split(1, 8, 1 << 22, None, 4096)


@pytest.mark.parametrize("tokens,bucket,chunk", [(8, 131072, 4096), (1, 131072, 2880), (64, 8192, 2048),
                                                 (16, 32768, 2048), (1, 32768, 1024), (8, 1024, 256), (64, 1024, 1024)])
def test_choices_at_the_measured_sizes(tokens, bucket, chunk):
    """The choices that the measurements on a B200 stand behind (8 kv heads, 740 resident blocks)."""
    assert decode_split(tokens, 8, bucket, None, 131072)[0] == chunk
