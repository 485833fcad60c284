"""The engine at the layer sizes the benchmark runs (hidden 2,048, feed-forward 8,192, 32 query heads on 8 kv
heads of 64, vocabulary 65,536; three layers: conv, attention, conv) against the plain implementation in
float64, in both precisions. The kernel variants that only large shapes select are on the path: the small-batch
products with 8, 16 and 32 warps, the persistent tcgen05 product from 2,048 rows, the tcgen05 prompt attention
with 32 heads, split-key decode attention over thousands of keys. One trace holds all schedules: a prompt with
a portion of 2,048 tokens, its last 32 tokens one by one, a second prompt in portions of changing size beside
the first one's decoded tokens, and a third request that takes over the pages the second gave back."""
from __future__ import annotations

import io
import json
import os

import numpy as np
import pytest

import plain_lfm2

pytestmark = pytest.mark.gpu

BENCH_SIZES = {
    "model_type": "lfm2", "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 3,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "conv_L_cache": 3, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096, "layer_types": ["conv", "full_attention", "conv"],
    "bos_token_id": 1, "eos_token_id": 7, "pad_token_id": 0,
}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from celeg_b200.weights import write_random_model
    folder = str(tmp_path_factory.mktemp("bench_sizes") / "model")
    write_random_model(folder, dict(BENCH_SIZES), 5)
    config, weights = plain_lfm2.load_model_folder(folder)
    rng = np.random.default_rng(50)
    long = rng.integers(0, 65536, size=2048 + 100 + 32).tolist()
    second = rng.integers(0, 65536, size=90).tolist()
    third = rng.integers(0, 65536, size=40).tolist()

    hidden = {}

    def wanted_rows(tokens, places):
        """Plain logits at ``places`` only: the head on 2,180 rows of 65,536 would be most of the work. The
        blocks' output of a sequence is kept, both precisions ask for the same rows."""
        key = tuple(tokens)
        if key not in hidden:
            x = weights["model.embed_tokens.weight"][np.asarray(tokens, dtype=np.int64)]
            for index, kind in enumerate(plain_lfm2.layer_kinds(config, weights)):
                x = plain_lfm2.block(x, index, kind, config, weights)
            hidden[key] = x
        z = plain_lfm2.rmsnorm(hidden[key][places], weights["model.embedding_norm.weight"],
                               plain_lfm2.norm_eps(config))
        return z @ weights["model.embed_tokens.weight"].T

    return folder, (long, second, third), wanted_rows


def test_plain_rows_are_the_plain_model(model):
    """The shortcut above gives what plain_lfm2.forward gives."""
    folder, (long, second, third), wanted_rows = model
    config, weights = plain_lfm2.load_model_folder(folder)
    assert np.allclose(wanted_rows(third, [0, 17, 39]), plain_lfm2.forward(config, weights, third)[[0, 17, 39]],
                       rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_schedules_at_the_benchmark_layer_sizes(model, dtype, tmp_path):
    from celeg_b200.engine.trace import replay
    folder, (long, second, third), wanted_rows = model
    steps, expect = [], []

    def step(entries, end=()):
        steps.append({"step": len(steps), "entries": entries, "end": list(end)})

    # 1: the long prompt: 2,048 tokens in one step, then 100 more, logits at a few places of each
    step([{"id": "long", "tokens": long[:2048], "want": [0, 1023, 2047]}])
    expect.append([("long", p) for p in (0, 1023, 2047)])
    step([{"id": "long", "tokens": long[2048:2148], "want": [0, 99]}])
    expect.append([("long", 2048), ("long", 2147)])
    # 2: its last 32 tokens one by one; beside them the second prompt in portions of changing size (down to two
    # tokens), then decoding too; the third request starts when the second has ended, on the second's pages
    cuts = [2, 17, 3, 33, 2, 16, 9, 8]
    assert sum(cuts) == len(second)
    at = 0
    for j in range(32):
        entries = [{"id": "long", "tokens": [long[2148 + j]], "want": [0]}]
        places = [("long", 2148 + j)]
        ended = []
        if j < len(cuts):
            n = cuts[j]
            entries.append({"id": "second", "tokens": second[at:at + n], "want": [n - 1]})
            places.append(("second", at + n - 1))
            at += n
            if j == len(cuts) - 1:
                ended.append("second")
        elif j >= 10:
            k = j - 10
            portion = third[:18] if k == 0 else third[18 + (k - 1):18 + k] if 18 + k <= len(third) else []
            if portion:
                start = 0 if k == 0 else 18 + (k - 1)
                entries.append({"id": "third", "tokens": portion, "want": [len(portion) - 1]})
                places.append(("third", start + len(portion) - 1))
        if j == 31:
            ended += ["long", "third"]
        step(entries, ended)
        expect.append(places)
    out_dir = str(tmp_path / f"out_{dtype}")
    text = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    # room for the long request and one of the short ones, in pages of 16: the third reuses the second's
    assert replay(folder, dtype, out_dir, 2240 + 128, text, io.StringIO(), max_batched_tokens=2048) == 0
    sequences = {"long": long, "second": second, "third": third}
    places_of = {name: sorted({p for places in expect for n, p in places if n == name}) for name in sequences}
    plain = {name: dict(zip(places_of[name], wanted_rows(sequences[name], places_of[name]))) for name in sequences}
    tol = {"float32": (3e-4, 3e-4), "bfloat16": (6e-2, 5e-2)}[dtype]
    for number, places in enumerate(expect):
        got = np.fromfile(os.path.join(out_dir, f"{number}.f32"), dtype="<f4").reshape(len(places), 65536)
        for row, (name, place) in enumerate(places):
            want = plain[name][place]
            err = np.abs(got[row] - want)
            assert (err <= tol[0] + tol[1] * np.abs(want)).all(), \
                f"{dtype} step {number} {name}[{place}]: max error {err.max():.3e}"
            cosine = float(np.dot(got[row], want) / (np.linalg.norm(got[row]) * np.linalg.norm(want)))
            assert cosine > (0.999999 if dtype == "float32" else 0.999), (number, name, place, cosine)
