"""The engine against the plain implementation through trace replay schedules, in float32 and
in bfloat16: whole, mostly whole then the last 32 one by one, portions of changing size down to
two tokens, and mixed with so few pages that pages and slots are used again."""
from __future__ import annotations

import io
import json
import os

import numpy as np
import pytest

import plain_lfm2
from tiny_models import write_tiny

pytestmark = pytest.mark.gpu

# float32 path against the float64 plain model; bfloat16 path against the same (bf16 weights are
# exact in both, so the gap is activation rounding only)
TOL = {"float32": dict(atol=2e-4, rtol=2e-4), "bfloat16": dict(atol=6e-2, rtol=5e-2)}


def run_trace(folder, dtype, steps, max_tokens, tmp_path, tag, page_tokens=16):
    from celeg_b200.engine.trace import replay
    out_dir = str(tmp_path / f"out_{tag}_{dtype}")
    text = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
    done = io.StringIO()
    assert replay(folder, dtype, out_dir, max_tokens, text, done, page_tokens=page_tokens) == 0
    assert done.getvalue().split() == [w for step in steps for w in ("done", str(step["step"]))]
    return out_dir


def read_logits(out_dir, step, vocab):
    data = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
    return data.reshape(-1, vocab)


def compare(got, want, dtype, what):
    tol = TOL[dtype]
    err = np.abs(got - want)
    bound = tol["atol"] + tol["rtol"] * np.abs(want)
    worst = np.unravel_index(np.argmax(err - bound), err.shape)
    assert (err <= bound).all(), (f"{what}: row {worst[0]} col {worst[1]} got {got[worst]} want {want[worst]} "
                                  f"(max err {err.max():.3e})")
    if dtype == "bfloat16":
        for row_got, row_want in zip(got, want):
            cos = float(np.dot(row_got, row_want) / (np.linalg.norm(row_got) * np.linalg.norm(row_want) + 1e-30))
            assert cos > 0.999, f"{what}: cosine {cos}"


def sequences(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    out = {}
    for name in ("A", "B", "C", "D"):
        folder = write_tiny(base, name)
        config, weights = plain_lfm2.load_model_folder(folder)
        out[name] = (folder, config, weights)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_requests(models, name, dtype, tmp_path):
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    seqs = sequences(vocab, [5, 17, 31, 130], seed=10)
    steps = [{"step": i, "entries": [{"id": f"r{i}", "tokens": s, "want": list(range(len(s)))}], "end": [f"r{i}"]}
             for i, s in enumerate(seqs)]
    out = run_trace(folder, dtype, steps, 192, tmp_path, "whole")
    for i, s in enumerate(seqs):
        compare(read_logits(out, i, vocab), plain_lfm2.forward(config, weights, s), dtype, f"{name} whole {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_one_by_one(models, name, dtype, tmp_path):
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    (seq,) = sequences(vocab, [97], seed=11)
    head = len(seq) - 32
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": seq[:head], "want": [head - 1]}], "end": []}]
    for j in range(32):
        steps.append({"step": j + 1, "entries": [{"id": "x", "tokens": [seq[head + j]], "want": [0]}],
                      "end": ["x"] if j == 31 else []})
    out = run_trace(folder, dtype, steps, 128, tmp_path, "decode")
    want = plain_lfm2.forward(config, weights, seq)
    compare(read_logits(out, 0, vocab), want[head - 1:head], dtype, f"{name} prefill end")
    for j in range(32):
        compare(read_logits(out, j + 1, vocab), want[head + j:head + j + 1], dtype, f"{name} decode {j}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_portions_of_changing_size(models, name, dtype, tmp_path):
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    (seq,) = sequences(vocab, [150], seed=12)
    cuts = [2, 3, 2, 16, 1, 17, 2, 31, 33, 2, 5, 2, 34]
    assert sum(cuts) == len(seq)
    steps, at = [], 0
    for i, n in enumerate(cuts):
        steps.append({"step": i, "entries": [{"id": "p", "tokens": seq[at:at + n], "want": list(range(n))}],
                      "end": ["p"] if i == len(cuts) - 1 else []})
        at += n
    out = run_trace(folder, dtype, steps, 192, tmp_path, "portions")
    want = plain_lfm2.forward(config, weights, seq)
    at = 0
    for i, n in enumerate(cuts):
        compare(read_logits(out, i, vocab), want[at:at + n], dtype, f"{name} portion {i} at {at}")
        at += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_mixed_requests_with_page_reuse(models, name, dtype, tmp_path):
    """Eight requests through a pool that holds four: portions of some beside decoded tokens of
    others; later requests get pages and slots that earlier ones gave back."""
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    lengths = [40, 64, 23, 57, 64, 35, 49, 18]
    seqs = sequences(vocab, lengths, seed=13)
    rng = np.random.default_rng(14)
    progress = [0] * len(seqs)
    live, waiting = [], list(range(len(seqs)))
    steps, expect = [], []
    number = 0
    while live or waiting:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, ended, places = [], [], []
        for r in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                    # left out of this step, goes on later
            left = lengths[r] - progress[r]
            # the last 8 tokens of every request go one by one, the rest in portions of 2..13
            n = 1 if left <= 8 else min(left - 8, int(rng.integers(2, 14)))
            want = sorted(set(rng.integers(0, n, size=2).tolist())) if n > 1 else [0]
            entries.append({"id": f"q{r}", "tokens": seqs[r][progress[r]:progress[r] + n], "want": want})
            places.extend((r, progress[r] + w) for w in want)
            progress[r] += n
            if progress[r] == lengths[r]:
                ended.append(f"q{r}")
                live.remove(r)
        if not entries:
            continue
        steps.append({"step": number, "entries": entries, "end": ended})
        expect.append(places)
        number += 1
    out = run_trace(folder, dtype, steps, 4 * 64, tmp_path, "mixed")
    full = [plain_lfm2.forward(config, weights, s) for s in seqs]
    for i, places in enumerate(expect):
        got = read_logits(out, i, vocab)
        want = np.stack([full[r][p] for r, p in places])
        compare(got, want, dtype, f"{name} mixed step {i} places {places}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_larger_than_one_pass_is_cut_inside(models, dtype, tmp_path):
    """Two requests bring 150 and 40 tokens in ONE step to a replay whose passes hold 16 tokens."""
    from celeg_b200.engine.trace import replay
    folder, config, weights = models["B"]
    vocab = config["vocab_size"]
    a, b = sequences(vocab, [150, 40], seed=15)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a, "want": [0, 17, 149]},
                                     {"id": "b", "tokens": b, "want": [39]}], "end": ["a"]},
             {"step": 1, "entries": [{"id": "b", "tokens": [5], "want": [0]}], "end": ["b"]}]
    out_dir = str(tmp_path / f"cut_{dtype}")
    text = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
    assert replay(folder, dtype, out_dir, 256, text, io.StringIO(), max_batched_tokens=16) == 0
    want_a = plain_lfm2.forward(config, weights, a)
    want_b = plain_lfm2.forward(config, weights, b + [5])
    compare(read_logits(out_dir, 0, vocab), np.stack([want_a[0], want_a[17], want_a[149], want_b[39]]), dtype, "cut")
    compare(read_logits(out_dir, 1, vocab), want_b[40:41], dtype, "after the cut")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_single_tokens_before_portions_in_one_step(models, name, dtype, tmp_path):
    """The shape of step the scheduler plans under load: decoded tokens of some requests first, then portions
    of others' prompts. The single tokens at the head of such a step take the decode attention, the portions the
    prompt attention, in the same pass. The decoding requests sit at very different depths (inside a first page,
    at a page's edge, beyond 128 keys), one portion is new and one continues a prompt."""
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    seqs = sequences(vocab, [72, 18, 135, 47, 40], seed=16)
    depth = [70, 16, 131]                       # r0..r2 are this deep when the mixed steps begin
    steps = [{"step": 0, "entries": [{"id": f"r{i}", "tokens": seqs[i][:depth[i]], "want": [depth[i] - 1]}
                                     for i in range(3)] +
                                    [{"id": "r4", "tokens": seqs[4][:9], "want": []}], "end": []}]
    # two mixed steps: r0..r2 one token each, r3 begins with 30 tokens then 17, r4 goes on with 2 then 29
    cuts3, cuts4 = [30, 17], [2, 29]
    at3, at4 = 0, 9
    for j in range(2):
        entries = [{"id": f"r{i}", "tokens": [seqs[i][depth[i] + j]], "want": [0]} for i in range(3)]
        entries.append({"id": "r3", "tokens": seqs[3][at3:at3 + cuts3[j]], "want": [0, cuts3[j] - 1]})
        entries.append({"id": "r4", "tokens": seqs[4][at4:at4 + cuts4[j]], "want": [cuts4[j] - 1]})
        steps.append({"step": j + 1, "entries": entries, "end": []})
        at3 += cuts3[j]
        at4 += cuts4[j]
    out = run_trace(folder, dtype, steps, 5 * 192, tmp_path, "single_then_portions")
    full = [plain_lfm2.forward(config, weights, s) for s in seqs]
    compare(read_logits(out, 0, vocab), np.stack([full[i][depth[i] - 1] for i in range(3)]), dtype, f"{name} prompts")
    at3, at4 = 0, 9
    for j in range(2):
        want = [full[i][depth[i] + j] for i in range(3)]
        want += [full[3][at3], full[3][at3 + cuts3[j] - 1], full[4][at4 + cuts4[j] - 1]]
        compare(read_logits(out, j + 1, vocab), np.stack(want), dtype, f"{name} mixed step {j}")
        at3 += cuts3[j]
        at4 += cuts4[j]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,requests", [("B", 20), ("D", 33), ("B", 64), ("D", 64)])
def test_many_requests_decoding_together(models, name, requests, dtype, tmp_path):
    """More requests than the small-batch kernels take (16): 20, 33 and 64 requests decode together, with the
    switches at their defaults. Prompts of 3 to 40 tokens go in first, eight requests to a step; then four
    steps in which every request brings one token; every row of every step against the plain model."""
    from celeg_b200.engine.trace import replay
    folder, config, weights = models[name]
    vocab = config["vocab_size"]
    rng = np.random.default_rng(17)
    lengths = rng.integers(3, 41, size=requests).tolist()
    seqs = sequences(vocab, [n + 4 for n in lengths], seed=18)
    steps = []
    for first in range(0, requests, 8):
        group = range(first, min(first + 8, requests))
        steps.append({"step": len(steps), "entries": [{"id": f"m{i}", "tokens": seqs[i][:lengths[i]],
                                                       "want": [lengths[i] - 1]} for i in group], "end": []})
    prompt_steps = len(steps)
    for j in range(4):
        steps.append({"step": len(steps), "entries": [{"id": f"m{i}", "tokens": [seqs[i][lengths[i] + j]], "want": [0]}
                                                      for i in range(requests)],
                      "end": [f"m{i}" for i in range(requests)] if j == 3 else []})
    out_dir = str(tmp_path / f"many_{name}_{requests}_{dtype}")
    text = io.StringIO("".join(json.dumps(step) + "\n" for step in steps))
    assert replay(folder, dtype, out_dir, requests * 64, text, io.StringIO(), max_requests=requests) == 0
    full = [plain_lfm2.forward(config, weights, s) for s in seqs]
    for number in range(prompt_steps):
        group = range(number * 8, min(number * 8 + 8, requests))
        compare(read_logits(out_dir, number, vocab), np.stack([full[i][lengths[i] - 1] for i in group]), dtype,
                f"{name} prompts {number}")
    for j in range(4):
        compare(read_logits(out_dir, prompt_steps + j, vocab),
                np.stack([full[i][lengths[i] + j] for i in range(requests)]), dtype, f"{name} decode step {j}")


def test_entries_without_tokens_and_ends_of_requests_that_hold_nothing(models, tmp_path):
    """An entry without tokens is a request left out of the step; ending a request that never brought a token,
    or that was ended before, gives nothing back and is no error; an id may come again after its end."""
    folder, config, weights = models["A"]
    vocab = config["vocab_size"]
    first, second = sequences(vocab, [21, 9], seed=33)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": first[:20], "want": [19]}, {"id": "b", "tokens": [], "want": []}],
         "end": ["b", "never"]},
        {"step": 1, "entries": [{"id": "a", "tokens": first[20:], "want": [0]}], "end": ["a"]},
        {"step": 2, "entries": [], "end": ["a"]},
        {"step": 3, "entries": [{"id": "a", "tokens": second, "want": [8]}], "end": ["a"]},
    ]
    out = run_trace(folder, "float32", steps, 64, tmp_path, "lenient")
    want = plain_lfm2.forward(config, weights, first)
    compare(read_logits(out, 0, vocab), want[19:20], "float32", "step 0")
    compare(read_logits(out, 1, vocab), want[20:21], "float32", "step 1")
    assert not os.path.exists(os.path.join(out, "2.f32"))
    compare(read_logits(out, 3, vocab), plain_lfm2.forward(config, weights, second)[8:9], "float32", "step 3")
