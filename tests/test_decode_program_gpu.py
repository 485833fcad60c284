"""The decode program (one persistent kernel for a whole decoding step, off by default) against
the plain implementation and against the same steps run as separate kernels: tiny models, a
configuration wide enough for several units per block and several stages per unit, 1 to 11 requests,
with and without CUDA graphs, a window over the cache, and decoding mixed with finishing requests."""
from __future__ import annotations

import copy

import numpy as np
import pytest
import torch

import plain_lfm2
from tiny_models import CONFIGS, write_tiny

pytestmark = pytest.mark.gpu

# wide enough that a product has more units than the GPU has SMs (inner 2,560 -> 160) and more than one
# stage per unit (k = 2,560 with a copied operand), head size 64 with groups of four query heads
WIDE = {"model_type": "lfm2", "vocab_size": 3000, "hidden_size": 1024, "num_hidden_layers": 3,
        "num_attention_heads": 16, "num_key_value_heads": 4, "max_position_embeddings": 1024, "norm_eps": 1e-5,
        "conv_L_cache": 3, "rope_theta": 1000000.0, "layer_types": ["conv", "full_attention", "conv"],
        "tie_word_embeddings": True, "intermediate_size": 2560}


@pytest.fixture()
def program_on(monkeypatch):
    monkeypatch.setenv("CELEG_B200_DECODE_PROGRAM", "1")


def _load(folder, batch, graphs, **kwargs):
    from celeg_b200.engine.loading import load_model
    return load_model(folder, "bfloat16", max_context=512, max_requests=max(batch, 1), use_graphs=graphs, **kwargs)


def _decode(loaded, prompts, forced):
    """Prefill every prompt in one step, then feed forced[s][i] to request i at step s; logits of every step."""
    from celeg_b200.engine.step import StepEntry
    batch = len(prompts)
    out = [loaded.step.run([StepEntry(i, prompts[i], [len(prompts[i]) - 1]) for i in range(batch)],
                           auto_begin=True).float().cpu().clone()]
    for tokens in forced:
        out.append(loaded.step.run([StepEntry(i, [tokens[i]], [0]) for i in range(batch)]).float().cpu().clone())
    loaded.step.raise_on_device_error()
    return out


def _built(loaded):
    return [p for p in loaded.model._programs.values() if p is not None]


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_program_follows_plain_model(tmp_path, program_on, name, graphs):
    folder = write_tiny(tmp_path, name)
    config, weights = plain_lfm2.load_model_folder(folder)
    vocab = config["vocab_size"]
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in (9, 30, 17)]
    forced = [[int(rng.integers(0, vocab)) for _ in prompts] for _ in range(20)]
    loaded = _load(folder, len(prompts), graphs)
    got = _decode(loaded, prompts, forced)
    assert _built(loaded), f"no program was built: {loaded.model.program_refusal}"
    for i, prompt in enumerate(prompts):
        seq = prompt + [step[i] for step in forced]
        want = plain_lfm2.forward(config, weights, seq)
        for s in range(len(forced) + 1):
            row = got[s][i].numpy()
            ref = want[len(prompt) - 1 + s]
            assert np.abs(row - ref).max() <= 6e-2 + 5e-2 * np.abs(ref).max(), f"{name} request {i} step {s}"
            cos = float(np.dot(row, ref) / (np.linalg.norm(row) * np.linalg.norm(ref) + 1e-30))
            assert cos > 0.999, f"{name} request {i} step {s}: cosine {cos}"


@pytest.mark.parametrize("batch", [1, 3, 8, 11])
def test_program_matches_separate_kernels_on_a_wide_model(tmp_path, monkeypatch, batch):
    from celeg_b200.weights import write_random_model
    folder = str(tmp_path / "wide")
    write_random_model(folder, copy.deepcopy(WIDE), 3, torch.bfloat16)
    rng = np.random.default_rng(5)
    vocab = WIDE["vocab_size"]
    prompts = [rng.integers(0, vocab, size=20 + 3 * i).tolist() for i in range(batch)]
    forced = [[int(rng.integers(0, vocab)) for _ in range(batch)] for _ in range(24)]
    monkeypatch.setenv("CELEG_B200_DECODE_PROGRAM", "0")
    reference = _decode(_load(folder, batch, False), prompts, forced)
    for graphs in (False, True):
        monkeypatch.setenv("CELEG_B200_DECODE_PROGRAM", "1")
        loaded = _load(folder, batch, graphs)
        got = _decode(loaded, prompts, forced)
        assert _built(loaded), f"no program was built: {loaded.model.program_refusal}"
        for s, (a, b) in enumerate(zip(reference, got)):
            scale = a.abs().max().item()
            # both are bfloat16 paths whose sums run in different orders: rounding-level differences only
            assert (a - b).abs().max().item() <= 0.03 * scale, f"batch {batch} graphs {graphs} step {s}"
            cos = torch.nn.functional.cosine_similarity(a, b, dim=1).min().item()
            assert cos > 0.9995, f"batch {batch} graphs {graphs} step {s}: cosine {cos}"


def test_program_with_requests_that_end_and_begin(tmp_path, program_on):
    """Requests finish at different steps and a new one begins on their pages and slot: programs for
    1, 2 and 3 rows run one after another over the same cache."""
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, "B")
    config, weights = plain_lfm2.load_model_folder(folder)
    vocab = config["vocab_size"]
    rng = np.random.default_rng(77)
    seqs = {name: rng.integers(0, vocab, size=n).tolist() for name, n in (("a", 40), ("b", 28), ("c", 33), ("d", 26))}
    loaded = _load(folder, 3, True, cache_tokens=192)
    heads = {"a": 20, "b": 20, "c": 20, "d": 20}
    got = {name: {} for name in seqs}

    def step(entries):
        logits = loaded.step.run([StepEntry(n, toks, want) for n, toks, want in entries], auto_begin=True).float().cpu()
        row = 0
        for n, toks, want in entries:
            for place in want:
                got[n][heads[n] - len(toks) + place] = logits[row].numpy().copy()
                row += 1

    live = ["a", "b", "c"]
    step([(n, seqs[n][:20], [19]) for n in live])
    while live:
        entries = []
        for n in live:
            entries.append((n, [seqs[n][heads[n]]], [0]))
            heads[n] += 1
        step(entries)
        for n in list(live):
            if heads[n] == len(seqs[n]):
                loaded.step.end(n)
                live.remove(n)
                if n == "b":                     # d takes over b's slot and pages
                    step([("d", seqs["d"][:20], [19])])
                    live.append("d")
    loaded.step.raise_on_device_error()
    assert len(_built(loaded)) >= 3
    for n, seq in seqs.items():
        want = plain_lfm2.forward(config, weights, seq)
        assert sorted(got[n]) == list(range(19, len(seq))), n
        for position, row in got[n].items():
            ref = want[position]
            assert np.abs(row - ref).max() <= 6e-2 + 5e-2 * np.abs(ref).max(), f"request {n} position {position}"
    loaded.manager.check_invariants()


def test_program_is_refused_for_float32_and_many_rows(tmp_path, program_on):
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, "A")
    loaded = load_model(folder, "float32", max_context=128, max_requests=2)
    loaded.step.run([StepEntry(0, [1, 2, 3], [2])], auto_begin=True)
    loaded.step.run([StepEntry(0, [4], [0])])
    assert not loaded.model._programs              # the float32 path never asks for a program
    loaded = load_model(folder, "bfloat16", max_context=128, max_requests=20)
    loaded.step.run([StepEntry(i, [1, 2, 3], [2]) for i in range(20)], auto_begin=True)
    loaded.step.run([StepEntry(i, [4], [0]) for i in range(20)])          # 20 rows: separate kernels
    assert not _built(loaded)
    loaded.step.raise_on_device_error()
