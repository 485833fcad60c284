"""The engine through its Python entry point and its parts on the GPU: greedy and seeded
generation against the plain implementation, long decoding, first tokens, parts alone, and a toy
mixer with state of its own that is registered, built and stepped from outside the package."""
from __future__ import annotations

import copy
import dataclasses
import io
import json

import numpy as np
import pytest
import torch

import plain_lfm2
from tiny_models import CONFIGS, TINY_A, TINY_B, write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("engine_models")
    out = {}
    for name in ("A", "B", "C"):
        folder = write_tiny(base, name)
        config, weights = plain_lfm2.load_model_folder(folder)
        out[name] = (folder, config, weights)
    return out


def prompts_of(vocab, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_matches_plain_model_float32(models, graphs):
    """The benchmark's workload in small, on tiny A: prompts of 5, 17 and 31 tokens, 16 greedy tokens each, run
    together through the scheduler."""
    from celeg_b200 import Engine
    folder, config, weights = models["A"]
    prompts = prompts_of(config["vocab_size"], [5, 17, 31], seed=20)
    engine = Engine(folder, dtype="float32", use_cuda_graph=graphs)
    got = engine.generate(prompts, max_new_tokens=16, temperature=0.0, repetition_penalty=1.0, eos_tokens=())
    for prompt, tokens in zip(prompts, got):
        assert tokens == plain_lfm2.generate(config, weights, prompt, 16, eos_tokens=())
    metrics = engine.metrics()
    assert metrics.completed == 3 and metrics.prefill_tokens == 53 and metrics.decode_tokens == 45
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == engine.options.max_active_requests


def test_greedy_generation_bfloat16_follows_plain_model(models):
    from celeg_b200 import Engine
    folder, config, weights = models["B"]
    prompts = prompts_of(config["vocab_size"], [9, 40], seed=21)
    engine = Engine(folder, dtype="bfloat16")
    got = engine.generate(prompts, max_new_tokens=12, temperature=0.0, repetition_penalty=1.0, eos_tokens=())
    for prompt, tokens in zip(prompts, got):
        # bf16 rounding may flip a near-tie; then the continuation differs, so compare step by
        # step against the plain model fed with the engine's own tokens
        sequence = list(prompt)
        for token in tokens:
            logits = plain_lfm2.forward(config, weights, sequence)[-1]
            best = float(logits.max())
            assert logits[token] >= best - 0.05, (token, int(logits.argmax()))
            sequence.append(token)


def test_seeded_sampling_is_independent_of_the_batch(models):
    """Tiny B's workload: chunked prefill beside decoding requests, temperature 0.8, seed 7. A
    request alone and the same request among others draw the same tokens (float32 path, so the
    logits agree to rounding), and they match the plain sampler fed with plain logits."""
    from celeg_b200 import Engine, EngineOptions
    folder, config, weights = models["B"]
    prompts = prompts_of(config["vocab_size"], [33, 1, 64, 20], seed=22)
    options = EngineOptions(max_active_requests=4, max_batched_tokens=24, prefill_chunk_tokens=7)
    kwargs = dict(max_new_tokens=24, temperature=0.8, top_k=50, top_p=0.95, repetition_penalty=1.1, seed=7,
                  eos_tokens=())
    together = Engine(folder, dtype="float32", options=options).generate(prompts, **kwargs)
    alone = Engine(folder, dtype="float32", options=options)
    for prompt, tokens in zip(prompts, together):
        assert alone.generate(prompt, **kwargs) == tokens
    want = plain_lfm2.generate(config, weights, prompts[0], 24, temperature=0.8, top_k=50, top_p=0.95,
                               repetition_penalty=1.1, seed=7)
    assert together[0] == want


def test_eos_stops_generation(models):
    from celeg_b200 import Engine
    folder, config, weights = models["A"]
    (prompt,) = prompts_of(config["vocab_size"], [11], seed=23)
    free_run = plain_lfm2.generate(config, weights, prompt, 10, eos_tokens=())
    stop = free_run[4]
    engine = Engine(folder, dtype="float32")
    got = engine.generate(prompt, max_new_tokens=10, temperature=0.0, repetition_penalty=1.0, eos_tokens=[stop])
    assert got == free_run[:free_run.index(stop) + 1]


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-4), ("bfloat16", 8e-2)])
def test_long_decoding(models, dtype, tol):
    """A short prompt, then 200 tokens decoded one by one with CUDA graphs on: pages fill and
    follow one another, the context bucket of the graph changes, positions grow."""
    from celeg_b200 import Engine, StepEntry
    folder, config, weights = models["A"]
    (sequence,) = prompts_of(config["vocab_size"], [215], seed=24)
    engine = Engine(folder, dtype=dtype, use_cuda_graph=True)
    want = plain_lfm2.forward(config, weights, sequence)
    got = [engine.forward([StepEntry("long", sequence[:15], [14])])[0].cpu().numpy()]
    for token in sequence[15:]:
        got.append(engine.forward([StepEntry("long", [token], [0])])[0].cpu().numpy())
    got = np.stack(got)
    err = np.abs(got - want[14:])
    assert err.max() < tol, f"worst at step {int(err.max(axis=1).argmax())}: {err.max():.3e}"
    engine.end("long")


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-4), ("bfloat16", 8e-2)])
def test_a_context_of_thousands_of_tokens(tmp_path, dtype, tol):
    """2,700 prompt tokens in portions of 1,000 (query tiles with more than forty blocks of keys behind them:
    every ring and barrier of the attention kernels wraps many times), then tokens decoded one by one with the
    keys split over many blocks that are merged, beside a short request that needs one block only."""
    from celeg_b200 import Engine, EngineOptions, StepEntry
    from celeg_b200.weights import write_random_model
    from tiny_models import TINY_D
    raw = copy.deepcopy(TINY_D)
    raw["max_position_embeddings"] = 4096
    folder = str(tmp_path / "long_context")
    write_random_model(folder, raw, 3, torch.bfloat16)
    config, weights = plain_lfm2.load_model_folder(folder)
    long_seq, short_seq = prompts_of(config["vocab_size"], [2712, 40], seed=29)
    want_long = plain_lfm2.forward(config, weights, long_seq)
    want_short = plain_lfm2.forward(config, weights, short_seq)
    engine = Engine(folder, dtype=dtype, max_context=4096, use_cuda_graph=True,
                    options=EngineOptions(max_batched_tokens=1024, prefill_chunk_tokens=1024))
    at = 0
    for size in (1000, 1000, 700):
        last = at + size == 2700
        out = engine.forward([StepEntry("long", long_seq[at:at + size], [size - 1] if last else [])])
        at += size
    got = [out[0].cpu().numpy()]
    engine.forward([StepEntry("short", short_seq[:28], [])])
    for step in range(12):
        out = engine.forward([StepEntry("long", [long_seq[2700 + step]], [0]),
                              StepEntry("short", [short_seq[28 + step]], [0])])
        got.append(out[0].cpu().numpy())
        assert np.abs(out[1].cpu().numpy() - want_short[28 + step]).max() < tol, f"short request, step {step}"
    err = np.abs(np.stack(got) - want_long[2699:2712])
    assert err.max() < tol, f"worst at step {int(err.max(axis=1).argmax())}: {err.max():.3e}"
    engine.end("long")
    engine.end("short")


def test_many_requests_decoding_over_thousands_of_keys(tmp_path):
    """Forty requests that hold the same 4,100-token prompt (each in pages of its own) decode together: the
    decode attention then cuts the keys into chunks of 2,048 (long contexts and enough requests to fill the GPU
    with few splits each) instead of 1,024 and fewer. Four steps, every request's logits against the plain model."""
    from celeg_b200 import Engine, EngineOptions, StepEntry
    from celeg_b200.parts.mixers import decode_split
    from celeg_b200.weights import write_random_model
    from tiny_models import TINY_D
    raw = copy.deepcopy(TINY_D)
    raw["max_position_embeddings"] = 8192
    folder = str(tmp_path / "many_long")
    write_random_model(folder, raw, 5, torch.bfloat16)
    config, weights = plain_lfm2.load_model_folder(folder)
    (sequence,) = prompts_of(config["vocab_size"], [4104], seed=53)
    want = plain_lfm2.forward(config, weights, sequence)
    requests, prompt = 40, 4100
    assert decode_split(requests, raw["num_key_value_heads"], 8192, None, 8192)[0] == 2048
    engine = Engine(folder, dtype="bfloat16", max_context=8192, use_cuda_graph=True,
                    options=EngineOptions(max_active_requests=requests, max_batched_tokens=2048,
                                          prefill_chunk_tokens=2048))
    for r in range(requests):
        for at in range(0, prompt, 2048):
            engine.forward([StepEntry(f"r{r}", sequence[at:min(at + 2048, prompt)], [])])
    for step in range(4):
        out = engine.forward([StepEntry(f"r{r}", [sequence[prompt + step]], [0]) for r in range(requests)])
        got = out.float().cpu().numpy()
        worst = np.abs(got - want[prompt + step][None, :]).max(axis=1)
        assert worst.max() < 8e-2, f"step {step}, request {int(worst.argmax())}: {worst.max():.3e}"
    engine.loaded.step.raise_on_device_error()
    for r in range(requests):
        engine.end(f"r{r}")


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-4), ("bfloat16", 6e-2)])
def test_first_tokens_of_a_sequence(models, dtype, tol):
    """Positions 0..5 one by one: fewer tokens than the conv kernel has taps, one key only."""
    from celeg_b200 import Engine, StepEntry
    for name in ("A", "B", "C"):
        folder, config, weights = models[name]
        (sequence,) = prompts_of(config["vocab_size"], [6], seed=25)
        engine = Engine(folder, dtype=dtype)
        want = plain_lfm2.forward(config, weights, sequence)
        for i, token in enumerate(sequence):
            got = engine.forward([StepEntry("first", [token], [0])])[0].cpu().numpy()
            assert np.abs(got - want[i]).max() < tol, (name, i)


def test_step_input_errors_name_the_request(models):
    from celeg_b200 import Engine, StepEntry
    from celeg_b200.engine.step import StepInputError
    folder, config, _ = models["A"]
    engine = Engine(folder, dtype="float32")
    with pytest.raises(StepInputError, match="'x'"):
        engine.forward([StepEntry("x", [1, 99999], [])])
    with pytest.raises(StepInputError, match="twice"):
        engine.forward([StepEntry("y", [1], []), StepEntry("y", [2], [])])
    with pytest.raises(StepInputError, match="wanted place"):
        engine.forward([StepEntry("z", [1, 2], [2])])
    with pytest.raises(StepInputError, match="context"):
        engine.forward([StepEntry("w", [1] * 300, [])])


def test_out_of_pages_leaves_everything_as_it_was(models):
    from celeg_b200 import Engine, EngineOptions, StepEntry
    from celeg_b200.cache import OutOfPages
    from celeg_b200.engine.step import StepInputError
    folder, config, weights = models["A"]
    engine = Engine(folder, dtype="float32", options=EngineOptions(logical_kv_pages=3, max_active_requests=2))
    sequence = prompts_of(config["vocab_size"], [40], seed=26)[0]
    engine.forward([StepEntry("a", sequence[:30], [])])              # 2 of 3 pages
    with pytest.raises(OutOfPages):
        engine.forward([StepEntry("a", sequence[30:32], []), StepEntry("b", sequence[:20], [])])
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.get("a").tokens == 30
    assert engine.loaded.manager.find("b") is None and engine.loaded.manager.free_slots == 1   # "b" was not begun
    with pytest.raises(StepInputError, match="context"):             # nor is a request that a faulty step names
        engine.forward([StepEntry("c", sequence[:2], []), StepEntry("a", [1] * 300, [])])
    assert engine.loaded.manager.find("c") is None and engine.loaded.manager.free_slots == 1
    got = engine.forward([StepEntry("a", sequence[30:40], [9])])[0].cpu().numpy()
    want = plain_lfm2.forward(config, weights, sequence)[39]
    assert np.abs(got - want).max() < 2e-4


# ------------------------------------------------------------------------- parts alone
def tiny_runtime(dtype, max_tokens=64):
    from celeg_b200.parts import Runtime
    return Runtime(torch.device("cuda:0"), dtype, max_tokens, max_requests=4, max_context=256)


def step_context(spans, page_tokens=16, slots=None):
    """spans: list of (start position, token count); every request gets fresh pages in order."""
    from celeg_b200.parts import StepContext
    positions, token_span, begins = [], [], [0]
    for index, (start, count) in enumerate(spans):
        positions += list(range(start, start + count))
        token_span += [index] * count
        begins.append(begins[-1] + count)
    max_pages = max((s + c + page_tokens - 1) // page_tokens for s, c in spans)
    table = np.full((len(spans), max_pages), -1, dtype=np.int32)
    page = 0
    for index, (start, count) in enumerate(spans):
        for logical in range((start + count + page_tokens - 1) // page_tokens):
            table[index, logical] = page
            page += 1
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    return StepContext(tokens=len(positions), spans=len(spans), token_ids=i32([0] * len(positions)),
                       positions=i32(positions), token_span=i32(token_span), span_begin=i32(begins),
                       span_slot=i32(slots or list(range(len(spans)))), block_tables=[i32(table)],
                       error_flag=torch.zeros(1, dtype=torch.int32, device="cuda"),
                       max_span=max(c for _, c in spans), max_context=max(s + c for s, c in spans),
                       context_bucket=256), page


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 4e-2)])
def test_parts_alone_against_their_plain_functions(dtype, tol):
    """Each part built from the registry with its own sizes, outside any model."""
    from celeg_b200.parts import PagedBinding, StateBinding, part_factory
    rng = np.random.default_rng(30)
    rt = tiny_runtime(dtype)
    w = lambda *shape, std=0.3: torch.tensor(rng.normal(size=shape) * std).to(torch.bfloat16)
    f64 = lambda t: t.to(torch.float64).numpy()
    hidden, tokens = 72, 23
    x_host = w(tokens, hidden, std=1.0)
    x = torch.zeros((64, hidden), dtype=dtype, device="cuda")
    x[:tokens] = x_host.to(dtype).cuda()
    out = torch.zeros((64, hidden), dtype=dtype, device="cuda")

    def check(got, want, scale=1.0):
        err = np.abs(got[:tokens].to(torch.float64).cpu().numpy() - want)
        # intermediate rounding scales with the size of the terms that were summed, not of the result
        bound = tol * scale * max(1.0, float(np.sqrt(np.mean(want * want))))
        assert err.max() <= bound, (err.max(), bound)

    # norm
    norm_w = (1 + 0.1 * torch.tensor(rng.normal(size=hidden))).to(torch.bfloat16)
    norm = part_factory("norm", "rmsnorm")({"width": hidden, "eps": 2e-5}, {"weight": norm_w}, rt)
    residual = torch.zeros((64, hidden), dtype=torch.float32, device="cuda")
    residual[:tokens] = x_host.float().cuda()
    norm.add_norm(residual, None, out, tokens)
    check(out, plain_lfm2.rmsnorm(f64(x_host), f64(norm_w), 2e-5))

    # feed-forward
    inner = 100
    ffn_w = {"gate": w(inner, hidden), "up": w(inner, hidden), "down": w(hidden, inner)}
    ffn = part_factory("feed_forward", "swiglu")({"hidden_size": hidden, "intermediate_size": inner}, ffn_w, {}, rt)
    step, _ = step_context([(0, tokens)])
    ffn.forward(x, out, step)
    check(out, plain_lfm2.swiglu(f64(x_host), f64(ffn_w["gate"]), f64(ffn_w["up"]), f64(ffn_w["down"])), 4.0)

    # short convolution, in two portions (5 taps, the second portion shorter than the kernel)
    taps = 5
    conv_w = {"in_proj": w(3 * hidden, hidden), "conv": w(hidden, 1, taps), "out_proj": w(hidden, hidden)}
    conv = part_factory("mixer", "short_conv")({"hidden_size": hidden, "taps": taps}, conv_w, {}, rt)
    assert conv.cache_need().elements == (taps - 1) * hidden
    state = torch.zeros((2, (taps - 1) * hidden + 8), dtype=torch.float32, device="cuda")
    conv.bind_cache(StateBinding(state=state[:, 4:], slot_stride=state.stride(0)))
    want = plain_lfm2.short_conv_mixer(f64(x_host), f64(conv_w["in_proj"]), f64(conv_w["conv"]),
                                       f64(conv_w["out_proj"]))
    cut = tokens - 3
    step, _ = step_context([(0, cut)], slots=[1])
    conv.forward(x, out, step)
    tail_in = torch.zeros_like(x)
    tail_in[:3] = x[cut:tokens]
    tail_out = torch.zeros_like(out)
    step, _ = step_context([(cut, 3)], slots=[1])
    conv.forward(tail_in, tail_out, step)
    got = torch.cat([out[:cut], tail_out[:3]])
    check(got, want, 4.0)
    assert float(state[0].abs().sum()) == 0.0

    # attention: 3 heads on 1 kv head, head size 24, in two portions over pages of 8
    heads, kv_heads, head_dim, theta, eps = 3, 1, 24, 5000.0, 1e-5
    attn_w = {"q_proj": w(heads * head_dim, hidden), "k_proj": w(kv_heads * head_dim, hidden),
              "v_proj": w(kv_heads * head_dim, hidden), "out_proj": w(hidden, heads * head_dim),
              "q_norm": (1 + 0.1 * torch.tensor(rng.normal(size=head_dim))).to(torch.bfloat16),
              "k_norm": (1 + 0.1 * torch.tensor(rng.normal(size=head_dim))).to(torch.bfloat16)}
    position = part_factory("position", "rope_split_half")(
        {"theta": theta, "head_dim": head_dim, "rotary_dim": head_dim}, rt)
    attention = part_factory("mixer", "attention")(
        {"hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
         "qk_norm_eps": eps, "window": None, "softmax_scale": head_dim ** -0.5}, attn_w, {"position": position}, rt)
    need = attention.cache_need()
    assert (need.kv_heads, need.head_dim, need.window) == (kv_heads, head_dim, None)
    k_cache = torch.zeros((8, kv_heads, 8, head_dim), dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    attention.bind_cache(PagedBinding(group=0, k=k_cache, v=v_cache, page_tokens=8))
    want = plain_lfm2.attention_mixer(f64(x_host), *(f64(attn_w[n]) for n in
                                                     ("q_proj", "k_proj", "v_proj", "out_proj", "q_norm", "k_norm")),
                                      heads, kv_heads, head_dim, theta, eps)
    step, _ = step_context([(0, cut)], page_tokens=8)
    attention.forward(x, out, step)
    step, _ = step_context([(cut, 3)], page_tokens=8)
    attention.forward(tail_in, tail_out, step)
    got = torch.cat([out[:cut], tail_out[:3]])
    check(got, want, 4.0)


# --------------------------------------------------------- a toy mixer from outside the package
def test_toy_mixer_with_its_own_state_is_registered_built_and_stepped(tmp_path):
    """An exponential moving average over the sequence, y_t = s_t W with s_t = a*s_{t-1} + x_t and
    per-request state s of fixed size, is defined here, registered, put into a model description
    in place of one LFM2 layer's mixer, and run through the engine's own loader, cache manager
    and step function in portions, against a plain computation."""
    from celeg_b200.cache import StateNeed
    from celeg_b200.config import (Architecture, Lfm2Config, PartSpec, TensorRef, build_lfm2_spec,
                                   register_architecture)
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.parts import register_part
    from celeg_b200.weights import write_random_model

    decay = 0.75

    @register_part("mixer", "toy_ema", replace=True)
    class ToyEma:
        def __init__(self, params, weights, parts, rt):
            self.rt = rt
            self.hidden = params["hidden_size"]
            self.decay = params["decay"]
            self.weight = rt.matrix(weights["proj"])
            self.binding = None
            self.mixed = rt.scratch("toy.mixed", self.hidden)

        def cache_need(self):
            return StateNeed(elements=self.hidden)

        def bind_cache(self, binding):
            self.binding = binding

        def forward(self, x, out, step):
            # plain torch on the device: a toy part is free to be slow
            state = self.binding.state
            begins = step.span_begin[:step.spans + 1].tolist()
            slots = step.span_slot[:step.spans].tolist()
            for index, slot in enumerate(slots):
                s = state[slot, :self.hidden].clone()
                for t in range(begins[index], begins[index + 1]):
                    s = self.decay * s + x[t].float()
                    self.mixed[t] = s.to(self.mixed.dtype)
                state[slot, :self.hidden] = s
            self.rt.linear(self.mixed, self.weight, out, step.tokens)

    def toy_spec(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        hidden = config.hidden_size
        toy = PartSpec(kind="toy_ema", params={"hidden_size": hidden, "decay": decay},
                       tensors={"proj": TensorRef("model.layers.1.toy.proj.weight", (hidden, hidden))})
        layers[1] = dataclasses.replace(layers[1], mixer=toy)
        return dataclasses.replace(spec, layers=tuple(layers), architecture="toy_lfm2")

    register_architecture(Architecture(
        name="toy_lfm2", parse_config=Lfm2Config.from_dict,
        resolve_config=lambda config, shapes: dataclasses.replace(
            config, tie_word_embeddings=True if config.tie_word_embeddings is None else config.tie_word_embeddings),
        build_spec=toy_spec, random_init=lfm2_random_init), replace=True)

    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "toy_lfm2"
    folder = write_random_model(str(tmp_path / "toy"), raw, 5)
    loaded = load_model(folder, dtype="float32", max_requests=3, cache_tokens=128, max_batched_tokens=64)
    assert loaded.model.state_layout.sizes[(1, "mixer")] == 64          # the toy's state sits in the slot beside the convs'
    assert len(loaded.model.state_layout.offsets) == 3       # two conv layers (0, 3) + the toy (1)

    config, weights = plain_lfm2.load_model_folder(folder)

    def plain_forward(tokens):
        x = weights["model.embed_tokens.weight"][np.asarray(tokens)]
        for index, kind in enumerate(config["layer_types"]):
            if index != 1:
                x = plain_lfm2.block(x, index, kind, config, weights)
                continue
            p = "model.layers.1."
            n = plain_lfm2.rmsnorm(x, weights[p + "operator_norm.weight"], config["norm_eps"])
            s, mixed = np.zeros(x.shape[1]), np.zeros_like(x)
            for t in range(len(tokens)):
                s = decay * s + n[t]
                mixed[t] = s
            h = x + mixed @ weights[p + "toy.proj.weight"].T
            n2 = plain_lfm2.rmsnorm(h, weights[p + "ffn_norm.weight"], config["norm_eps"])
            x = h + plain_lfm2.swiglu(n2, weights[p + "feed_forward.w1.weight"], weights[p + "feed_forward.w3.weight"],
                                      weights[p + "feed_forward.w2.weight"])
        z = plain_lfm2.rmsnorm(x, weights["model.embedding_norm.weight"], config["norm_eps"])
        return z @ weights["model.embed_tokens.weight"].T

    sequences = prompts_of(config["vocab_size"], [30, 21], seed=31)
    want = [plain_forward(s) for s in sequences]
    step = loaded.step
    cuts = [(7, 2), (1, 9), (10, 1), (12, 9)]                   # portions of the two requests, step by step
    at = [0, 0]
    for a, b in cuts:
        entries = [StepEntry("r0", sequences[0][at[0]:at[0] + a], list(range(a))),
                   StepEntry("r1", sequences[1][at[1]:at[1] + b], list(range(b)))]
        logits = step.run(entries, auto_begin=True).cpu().numpy()
        assert np.abs(logits[:a] - want[0][at[0]:at[0] + a]).max() < 3e-4
        assert np.abs(logits[a:] - want[1][at[1]:at[1] + b]).max() < 3e-4
        at = [at[0] + a, at[1] + b]
    step.end("r0")
    # a new request in r0's slot starts from a cleared state
    logits = step.run([StepEntry("r2", sequences[0][:5], [4])], auto_begin=True).cpu().numpy()
    assert np.abs(logits[0] - want[0][4]).max() < 3e-4


def test_toy_routed_feed_forward_and_toy_position_encoding(tmp_path):
    """Two more parts from outside the package, put into a model description without a change to the
    framework's files: a feed-forward that routes every token to one of three small experts (router logits
    and the gate in float32), and a position encoding that rotates neighbouring pairs (2i, 2i+1) instead of
    halves, which has no tables for the fused q/k kernel and so goes through ``apply``. Run in portions and
    token by token through the engine's loader, cache and step function, against a plain computation."""
    from celeg_b200.config import (Architecture, Lfm2Config, PartSpec, TensorRef, build_lfm2_spec,
                                   register_architecture)
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.parts import register_part
    from celeg_b200.weights import write_random_model

    experts, inner = 3, 40

    @register_part("feed_forward", "toy_routed", replace=True)
    class ToyRouted:
        def __init__(self, params, weights, parts, rt):
            self.rt = rt
            self.router = rt.vector(weights["router"])                    # float32 [experts, hidden]
            self.up = [rt.matrix(weights[f"up{e}"]) for e in range(params["experts"])]
            self.down = [rt.matrix(weights[f"down{e}"]) for e in range(params["experts"])]
            self.hidden_act = rt.scratch("toy.routed.act", params["inner"])
            self.expert_out = rt.scratch("toy.routed.out", params["hidden_size"])

        def forward(self, x, out, step):
            t = step.tokens
            logits = x[:t].float() @ self.router.t()
            gate = torch.softmax(logits, dim=-1)
            chosen = logits.argmax(dim=-1)
            out[:t] = 0
            for e in range(len(self.up)):                                 # every expert over all rows, then masked:
                self.rt.linear(x, self.up[e], self.hidden_act, t)         # a toy part is free to be slow
                self.hidden_act[:t] = torch.relu(self.hidden_act[:t])
                self.rt.linear(self.hidden_act, self.down[e], self.expert_out, t)
                weight = torch.where(chosen == e, gate[:, e], torch.zeros_like(gate[:, e]))
                out[:t] += (self.expert_out[:t].float() * weight[:, None]).to(out.dtype)

    @register_part("position", "toy_rope_pairs", replace=True)
    class ToyPairRope:
        def __init__(self, params, rt):
            half = params["head_dim"] // 2
            self.inv_freq = (params["theta"] ** (-torch.arange(half, dtype=torch.float64) / half)).to(
                torch.float32).to(rt.device)

        def fused(self):
            return None                                                   # no tables: the mixer calls apply()

        def apply(self, q, k, positions, tokens):
            angle = positions[:tokens].float()[:, None] * self.inv_freq[None, :]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for view in (q, k):
                even, odd = view[..., 0::2].float().clone(), view[..., 1::2].float().clone()
                view[..., 0::2] = (even * cos - odd * sin).to(view.dtype)
                view[..., 1::2] = (odd * cos + even * sin).to(view.dtype)

    def toy_spec(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        hidden = config.hidden_size
        tensors = {"router": TensorRef("model.layers.0.toy_ff.router.weight", (experts, hidden))}
        for e in range(experts):
            tensors[f"up{e}"] = TensorRef(f"model.layers.0.toy_ff.experts.{e}.up.weight", (inner, hidden))
            tensors[f"down{e}"] = TensorRef(f"model.layers.0.toy_ff.experts.{e}.down.weight", (hidden, inner))
        layers[0] = dataclasses.replace(layers[0], feed_forward=PartSpec(
            kind="toy_routed", params={"hidden_size": hidden, "experts": experts, "inner": inner}, tensors=tensors))
        attention = layers[2].mixer
        position = PartSpec(kind="toy_rope_pairs", params={"theta": 300.0, "head_dim": config.head_dim})
        layers[2] = dataclasses.replace(layers[2], mixer=dataclasses.replace(attention, parts={"position": position}))
        return dataclasses.replace(spec, layers=tuple(layers), architecture="toy_routed_lfm2")

    register_architecture(Architecture(
        name="toy_routed_lfm2", parse_config=Lfm2Config.from_dict,
        resolve_config=lambda config, shapes: dataclasses.replace(
            config, tie_word_embeddings=True if config.tie_word_embeddings is None else config.tie_word_embeddings),
        build_spec=toy_spec, random_init=lfm2_random_init), replace=True)

    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "toy_routed_lfm2"
    folder = write_random_model(str(tmp_path / "toy_routed"), raw, 9, torch.float32)
    loaded = load_model(folder, dtype="float32", max_requests=2, cache_tokens=128, max_batched_tokens=64)
    config, weights = plain_lfm2.load_model_folder(folder)
    head_dim = config["hidden_size"] // config["num_attention_heads"]

    def pair_rope(x, positions):
        half = head_dim // 2
        inv_freq = (300.0 ** (-np.arange(half) / half)).astype(np.float32).astype(np.float64)
        angle = positions[:, None] * inv_freq[None, :]
        cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
        out = np.empty_like(x)
        out[..., 0::2] = x[..., 0::2] * cos - x[..., 1::2] * sin
        out[..., 1::2] = x[..., 1::2] * cos + x[..., 0::2] * sin
        return out

    def plain_forward(tokens):
        count = len(tokens)
        x = weights["model.embed_tokens.weight"][np.asarray(tokens)]
        for index, kind in enumerate(config["layer_types"]):
            p = f"model.layers.{index}."
            if index == 0:
                n = plain_lfm2.rmsnorm(x, weights[p + "operator_norm.weight"], config["norm_eps"])
                h = x + plain_lfm2.short_conv_mixer(n, weights[p + "conv.in_proj.weight"], weights[p + "conv.conv.weight"],
                                                    weights[p + "conv.out_proj.weight"])
                n2 = plain_lfm2.rmsnorm(h, weights[p + "ffn_norm.weight"], config["norm_eps"])
                logits = n2 @ weights[p + "toy_ff.router.weight"].T
                gate = np.exp(logits - logits.max(axis=-1, keepdims=True))
                gate /= gate.sum(axis=-1, keepdims=True)
                routed = np.zeros_like(h)
                for t in range(count):
                    e = int(logits[t].argmax())
                    act = np.maximum(n2[t] @ weights[p + f"toy_ff.experts.{e}.up.weight"].T, 0.0)
                    routed[t] = gate[t, e] * (act @ weights[p + f"toy_ff.experts.{e}.down.weight"].T)
                x = h + routed
            elif index == 2:
                heads, kv_heads = config["num_attention_heads"], config["num_key_value_heads"]
                n = plain_lfm2.rmsnorm(x, weights[p + "operator_norm.weight"], config["norm_eps"])
                q = (n @ weights[p + "self_attn.q_proj.weight"].T).reshape(count, heads, head_dim)
                k = (n @ weights[p + "self_attn.k_proj.weight"].T).reshape(count, kv_heads, head_dim)
                v = (n @ weights[p + "self_attn.v_proj.weight"].T).reshape(count, kv_heads, head_dim)
                positions = np.arange(count, dtype=np.float64)
                q = pair_rope(plain_lfm2.rmsnorm(q, weights[p + "self_attn.q_layernorm.weight"], config["norm_eps"]), positions)
                k = pair_rope(plain_lfm2.rmsnorm(k, weights[p + "self_attn.k_layernorm.weight"], config["norm_eps"]), positions)
                mixed = np.zeros((count, heads, head_dim))
                for head in range(heads):
                    kv = head // (heads // kv_heads)
                    scores = (q[:, head] @ k[:, kv].T) / np.sqrt(head_dim)
                    scores = np.where(np.arange(count)[None, :] > np.arange(count)[:, None], -np.inf, scores)
                    scores = np.exp(scores - scores.max(axis=-1, keepdims=True))
                    mixed[:, head] = (scores / scores.sum(axis=-1, keepdims=True)) @ v[:, kv]
                h = x + mixed.reshape(count, -1) @ weights[p + "self_attn.out_proj.weight"].T
                n2 = plain_lfm2.rmsnorm(h, weights[p + "ffn_norm.weight"], config["norm_eps"])
                x = h + plain_lfm2.swiglu(n2, weights[p + "feed_forward.w1.weight"], weights[p + "feed_forward.w3.weight"],
                                          weights[p + "feed_forward.w2.weight"])
            else:
                x = plain_lfm2.block(x, index, kind, config, weights)
        z = plain_lfm2.rmsnorm(x, weights["model.embedding_norm.weight"], config["norm_eps"])
        return z @ weights["model.embed_tokens.weight"].T

    (sequence,) = prompts_of(config["vocab_size"], [34], seed=33)
    want = plain_forward(sequence)
    step = loaded.step
    at = 0
    for size in (9, 2, 12, 1, 1, 7, 1, 1):
        logits = step.run([StepEntry("toy", sequence[at:at + size], list(range(size)))], auto_begin=True).cpu().numpy()
        worst = np.abs(logits - want[at:at + size]).max(axis=1)
        assert worst.max() < 3e-4, f"tokens {at}..{at + size}: {np.round(worst, 5).tolist()}"
        at += size
    assert at == len(sequence)
    step.raise_on_device_error()


def test_cli_generates_and_dumps_logits(models, tmp_path, capsys):
    from celeg_b200.cli import main
    folder, config, weights = models["A"]
    prompt = prompts_of(config["vocab_size"], [12], seed=32)[0]
    dump = str(tmp_path / "last.f32")
    code = main(["--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6",
                 "--dtype", "fp32", "--temperature", "0", "--repetition-penalty", "1.0", "--runtime-tokens",
                 "--dump-logits", dump, "--runtime-metrics", "--context", "128"])
    assert code == 0
    captured = capsys.readouterr()
    want = [t for t in plain_lfm2.generate(config, weights, prompt, 6, eos_tokens=(7,))]
    assert f"CELEG_GENERATED_TOKEN_IDS=[{','.join(map(str, want))}]" in captured.out
    assert "runtime.decode_tokens_per_second=" in captured.err
    logits = np.fromfile(dump, dtype="<f4")
    assert np.abs(logits - plain_lfm2.forward(config, weights, prompt)[-1]).max() < 2e-4
    assert main(["--model", folder, "--prompt", "hello"]) == 1
    assert "error:" in capsys.readouterr().err


def test_many_requests_through_a_small_pool(models):
    """Thirty requests of random lengths through four slots and a pool that holds about two of them
    (MAX_UTILIZATION): admission waits, pages and slots are reused, requests that find no page are
    skipped or preempted and prefilled again; every request still produces exactly the tokens it
    produces alone (float32, greedy)."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams, SchedulerPolicy
    folder, config, weights = models["A"]
    rng = np.random.default_rng(40)
    lengths = rng.integers(1, 60, size=30).tolist()
    prompts = prompts_of(config["vocab_size"], lengths, seed=41)
    new_tokens = rng.integers(1, 24, size=30).tolist()
    options = EngineOptions(max_active_requests=4, max_batched_tokens=32, prefill_chunk_tokens=13, page_tokens=16,
                            logical_kv_pages=9, scheduler_policy=SchedulerPolicy.MAX_UTILIZATION)
    engine = Engine(folder, dtype="float32", options=options)
    greedy = SamplingParams(temperature=0.0, top_k=1, repetition_penalty=1.0)
    ids = [engine.submit(p, RequestOptions(max_new_tokens=n, eos_tokens=(), generation=greedy))
           for p, n in zip(prompts, new_tokens)]
    outputs = {i: [] for i in ids}
    pending = set(ids)
    steps = 0
    while pending:
        assert engine.step() or not engine.scheduler.has_work()
        engine.loaded.manager.check_invariants()
        for i in list(pending):
            result = engine.poll(i)
            outputs[i].extend(result.tokens)
            if result.finished:
                assert result.status.value == "finished", result.error
                pending.discard(i)
        steps += 1
        assert steps < 3000
    metrics = engine.metrics()
    assert metrics.completed == 30 and metrics.failed == 0
    assert metrics.max_step_requests > 1
    assert engine.loaded.manager.free_slots == 4
    assert all(g.pool.free_pages == g.pool.total_pages for g in engine.loaded.manager.groups)
    alone = Engine(folder, dtype="float32")
    for request_id, prompt, n in list(zip(ids, prompts, new_tokens))[::3]:
        want = alone.generate(prompt, max_new_tokens=n, temperature=0.0, repetition_penalty=1.0, eos_tokens=())
        assert outputs[request_id] == want, request_id
    for request_id, prompt, n in list(zip(ids, prompts, new_tokens))[1::7]:
        assert outputs[request_id] == plain_lfm2.generate(config, weights, prompt, n, eos_tokens=()), request_id
    for request_id, n in zip(ids, new_tokens):
        assert len(outputs[request_id]) == n


def test_seeded_sampling_survives_preemption(models):
    """Temperature 0.8 with a seed per request through a pool so small that requests are preempted (pages and
    slot given back, generator state kept, prompt + generated tokens prefilled again): every request still draws
    exactly what it draws alone and what the plain sampler draws from the plain model's logits (float32)."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams, SchedulerPolicy
    folder, config, weights = models["B"]
    rng = np.random.default_rng(42)
    # every request is admitted with three pages and needs five before it ends; the pool holds eight, so two
    # live requests grow to four pages each and then neither can take its fifth
    lengths = rng.integers(18, 31, size=10).tolist()
    prompts = prompts_of(config["vocab_size"], lengths, seed=43)
    new_tokens = rng.integers(45, 61, size=10).tolist()
    options = EngineOptions(max_active_requests=4, max_batched_tokens=32, prefill_chunk_tokens=11, page_tokens=16,
                            logical_kv_pages=8, scheduler_policy=SchedulerPolicy.MAX_UTILIZATION)
    engine = Engine(folder, dtype="float32", options=options)

    def params(i):
        return SamplingParams(temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1, seed=100 + i)

    ids = [engine.submit(p, RequestOptions(max_new_tokens=n, eos_tokens=(), generation=params(i)))
           for i, (p, n) in enumerate(zip(prompts, new_tokens))]
    outputs = {i: [] for i in ids}
    pending = set(ids)
    steps = 0
    while pending:
        engine.step()
        engine.loaded.manager.check_invariants()
        for i in list(pending):
            result = engine.poll(i)
            outputs[i].extend(result.tokens)
            if result.finished:
                assert result.status.value == "finished", result.error
                pending.discard(i)
        steps += 1
        assert steps < 6000
    assert engine.metrics().preempted > 0, "the pool was meant to be too small for four live requests"
    alone = Engine(folder, dtype="float32")
    for index, (request_id, prompt, n) in enumerate(zip(ids, prompts, new_tokens)):
        kwargs = dict(max_new_tokens=n, temperature=0.8, top_k=40, top_p=0.95, repetition_penalty=1.1,
                      seed=100 + index, eos_tokens=())
        assert outputs[request_id] == alone.generate(prompt, **kwargs), f"request {index} against itself alone"
        if index % 3 == 0:
            want = plain_lfm2.generate(config, weights, prompt, n, temperature=0.8, top_k=40, top_p=0.95,
                                       repetition_penalty=1.1, seed=100 + index)
            assert outputs[request_id] == want, f"request {index} against the plain model"


def test_worker_thread_serves_requests_submitted_from_other_threads(models):
    """``Engine.start()`` runs the steps on a worker thread (celeg: src/runtime/concurrency/worker.cpp:48-67);
    three client threads submit and poll meanwhile; ``stop()`` joins it. Outputs equal the plain model's."""
    import threading
    import time
    from celeg_b200 import Engine, EngineOptions
    folder, config, weights = models["A"]
    prompts = prompts_of(config["vocab_size"], [5, 9, 14, 22, 31, 40], seed=44)
    engine = Engine(folder, dtype="float32", options=EngineOptions(max_active_requests=4, max_batched_tokens=48,
                                                                   prefill_chunk_tokens=16))
    engine.start()
    assert engine.running()
    engine.start()                                   # a second start changes nothing
    results, errors = {}, []

    def client(indices):
        try:
            mine = {i: engine.submit(prompts[i], max_new_tokens=10, temperature=0.0, repetition_penalty=1.0,
                                     eos_tokens=()) for i in indices}
            got = {i: [] for i in indices}
            deadline = time.monotonic() + 120
            while mine and time.monotonic() < deadline:
                for i, request_id in list(mine.items()):
                    result = engine.poll(request_id)
                    got[i].extend(result.tokens)
                    if result.finished:
                        assert result.status.value == "finished", result.error
                        engine.release(request_id)
                        del mine[i]
                time.sleep(0.001)
            assert not mine, "requests were not served in time"
            results.update(got)
        except Exception as exc:                     # reported by the main thread
            errors.append(exc)

    threads = [threading.Thread(target=client, args=(indices,)) for indices in ([0, 3], [1, 4], [2, 5])]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join(timeout=180)
    engine.stop()
    assert not engine.running()
    engine.stop()                                    # a second stop changes nothing
    assert not errors, errors
    for i, prompt in enumerate(prompts):
        assert results[i] == plain_lfm2.generate(config, weights, prompt, 10, eos_tokens=()), i
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == 4
    # the engine still steps by hand after the worker has gone
    assert engine.generate(prompts[0], max_new_tokens=4, temperature=0.0, repetition_penalty=1.0,
                           eos_tokens=()) == results[0][:4]


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_bfloat16_path_agrees_with_float32_path(tmp_path, name):
    """The serving path against the true 32-bit path of the same engine on whole prompts of 150 tokens: the
    same token has the highest logit at 95 % of the positions or more, every row's error is at most 3 % of the
    row's norm, and greedy continuations agree until a first difference at a position where the 32-bit path
    itself saw a near tie."""
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, name)
    config = CONFIGS[name][0]
    prompts = prompts_of(config["vocab_size"], [150, 150, 150], seed=45)
    rows = {}
    for dtype in ("float32", "bfloat16"):
        loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=512, max_batched_tokens=160)
        out = []
        for i, prompt in enumerate(prompts):
            logits = loaded.step.run([StepEntry(f"p{i}", prompt, list(range(len(prompt))))], auto_begin=True)
            out.append(logits.float().cpu().numpy().copy())
            loaded.step.end(f"p{i}")
        loaded.step.raise_on_device_error()
        rows[dtype] = np.concatenate(out)
    exact, served = rows["float32"], rows["bfloat16"]
    agreement = float((exact.argmax(axis=1) == served.argmax(axis=1)).mean())
    assert agreement >= 0.95, f"top-1 agreement {agreement:.3f}"
    relative = np.linalg.norm(served - exact, axis=1) / np.linalg.norm(exact, axis=1)
    assert float(relative.max()) <= 0.03, f"largest relative row error {relative.max():.4f}"
    # where the top token differs, the 32-bit path's own margin between the two candidates is small
    for row in np.nonzero(exact.argmax(axis=1) != served.argmax(axis=1))[0]:
        margin = exact[row].max() - exact[row, served[row].argmax()]
        assert margin <= 0.02 * np.linalg.norm(exact[row]) / np.sqrt(exact.shape[1]) * 10, (row, margin)


def test_run_order_names_a_layer_twice_and_shares_a_cache(tmp_path):
    """The order in which layers run is data. Here tiny A runs as 0, 1, 2, 3, 1, 2': the conv layer 1 a
    second time with a state of its own, and the attention layer 2 a second time reading the keys and
    values its first run wrote (it computes only queries there). Checked against a plain computation,
    whole and in portions."""
    from celeg_b200.config import (Architecture, ExecutionEntry, Lfm2Config, build_lfm2_spec, register_architecture)
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.weights import write_random_model

    def spec_with_order(config):
        spec = build_lfm2_spec(config)
        order = tuple(ExecutionEntry(i) for i in range(4)) + (ExecutionEntry(1), ExecutionEntry(2, cache_of=2))
        return dataclasses.replace(spec, order=order, architecture="lfm2_twice")

    register_architecture(Architecture(name="lfm2_twice", parse_config=Lfm2Config.from_dict,
                                       resolve_config=lambda c, shapes: c.resolved_with(shapes),
                                       build_spec=spec_with_order, random_init=lfm2_random_init), replace=True)
    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "lfm2_twice"
    folder = write_random_model(str(tmp_path / "twice"), raw, 6)
    loaded = load_model(folder, dtype="float32", max_requests=2, cache_tokens=128, max_batched_tokens=64)
    assert len(loaded.model.state_layout.offsets) == 4            # conv layers 0, 1, 3 and the second run of 1
    assert [len(m) for m in loaded.model.group_members] == [1]    # one attention cache, shared by both runs

    config, w = plain_lfm2.load_model_folder(folder)
    eps, d, heads, kv_heads = config["norm_eps"], 16, 4, 2

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        for index, kind in enumerate(config["layer_types"]):
            if index == 2:
                before_attention = x
            x = plain_lfm2.block(x, index, kind, config, w)
        x = plain_lfm2.block(x, 1, "conv", config, w)             # layer 1 again, from an empty state
        # layer 2 again: queries from the current stream, keys and values from its first run
        p = "model.layers.2."
        positions = np.arange(len(tokens))
        n_first = plain_lfm2.rmsnorm(before_attention, w[p + "operator_norm.weight"], eps)
        k = (n_first @ w[p + "self_attn.k_proj.weight"].T).reshape(-1, kv_heads, d)
        v = (n_first @ w[p + "self_attn.v_proj.weight"].T).reshape(-1, kv_heads, d)
        k = plain_lfm2.rope_split_half(plain_lfm2.rmsnorm(k, w[p + "self_attn.k_layernorm.weight"], eps), positions,
                                       config["rope_theta"])
        n_now = plain_lfm2.rmsnorm(x, w[p + "operator_norm.weight"], eps)
        q = (n_now @ w[p + "self_attn.q_proj.weight"].T).reshape(-1, heads, d)
        q = plain_lfm2.rope_split_half(plain_lfm2.rmsnorm(q, w[p + "self_attn.q_layernorm.weight"], eps), positions,
                                       config["rope_theta"])
        attended = np.zeros((len(tokens), heads, d))
        for h in range(heads):
            scores = (q[:, h] @ k[:, h // 2].T) / np.sqrt(d)
            scores = np.where(np.arange(len(tokens))[None, :] > positions[:, None], -np.inf, scores)
            weights_ = np.exp(scores - scores.max(axis=-1, keepdims=True))
            weights_ /= weights_.sum(axis=-1, keepdims=True)
            attended[:, h] = weights_ @ v[:, h // 2]
        hidden = x + attended.reshape(len(tokens), -1) @ w[p + "self_attn.out_proj.weight"].T
        n2 = plain_lfm2.rmsnorm(hidden, w[p + "ffn_norm.weight"], eps)
        x = hidden + plain_lfm2.swiglu(n2, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                                       w[p + "feed_forward.w2.weight"])
        z = plain_lfm2.rmsnorm(x, w["model.embedding_norm.weight"], eps)
        return z @ w["model.embed_tokens.weight"].T

    (sequence,) = prompts_of(config["vocab_size"], [37], seed=42)
    want = plain_forward(sequence)
    step = loaded.step
    whole = step.run([StepEntry("whole", sequence, list(range(37)))], auto_begin=True).cpu().numpy()
    assert np.abs(whole - want).max() < 3e-4
    step.end("whole")
    at = 0
    for n in (5, 2, 17, 1, 1, 11):
        got = step.run([StepEntry("cut", sequence[at:at + n], list(range(n)))], auto_begin=True).cpu().numpy()
        assert np.abs(got - want[at:at + n]).max() < 3e-4, at
        at += n


@pytest.mark.parametrize("name,dtype,tol", [("B", "float32", 4e-4), ("D", "float32", 4e-4), ("D", "bfloat16", 8e-2)])
def test_a_layer_with_a_window_has_pages_of_its_own_and_gives_them_back(tmp_path, name, dtype, tol):
    """One attention layer of the model sees the last 24 keys only. Its pages form a group of their own beside
    the layers that see all keys; pages the window has passed go back to the pool and are used again (the
    group's pool is far smaller than the sequence). A long and a short request, in portions and token by
    token, against the plain implementation with the same window."""
    from celeg_b200.config import Architecture, Lfm2Config, build_lfm2_spec, register_architecture
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.weights import write_random_model

    window = 24
    raw, seed = copy.deepcopy(CONFIGS[name][0]), CONFIGS[name][1]
    kinds = raw["layer_types"]
    windowed = max(i for i, kind in enumerate(kinds) if kind == "full_attention")

    def spec_with_window(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        mixer = layers[windowed].mixer
        layers[windowed] = dataclasses.replace(layers[windowed], mixer=dataclasses.replace(
            mixer, params={**mixer.params, "window": window}))
        return dataclasses.replace(spec, layers=tuple(layers), architecture="lfm2_windowed")

    register_architecture(Architecture(name="lfm2_windowed", parse_config=Lfm2Config.from_dict,
                                       resolve_config=lambda c, shapes: c.resolved_with(shapes),
                                       build_spec=spec_with_window, random_init=lfm2_random_init), replace=True)
    raw["model_type"] = "lfm2_windowed"
    folder = write_random_model(str(tmp_path / "windowed"), raw, seed, torch.bfloat16)
    loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=208, page_tokens=8, max_batched_tokens=64,
                        use_graphs=True)
    groups = loaded.model.group_members
    assert sorted(len(m) for m in groups) == sorted([1, sum(k == "full_attention" for k in kinds) - 1])
    config, w = plain_lfm2.load_model_folder(folder)
    heads, kv_heads = config["num_attention_heads"], config["num_key_value_heads"]
    head_dim = config.get("head_dim") or config["hidden_size"] // heads
    eps = config["norm_eps"]

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        for index, kind in enumerate(kinds):
            if index != windowed:
                x = plain_lfm2.block(x, index, kind, config, w)
                continue
            p = f"model.layers.{index}."
            n = plain_lfm2.rmsnorm(x, w[p + "operator_norm.weight"], eps)
            h = x + plain_lfm2.attention_mixer(
                n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"],
                w[p + "self_attn.out_proj.weight"], w[p + "self_attn.q_layernorm.weight"],
                w[p + "self_attn.k_layernorm.weight"], heads, kv_heads, head_dim, config["rope_theta"], eps,
                window=window)
            n2 = plain_lfm2.rmsnorm(h, w[p + "ffn_norm.weight"], eps)
            x = h + plain_lfm2.swiglu(n2, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                                      w[p + "feed_forward.w2.weight"])
        z = plain_lfm2.rmsnorm(x, w["model.embedding_norm.weight"], eps)
        head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
        return z @ head.T

    long_seq, short_seq = prompts_of(config["vocab_size"], [170, 30], seed=44)
    want = {"long": plain_forward(long_seq), "short": plain_forward(short_seq)}
    seqs = {"long": long_seq, "short": short_seq}
    step = loaded.step
    heads_at = {"long": 0, "short": 0}

    def run(portions):
        entries = [StepEntry(n, seqs[n][heads_at[n]:heads_at[n] + size], list(range(size))) for n, size in portions]
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        row = 0
        for n, size in portions:
            ref = want[n][heads_at[n]:heads_at[n] + size]
            worst = np.abs(logits[row:row + size] - ref).max()
            assert worst < tol, f"request {n}, tokens {heads_at[n]}..{heads_at[n] + size}: {worst:.3e}"
            row += size
            heads_at[n] += size

    run([("long", 40)])
    run([("long", 33), ("short", 9)])
    run([("long", 2), ("short", 21)])
    for _ in range(60):                          # decoded one by one; the short request ends on the way
        portions = [("long", 1)]
        if heads_at["short"] < len(short_seq):
            portions.append(("short", 1))
        run(portions)
        if heads_at["short"] == len(short_seq) and "short" in loaded.manager.live_requests():
            step.end("short")
    run([("long", 35)])
    assert heads_at["long"] == 170
    step.raise_on_device_error()
    loaded.manager.check_invariants()
    # the windowed group holds only what the window still needs: far fewer pages than the 170 tokens
    held = [len(loaded.manager.get("long").held_pages(g)) for g in range(len(groups))]
    assert min(held) <= (window + 8 - 1) // 8 + 2 and max(held) >= 170 // 8, held


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-4), ("bfloat16", 8e-2)])
def test_toy_block_with_post_norms_and_two_mixers(tmp_path, dtype, tol):
    """A block that the four named parts do not cover, described with a layer's ``extra_parts`` and run by an
    arrangement defined here: a sandwich (a norm AFTER the mixer and after the feed-forward, as some
    architectures have) whose mixer stage is an attention and a short convolution side by side:

        a = PostNorm1(Attention(N1(x)) + ShortConv(N1(x)));  h = x + a;  y = h + PostNorm2(FeedForward(N2(h)))

    Both mixers hold a cache (pages for one, a state slot for the other) at the same position of the run
    order. Nothing of the package changes; prompts in portions and decoded tokens against a plain computation."""
    from celeg_b200.config import Architecture, Lfm2Config, PartSpec, TensorRef, build_lfm2_spec, register_architecture
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.parts import register_part
    from celeg_b200.weights import write_random_model

    @register_part("arrangement", "toy_sandwich_two_mixers", replace=True)
    class ToySandwich:
        def __init__(self, layer_parts, rt):
            self.parts = layer_parts
            hidden = layer_parts["mixer_norm"].width
            self.normed = rt.scratch("toy.sandwich.normed", hidden)
            self.out_a = rt.scratch("toy.sandwich.out_a", hidden)
            self.out_b = rt.scratch("toy.sandwich.out_b", hidden)
            self.post = rt.scratch("toy.sandwich.post", hidden)
            self.zero = torch.zeros_like(rt.scratch("toy.sandwich.zero", hidden, torch.float32))

        def _post_norm(self, norm, value, t):
            """norm(value) with the norm kernels' interface: a float32 'residual' of zeros plus the value."""
            self.zero[:t].zero_()
            norm.add_norm(self.zero, value, self.post, t)
            return self.post

        def run(self, stream, step):
            t = step.tokens
            x = stream.normed(self.parts["mixer_norm"], self.normed, t)
            stream.expect(self.out_a, None, t)
            self.parts["mixer"].forward(x, self.out_a, step)
            self.parts["second_mixer"].forward(x, self.out_b, step)
            self.out_a[:t] = (self.out_a[:t].float() + self.out_b[:t].float()).to(self.out_a.dtype)
            stream.add_later(self._post_norm(self.parts["post_mixer_norm"], self.out_a, t))
            x = stream.normed(self.parts["feed_forward_norm"], self.normed, t)
            stream.expect(self.out_a, None, t)
            self.parts["feed_forward"].forward(x, self.out_a, step)
            self.out_b[:t] = self._post_norm(self.parts["post_feed_forward_norm"], self.out_a, t)[:t]
            stream.add_later(self.out_b)

    def toy_spec(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        hidden = config.hidden_size

        def rms(name):
            return PartSpec(kind="rmsnorm", category="norm", params={"width": hidden, "eps": config.norm_eps},
                            tensors={"weight": TensorRef(name, (hidden,))})

        # layer 2 of tiny A is the attention layer: give it layer 1's kind of mixer as a second one
        base = "model.layers.2"
        second = PartSpec(kind="short_conv", category="mixer", params={"hidden_size": hidden, "taps": config.conv_L_cache},
                          tensors={"in_proj": TensorRef(f"{base}.toy_conv.in_proj.weight", (3 * hidden, hidden)),
                                   "conv": TensorRef(f"{base}.toy_conv.conv.weight", (hidden, config.conv_L_cache)),
                                   "out_proj": TensorRef(f"{base}.toy_conv.out_proj.weight", (hidden, hidden))})
        layers[2] = dataclasses.replace(
            layers[2], arrangement="toy_sandwich_two_mixers",
            extra_parts={"second_mixer": second, "post_mixer_norm": rms(f"{base}.toy_post_mixer_norm.weight"),
                         "post_feed_forward_norm": rms(f"{base}.toy_post_ffn_norm.weight")})
        return dataclasses.replace(spec, layers=tuple(layers), architecture="toy_sandwich_lfm2")

    def init(config, name, shape):
        if name.endswith("toy_conv.conv.weight"):
            return "conv"
        return lfm2_random_init(config, name, shape)

    register_architecture(Architecture(
        name="toy_sandwich_lfm2", parse_config=Lfm2Config.from_dict,
        resolve_config=lambda config, shapes: dataclasses.replace(
            config, tie_word_embeddings=True if config.tie_word_embeddings is None else config.tie_word_embeddings),
        build_spec=toy_spec, random_init=init), replace=True)
    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "toy_sandwich_lfm2"
    folder = write_random_model(str(tmp_path / "toy_sandwich"), raw, 12, torch.bfloat16)
    loaded = load_model(folder, dtype=dtype, max_requests=3, cache_tokens=192, max_batched_tokens=64, use_graphs=True)
    # two caches at position 2: pages for the attention, a state place for the second mixer
    assert set(loaded.model.bindings[2]) == {"mixer", "second_mixer"}
    assert (2, "second_mixer") in loaded.model.state_layout.offsets
    config, w = plain_lfm2.load_model_folder(folder)
    eps = config["norm_eps"]
    heads, kv_heads, head_dim = config["num_attention_heads"], config["num_key_value_heads"], plain_lfm2.head_dim(config)

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        for index, kind in enumerate(plain_lfm2.layer_kinds(config, w)):
            if index != 2:
                x = plain_lfm2.block(x, index, kind, config, w)
                continue
            p = "model.layers.2."
            n = plain_lfm2.rmsnorm(x, w[p + "operator_norm.weight"], eps)
            attended = plain_lfm2.attention_mixer(
                n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"],
                w[p + "self_attn.out_proj.weight"], w[p + "self_attn.q_layernorm.weight"],
                w[p + "self_attn.k_layernorm.weight"], heads, kv_heads, head_dim, config["rope_theta"], eps)
            convolved = plain_lfm2.short_conv_mixer(n, w[p + "toy_conv.in_proj.weight"], w[p + "toy_conv.conv.weight"],
                                                    w[p + "toy_conv.out_proj.weight"])
            h = x + plain_lfm2.rmsnorm(attended + convolved, w[p + "toy_post_mixer_norm.weight"], eps)
            n2 = plain_lfm2.rmsnorm(h, w[p + "ffn_norm.weight"], eps)
            f = plain_lfm2.swiglu(n2, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                                  w[p + "feed_forward.w2.weight"])
            x = h + plain_lfm2.rmsnorm(f, w[p + "toy_post_ffn_norm.weight"], eps)
        z = plain_lfm2.rmsnorm(x, w["model.embedding_norm.weight"], eps)
        return z @ w["model.embed_tokens.weight"].T

    first, second = prompts_of(config["vocab_size"], [60, 25], seed=46)
    want = {"first": plain_forward(first), "second": plain_forward(second)}
    seqs = {"first": first, "second": second}
    at = {"first": 0, "second": 0}
    step = loaded.step

    def run(portions):
        entries = [StepEntry(n, seqs[n][at[n]:at[n] + size], list(range(size))) for n, size in portions]
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        row = 0
        for n, size in portions:
            worst = np.abs(logits[row:row + size] - want[n][at[n]:at[n] + size]).max()
            assert worst < tol, f"request {n}, tokens {at[n]}..{at[n] + size}: {worst:.3e}"
            row += size
            at[n] += size

    run([("first", 33)])
    run([("first", 2), ("second", 17)])
    for _ in range(8):                              # decoded one by one, both together (a graph from the second step on)
        run([("first", 1), ("second", 1)])
    step.end("second")
    run([("first", 17)])
    assert at["first"] == 60
    step.raise_on_device_error()
    loaded.manager.check_invariants()


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-4), ("bfloat16", 8e-2)])
def test_toy_norm_and_toy_arrangement(tmp_path, dtype, tol):
    """A norm that is no RMSNorm (mean-centred, with a bias) and a block arrangement that is not pre-norm
    residual (mixer and feed-forward side by side: y = x + Mixer(N1(x)) + FeedForward(N2(x))), both defined
    here and registered. The norm cannot be split over the products around it and the arrangement names no
    first norm, so on the bfloat16 path their neighbours fall back to the unsplit form; decoded tokens (few
    rows) and prompt portions, against a plain computation."""
    from celeg_b200.config import Architecture, Lfm2Config, PartSpec, TensorRef, build_lfm2_spec, register_architecture
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.parts import register_part
    from celeg_b200.weights import write_random_model

    toy_eps = 1e-4

    @register_part("norm", "toy_centred", replace=True)
    class ToyCentredNorm:
        def __init__(self, params, weights, rt):
            self.width = int(params["width"])
            self.weight = rt.vector(weights["weight"])
            self.bias = rt.vector(weights["bias"])

        def add_norm(self, residual, delta, out, n_rows, rows=None):
            if rows is None:
                if delta is not None:
                    residual[:n_rows] += delta[:n_rows].float()
                x = residual[:n_rows]
            else:
                index = rows[:n_rows].long()
                x = residual[index] + (delta[index].float() if delta is not None else 0.0)
            x = x - x.mean(dim=-1, keepdim=True)
            y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + toy_eps) * self.weight + self.bias
            out[:n_rows] = y.to(out.dtype)

    @register_part("arrangement", "toy_side_by_side", replace=True)
    class ToySideBySide:
        def __init__(self, layer_parts, rt):
            self.parts = layer_parts
            hidden = layer_parts["mixer_norm"].width
            self.normed_a = rt.scratch("toy.side.normed_a", hidden)
            self.normed_b = rt.scratch("toy.side.normed_b", hidden)
            self.delta_a = rt.scratch("toy.side.delta_a", hidden)
            self.delta_b = rt.scratch("toy.side.delta_b", hidden)

        def run(self, stream, step):
            t = step.tokens
            xa = stream.normed(self.parts["mixer_norm"], self.normed_a, t)     # adds what was pending
            xb = stream.normed(self.parts["feed_forward_norm"], self.normed_b, t)
            stream.expect(self.delta_a, None, t)
            self.parts["mixer"].forward(xa, self.delta_a, step)
            self.parts["feed_forward"].forward(xb, self.delta_b, step)
            self.delta_a[:t] = (self.delta_a[:t].float() + self.delta_b[:t].float()).to(self.delta_a.dtype)
            stream.add_later(self.delta_a)

    def toy_spec(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        hidden = config.hidden_size

        def centred(name):
            return PartSpec(kind="toy_centred", params={"width": hidden},
                            tensors={"weight": TensorRef(name + ".weight", (hidden,)),
                                     "bias": TensorRef(name + ".bias", (hidden,))})

        layers[1] = dataclasses.replace(layers[1], mixer_norm=centred("model.layers.1.toy_norm"))
        layers[2] = dataclasses.replace(layers[2], feed_forward_norm=centred("model.layers.2.toy_ffn_norm"))
        layers[3] = dataclasses.replace(layers[3], arrangement="toy_side_by_side")
        return dataclasses.replace(spec, layers=tuple(layers), final_norm=centred("model.toy_final_norm"),
                                   architecture="toy_norms_lfm2")

    def init(config, name, shape):
        if name.endswith(".bias"):
            return "linear"
        return "norm" if "toy_" in name and name.endswith(".weight") else lfm2_random_init(config, name, shape)

    register_architecture(Architecture(
        name="toy_norms_lfm2", parse_config=Lfm2Config.from_dict,
        resolve_config=lambda config, shapes: dataclasses.replace(
            config, tie_word_embeddings=True if config.tie_word_embeddings is None else config.tie_word_embeddings),
        build_spec=toy_spec, random_init=init), replace=True)
    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "toy_norms_lfm2"
    folder = write_random_model(str(tmp_path / "toy_norms"), raw, 11, torch.bfloat16)
    loaded = load_model(folder, dtype=dtype, max_requests=3, cache_tokens=192, max_batched_tokens=64, use_graphs=True)
    config, w = plain_lfm2.load_model_folder(folder)
    eps = config["norm_eps"]

    def centred_norm(x, name):
        x = x - x.mean(axis=-1, keepdims=True)
        return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + toy_eps) * w[name + ".weight"] + w[name + ".bias"]

    def conv_of(index, n):
        p = f"model.layers.{index}."
        return plain_lfm2.short_conv_mixer(n, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"], w[p + "conv.out_proj.weight"])

    def ffn_of(index, n):
        p = f"model.layers.{index}."
        return plain_lfm2.swiglu(n, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"], w[p + "feed_forward.w2.weight"])

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        x = plain_lfm2.block(x, 0, "conv", config, w)
        h = x + conv_of(1, centred_norm(x, "model.layers.1.toy_norm"))
        x = h + ffn_of(1, plain_lfm2.rmsnorm(h, w["model.layers.1.ffn_norm.weight"], eps))
        p = "model.layers.2."
        n = plain_lfm2.rmsnorm(x, w[p + "operator_norm.weight"], eps)
        h = x + plain_lfm2.attention_mixer(
            n, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"], w[p + "self_attn.v_proj.weight"],
            w[p + "self_attn.out_proj.weight"], w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
            config["num_attention_heads"], config["num_key_value_heads"], 16, config["rope_theta"], eps)
        x = h + ffn_of(2, centred_norm(h, "model.layers.2.toy_ffn_norm"))
        x = (x + conv_of(3, plain_lfm2.rmsnorm(x, w["model.layers.3.operator_norm.weight"], eps))
             + ffn_of(3, plain_lfm2.rmsnorm(x, w["model.layers.3.ffn_norm.weight"], eps)))
        return centred_norm(x, "model.toy_final_norm") @ w["model.embed_tokens.weight"].T

    sequences = prompts_of(config["vocab_size"], [40, 33, 26], seed=45)
    want = [plain_forward(s) for s in sequences]
    step = loaded.step
    at = [0, 0, 0]

    def run(sizes):
        entries, rows = [], []
        for i, size in enumerate(sizes):
            if size:
                entries.append(StepEntry(f"r{i}", sequences[i][at[i]:at[i] + size], list(range(size))))
                rows.append((i, size))
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        row = 0
        for i, size in rows:
            worst = np.abs(logits[row:row + size] - want[i][at[i]:at[i] + size]).max()
            assert worst < tol, f"request {i}, tokens {at[i]}..{at[i] + size}: {worst:.3e}"
            row += size
            at[i] += size

    run([12, 0, 5])
    run([3, 20, 1])
    for _ in range(10):                 # three rows a step: the small-batch path, captured in a graph
        run([1, 1, 1])
    run([15, 3, 10])
    step.raise_on_device_error()


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-4), ("bfloat16", 8e-2)])
def test_scale_factors_of_a_model_description(tmp_path, dtype, tol):
    """The factors a model description may carry and LFM2 leaves at one: on the embedding, on the logits, and
    a softmax scale that is not 1/sqrt(head size). Prompt portions and decoded tokens against the plain
    computation with the same factors."""
    from celeg_b200.config import Architecture, Lfm2Config, build_lfm2_spec, register_architecture
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.weights import write_random_model

    on_embedding, on_logits, softmax_scale = 3.0, 0.25, 0.4

    def scaled_spec(config):
        spec = build_lfm2_spec(config)
        layers = list(spec.layers)
        mixer = layers[2].mixer
        layers[2] = dataclasses.replace(layers[2], mixer=dataclasses.replace(
            mixer, params={**mixer.params, "softmax_scale": softmax_scale}))
        return dataclasses.replace(spec, layers=tuple(layers), embedding_multiplier=on_embedding,
                                   logits_multiplier=on_logits, architecture="lfm2_scaled")

    register_architecture(Architecture(name="lfm2_scaled", parse_config=Lfm2Config.from_dict,
                                       resolve_config=lambda c, shapes: c.resolved_with(shapes),
                                       build_spec=scaled_spec, random_init=lfm2_random_init), replace=True)
    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "lfm2_scaled"
    folder = write_random_model(str(tmp_path / "scaled"), raw, 13, torch.bfloat16)
    loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=128, max_batched_tokens=64, use_graphs=True)
    config, w = plain_lfm2.load_model_folder(folder)
    w = dict(w)
    # q . k * s = (q * s * sqrt(d)) . k / sqrt(d), and q is linear in its norm weight
    w["model.layers.2.self_attn.q_layernorm.weight"] = w["model.layers.2.self_attn.q_layernorm.weight"] * softmax_scale * 4.0

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)] * on_embedding
        for index, kind in enumerate(config["layer_types"]):
            x = plain_lfm2.block(x, index, kind, config, w)
        z = plain_lfm2.rmsnorm(x, w["model.embedding_norm.weight"], config["norm_eps"])
        return (z @ w["model.embed_tokens.weight"].T) * on_logits

    sequences = prompts_of(config["vocab_size"], [30, 24], seed=46)
    want = [plain_forward(seq) for seq in sequences]
    step = loaded.step
    at = [0, 0]
    for sizes in ((11, 4), (2, 9)) + ((1, 1),) * 8 + ((9, 3),):
        entries = [StepEntry(f"r{i}", sequences[i][at[i]:at[i] + n], list(range(n))) for i, n in enumerate(sizes)]
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        row = 0
        for i, n in enumerate(sizes):
            worst = np.abs(logits[row:row + n] - want[i][at[i]:at[i] + n]).max()
            assert worst < tol, f"request {i}, tokens {at[i]}..{at[i] + n}: {worst:.3e}"
            row += n
            at[i] += n
    step.raise_on_device_error()


@pytest.mark.parametrize("dtype,tol", [("float32", 4e-4), ("bfloat16", 8e-2)])
def test_toy_ends_of_a_model_registered_from_outside(tmp_path, dtype, tol):
    """The two ends of a model are parts too. A toy architecture, defined here, names ends of its own: an
    input that normalises the embedded rows with a weight of its own before the first block, and an output
    that caps the logits (cap * tanh(logits / cap)) and has an untied head. Nothing in the package changes;
    prompt portions and decoded tokens (graphs included) against the plain computation."""
    from celeg_b200 import kernels
    from celeg_b200.config import Architecture, Lfm2Config, build_lfm2_spec, register_architecture
    from celeg_b200.config.lfm2_arch import lfm2_random_init
    from celeg_b200.config.spec import PartSpec, TensorRef
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.parts import register_part
    from celeg_b200.weights import write_random_model

    cap = 1.5

    class NormedEmbedding:
        def __init__(self, params, weights, parts, rt):
            self.rt = rt
            self.table = rt.matrix(weights["table"])
            self.vocab_size = int(self.table.shape[0])
            self.norm = parts["norm"]
            self.raw = rt.scratch("toy.embedded", int(self.table.shape[1]), torch.float32)
            self.normed = rt.scratch("toy.embedded_normed", int(self.table.shape[1]))

        def run(self, stream, step, first=None):
            rows = step.tokens
            kernels.embedding(self.table, step.token_ids[:rows], self.raw)
            # norm(raw) in the path's precision, then widened into the float32 stream
            self.norm.add_norm(self.raw, None, self.normed, rows)
            stream.residual[:rows].copy_(self.normed[:rows])

    class CappedHead:
        def __init__(self, params, weights, parts, rt):
            self.rt = rt
            self.norm = parts["norm"]
            self.head = rt.matrix(weights["head"])
            self.cap = float(params["cap"])
            self.normed = rt.scratch("toy.final_normed", int(self.head.shape[1]))

        def run(self, stream, step, logit_rows, n_logits, logits):
            gather = None if step.logits_of_all_rows else logit_rows
            normed = stream.normed(self.norm, self.normed, n_logits, gather=gather)
            self.rt.linear(normed, self.head, logits, n_logits)
            view = logits[:n_logits]
            view.div_(self.cap).tanh_().mul_(self.cap)

    register_part("input", "toy_normed_embedding", NormedEmbedding, replace=True)
    register_part("output", "toy_capped_head", CappedHead, replace=True)

    def toy_spec(config):
        spec = build_lfm2_spec(config)
        hidden = config.hidden_size
        norm = dataclasses.replace(spec.final_norm, tensors={"weight": TensorRef("model.input_norm.weight", (hidden,))})
        return dataclasses.replace(
            spec, architecture="lfm2_toy_ends",
            input=PartSpec("toy_normed_embedding", tensors={"table": spec.embedding}, parts={"norm": norm},
                           category="input"),
            output=PartSpec("toy_capped_head", params={"cap": cap},
                            tensors={"head": TensorRef("lm_head.weight", (config.vocab_size, hidden))},
                            parts={"norm": spec.final_norm}, category="output"))

    register_architecture(Architecture(name="lfm2_toy_ends", parse_config=Lfm2Config.from_dict,
                                       resolve_config=lambda c, shapes: c.resolved_with(shapes),
                                       build_spec=toy_spec, random_init=lfm2_random_init), replace=True)
    raw = copy.deepcopy(TINY_A)
    raw["model_type"] = "lfm2_toy_ends"
    folder = write_random_model(str(tmp_path / "toy_ends"), raw, 17, torch.bfloat16)
    loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=128, max_batched_tokens=64, use_graphs=True)
    config, w = plain_lfm2.load_model_folder(folder)

    def plain_forward(tokens):
        x = w["model.embed_tokens.weight"][np.asarray(tokens)]
        x = plain_lfm2.rmsnorm(x, w["model.input_norm.weight"], config["norm_eps"])
        if dtype == "bfloat16":                           # the toy input rounds its normalised rows to the path's precision
            x = torch.from_numpy(x).to(torch.bfloat16).to(torch.float64).numpy()
        for index, kind in enumerate(config["layer_types"]):
            x = plain_lfm2.block(x, index, kind, config, w)
        z = plain_lfm2.rmsnorm(x, w["model.embedding_norm.weight"], config["norm_eps"])
        return cap * np.tanh((z @ w["lm_head.weight"].T) / cap)

    sequences = prompts_of(config["vocab_size"], [30, 24], seed=52)
    want = [plain_forward(seq) for seq in sequences]
    step = loaded.step
    at = [0, 0]
    for sizes in ((11, 4), (2, 9)) + ((1, 1),) * 8 + ((9, 3),):
        entries = [StepEntry(f"r{i}", sequences[i][at[i]:at[i] + n], list(range(n))) for i, n in enumerate(sizes)]
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        row = 0
        for i, n in enumerate(sizes):
            worst = np.abs(logits[row:row + n] - want[i][at[i]:at[i] + n]).max()
            assert worst < tol, f"request {i}, tokens {at[i]}..{at[i] + n}: {worst:.3e}"
            row += n
            at[i] += n
    step.raise_on_device_error()
    assert type(loaded.model.input).__name__ == "NormedEmbedding" and type(loaded.model.output).__name__ == "CappedHead"


@pytest.mark.parametrize("name,dtype,tol", [("A", "float32", 3e-4), ("D", "bfloat16", 8e-2)])
def test_equal_prompt_portions_are_replayed_from_a_graph(tmp_path, name, dtype, tol):
    """A prompt cut into equal portions: the third portion of a shape is captured in a CUDA graph, the later
    ones are replayed from it (other contexts, other pages, the same launch shapes); a portion of another
    length and a step that mixes a portion with a decoded token run kernel by kernel or get graphs of their
    own. All of it against the plain implementation; the same again without graphs gives the same bits on the
    float32 path (whose products sum every element in an order that does not depend on the batch) and the same
    values to rounding on the bfloat16 path (a replayed step runs on a padded launch shape, for which the library
    may choose another kernel)."""
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, name)
    config, weights = plain_lfm2.load_model_folder(folder)
    long_seq, other = prompts_of(config["vocab_size"], [6 * 24 + 10, 30], seed=47)
    want_long = plain_lfm2.forward(config, weights, long_seq)
    want_other = plain_lfm2.forward(config, weights, other)

    def run(use_graphs):
        loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=256, max_batched_tokens=64,
                            use_graphs=use_graphs)
        step = loaded.step
        rows = []
        at = 0
        for _ in range(6):                                        # six portions of 24 tokens, the last row wanted
            rows.append(step.run([StepEntry("long", long_seq[at:at + 24], [23])], auto_begin=True).float().cpu().numpy()[0])
            at += 24
        graphed_after_equal_portions = step.kernel_steps_graphed
        rows.append(step.run([StepEntry("long", long_seq[at:at + 10], [9])]).float().cpu().numpy()[0])   # another length
        for start in (0, 12):                                     # a second request: two portions of 12 beside nothing
            step.run([StepEntry("other", other[start:start + 12], [])], auto_begin=True)
        mixed = step.run([StepEntry("other", other[24:30], [5]), StepEntry("long", [long_seq[5]], [0])])
        rows.append(mixed.float().cpu().numpy()[0])
        step.raise_on_device_error()
        return np.stack(rows), graphed_after_equal_portions

    got, graphed = run(True)
    assert graphed == 4                      # two portions ran kernel by kernel, the third was captured
    ref, not_graphed = run(False)
    assert not_graphed == 0
    if dtype == "float32":
        assert np.array_equal(got, ref)
    else:
        assert np.abs(got - ref).max() < tol
    for i in range(6):
        assert np.abs(got[i] - want_long[24 * i + 23]).max() < tol, f"portion {i}"
    assert np.abs(got[6] - want_long[153]).max() < tol
    assert np.abs(got[7] - want_other[29]).max() < tol


@pytest.mark.parametrize("name", ["B", "D"])
def test_every_product_on_the_tcgen05_kernel(tmp_path, name):
    """``KernelOptions(tensor_core_products="all")``: every product of more than 16 rows, the gate+up product with its activation
    included, runs on this package's TMA + tcgen05 kernel instead of the library's (by default only gate+up of
    2,048 rows and more does). A prompt whole, in portions and beside decoded tokens, against the plain model."""
    from celeg_b200 import KernelOptions
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, name)
    config, weights = plain_lfm2.load_model_folder(folder)
    first, second = prompts_of(config["vocab_size"], [300, 150], seed=48)
    want = [plain_lfm2.forward(config, weights, first), plain_lfm2.forward(config, weights, second)]
    loaded = load_model(folder, dtype="bfloat16", max_requests=2, cache_tokens=512, max_batched_tokens=320,
                        kernel_options=KernelOptions(tensor_core_products="all"))
    step = loaded.step
    tol = 8e-2
    whole = step.run([StepEntry("whole", first, [0, 150, 299])], auto_begin=True).float().cpu().numpy()
    for row, place in enumerate((0, 150, 299)):
        assert np.abs(whole[row] - want[0][place]).max() < tol, f"whole prompt, place {place}"
    step.end("whole")
    got = step.run([StepEntry("a", first[:170], [169]), StepEntry("b", second[:131], [130])], auto_begin=True).float().cpu().numpy()
    assert np.abs(got[0] - want[0][169]).max() < tol and np.abs(got[1] - want[1][130]).max() < tol
    got = step.run([StepEntry("a", first[170:299], [128]), StepEntry("b", [second[131]], [0])]).float().cpu().numpy()
    assert np.abs(got[0] - want[0][298]).max() < tol and np.abs(got[1] - want[1][131]).max() < tol
    step.raise_on_device_error()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_that_end_on_a_token_while_the_next_step_is_in_flight(models, dtype):
    """The scheduler enqueues the step after the one it reads while every request decodes. A request
    that ends on an end-of-sequence token has then one position computed in vain: its output must stop at
    that token, the others must continue as if nothing happened, and slot and pages must come back."""
    from celeg_b200 import Engine
    folder, config, weights = models["A"]
    prompts = prompts_of(config["vocab_size"], [7, 19, 12, 26], seed=29)
    free = [plain_lfm2.generate(config, weights, prompt, 24, eos_tokens=()) for prompt in prompts]
    # each request stops at a token of its own free-running output: after 3, 9, 15 and (none) tokens
    stops = [(free[0][3],), (free[1][9],), (free[2][15],), ()]
    engine = Engine(folder, dtype=dtype)
    assert engine.scheduler._runs_ahead
    ids = [engine.submit(prompt, max_new_tokens=24, temperature=0.0, repetition_penalty=1.0, eos_tokens=stop)
           for prompt, stop in zip(prompts, stops)]
    while engine.scheduler.has_work():
        engine.step()
    agree = 0
    for request_id, prompt, stop in zip(ids, prompts, stops):
        want = plain_lfm2.generate(config, weights, prompt, 24, eos_tokens=stop)
        got = engine.poll(request_id).tokens
        assert engine.status(request_id).value == "finished"
        if dtype == "float32":
            assert got == want
        agree += got == want
    assert agree >= 3
    engine.loaded.step.raise_on_device_error()
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == engine.options.max_active_requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_ahead_with_requests_that_end_at_different_steps(models, dtype, monkeypatch):
    """Twelve requests with 3 to 25 new tokens each, some drawn with a seed, one ending on a token of its own:
    in nearly every step some request produces its last token. The step after is still enqueued early for the
    others and takes their tokens from the device, from the rows they had in the step before. Outputs against
    the plain model; steps with fewer rows than their predecessor must have been launched ahead."""
    from celeg_b200 import Engine, EngineOptions
    from celeg_b200.engine import engine as engine_module
    folder, config, weights = models["A"]
    lengths = [5, 9, 3, 14, 7, 11, 4, 8, 6, 10, 12, 2]
    news = [3, 25, 6, 9, 14, 4, 17, 8, 21, 5, 12, 10]
    prompts = prompts_of(config["vocab_size"], lengths, seed=61)
    sampled = {1, 4, 8}                                 # these draw with a seed, the others are greedy
    free = plain_lfm2.generate(config, weights, prompts[3], news[3], eos_tokens=())
    stops = {3: (free[5],)}
    shrunk = []
    original = engine_module._Runner.launch

    def launch(self, entries, sample_rows, tokens_on_device=False, source_rows=None):
        if source_rows is not None:
            shrunk.append(len(source_rows))
        return original(self, entries, sample_rows, tokens_on_device, source_rows)
    monkeypatch.setattr(engine_module._Runner, "launch", launch)
    engine = Engine(folder, dtype=dtype, options=EngineOptions(max_active_requests=16, max_batched_tokens=64))
    ids = []
    for i, (prompt, new) in enumerate(zip(prompts, news)):
        if i in sampled:
            ids.append(engine.submit(prompt, max_new_tokens=new, temperature=0.8, top_k=20, top_p=0.9,
                                     repetition_penalty=1.1, seed=100 + i, eos_tokens=()))
        else:
            ids.append(engine.submit(prompt, max_new_tokens=new, temperature=0.0, repetition_penalty=1.0,
                                     eos_tokens=stops.get(i, ())))
    while engine.scheduler.has_work():
        engine.step()
    agree = 0
    for i, (request_id, prompt, new) in enumerate(zip(ids, prompts, news)):
        if i in sampled:
            want = plain_lfm2.generate(config, weights, prompt, new, temperature=0.8, top_k=20, top_p=0.9,
                                       repetition_penalty=1.1, seed=100 + i, eos_tokens=())
        else:
            want = plain_lfm2.generate(config, weights, prompt, new, eos_tokens=stops.get(i, ()))
        got = engine.poll(request_id).tokens
        assert engine.status(request_id).value == "finished"
        if dtype == "float32":
            assert got == want, (i, got, want)
        agree += got == want
    assert agree >= 9
    assert len(shrunk) >= 4, shrunk
    engine.loaded.step.raise_on_device_error()
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == engine.options.max_active_requests


@pytest.mark.parametrize("name,dtype,tol", [("A", "float32", 4e-4), ("B", "bfloat16", 8e-2), ("D", "bfloat16", 8e-2)])
def test_steps_of_changing_mix_are_padded_to_launch_shapes_and_replayed(tmp_path, name, dtype, tol):
    """Steps of the form the scheduler plans under load: decoded tokens of a changing number of requests first,
    then one or two prompt portions of changing lengths. No two of them have the same shape, yet from its
    third coming on a launch shape from the coarse grid (spare single tokens, one spare portion) is replayed
    from a CUDA graph. Every wanted row of every step against the plain model; graphs must have been used."""
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, name)
    config, weights = plain_lfm2.load_model_folder(folder)
    rng = np.random.default_rng(47)
    count = 14
    lengths = rng.integers(30, 90, size=count).tolist()
    seqs = prompts_of(config["vocab_size"], lengths, seed=48)
    want = [plain_lfm2.forward(config, weights, s) for s in seqs]
    loaded = load_model(folder, dtype=dtype, max_requests=16, cache_tokens=12 * 96, max_batched_tokens=96,
                        use_graphs=True)
    step = loaded.step
    at = [0] * count
    decoding, waiting, prefilling = [], list(range(count)), []
    steps = 0
    while decoding or waiting or prefilling:
        entries, places = [], []
        for r in list(decoding):                           # single tokens first
            entries.append(StepEntry(f"r{r}", [seqs[r][at[r]]], [0]))
            places.append((r, at[r]))
            at[r] += 1
        budget = 2                                         # then up to two portions
        while len(prefilling) < budget and waiting and len(decoding) + len(prefilling) < 10:
            prefilling.append(waiting.pop(0))
        started = []
        for r in list(prefilling)[:budget]:
            # a request's prompt is all but its last 12 tokens, which it then decodes one by one
            left = lengths[r] - 12 - at[r]
            n = int(min(left, rng.integers(2, 30)))
            last = n == left
            entries.append(StepEntry(f"r{r}", seqs[r][at[r]:at[r] + n], [n - 1] if last else []))
            if last:
                places.append((r, at[r] + n - 1))
                started.append(r)
            at[r] += n
        logits = step.run(entries, auto_begin=True).float().cpu().numpy()
        assert logits.shape[0] == len(places)
        for row, (r, place) in enumerate(places):
            worst = np.abs(logits[row] - want[r][place]).max()
            assert worst < tol, f"step {steps}, request {r}, place {place}: {worst:.3e}"
        for r in started:
            prefilling.remove(r)
            decoding.append(r)
        for r in list(decoding):
            if at[r] == lengths[r]:
                decoding.remove(r)
                step.end(f"r{r}")
        steps += 1
        assert steps < 2000
    step.raise_on_device_error()
    loaded.manager.check_invariants()
    padded = [k for k in step._graphs if k and k[0] == "padded prompt"]
    assert len(padded) >= 2 and step.kernel_steps_graphed > steps // 3, (len(padded), step.kernel_steps_graphed, steps)


@pytest.mark.parametrize("name,dtype,tol,seed", [("A", "float32", 4e-4, 1), ("B", "bfloat16", 8e-2, 2),
                                                  ("C", "float32", 4e-4, 0), ("D", "bfloat16", 8e-2, 1),
                                                  ("D", "float32", 4e-4, 3)])
def test_random_steps_under_random_cache_shapes(tmp_path, name, dtype, tol, seed):
    """Page size, live requests, token budget, context limit, pool size and graphs drawn at random; then steps
    drawn at random: each live request is left out, brings a portion of some length or one token, in the
    scheduler's order (single tokens first) or in any; places wanted at the end, nowhere or anywhere; requests
    end early; a refused step (no pages) must leave everything as it was, and the request that holds most then
    gives its pages back. Every wanted row against the plain model."""
    import random
    from celeg_b200.cache import OutOfPages
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    folder = write_tiny(tmp_path, name)
    config, weights = plain_lfm2.load_model_folder(folder)
    rng = random.Random(seed * 13 + ord(name))
    page_tokens = rng.choice([4, 8, 16, 64])
    max_requests = rng.choice([2, 3, 4, 8])
    budget = rng.choice([32, 64, 128, 256])
    context = rng.choice([None, 96, 200])
    longest = min(context or config["max_position_embeddings"], rng.choice([40, 90, 150, 250]))
    cache_tokens = max((-(-longest // page_tokens) + 1) * page_tokens,
                       int(max_requests * longest * rng.choice([0.4, 0.7, 1.2])))
    loaded = load_model(folder, dtype=dtype, max_requests=max_requests, cache_tokens=cache_tokens,
                        page_tokens=page_tokens, max_batched_tokens=budget, use_graphs=rng.random() < 0.7,
                        max_context=context)
    step = loaded.step
    live, made, total, steps = {}, 0, rng.randint(6, 14), 0      # id -> [tokens, plain logits, at, ends at, decodes from]
    while live or made < total:
        while len(live) < max_requests and made < total and rng.random() < 0.7:
            n = rng.randint(3, longest)
            sequence = [rng.randrange(config["vocab_size"]) for _ in range(n)]
            live[f"q{made}"] = [sequence, None, 0, n if rng.random() < 0.7 else rng.randint(2, n), rng.randint(1, n)]
            made += 1
        left, chosen = budget, []
        order = list(live)
        rng.shuffle(order)
        for rid in order:
            _, _, at, ends_at, decodes_from = live[rid]
            if rng.random() < 0.15 or left <= 0:
                continue
            n = 1 if at >= decodes_from or rng.random() < 0.1 else \
                min(decodes_from - at, rng.choice([2, 3, 5, 8, 17, 33, 64, 128]))
            n = min(n, ends_at - at, left)
            if n > 0:
                left -= n
                chosen.append((rid, n))
        if rng.random() < 0.5:
            chosen.sort(key=lambda c: c[1] != 1)
        entries, places = [], []
        for rid, n in chosen:
            sequence, _, at, _, _ = live[rid]
            kind = rng.random()
            wanted = [n - 1] if kind < 0.5 else [] if kind < 0.7 else \
                sorted(rng.sample(range(n), rng.randint(1, min(n, 3))))
            entries.append(StepEntry(rid, sequence[at:at + n], wanted))
            places.extend((rid, at + w) for w in wanted)
        if not entries:
            continue
        try:
            out = step.run(entries, auto_begin=True)
        except OutOfPages:
            loaded.manager.check_invariants()
            rid = max(live, key=lambda r: live[r][2])
            if live[rid][2] > 0:
                step.end(rid)
            del live[rid]
            continue
        logits = out.float().cpu().numpy() if places else np.zeros((0, 1))
        assert logits.shape[0] == len(places)
        for row, (rid, place) in enumerate(places):
            if live[rid][1] is None:
                live[rid][1] = plain_lfm2.forward(config, weights, live[rid][0])
            worst = float(np.abs(logits[row] - live[rid][1][place]).max())
            assert worst < tol, f"step {steps}, request {rid}, place {place}: {worst:.3e}"
        for entry in entries:
            live[entry.request_id][2] += len(entry.tokens)
        for rid in list(live):
            if live[rid][2] >= live[rid][3]:
                step.end(rid)
                del live[rid]
        steps += 1
        assert steps < 5000
    step.raise_on_device_error()
    loaded.manager.check_invariants()
    assert loaded.manager.free_slots == max_requests
    assert all(group.pool.used_pages == 0 for group in loaded.manager.groups)


@pytest.mark.parametrize("seed", [3, 6, 9, 11, 101, 317])
def test_random_configurations_and_kernel_options_against_the_plain_model(tmp_path, seed):
    """Every size of the configuration drawn at random (widths that are odd numbers, 1 to 8 key/value heads with
    1 to 7 query heads each, head sizes 16 to 128 in steps of 16 and others up to 320, any feed-forward width
    and vocabulary, 2 to 4 taps, any order of layers), and the switches of the kernel path too: the logits of a
    prompt in two portions and of the rest token by token, on both paths, with and without graphs, against the
    plain model."""
    import copy
    import random
    from celeg_b200 import KernelOptions
    from celeg_b200.engine.loading import load_model
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.weights import write_random_model
    rng = random.Random(1000 + seed)
    layers = rng.randint(1, 5)
    types = [rng.choice(["conv", "full_attention"]) for _ in range(layers)]
    if "full_attention" not in types:
        types[rng.randrange(layers)] = "full_attention"
    kv_heads = rng.choice([1, 2, 3, 4, 5, 8])
    raw = {"model_type": "lfm2", "vocab_size": rng.randint(50, 3000),
           "hidden_size": rng.randint(2, 40) * rng.choice([1, 2, 8, 16, 64]),
           "num_hidden_layers": layers, "num_attention_heads": kv_heads * rng.choice([1, 2, 3, 4, 7]),
           "num_key_value_heads": kv_heads, "head_dim": rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 24, 40, 200, 320]),
           "max_position_embeddings": 512, "norm_eps": rng.choice([1e-5, 1e-6, 3e-4]),
           "conv_L_cache": rng.choice([2, 3, 4]), "rope_theta": rng.choice([1e4, 1e6, 5e5]), "layer_types": types,
           "tie_word_embeddings": rng.random() < 0.5,
           "intermediate_size": rng.randint(8, 400) if rng.random() < 0.5 else rng.randint(1, 30) * rng.choice([16, 128]),
           "conv_bias": False, "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0}
    folder = str(tmp_path / "model")
    write_random_model(folder, copy.deepcopy(raw), seed, torch.bfloat16)
    config, weights = plain_lfm2.load_model_folder(folder)
    n = rng.randint(20, 150)
    sequence = [rng.randrange(raw["vocab_size"]) for _ in range(n)]
    cut = rng.randint(2, n - 8)
    middle = cut + (n - cut) // 2
    want = plain_lfm2.forward(config, weights, sequence)
    scale = max(1.0, float(np.abs(want).max()))
    for dtype, tol in (("float32", 6e-4), ("bfloat16", 1e-1)):
        for graphs in (False, True):
            options = KernelOptions(tensor_core_products=rng.choice(["none", "swiglu", "all"]),
                                    tensor_core_min_rows=rng.choice([1, 17, 64, 2048]),
                                    tensor_core_min_width=rng.choice([1, 1536]),
                                    tensor_core_variant=rng.choice([-1, -1, 0, 1, 2, 3]),
                                    split_norms=rng.random() < 0.5, fuse_decode_qk=rng.random() < 0.5,
                                    tcgen05_attention=rng.random() < 0.5, prefetch_mb=rng.choice([0.0, 8.0]),
                                    fuse_small_batches=rng.random() < 0.5)
            loaded = load_model(folder, dtype=dtype, max_requests=2, cache_tokens=512, page_tokens=rng.choice([16, 64]),
                                max_batched_tokens=256, use_graphs=graphs, kernel_options=options)
            step = loaded.step
            rows = [step.run([StepEntry("a", sequence[:cut], list(range(cut)))], auto_begin=True).float().cpu().numpy()]
            rows.append(step.run([StepEntry("a", sequence[cut:middle], list(range(middle - cut)))]).float().cpu().numpy())
            for token in sequence[middle:]:
                rows.append(step.run([StepEntry("a", [token], [0])]).float().cpu().numpy().copy())
            step.raise_on_device_error()
            worst = np.abs(np.concatenate(rows, axis=0) - want).max(axis=1)
            assert worst.max() < tol * scale, (raw, options, dtype, graphs, int(worst.argmax()), float(worst.max()))
            del loaded, step
