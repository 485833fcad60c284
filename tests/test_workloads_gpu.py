"""The scheduler workloads of ``bench.py --workload`` at tiny sizes: the same driver
(``bench.drive_workload``: submit everything, step and poll until all are terminal) with 64 requests
of very different prompt lengths in portions beside decoded tokens, and with 256 requests that draw
at temperature 1.0 with a seed each. A sample of the outputs is compared with the plain
implementation, token by token, on the float32 path; the record's counters are checked against what
the run must have done."""
from __future__ import annotations

import numpy as np
import pytest

import bench
import plain_lfm2
from tiny_models import write_tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    base = tmp_path_factory.mktemp("workload_models")
    out = {}
    for name in ("A", "B"):
        folder = write_tiny(base, name)
        config, weights = plain_lfm2.load_model_folder(folder)
        out[name] = (folder, config, weights)
    return out


def test_64_requests_of_mixed_lengths_in_portions_beside_decoding(models):
    """The 700M workload in small on tiny A: 64 live requests, prompts of 5 to 120 tokens in portions of at most
    32 under a budget of 96 tokens a step, so most steps hold portions of some requests beside decoded tokens
    of others; 16 greedy tokens each; so few pages that admission has to wait for finished requests."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams
    folder, config, weights = models["A"]
    rng = np.random.default_rng(60)
    lengths = rng.integers(5, 121, size=64).tolist()
    prompts = [rng.integers(0, config["vocab_size"], size=n).tolist() for n in lengths]
    options = EngineOptions(max_active_requests=64, max_batched_tokens=96, prefill_chunk_tokens=32, page_tokens=16,
                            logical_kv_pages=180)
    engine = Engine(folder, dtype="float32", options=options)
    request_options = [RequestOptions(max_new_tokens=16, eos_tokens=(),
                                      generation=SamplingParams(temperature=0.0, top_k=1, repetition_penalty=1.0))
                       for _ in prompts]
    result = bench.drive_workload(engine, prompts, request_options)
    record = result["record"]
    assert not result["errors"]
    assert record["generated_tokens"] == 64 * 16 and record["prompt_tokens"] == sum(lengths)
    assert record["max_step_tokens"] <= 96 and record["max_step_requests"] > 4
    assert 0 < record["pages"]["high_water"] <= record["pages"]["total"] == 180
    assert record["ttft_ms"]["p99"] >= record["ttft_ms"]["p50"] > 0 and record["itl_ms"]["mean"] > 0
    host = record["host_ms_per_step"]
    assert host["launch"] > 0 and host["plan"] > 0 and host["commit"] > 0 and record["gpu_ms_per_step"] > 0
    assert abs(host["check"] + host["stage"] + host["forward"] + host["sample"] - host["launch"]) < 0.5 * host["launch"]
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == 64
    assert all(group.pool.used_pages == 0 for group in engine.loaded.manager.groups)
    for index in (0, 7, 13, 29, 41, 63):
        assert result["outputs"][index] == plain_lfm2.generate(config, weights, prompts[index], 16, eos_tokens=())


def test_256_requests_drawing_with_a_seed_each(models):
    """The 350M workload in small on tiny B: 256 live requests of 24 prompt tokens, 12 tokens each at
    temperature 1.0 with top-k 50 and the request's own seed; what a request draws must not depend on the
    255 others."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams
    folder, config, weights = models["B"]
    rng = np.random.default_rng(61)
    prompts = [rng.integers(0, config["vocab_size"], size=24).tolist() for _ in range(256)]
    options = EngineOptions(max_active_requests=256, max_batched_tokens=1024, prefill_chunk_tokens=24, page_tokens=16)
    engine = Engine(folder, max_context=64, dtype="float32", options=options)
    request_options = [RequestOptions(max_new_tokens=12, eos_tokens=(),
                                      generation=SamplingParams(temperature=1.0, top_k=50, top_p=1.0,
                                                                repetition_penalty=1.0, seed=i + 1))
                       for i in range(256)]
    result = bench.drive_workload(engine, prompts, request_options)
    record = result["record"]
    assert not result["errors"]
    assert record["generated_tokens"] == 256 * 12 and record["max_step_requests"] == 256
    assert record["decode_only"]["steps"] >= 8 and record["decode_only"]["gb_per_step"] > 0
    engine.loaded.manager.check_invariants()
    for index in (0, 100, 255):
        want = plain_lfm2.generate(config, weights, prompts[index], 12, temperature=1.0, top_k=50, top_p=1.0,
                                   repetition_penalty=1.0, seed=index + 1)
        assert result["outputs"][index] == want


def test_256_requests_with_a_warp_per_attention_item(models):
    """The decode attention's form for very many requests with short contexts (one warp a (token, kv head)
    item), inside the engine: 256 requests on tiny B in bfloat16, greedy, once with that form and once with the
    four-warp form. Both sum a row's keys in different orders, so a token may differ where two logits are
    nearly equal: nearly all requests must agree, and every request's first token with the plain model's."""
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams, kernels
    folder, config, weights = models["B"]
    rng = np.random.default_rng(62)
    prompts = [rng.integers(0, config["vocab_size"], size=int(n)).tolist() for n in rng.integers(3, 40, size=256)]
    options = EngineOptions(max_active_requests=256, max_batched_tokens=1024, prefill_chunk_tokens=64, page_tokens=16)
    request_options = [RequestOptions(max_new_tokens=10, eos_tokens=(),
                                      generation=SamplingParams(temperature=0.0, top_k=1, repetition_penalty=1.0))
                       for _ in prompts]
    outputs = {}
    try:
        for name, items in (("one warp", 1), ("four warps", 1 << 40)):
            kernels.library().celeg_attention_decode_solo_items(items)
            engine = Engine(folder, max_context=64, dtype="bfloat16", options=options)
            result = bench.drive_workload(engine, prompts, request_options)
            assert not result["errors"]
            engine.loaded.step.raise_on_device_error()
            engine.loaded.manager.check_invariants()
            outputs[name] = result["outputs"]
            del engine
    finally:
        kernels.library().celeg_attention_decode_solo_items(1536)
    same = sum(1 for a, b in zip(outputs["one warp"], outputs["four warps"]) if a == b)
    assert same >= 240, same
    first = 0
    for index in range(0, 256, 16):
        want = plain_lfm2.generate(config, weights, prompts[index], 1, eos_tokens=())
        first += outputs["one warp"][index][:1] == want
    assert first >= 14, first


@pytest.mark.parametrize("name,seed", [("A", 0), ("A", 1), ("A", 12), ("B", 0), ("B", 5), ("B", 13)])
def test_random_requests_under_random_engine_options(models, name, seed):
    """Options drawn at random (policy, live requests, token budget, portion size, page size down to 4 tokens,
    pool size down to little more than one request) with a context limit of 96 tokens, so that a table row holds
    fewer pages than a padded launch shape's spare portion may want; requests of random lengths, greedy or drawing
    with a seed, some ending on a token, submitted a few at a time while the engine steps. Every request's output
    against the plain implementation."""
    import random
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams
    from celeg_b200.engine.scheduler import SchedulerPolicy
    folder, config, weights = models[name]
    rng = random.Random(seed * 7 + (1 if name == "B" else 0))
    policy = rng.choice([SchedulerPolicy.GUARANTEED_NO_EVICT, SchedulerPolicy.MAX_UTILIZATION])
    max_active = rng.choice([2, 4, 8, 12])
    page_tokens = rng.choice([4, 8, 16])
    pools = [0, max(12, 90 // page_tokens * max_active // 2), 96 // page_tokens + rng.randint(1, 12)]
    options = EngineOptions(max_active_requests=max_active, max_batched_tokens=rng.choice([16, 24, 48, 96]),
                            prefill_chunk_tokens=rng.choice([4, 7, 16, 32]), page_tokens=page_tokens,
                            logical_kv_pages=rng.choice(pools), scheduler_policy=policy)
    engine = Engine(folder, max_context=96, dtype="float32", options=options)
    requests = []
    for _ in range(rng.randint(10, 24)):
        prompt = [rng.randrange(config["vocab_size"]) for _ in range(rng.randint(1, 50))]
        new = rng.randint(1, 24)
        if rng.random() < 0.5:
            params = dict(temperature=0.8, top_k=rng.choice([5, 50]), top_p=rng.choice([1.0, 0.9]),
                          repetition_penalty=rng.choice([1.0, 1.2]), seed=rng.randint(1, 1000))
        else:
            params = dict(temperature=0.0, top_k=1, top_p=1.0, repetition_penalty=1.0, seed=1)
        free = plain_lfm2.generate(config, weights, prompt, new, eos_tokens=(), **params)
        eos = (free[rng.randrange(len(free))],) if rng.random() < 0.3 else ()
        want = plain_lfm2.generate(config, weights, prompt, new, eos_tokens=eos, **params)
        requests.append((prompt, RequestOptions(max_new_tokens=new, eos_tokens=eos,
                                                generation=SamplingParams(**params)), want))
    submitted, pending, steps = [], list(range(len(requests))), 0
    while pending or engine.scheduler.has_work():
        for _ in range(rng.randint(0, 3)):
            if pending:
                index = pending.pop(0)
                submitted.append((index, engine.submit(requests[index][0], requests[index][1])))
        engine.step()
        steps += 1
        assert steps < 5000
    for index, request_id in submitted:
        result = engine.poll(request_id)
        assert engine.status(request_id).value == "finished", (index, result.error)
        assert result.tokens == requests[index][2], index
    engine.loaded.step.raise_on_device_error()
    engine.loaded.manager.check_invariants()
    assert engine.loaded.manager.free_slots == max_active
