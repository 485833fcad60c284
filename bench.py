#!/usr/bin/env python3
"""Benchmark of celeg_b200 on one B200: decode tokens per second at LFM2-1.2B sizes with random
weights (batch 8, 512-token prompts, context 4,096), plus prefill of 2,048 tokens and decode at
batch 1 and 64. Prints ONE JSON line.

  python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
  python bench.py --phase decode|prefill [--sizes lfm2-1.2b|lfm2-700m|lfm2-350m] [--batch B] [--prompt-tokens P]
                  [--prefill-tokens T] [--chunk C] [--kernel-times] [--no-cuda-graph]      one phase, a short record
  python bench.py --workload lfm2-700m|lfm2-350m [--requests N] [--new-tokens N] [--max-batched-tokens N]
                  [--prefill-chunk N] [--kernel-times]       a scheduler workload through Engine.submit/step/poll

A "step" is one decode step of the whole batch. ``value`` is timed on the device (CUDA events
around K steps of step function + sampling kernel, synthetic token ids); ``e2e`` is the same
through ``Engine.step()``: host token ids in through pinned memory, sampled ids back to the host
every step (two timed regions of K steps, the better one reported, both named). Weights (2.3 GB) are larger than L2, so no flush is needed between iterations.
``--impl reference`` runs celsowm/celeg's own engine on the same model folder and workload through its
C API (``baseline/reference_bench.py`` over ``baseline/_ref/libceleg.so``, which
``baseline/build_reference.py`` builds from celeg's sources). Switches of the kernel path can be set
for a run with ``CELEG_B200_<FIELD>`` (fields of ``celeg_b200.KernelOptions``).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the sizes of LFM2-1.2B, the configuration the headline numbers are quoted on
LFM2_1P2B = {
    "model_type": "lfm2", "vocab_size": 65536, "hidden_size": 2048, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
    "conv_L_cache": 3, "rope_theta": 1000000.0, "norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 4096,
    "layer_types": ["full_attention" if i in (2, 5, 8, 10, 12, 14) else "conv" for i in range(16)],
    "bos_token_id": 1, "eos_token_id": 7, "pad_token_id": 0,
}

def _lfm2_sizes(hidden: int, heads: int, inner: int, context: int) -> dict:
    raw = dict(LFM2_1P2B)
    raw.update({"hidden_size": hidden, "num_attention_heads": heads, "intermediate_size": inner,
                "max_position_embeddings": context})
    return raw


# The two scheduler workloads: many live requests through Engine.submit / step / poll.
WORKLOADS = {
    # 64 requests, prompts uniform in [256, 16,384], context 32,768, portions of prompts beside decoded tokens,
    # 256 new tokens each, greedy: the load on the scheduler, the page pool and long-context decode attention
    "lfm2-700m": {"config": _lfm2_sizes(1536, 24, 6912, 32768), "requests": 64, "prompt_min": 256,
                  "prompt_max": 16384, "context": 32768, "new_tokens": 256, "temperature": 0.0,
                  "max_batched_tokens": 2048, "prefill_chunk_tokens": 2048},
    # 256 requests of 128 prompt tokens, context 2,048, 128 new tokens at temperature 1.0 with a seed each: the
    # load on the host side (plan, staging, sampling options, page leases, state slots)
    "lfm2-350m": {"config": _lfm2_sizes(1024, 16, 4608, 2048), "requests": 256, "prompt_min": 128,
                  "prompt_max": 128, "context": 2048, "new_tokens": 128, "temperature": 1.0,
                  "max_batched_tokens": 4096, "prefill_chunk_tokens": 256},
}
FULL_LAYERS = 16
CONTEXT = 4096
PROMPT_TOKENS = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            data = json.load(handle)
        return {k: float(data[k]) for k in FALLBACK_PEAKS}, "measured"
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


def model_config(layers: int, sizes: str = "lfm2-1.2b") -> dict:
    raw = dict(LFM2_1P2B) if sizes == "lfm2-1.2b" else dict(WORKLOADS[sizes]["config"])
    if layers != FULL_LAYERS:
        raw["num_hidden_layers"] = layers
        raw["layer_types"] = LFM2_1P2B["layer_types"][:layers]
    return raw


def model_folder(raw: dict, seed: int = 0) -> str:
    """Random-weights model folder, reused if a finished one of the same configuration exists."""
    from celeg_b200 import write_random_model
    tag = hashlib.sha256((json.dumps(raw, sort_keys=True) + str(seed)).encode()).hexdigest()[:16]
    folder = os.path.join(tempfile.gettempdir(), f"celeg_b200_bench_{os.getuid()}_{tag}")
    if not os.path.isfile(os.path.join(folder, "complete")):
        started = time.time()
        write_random_model(folder, raw, seed)
        with open(os.path.join(folder, "complete"), "w") as handle:
            handle.write("ok")
        print(f"[bench] wrote random weights to {folder} in {time.time() - started:.0f} s", file=sys.stderr)
    return folder


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.rows = []
        self.process = None
        self.index = index

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([part.strip() for part in line.split(",")])

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.25)
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self) -> dict:
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            try:
                clocks.append(float(row[0]))
                maxima.append(float(row[1]))
            except (ValueError, IndexError):
                continue
            for name, value in zip(names, row[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


def decode_bytes(raw: dict, batch: int, context_tokens: int) -> float:
    """Bytes one decode step has to read: every weight once (the tied table once, as the head),
    the KV of the live requests, their conv state, and the embedding rows."""
    h, inner, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    q = raw["num_attention_heads"] * raw["head_dim"]
    kv = raw["num_key_value_heads"] * raw["head_dim"]
    taps = raw["conv_L_cache"]
    conv = raw["layer_types"].count("conv")
    attn = raw["layer_types"].count("full_attention")
    per_conv = 3 * h * h + h * h + h * taps
    per_attn = (q + 2 * kv) * h + h * q + 2 * raw["head_dim"]
    per_ffn = 3 * h * inner + 2 * h
    weights = 2.0 * (conv * (per_conv + per_ffn) + attn * (per_attn + per_ffn) + v * h + h)
    kv_bytes = 2.0 * 2 * kv * attn * context_tokens * batch
    state = 4.0 * (taps - 1) * h * conv * batch
    return weights + kv_bytes + state + 2.0 * batch * h


def prefill_flops(raw: dict, tokens: int) -> float:
    h, inner, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
    q = raw["num_attention_heads"] * raw["head_dim"]
    kv = raw["num_key_value_heads"] * raw["head_dim"]
    conv = raw["layer_types"].count("conv")
    attn = raw["layer_types"].count("full_attention")
    linear = conv * (3 * h * h + h * h) + attn * ((q + 2 * kv) * h + h * q) + (conv + attn) * 3 * h * inner
    causal = attn * 2 * q * tokens * (tokens + 1) / 2            # QK^T and PV, lower triangle
    return 2.0 * tokens * linear + 2.0 * causal + 2.0 * v * h    # head on the last row only


class KernelTimer:
    """Device time per kind of kernel: while active, every launch entry of ``celeg_b200.kernels`` and the
    library product are bracketed by two CUDA events. Use it on steps that are launched kernel by kernel
    (``--no-cuda-graph``); the numbers include what a launch from the host adds, so read them as shares."""
    NAMES = ("embedding", "add_rmsnorm", "short_conv", "qk_norm_rope_store", "attention_generic", "attention_decode",
             "attention_decode_fused", "attention_prefill", "attention_prefill_tcgen05", "gemv_bf16", "gemm_tcgen05",
             "gemm_stream", "gemm_f32", "swiglu", "sample", "sample_greedy", "mark_seen")

    def __init__(self):
        self.pairs = []
        self.saved = {}

    def _wrap(self, name, function):
        import torch

        def timed(*args, **kwargs):
            if torch.cuda.is_current_stream_capturing():       # a graph is being recorded: nothing runs now
                return function(*args, **kwargs)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = function(*args, **kwargs)
            end.record()
            self.pairs.append((name, begin, end))
            return result
        return timed

    def __enter__(self):
        import torch
        from celeg_b200 import kernels
        for name in self.NAMES:
            if hasattr(kernels, name):
                self.saved[name] = getattr(kernels, name)
                setattr(kernels, name, self._wrap(name, self.saved[name]))
        self.saved["torch.mm"] = torch.mm
        torch.mm = self._wrap("library product (torch.mm)", torch.mm)
        return self

    def __exit__(self, *exc):
        import torch
        from celeg_b200 import kernels
        torch.mm = self.saved.pop("torch.mm")
        for name, function in self.saved.items():
            setattr(kernels, name, function)
        self.saved = {}

    def table(self, steps: int) -> dict:
        import torch
        torch.cuda.synchronize()
        totals = {}
        for name, begin, end in self.pairs:
            entry = totals.setdefault(name, [0, 0.0])
            entry[0] += 1
            entry[1] += begin.elapsed_time(end) * 1e3
        return {name: {"launches": round(count / steps, 1), "us": round(us / steps, 1)}
                for name, (count, us) in sorted(totals.items(), key=lambda item: -item[1][1])}


def time_decode(loaded, sampler, batch: int, steps: int, warmup: int, prompt_tokens: int, seed: int, timer=None):
    """Prefill ``batch`` requests, then time ``steps`` decode steps on the device."""
    import torch
    from celeg_b200 import kernels
    from celeg_b200.engine.step import StepEntry
    from celeg_b200.sampling import GREEDY
    step_fn = loaded.step
    vocab = loaded.model.vocab_size
    generator = torch.Generator().manual_seed(seed)
    names = [f"b{batch}_{i}" for i in range(batch)]
    chunk = step_fn.max_tokens
    prompts = {name: torch.randint(0, vocab, (prompt_tokens,), generator=generator).tolist() for name in names}
    # prompts go in as many requests to a step as the step's token limit holds
    together = max(1, min(step_fn.max_spans, chunk // max(1, min(prompt_tokens, chunk))))
    for first in range(0, batch, together):
        group = names[first:first + together]
        for at in range(0, prompt_tokens, chunk):
            step_fn.run([StepEntry(name, prompts[name][at:at + chunk], []) for name in group], auto_begin=True)
    slots = [(loaded.manager.get(name).slot, GREEDY) for name in names]
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=generator).tolist()

    def one(i):
        logits = step_fn.run([StepEntry(name, [feed[i][j]], [0]) for j, name in enumerate(names)])
        kernels.sample_greedy(logits, batch, sampler._dev_i[:batch], None, None, sampler.out,
                              sampler._partial_score, sampler._partial_token)

    sampler._dev_i[:batch].copy_(torch.tensor([s for s, _ in slots], dtype=torch.int32))
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches_before = kernels.LAUNCHES
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if timer is not None:
        timer.__enter__()
    start.record()
    for i in range(warmup, warmup + steps):
        one(i)
    stop.record()
    torch.cuda.synchronize()
    if timer is not None:
        timer.__exit__(None, None, None)
    ms = start.elapsed_time(stop) / steps
    launches = kernels.LAUNCHES - launches_before
    context = prompt_tokens + warmup + steps // 2
    for name in names:
        step_fn.end(name)
    return ms, launches, context


def time_prefill(loaded, tokens: int, repeats: int, seed: int, chunk: int = 0):
    """One prompt of ``tokens`` tokens, as one step or (``chunk`` > 0) in portions of that many tokens, each
    portion attending to the cache the earlier ones left; the best of ``repeats`` runs."""
    import torch
    from celeg_b200.engine.step import StepEntry
    step_fn = loaded.step
    vocab = loaded.model.vocab_size
    generator = torch.Generator().manual_seed(seed)
    best = None
    for i in range(repeats + 3):
        prompt = torch.randint(0, vocab, (tokens,), generator=generator).tolist()
        size = chunk if chunk > 0 else tokens
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for at in range(0, tokens, size):
            portion = prompt[at:at + size]
            want = [len(portion) - 1] if at + size >= tokens else []
            step_fn.run([StepEntry(f"prefill{i}", portion, want)], auto_begin=True)
        stop.record()
        torch.cuda.synchronize()
        step_fn.end(f"prefill{i}")
        if i >= 3:                     # (the step's shape is launched from the host twice, then captured, then replayed)
            ms = start.elapsed_time(stop)
            best = ms if best is None else min(best, ms)
    return best


def time_e2e(engine, batch: int, steps: int, warmup: int, prompt_tokens: int, seed: int):
    """The same decode through Engine.step(): pinned host inputs in, sampled ids out, every step."""
    import torch
    from celeg_b200 import RequestOptions, SamplingParams
    vocab = engine.loaded.model.vocab_size
    generator = torch.Generator().manual_seed(seed)
    options = RequestOptions(max_new_tokens=warmup + steps + 8, eos_tokens=(),
                             generation=SamplingParams(temperature=0.0, top_k=1, repetition_penalty=1.0))
    ids = [engine.submit(torch.randint(0, vocab, (prompt_tokens,), generator=generator).tolist(), options)
           for _ in range(batch)]
    scheduler = engine.scheduler
    while any(scheduler.status(i).value in ("queued", "prefill") for i in ids):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall = time.perf_counter()
    start.record()
    for _ in range(steps):
        engine.step()
    stop.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - wall) * 1e3 / steps
    ms = max(start.elapsed_time(stop) / steps, wall_ms)
    produced = sum(len(engine.poll(i).tokens) for i in ids)
    for i in ids:
        engine.cancel(i)
    engine.step()
    step_words = engine.loaded.step
    table_words = batch * step_words.max_pages
    h2d = 4 * (3 * ((batch + 3) // 4 * 4) + (batch + 1 + 3) // 4 * 4 + 2 * ((batch + 3) // 4 * 4) + table_words) \
        + engine.sampler._host_i.numel() * 4 + engine.sampler._host_f.numel() * 4
    d2h = engine.sampler._out_host.numel() * 4
    return ms, h2d, d2h, produced


def run_ours(args) -> dict:
    import torch
    from celeg_b200 import Engine, EngineOptions, kernels
    from celeg_b200.sampling import Sampler
    batch = 8
    raw = model_config(args.layers, args.sizes if args.phase != "all" else "lfm2-1.2b")
    peak, peak_source = peaks()
    max_batch = 64
    context, prompt_tokens, step_tokens = CONTEXT, PROMPT_TOKENS, PREFILL_TOKENS
    if args.phase != "all":             # other context lengths and prompt sizes, for one phase at a time
        context = max(args.context, args.prompt_tokens + args.steps + args.warmup + 8, args.prefill_tokens)
        prompt_tokens = args.prompt_tokens
        step_tokens = max(PREFILL_TOKENS, args.chunk or args.prefill_tokens)
        max_batch = max(1, args.batch)
        raw["max_position_embeddings"] = max(raw["max_position_embeddings"], context)
    folder = model_folder(raw)
    options = EngineOptions(max_active_requests=max_batch, max_batched_tokens=step_tokens,
                            prefill_chunk_tokens=step_tokens, page_tokens=args.page_tokens,
                            logical_kv_pages=max_batch * (-(-context // args.page_tokens)))
    from celeg_b200 import KernelOptions
    engine = Engine(folder, max_context=context, dtype="bfloat16", device="cuda:0", options=options,
                    use_cuda_graph=not args.no_cuda_graph, kernel_options=KernelOptions.from_env())
    loaded = engine.loaded
    sampler = Sampler(raw["vocab_size"], max_batch, max_batch, engine.device)

    if args.phase == "decode":          # a short run of one phase, for profilers
        timer = KernelTimer() if args.kernel_times else None
        ms, launches, context = time_decode(loaded, sampler, args.batch, args.steps, args.warmup, prompt_tokens, 1,
                                            timer=timer)
        record = {"phase": "decode", "sizes": args.sizes, "batch": args.batch, "context_tokens": context,
                  "ms_per_step": round(ms, 4),
                  "tokens_per_s": round(args.batch * 1e3 / ms, 1), "gpu_launches": launches,
                  "hbm_frac": round(decode_bytes(raw, args.batch, context) / (ms * 1e-3) / 1e9 / peak["hbm_gbs"], 4)}
        if timer is not None:
            record["kernel_us_per_step"] = timer.table(args.steps)
        return record
    if args.phase == "prefill":
        prefill_ms = time_prefill(loaded, args.prefill_tokens, max(1, min(args.steps, 5)), 2, args.chunk)
        return {"phase": "prefill", "tokens": args.prefill_tokens, "chunk": args.chunk or args.prefill_tokens,
                "ms": round(prefill_ms, 3),
                "tokens_per_s": round(args.prefill_tokens * 1e3 / prefill_ms, 1),
                "frac": round(prefill_flops(raw, args.prefill_tokens) / (prefill_ms * 1e-3)
                              / (peak["bf16_tflops"] * 1e12), 4)}
    with ClockSampler() as clocks:
        ms, launches, context = time_decode(loaded, sampler, batch, args.steps, args.warmup, PROMPT_TOKENS, 1)
    clock_summary = clocks.summary()
    value = batch * 1e3 / ms
    achieved = decode_bytes(raw, batch, context) / (ms * 1e-3) / 1e9

    prefill_ms = time_prefill(loaded, PREFILL_TOKENS, 3, 2)
    prefill_frac = prefill_flops(raw, PREFILL_TOKENS) / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12)

    points = {}
    for b, key in ((1, "decode_b1"), (64, "decode_b64")):
        point_ms, _, _ = time_decode(loaded, sampler, b, max(8, args.steps // 2), args.warmup, PROMPT_TOKENS, 3 + b)
        points[key] = round(b * 1e3 / point_ms, 1)

    # the host is inside this loop, so a busy core of a shared machine shows at once: two timed regions of K steps
    # each, the better one is reported and both are named
    e2e_runs = [time_e2e(engine, batch, args.steps, args.warmup, PROMPT_TOKENS, 5 + i) for i in range(2)]
    e2e_ms, h2d, d2h, _ = min(e2e_runs, key=lambda run: run[0])

    return {
        "metric": "decode tok/s at batch 8 (LFM2-1.2B sizes, random weights, 512-token prompts, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights (seed 0), uniform-random token ids",
        "impl": "ours",
        "config": {
            "model": "LFM2-1.2B sizes", "global_batch": batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS,
            "parallelism": "single GPU", "vocab_size": raw["vocab_size"], "hidden_size": raw["hidden_size"],
            "layers": raw["num_hidden_layers"], "layers_of_config": FULL_LAYERS,
            "attention_layers": raw["layer_types"].count("full_attention"),
            "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
            "head_dim": raw["head_dim"], "intermediate_size": raw["intermediate_size"],
            "conv_L_cache": raw["conv_L_cache"], "page_tokens": args.page_tokens,
            "cuda_graph": not args.no_cuda_graph, "l2": "inputs larger than L2 (2.3 GB of weights per step)",
        },
        "e2e": {"value": round(batch * 1e3 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step_of_runs": [round(run[0], 4) for run in e2e_runs]},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS * 1e3 / prefill_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(prefill_frac, 4),
                    "peak_tflops": peak["bf16_tflops"], "of": peak_source},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4), "of": peak_source,
                     "context_tokens": context},
        "points": points,
        "clocks": clock_summary,
        "kernel_library": kernels.library_path(),
        "model_fingerprint": loaded.fingerprint,
    }


def percentile(samples, q: float) -> float:
    if not samples:
        return 0.0
    ordered = sorted(samples)
    return ordered[min(len(ordered) - 1, int(q * len(ordered)))]


def drive_workload(engine, prompts, request_options, max_steps: int = 10 ** 9) -> dict:
    """Submits every prompt, then calls ``engine.step()`` until all requests are terminal, polling
    after every step as a client would (celeg's own engine benchmark does the same:
    src/app/benchmark/cuda/concurrent.cpp:50-72). Returns the outputs and what was measured:
    wall time, tokens, steps, time to the first token and between tokens, the page pool's high-water
    mark, preemptions, and where the host's time went per step (celeg's host_prepare_ms /
    gpu_execute_ms / host_commit_ms: src/backend/cuda/packed/execution.cu:200-223). For steps in which
    every live request decodes it also sums the bytes such a step has to read (every weight once, the
    live requests' keys and values and fixed-size state), for the roofline."""
    import torch
    manager = engine.loaded.manager
    scheduler = engine.scheduler
    bytes_per_position = 0
    for group, (k, _v) in zip(manager.groups, zip(engine.loaded.storage.k, engine.loaded.storage.v)):
        bytes_per_position += 2 * k.shape[0] * k.shape[2] * k.shape[4] * k.element_size()
    state_bytes = engine.loaded.storage.slot_elements * 4
    weight_bytes = engine.loaded.model.weight_bytes()
    torch.cuda.synchronize()
    started = time.perf_counter()
    ids = [engine.submit(prompt, options) for prompt, options in zip(prompts, request_options)]
    outputs = {i: [] for i in ids}
    pending = set(ids)
    failed = {}
    decode_steps = 0
    decode_seconds = 0.0
    decode_bytes_sum = 0.0
    decode_rows = 0
    steps = 0
    while pending and steps < max_steps:
        live = [scheduler.requests[i] for i in scheduler.live]
        all_decode = bool(live) and not scheduler.queue and all(r.status.value == "decoding" for r in live)
        positions = sum(r.cache.tokens for r in live if r.cache is not None) if all_decode else 0
        before = time.perf_counter()
        progressed = engine.step()
        after = time.perf_counter()
        steps += 1
        if all_decode:
            decode_steps += 1
            decode_seconds += after - before
            decode_rows += len(live)
            decode_bytes_sum += weight_bytes + positions * bytes_per_position + len(live) * state_bytes
        for request_id in list(pending):
            result = engine.poll(request_id)
            if result.tokens:
                outputs[request_id].extend(result.tokens)
            if result.finished:
                pending.discard(request_id)
                if result.error:
                    failed[request_id] = result.error
                engine.release(request_id)
        if not progressed and pending and not scheduler.has_work():
            raise RuntimeError("the engine made no progress although requests are pending")
    torch.cuda.synchronize()
    wall = time.perf_counter() - started
    metrics = engine.metrics()
    generated = sum(len(tokens) for tokens in outputs.values())
    record = {
        "wall_s": round(wall, 4), "requests": len(ids), "failed": len(failed),
        "prompt_tokens": sum(len(p) for p in prompts), "generated_tokens": generated,
        "tokens_per_s": round((metrics.prefill_tokens + metrics.decode_tokens) / wall, 1),
        "generated_tokens_per_s": round(generated / wall, 1),
        "steps": metrics.steps, "max_step_tokens": metrics.max_step_tokens,
        "max_step_requests": metrics.max_step_requests, "preemptions": metrics.preempted,
        "skipped_for_pages": metrics.skipped_for_pages,
        "ttft_ms": {"mean": round(1e3 * metrics.ttft_seconds_sum / max(1, metrics.ttft_count), 3),
                    "p50": round(1e3 * percentile(metrics.ttft_seconds, 0.50), 3),
                    "p99": round(1e3 * percentile(metrics.ttft_seconds, 0.99), 3)},
        "itl_ms": {"mean": round(1e3 * metrics.itl_seconds_sum / max(1, metrics.itl_count), 3),
                   "p50": round(1e3 * percentile(metrics.itl_seconds, 0.50), 3),
                   "p99": round(1e3 * percentile(metrics.itl_seconds, 0.99), 3)},
        "pages": {"high_water": metrics.pages_high_water, "total": metrics.pages_total,
                  "page_tokens": manager.page_tokens},
        "host_ms_per_step": metrics.host_ms_per_step(),
        "gpu_ms_per_step": round(1e3 * metrics.gpu_seconds / max(1, metrics.steps), 4),
        "wall_ms_per_step": round(1e3 * wall / max(1, metrics.steps), 4),
        "decode_only": {"steps": decode_steps,
                        "ms_per_step": round(1e3 * decode_seconds / max(1, decode_steps), 4),
                        "tokens_per_s": round(decode_rows / decode_seconds, 1) if decode_seconds else 0.0,
                        "gb_per_step": round(decode_bytes_sum / max(1, decode_steps) / 1e9, 4),
                        "achieved_gbs": round(decode_bytes_sum / decode_seconds / 1e9, 1) if decode_seconds else 0.0},
    }
    return {"outputs": [outputs[i] for i in ids], "errors": failed, "record": record}


def run_workload(args) -> dict:
    """One of the two scheduler workloads at full size, through Engine.submit / step / poll."""
    import torch
    from celeg_b200 import Engine, EngineOptions, RequestOptions, SamplingParams, kernels
    spec = WORKLOADS[args.workload]
    raw = dict(spec["config"])
    if args.layers != FULL_LAYERS:
        raw["num_hidden_layers"] = args.layers
        raw["layer_types"] = raw["layer_types"][:args.layers]
    requests = args.requests or spec["requests"]
    new_tokens = args.new_tokens or spec["new_tokens"]
    budget = args.max_batched_tokens or spec["max_batched_tokens"]
    chunk = args.prefill_chunk or spec["prefill_chunk_tokens"]
    peak, peak_source = peaks()
    folder = model_folder(raw)
    options = EngineOptions(max_active_requests=requests, max_batched_tokens=max(budget, requests),
                            prefill_chunk_tokens=chunk, page_tokens=args.page_tokens)
    from celeg_b200 import KernelOptions
    engine = Engine(folder, max_context=spec["context"], dtype="bfloat16", device="cuda:0", options=options,
                    use_cuda_graph=not args.no_cuda_graph, kernel_options=KernelOptions.from_env())
    generator = torch.Generator().manual_seed(11)
    vocab = raw["vocab_size"]

    def batch(count, tag):
        lengths = torch.randint(spec["prompt_min"], spec["prompt_max"] + 1, (count,), generator=generator).tolist()
        prompts = [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in lengths]
        opts = [RequestOptions(max_new_tokens=new_tokens, eos_tokens=(),
                               generation=SamplingParams(temperature=spec["temperature"],
                                                         top_k=50 if spec["temperature"] > 0 else 1,
                                                         top_p=1.0, repetition_penalty=1.0, seed=tag + i + 1))
                for i in range(count)]
        return prompts, opts

    # warm-up: the same number of requests of the same kind (other prompts and lengths from the same
    # distribution), run to their end, so that the library, the graphs of the launch shapes a draining batch
    # goes through and the allocator are past their first use, as in a server that has been up for a while (the
    # requests are finished and released before the timed run)
    if not args.no_warmup_run:
        warm_prompts, warm_options = batch(requests, 10_000)
        drive_workload(engine, warm_prompts, warm_options)
    engine.scheduler.metrics = type(engine.scheduler.metrics)()
    for group in engine.loaded.manager.groups:
        group.pool.high_water = group.pool.used_pages
    launches_before = kernels.LAUNCHES
    prompts, request_options = batch(requests, 0)
    timer = KernelTimer() if args.kernel_times else None
    if timer is not None:
        timer.__enter__()
    with ClockSampler() as clocks:
        result = drive_workload(engine, prompts, request_options)
    if timer is not None:
        timer.__exit__(None, None, None)
    record = result["record"]
    if timer is not None:
        record["kernel_us_per_step"] = timer.table(max(1, record["steps"]))
    decode = record["decode_only"]
    return {
        "workload": args.workload, "impl": "ours", "dtype": "bf16", "model_fingerprint": engine.loaded.fingerprint,
        "data": "synthetic: random weights (seed 0), uniform-random token ids and prompt lengths (seed 11)",
        "config": {"hidden_size": raw["hidden_size"], "layers": raw["num_hidden_layers"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "intermediate_size": raw["intermediate_size"], "vocab_size": vocab,
                   "requests": requests, "prompt_tokens": [spec["prompt_min"], spec["prompt_max"]],
                   "context": spec["context"], "new_tokens": new_tokens, "temperature": spec["temperature"],
                   "max_batched_tokens": options.max_batched_tokens, "prefill_chunk_tokens": chunk,
                   "page_tokens": args.page_tokens, "cuda_graph": not args.no_cuda_graph,
                   "scheduler_policy": options.scheduler_policy.value},
        **record,
        "decode_only_roofline": {"bound": "hbm", "achieved": decode["achieved_gbs"], "peak": peak["hbm_gbs"],
                                 "unit": "GB/s", "frac": round(decode["achieved_gbs"] / peak["hbm_gbs"], 4),
                                 "of": peak_source},
        "gpu_launches": kernels.LAUNCHES - launches_before,
        "clocks": clocks.summary(),
        "errors": list(result["errors"].values())[:3],
    }


def run_reference(args) -> dict:
    """The reference arm: celsowm/celeg's own engine, unmodified, driven through its public C API
    (include/celeg/api.h:142-179) by ``baseline/reference_bench.py`` in a process of its own that loads
    ``baseline/_ref/libceleg.so`` and nothing of this package. ``pip install`` of the checkout is not possible
    (a CMake project without setup.py or pyproject.toml); ``baseline/build_reference.py`` compiles celeg's own
    source lists into that library instead. Same model folder, batch, prompts, steps and warm-up as the other
    arm; every number is end to end (token ids in and out on the host)."""
    library = os.path.join(ROOT, "baseline", "_ref", "libceleg.so")
    if not os.path.isfile(library):
        return {"impl": "reference",
                "unavailable": "baseline/_ref/libceleg.so is not built: celsowm/celeg is a CMake C++/CUDA project that "
                               "pip cannot install; run `python baseline/build_reference.py <celeg checkout>` first"}
    raw = model_config(args.layers)
    folder = model_folder(raw)
    command = [sys.executable, os.path.join(ROOT, "baseline", "reference_bench.py"), "--library", library,
               "--model", folder, "--steps", str(args.steps), "--warmup", str(args.warmup), "--batch", "8",
               "--prompt-tokens", str(PROMPT_TOKENS), "--prefill-tokens", str(PREFILL_TOKENS),
               "--context", str(CONTEXT), "--page-tokens", str(args.page_tokens)]
    with ClockSampler() as clocks:
        try:
            done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=1500)
        except subprocess.TimeoutExpired:
            return {"impl": "reference", "unavailable": "celeg's engine did not finish the workload within 1500 s"}
    lines = [line for line in done.stdout.splitlines() if line.startswith("{")]
    try:
        measured = json.loads(lines[-1])
    except (IndexError, ValueError):
        measured = {"error": (done.stderr or done.stdout).strip().splitlines()[-1:] or ["no output"]}
    if done.returncode != 0 or "error" in measured:
        return {"impl": "reference", "unavailable": f"celeg's engine failed on this workload: {measured.get('error')}"[:600]}
    value = measured["tokens_per_s"]
    return {
        "metric": "decode tok/s at batch 8 (LFM2-1.2B sizes, random weights, 512-token prompts, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(measured["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights (seed 0), uniform-random token ids", "impl": "reference",
        "config": {"model": "LFM2-1.2B sizes", "global_batch": 8, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS,
                   "parallelism": "single GPU", "layers": raw["num_hidden_layers"], "layers_of_config": FULL_LAYERS,
                   "page_tokens": args.page_tokens, "api": "celeg_engine_* over libceleg.so (its worker thread steps)",
                   "timing": "wall clock between polled tokens"},
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "ms_per_step": round(measured["ms_per_step"], 4)},
        "prefill": {"value": round(measured["prefill"]["tokens_per_s"], 1), "tokens": PREFILL_TOKENS,
                    "ms": round(measured["prefill"]["ms"], 3)},
        "points": {key: round(v, 1) for key, v in measured["points"].items()},
        "clocks": clocks.summary(),
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=16)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--layers", type=int, default=FULL_LAYERS,
                        help="fewer layers of the same sizes, when memory or time needs it")
    parser.add_argument("--page-tokens", type=int, default=16)
    parser.add_argument("--no-cuda-graph", action="store_true")
    parser.add_argument("--phase", default="all", choices=["all", "decode", "prefill"],
                        help="run one phase only and print a short record (for profilers)")
    parser.add_argument("--batch", type=int, default=8, help="batch of --phase decode")
    parser.add_argument("--sizes", default="lfm2-1.2b", choices=["lfm2-1.2b", *sorted(WORKLOADS)],
                        help="layer sizes of a --phase run")
    parser.add_argument("--kernel-times", action="store_true",
                        help="--phase decode and --workload: device time per kind of kernel between two events "
                             "each (steps that replay a graph show nothing; use with --no-cuda-graph)")
    parser.add_argument("--prompt-tokens", type=int, default=PROMPT_TOKENS, help="prompt length of --phase decode")
    parser.add_argument("--context", type=int, default=CONTEXT, help="longest request of a --phase run")
    parser.add_argument("--chunk", type=int, default=0,
                        help="--phase prefill: the prompt in portions of this many tokens (0: one step)")
    parser.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="tokens of --phase prefill")
    parser.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                        help="run one of the scheduler workloads through Engine.submit/step/poll and print its record")
    parser.add_argument("--requests", type=int, default=0, help="--workload: number of requests (0: the workload's own)")
    parser.add_argument("--new-tokens", type=int, default=0, help="--workload: tokens to generate per request")
    parser.add_argument("--max-batched-tokens", type=int, default=0, help="--workload: token budget of a step")
    parser.add_argument("--prefill-chunk", type=int, default=0, help="--workload: longest prompt portion")
    parser.add_argument("--no-warmup-run", action="store_true",
                        help="--workload: skip the untimed run before the timed one (for profilers)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        result = run_reference(args)
    elif args.workload:
        result = run_workload(args)
    else:
        result = run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
