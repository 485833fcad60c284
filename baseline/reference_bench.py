#!/usr/bin/env python3
"""The reference arm of bench.py: drives celsowm/celeg's own, unmodified engine through its public C API
(include/celeg/api.h:142-179: celeg_engine_create / _submit / _step / _poll) from ``baseline/_ref/libceleg.so``,
which ``baseline/build_reference.py`` builds from the reference checkout. This process loads that library only:
nothing of this repository's package, kernels or engine is imported here. Token ids go in and come out on the
host, so every number is end to end: wall clock between tokens arriving at ``celeg_engine_poll``.

  python baseline/reference_bench.py --model DIR --steps K --warmup W   -> one JSON line

Same workload as bench.py's own arm: ``batch`` requests of 512 random prompt tokens, greedy, K timed tokens per
request after W untimed ones; a prompt of 2,048 tokens alone (time to its first token); decode at batch 1 and 64.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import random
import sys
import time
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_float, c_int, c_int32, c_size_t, c_uint32,
                    c_uint64, c_void_p)

HERE = os.path.dirname(os.path.abspath(__file__))


class GenerationOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("temperature", c_float), ("top_k", c_int32), ("top_p", c_float),
                ("repetition_penalty", c_float), ("seed", c_uint64)]


class CudaModelOptions(Structure):
    _fields_ = [("flags", c_uint32), ("weight_mode", c_int32), ("kv_cache_mode", c_int32), ("gemm_backend", c_int32),
                ("attention_mode", c_int32), ("attention_chunk_tokens", c_int32),
                ("attention_auto_threshold", c_int32), ("lt_workspace_mb", c_int32), ("lt_heuristics", c_int32)]


class CudaEngineOptions(Structure):
    _fields_ = [("max_active_requests", c_int32), ("max_batched_tokens", c_int32), ("prefill_chunk_tokens", c_int32),
                ("page_tokens", c_int32), ("logical_kv_pages", c_uint64), ("scheduler_policy", c_int32)]


class CudaBackendOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("model", CudaModelOptions), ("engine", CudaEngineOptions)]


class EngineOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("backend_id", c_char_p), ("max_context", c_int32),
                ("backend_options", c_void_p), ("backend_options_size", c_uint32), ("generation", GenerationOptions)]


class RequestOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("max_new_tokens", c_uint32), ("eos_token_id", c_int32),
                ("priority", c_int32), ("generation", GenerationOptions)]


def load_library(path: str):
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    lib.celeg_engine_options_init.argtypes = [POINTER(EngineOptions), c_char_p, c_void_p, c_uint32]
    lib.celeg_cuda_backend_options_init.argtypes = [POINTER(CudaBackendOptions)]
    lib.celeg_request_options_init.argtypes = [POINTER(RequestOptions)]
    lib.celeg_engine_create.restype = c_void_p
    lib.celeg_engine_create.argtypes = [c_char_p, POINTER(EngineOptions)]
    lib.celeg_engine_destroy.argtypes = [c_void_p]
    lib.celeg_engine_submit.argtypes = [c_void_p, POINTER(c_int32), c_size_t, POINTER(RequestOptions),
                                        POINTER(c_uint64)]
    lib.celeg_engine_poll.argtypes = [c_void_p, c_uint64, POINTER(c_int32), c_size_t, POINTER(c_size_t),
                                      POINTER(c_int)]
    lib.celeg_engine_status.argtypes = [c_void_p, c_uint64, POINTER(c_int)]
    lib.celeg_engine_cancel.argtypes = [c_void_p, c_uint64]
    lib.celeg_engine_step.argtypes = [c_void_p, POINTER(c_int)]
    lib.celeg_engine_last_error.restype = c_char_p
    lib.celeg_engine_last_error.argtypes = [c_void_p]
    return lib


class ReferenceEngine:
    def __init__(self, lib, model: str, context: int, max_requests: int, max_batched_tokens: int, chunk: int,
                 page_tokens: int):
        self.lib = lib
        backend = CudaBackendOptions()
        lib.celeg_cuda_backend_options_init(byref(backend))
        backend.engine.max_active_requests = max_requests
        backend.engine.max_batched_tokens = max_batched_tokens
        backend.engine.prefill_chunk_tokens = chunk
        backend.engine.page_tokens = page_tokens
        # celeg_cuda_backend_options_init asks for automatic attention, which celeg refuses without its
        # fast-attention switch, and the C API has no field for that switch ("segmented or automatic attention
        # requires --fast-attention", src/backend/cuda/execution_plan.cpp:38): single-pass attention is what the
        # API can run
        backend.model.attention_mode = 0
        self._backend = backend
        options = EngineOptions()
        lib.celeg_engine_options_init(byref(options), b"cuda", ctypes.addressof(backend), ctypes.sizeof(backend))
        options.max_context = context
        self.handle = lib.celeg_engine_create(model.encode(), byref(options))
        if not self.handle:
            raise RuntimeError("celeg_engine_create failed: " + (lib.celeg_engine_last_error(None) or b"").decode())
        self._out = (c_int32 * 4096)()

    def check(self, status: int, what: str) -> None:
        if status != 0:
            raise RuntimeError(f"{what} returned status {status}: "
                               f"{(self.lib.celeg_engine_last_error(self.handle) or b'').decode()}")

    def submit(self, tokens, max_new_tokens: int) -> int:
        request = RequestOptions()
        self.lib.celeg_request_options_init(byref(request))
        request.max_new_tokens = max_new_tokens
        request.eos_token_id = -1                        # no token ends a request: they run to max_new_tokens
        request.generation.temperature = 0.0
        request.generation.top_k = 1
        request.generation.top_p = 1.0
        request.generation.repetition_penalty = 1.0
        array = (c_int32 * len(tokens))(*tokens)
        request_id = c_uint64(0)
        self.check(self.lib.celeg_engine_submit(self.handle, array, len(tokens), byref(request), byref(request_id)),
                   "celeg_engine_submit")
        return request_id.value

    def step(self) -> bool:
        progressed = c_int(0)
        self.check(self.lib.celeg_engine_step(self.handle, byref(progressed)), "celeg_engine_step")
        return bool(progressed.value)

    def status(self, request_id: int) -> int:
        value = c_int(0)
        self.check(self.lib.celeg_engine_status(self.handle, request_id, byref(value)), "celeg_engine_status")
        return value.value

    def poll(self, request_id: int):
        count, finished = c_size_t(0), c_int(0)
        self.check(self.lib.celeg_engine_poll(self.handle, request_id, self._out, len(self._out), byref(count),
                                              byref(finished)), "celeg_engine_poll")
        return list(self._out[:count.value]), bool(finished.value)

    def cancel(self, request_id: int) -> None:
        self.lib.celeg_engine_cancel(self.handle, request_id)

    def close(self) -> None:
        if self.handle:
            self.lib.celeg_engine_destroy(self.handle)
            self.handle = None


def submit_one_by_one(engine: ReferenceEngine, prompts, max_new_tokens: int):
    """Submits the prompts one after the other, each when the one before has left prefill.

    On B200 celeg's ragged prefill pass (two or more requests' prompt portions in one pass) ended with "an
    illegal memory access was encountered" (reported at src/backend/cuda/kernels/embedding.cu:176) every time it
    ran, with 8 requests of 512 tokens under token budgets of 512 and of 2,048; a single request's prompt and
    decoding rows of several requests ran clean. The C API has no switch for that pass, so the client keeps at
    most one request in prefill at a time, as staggered arrivals would."""
    ids = []
    for prompt in prompts:
        request = engine.submit(prompt, max_new_tokens)
        deadline = time.perf_counter() + 300.0
        while engine.status(request) in (0, 1):
            if time.perf_counter() > deadline:
                raise RuntimeError("a request did not leave prefill within 300 s")
            time.sleep(0.0005)
        if engine.status(request) == 5:
            raise RuntimeError("celeg's engine failed a request during its prompt")
        ids.append(request)
    return ids


def warm_lanes(engine: ReferenceEngine, vocab: int, batch: int, rng: random.Random) -> None:
    """celeg sets a lane up at its first use (seconds each); have ``batch`` lanes live at once before timing."""
    ids = submit_one_by_one(engine, [[rng.randrange(vocab) for _ in range(16)] for _ in range(batch)], 30000)
    for i in ids:
        engine.cancel(i)
    wait_until_idle(engine, ids)


def time_decode(engine: ReferenceEngine, vocab: int, batch: int, prompt_tokens: int, steps: int, warmup: int,
                rng: random.Random):
    """celeg's engine runs its steps on its own worker thread when it is created through the C API (the API has
    no switch for it: include/celeg/backend/cuda/concurrency.hpp:20, src/backend/cuda/runtime/engine.cpp:98), so
    the client only submits and polls. All requests decode together; the clock starts when every request has
    given ``warmup`` tokens more than it had when the last one began to decode, and stops ``steps`` tokens per
    request later."""
    prompts = [[rng.randrange(vocab) for _ in range(prompt_tokens)] for _ in range(batch)]
    ids = submit_one_by_one(engine, prompts, 3000)
    got = {i: 0 for i in ids}
    floor = None
    started = None
    deadline = time.perf_counter() + 300.0
    while True:
        finished_any = False
        for i in ids:
            tokens, finished = engine.poll(i)
            got[i] += len(tokens)
            finished_any = finished_any or finished
        if floor is None:
            floor = dict(got)                     # tokens each request had when all were decoding
        least = min(got[i] - floor[i] for i in ids)
        now = time.perf_counter()
        if started is None and least >= warmup:
            started, base = now, sum(got.values())
        if least >= warmup + steps:
            elapsed = now - started
            produced = sum(got.values()) - base
            break
        if finished_any:
            raise RuntimeError("a request ended before the timed tokens were out (failed, or out of new tokens)")
        if now > deadline:
            raise RuntimeError(f"only {least} tokens per request after 300 s")
        time.sleep(0.0002)
    for i in ids:
        engine.cancel(i)
    wait_until_idle(engine, ids)
    return 1e3 * elapsed * batch / produced, produced


def wait_until_idle(engine: ReferenceEngine, ids) -> None:
    deadline = time.perf_counter() + 60.0
    while any(engine.status(i) in (0, 1, 2) for i in ids) and time.perf_counter() < deadline:
        time.sleep(0.001)


def time_prefill(engine: ReferenceEngine, vocab: int, tokens: int, repeats: int, rng: random.Random) -> float:
    """Time from submitting a prompt of ``tokens`` tokens to its first token on the host; best of ``repeats``."""
    best = None
    for attempt in range(repeats + 1):
        prompt = [rng.randrange(vocab) for _ in range(tokens)]
        started = time.perf_counter()
        request = engine.submit(prompt, 1)
        deadline = started + 600.0
        while True:
            produced, finished = engine.poll(request)
            if produced or finished:
                break
            if time.perf_counter() > deadline:
                raise RuntimeError("no first token after 600 s")
            time.sleep(0.0001)
        elapsed = 1e3 * (time.perf_counter() - started)
        wait_until_idle(engine, [request])
        if attempt > 0:
            best = elapsed if best is None else min(best, elapsed)
    return best


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--library", default=os.path.join(HERE, "_ref", "libceleg.so"))
    parser.add_argument("--model", required=True)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=16)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-tokens", type=int, default=512)
    parser.add_argument("--prefill-tokens", type=int, default=2048)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--page-tokens", type=int, default=16)
    parser.add_argument("--points", default="1")
    args = parser.parse_args()
    with open(os.path.join(args.model, "config.json"), "r", encoding="utf-8") as handle:
        vocab = int(json.load(handle)["vocab_size"])
    lib = load_library(args.library)
    rng = random.Random(1)
    points = [int(p) for p in args.points.split(",") if p]
    # celeg's own defaults for the token budget of a pass (512) and the longest prompt portion (256); a context
    # that leaves the lanes' first use (warm_lanes) room to decode while the other lanes start
    engine = ReferenceEngine(lib, args.model, max(args.context, 32768), max(args.batch, *points, 1), 512, 256,
                             args.page_tokens)
    warm_lanes(engine, vocab, max(args.batch, *points, 1), rng)
    ms, produced = time_decode(engine, vocab, args.batch, args.prompt_tokens, args.steps, args.warmup, rng)
    result = {"ms_per_step": ms, "tokens_per_s": args.batch * 1e3 / ms, "produced": produced}
    prefill_ms = time_prefill(engine, vocab, args.prefill_tokens, 2, rng)
    result["prefill"] = {"tokens": args.prefill_tokens, "ms": prefill_ms,
                         "tokens_per_s": args.prefill_tokens * 1e3 / prefill_ms}
    result["points"] = {}
    for batch in points:
        point_ms, _ = time_decode(engine, vocab, batch, args.prompt_tokens, max(8, args.steps // 2), args.warmup, rng)
        result["points"][f"decode_b{batch}"] = batch * 1e3 / point_ms
    engine.close()
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    try:
        sys.exit(main())
    except Exception as error:                       # the caller prints this as the reason
        print(json.dumps({"error": f"{type(error).__name__}: {error}"}))
        sys.exit(1)
