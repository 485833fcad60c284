"""The C interface (include/celeg_b200/api.h). On the GPU: a tiny model is driven through the exported C
symbols alone, once from this process with ctypes (the running interpreter is used) and once from a C
program compiled here with gcc (the library starts an interpreter of its own), and the tokens are the plain
model's. Without a GPU: sizes of option structs, defaults, and that a failed create says why."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import (POINTER, Structure, byref, c_char_p, c_double, c_float, c_int, c_int32, c_size_t, c_uint32,
                    c_uint64, c_void_p)

import numpy as np
import pytest

ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir)


class Generation(Structure):
    _fields_ = [("struct_size", c_uint32), ("temperature", c_float), ("top_k", c_int32), ("top_p", c_float),
                ("repetition_penalty", c_float), ("seed", c_uint64)]


class EngineOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("max_context", c_int32), ("dtype", c_int32), ("device", c_int32),
                ("cuda_graph", c_int32), ("max_active_requests", c_int32), ("max_batched_tokens", c_int32),
                ("prefill_chunk_tokens", c_int32), ("page_tokens", c_int32), ("logical_kv_pages", c_uint64),
                ("scheduler_policy", c_int32)]


class RequestOptions(Structure):
    _fields_ = [("struct_size", c_uint32), ("max_new_tokens", c_uint32), ("eos_token_id", c_int32),
                ("priority", c_int32), ("generation", Generation)]


class Metrics(Structure):
    _fields_ = ([("struct_size", c_uint32)] +
                [(name, c_uint64) for name in ("submitted", "completed", "cancelled", "failed", "preempted", "steps",
                                               "prefill_tokens", "decode_tokens", "active_requests", "queued_requests",
                                               "pages_used", "pages_total", "pages_high_water")] +
                [("ttft_ms_sum", c_double), ("ttft_samples", c_uint64), ("itl_ms_sum", c_double),
                 ("itl_samples", c_uint64), ("host_ms_sum", c_double), ("gpu_ms_sum", c_double)])


@pytest.fixture(scope="module")
def api():
    from celeg_b200.capi.build import ensure_built
    lib = ctypes.CDLL(ensure_built())
    lib.celeg_b200_engine_create.restype = c_void_p
    lib.celeg_b200_engine_create.argtypes = [c_char_p, POINTER(EngineOptions)]
    lib.celeg_b200_engine_destroy.argtypes = [c_void_p]
    lib.celeg_b200_engine_submit.argtypes = [c_void_p, POINTER(c_int32), c_size_t, POINTER(RequestOptions),
                                             POINTER(c_uint64)]
    lib.celeg_b200_engine_poll.argtypes = [c_void_p, c_uint64, POINTER(c_int32), c_size_t, POINTER(c_size_t),
                                           POINTER(c_int)]
    lib.celeg_b200_engine_status.argtypes = [c_void_p, c_uint64, POINTER(c_int)]
    lib.celeg_b200_engine_cancel.argtypes = [c_void_p, c_uint64]
    lib.celeg_b200_engine_release.argtypes = [c_void_p, c_uint64]
    lib.celeg_b200_engine_step.argtypes = [c_void_p, POINTER(c_int)]
    lib.celeg_b200_engine_get_metrics.argtypes = [c_void_p, POINTER(Metrics)]
    lib.celeg_b200_engine_fingerprint.argtypes = [c_void_p, c_char_p, c_size_t]
    lib.celeg_b200_engine_last_error.restype = c_char_p
    lib.celeg_b200_engine_last_error.argtypes = [c_void_p]
    lib.celeg_b200_engine_options_init.argtypes = [POINTER(EngineOptions)]
    lib.celeg_b200_request_options_init.argtypes = [POINTER(RequestOptions)]
    return lib


def test_option_structs_carry_their_size_and_celegs_defaults(api):
    options = EngineOptions()
    api.celeg_b200_engine_options_init(byref(options))
    assert options.struct_size == ctypes.sizeof(EngineOptions)
    assert (options.max_active_requests, options.max_batched_tokens, options.prefill_chunk_tokens,
            options.page_tokens, options.cuda_graph, options.dtype) == (8, 512, 256, 16, 1, 0)
    request = RequestOptions()
    api.celeg_b200_request_options_init(byref(request))
    assert request.struct_size == ctypes.sizeof(RequestOptions)
    assert request.generation.struct_size == ctypes.sizeof(Generation)
    assert (request.max_new_tokens, request.eos_token_id, request.generation.top_k, request.generation.seed) == (128, -1, 50, 1)
    assert abs(request.generation.temperature - 0.1) < 1e-6 and abs(request.generation.repetition_penalty - 1.05) < 1e-6


def test_a_failed_create_says_why(api, tmp_path):
    options = EngineOptions()
    api.celeg_b200_engine_options_init(byref(options))
    assert api.celeg_b200_engine_create(str(tmp_path / "nothing_here").encode(), byref(options)) is None
    assert b"config.json" in api.celeg_b200_engine_last_error(None)
    options.struct_size = 8                                  # a caller built against an older, smaller struct
    assert api.celeg_b200_engine_create(b"x", byref(options)) is None
    assert b"smaller" in api.celeg_b200_engine_last_error(None)
    assert api.celeg_b200_engine_create(None, byref(options)) is None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [1, 0])
def test_tiny_model_through_the_c_symbols(api, tmp_path, dtype):
    import plain_lfm2
    from tiny_models import write_tiny
    folder = write_tiny(tmp_path, "A")
    config, weights = plain_lfm2.load_model_folder(folder)
    rng = np.random.default_rng(70)
    prompts = [rng.integers(0, config["vocab_size"], size=n).tolist() for n in (5, 23, 40)]
    options = EngineOptions()
    api.celeg_b200_engine_options_init(byref(options))
    options.dtype = dtype
    options.max_active_requests = 4
    options.max_batched_tokens = 32
    options.prefill_chunk_tokens = 9
    engine = api.celeg_b200_engine_create(folder.encode(), byref(options))
    assert engine, api.celeg_b200_engine_last_error(None)
    ids = []
    for prompt in prompts:
        request = RequestOptions()
        api.celeg_b200_request_options_init(byref(request))
        request.max_new_tokens = 12
        request.eos_token_id = -2
        request.generation.temperature = 0.0
        request.generation.top_k = 1
        request.generation.repetition_penalty = 1.0
        request_id = c_uint64(0)
        array = (c_int32 * len(prompt))(*prompt)
        assert api.celeg_b200_engine_submit(engine, array, len(prompt), byref(request), byref(request_id)) == 0
        ids.append(request_id.value)
    status = c_int(-1)
    assert api.celeg_b200_engine_status(engine, ids[0], byref(status)) == 0 and status.value == 0     # queued
    outputs = {i: [] for i in ids}
    buffer = (c_int32 * 5)()                                     # smaller than an output: several polls drain it
    done = set()
    for _ in range(500):
        progressed = c_int(0)
        assert api.celeg_b200_engine_step(engine, byref(progressed)) == 0, api.celeg_b200_engine_last_error(engine)
        for i in ids:
            count, finished = c_size_t(0), c_int(0)
            assert api.celeg_b200_engine_poll(engine, i, buffer, 5, byref(count), byref(finished)) == 0
            outputs[i].extend(buffer[:count.value])
            if finished.value:
                done.add(i)
        if len(done) == len(ids):
            break
    assert len(done) == len(ids)
    for i, prompt in zip(ids, prompts):
        want = plain_lfm2.generate(config, weights, prompt, 12, eos_tokens=())
        if dtype == 1:
            assert outputs[i] == want
        else:
            assert len(outputs[i]) == 12 and outputs[i][:3] == want[:3]
    # errors: an unknown request, an option out of range, a struct that is too small
    count, finished = c_size_t(0), c_int(0)
    assert api.celeg_b200_engine_poll(engine, 999, buffer, 5, byref(count), byref(finished)) == 4      # NOT_FOUND
    assert b"999" in api.celeg_b200_engine_last_error(engine)
    bad = RequestOptions()
    api.celeg_b200_request_options_init(byref(bad))
    bad.generation.top_k = 0
    request_id = c_uint64(0)
    array = (c_int32 * 3)(1, 2, 3)
    assert api.celeg_b200_engine_submit(engine, array, 3, byref(bad), byref(request_id)) == 1           # INVALID_ARGUMENT
    assert b"top_k" in api.celeg_b200_engine_last_error(engine)
    bad.struct_size = 4
    assert api.celeg_b200_engine_submit(engine, array, 3, byref(bad), byref(request_id)) == 1
    assert api.celeg_b200_engine_release(engine, ids[0]) == 0
    assert api.celeg_b200_engine_release(engine, ids[0]) == 4
    metrics = Metrics()
    metrics.struct_size = ctypes.sizeof(Metrics)
    assert api.celeg_b200_engine_get_metrics(engine, byref(metrics)) == 0
    assert metrics.completed == 3 and metrics.prefill_tokens == 68 and metrics.pages_used == 0
    assert metrics.pages_high_water > 0 and metrics.gpu_ms_sum > 0
    text = ctypes.create_string_buffer(80)
    assert api.celeg_b200_engine_fingerprint(engine, text, 80) == 0 and len(text.value) == 64
    assert api.celeg_b200_engine_fingerprint(engine, text, 10) == 3                                     # BUFFER_TOO_SMALL
    api.celeg_b200_engine_destroy(engine)


@pytest.mark.gpu
def test_a_c_program_drives_the_engine(tmp_path):
    """A program that knows the header only, compiled with gcc: the library starts its own interpreter."""
    import plain_lfm2
    from celeg_b200.capi.build import ensure_built
    from tiny_models import write_tiny
    library = ensure_built()
    folder = write_tiny(tmp_path, "B")
    config, weights = plain_lfm2.load_model_folder(folder)
    program = str(tmp_path / "drive_engine")
    build = subprocess.run(["gcc", "-std=c11", "-O1", "-I", os.path.join(ROOT, "include"),
                            os.path.join(ROOT, "tests", "capi", "drive_engine.c"), "-o", program,
                            f"-L{os.path.dirname(library)}", f"-Wl,-rpath,{os.path.dirname(library)}",
                            "-lceleg_b200_api"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    prompt = np.random.default_rng(71).integers(0, config["vocab_size"], size=19).tolist()
    env = {key: value for key, value in os.environ.items() if not key.startswith("PYTHON")}
    run = subprocess.run([program, folder, "1", "10", *[str(t) for t in prompt]], capture_output=True, text=True,
                         timeout=600, env=env)
    assert run.returncode == 0, run.stdout + run.stderr
    lines = dict(line.split(":", 1) for line in run.stdout.strip().splitlines())
    assert [int(t) for t in lines["tokens"].split()] == plain_lfm2.generate(config, weights, prompt, 10, eos_tokens=())
    assert len(lines["fingerprint"].strip()) == 64
