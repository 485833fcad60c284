"""What the C interface (include/celeg_b200/api.h) calls: plain functions over simple values, so that the C
side needs no knowledge of the engine's classes. Every function raises on failure; the C side turns
``ValueError`` / ``TypeError`` into INVALID_ARGUMENT, ``KeyError`` into NOT_FOUND, a missing kernel library
into BACKEND_UNAVAILABLE and everything else into ERROR, with the message kept for ``last_error``."""
from __future__ import annotations

from typing import List, Optional, Tuple

_STATUS_CODE = {"queued": 0, "prefill": 1, "decoding": 2, "finished": 3, "cancelled": 4, "failed": 5}
NO_EOS = -2            # request option eos_token_id: no token ends the request
MODEL_EOS = -1         # the stop ids of the model's configuration


def create(model_path: str, max_context: int, dtype: int, device: int, cuda_graph: int, max_active_requests: int,
           max_batched_tokens: int, prefill_chunk_tokens: int, page_tokens: int, logical_kv_pages: int,
           scheduler_policy: int):
    from ..engine.engine import Engine
    from ..engine.scheduler import EngineOptions, SchedulerPolicy
    if dtype not in (0, 1):
        raise ValueError(f"dtype must be 0 (bfloat16) or 1 (float32), got {dtype}")
    if scheduler_policy not in (0, 1):
        raise ValueError(f"scheduler_policy must be 0 or 1, got {scheduler_policy}")
    options = EngineOptions(max_active_requests=max_active_requests, max_batched_tokens=max_batched_tokens,
                            prefill_chunk_tokens=prefill_chunk_tokens, page_tokens=page_tokens,
                            logical_kv_pages=logical_kv_pages,
                            scheduler_policy=(SchedulerPolicy.GUARANTEED_NO_EVICT, SchedulerPolicy.MAX_UTILIZATION)[scheduler_policy])
    return Engine(model_path, max_context=max_context or None, dtype="bfloat16" if dtype == 0 else "float32",
                  device=f"cuda:{device}", options=options, use_cuda_graph=bool(cuda_graph))


def submit(engine, tokens: List[int], max_new_tokens: int, eos_token_id: int, priority: int, temperature: float,
           top_k: int, top_p: float, repetition_penalty: float, seed: int) -> int:
    from ..engine.scheduler import RequestOptions
    from ..sampling.params import SamplingParams
    if eos_token_id == MODEL_EOS:
        eos = None
    elif eos_token_id == NO_EOS:
        eos = ()
    elif eos_token_id >= 0:
        eos = (eos_token_id,)
    else:
        raise ValueError(f"eos_token_id must be a token id, -1 (the model's) or -2 (none), got {eos_token_id}")
    options = RequestOptions(max_new_tokens=max_new_tokens, eos_tokens=eos, priority=priority,
                             generation=SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p,
                                                       repetition_penalty=repetition_penalty, seed=seed))
    return engine.submit(tokens, options)


def poll(engine, request_id: int, capacity: int) -> Tuple[List[int], bool]:
    result = engine.poll(request_id, capacity)
    return result.tokens, bool(result.finished)


def status(engine, request_id: int) -> int:
    return _STATUS_CODE[engine.status(request_id).value]


def cancel(engine, request_id: int) -> None:
    if not engine.cancel(request_id):
        raise KeyError(f"request {request_id} is unknown or already terminal")


def release(engine, request_id: int) -> None:
    if not engine.release(request_id):
        raise KeyError(f"request {request_id} is unknown or not terminal")


def step(engine) -> bool:
    return bool(engine.step())


def start(engine) -> None:
    engine.start()


def stop(engine) -> None:
    engine.stop()


def fingerprint(engine) -> str:
    return engine.loaded.fingerprint


def metrics(engine) -> tuple:
    m = engine.metrics()
    host = m.host_plan_seconds + m.host_launch_seconds + m.host_commit_seconds
    return (m.submitted, m.completed, m.cancelled, m.failed, m.preempted, m.steps, m.prefill_tokens, m.decode_tokens,
            m.active_requests, m.queued_requests, m.pages_used, m.pages_total, m.pages_high_water,
            1e3 * m.ttft_seconds_sum, m.ttft_count, 1e3 * m.itl_seconds_sum, m.itl_count, 1e3 * host,
            1e3 * m.gpu_seconds)


def destroy(engine) -> None:
    engine.stop()


def classify(exc: BaseException) -> int:
    """The status code of include/celeg_b200/api.h for an exception."""
    from ..kernels import KernelLibraryError
    if isinstance(exc, KernelLibraryError):
        return 5
    if isinstance(exc, KeyError):
        return 4
    if isinstance(exc, (ValueError, TypeError)):
        return 1
    return 2
