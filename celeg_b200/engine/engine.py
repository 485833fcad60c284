"""The Python entry point: an engine over one model folder, with celeg's engine calls
(``ConcurrentEngine``: include/celeg/backend/cuda/concurrency.hpp:36-70; C API
include/celeg/api.h:142-179): submit, step, poll, status, cancel, release, metrics; plus
``generate`` for the common case and ``forward`` for the raw step."""
from __future__ import annotations

import threading
import time
from typing import Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

from ..parts.options import KernelOptions
from ..sampling import Sampler, SamplingParams
from .loading import LoadedModel, load_model
from .scheduler import (EngineOptions, Metrics, PollResult, RequestOptions, RequestStatus, Scheduler,
                        SchedulerPolicy)
from .step import DeviceCheckError, StepEntry, device_error_text


class _Runner:
    """What the scheduler drives: the step function and the sampler. Every launch is bracketed by two
    timing events and followed by a copy of the kernels' error flag to pinned memory; ``collect`` waits
    for the launch's last event, reads both, and raises if a kernel flagged an index that the host
    should have made impossible, so that such a step's logits never become tokens."""

    IN_FLIGHT = 4          # launches whose events and flag copies may be unread at a time (two are)

    def __init__(self, loaded: LoadedModel, sampler: Sampler):
        self.loaded = loaded
        self.sampler = sampler
        self._begin = [torch.cuda.Event(enable_timing=True) for _ in range(self.IN_FLIGHT)]
        self._end = [torch.cuda.Event(enable_timing=True) for _ in range(self.IN_FLIGHT)]
        self._flags = torch.zeros(self.IN_FLIGHT, dtype=torch.int32).pin_memory()
        self._next = 0
        self._sample_seconds = 0.0
        self._gpu_seconds = 0.0
        self._reported = dict(loaded.step.host_seconds)
        # the tokens a step feeds count as seen by their requests: marked on the way into the model, so that
        # the marking is part of the step's graph
        loaded.step.set_before_forward(sampler.mark_step)

    def reset_request(self, slot: int, seed: int) -> None:
        self.sampler.reset_slot(slot, seed)

    def padded_singles(self, count: int) -> int:
        """Rows that ``count`` decoded tokens take in a step that also holds prompt portions (the step function
        pads such a step to a launch shape)."""
        return self.loaded.step.padded_single_rows(count)

    def save_generator(self, slot: int) -> int:
        return self.sampler.get_rng(slot)

    def run(self, entries: Sequence[StepEntry], sample_rows: Sequence[Tuple[int, SamplingParams]]) -> List[int]:
        return self.collect(self.launch(entries, sample_rows))

    def launch(self, entries: Sequence[StepEntry], sample_rows: Sequence[Tuple[int, SamplingParams]],
               tokens_on_device: bool = False, source_rows: Optional[Sequence[int]] = None):
        """Enqueues a step and its draw without waiting. ``tokens_on_device``: the entries' tokens are
        placeholders, the real ones are what the launch before drew: row i of this step takes the token of that
        launch's row ``source_rows[i]`` (None: the same rows in the same order)."""
        step = self.loaded.step
        index = self._next
        self._next = (index + 1) % self.IN_FLIGHT
        self._begin[index].record()
        logits = step.run(entries, token_source=self.sampler.out if tokens_on_device else None,
                          source_rows=source_rows if tokens_on_device else None)
        started = time.perf_counter()
        drawn = self.sampler.launch(logits, sample_rows, also_copy=(self._flags[index:index + 1], step.error_flag))
        self._end[index].record()
        self._sample_seconds += time.perf_counter() - started
        return index, drawn

    def collect(self, handle) -> List[int]:
        index, drawn = handle
        tokens = self.sampler.read(drawn)                  # (waits for the copy of the tokens and of the flag)
        self._end[index].synchronize()
        self._gpu_seconds += self._begin[index].elapsed_time(self._end[index]) * 1e-3
        code = int(self._flags[index])
        if code:
            step = self.loaded.step
            step.error_flag.zero_()
            raise DeviceCheckError(device_error_text(code))
        return tokens

    def report_times(self, metrics: Metrics) -> None:
        """Adds the host seconds spent since the last call, by phase, and the steps' device time."""
        now = self.loaded.step.host_seconds
        for name in ("check", "stage", "forward"):
            setattr(metrics, f"host_{name}_seconds",
                    getattr(metrics, f"host_{name}_seconds") + now[name] - self._reported[name])
        self._reported = dict(now)
        metrics.host_sample_seconds += self._sample_seconds
        metrics.gpu_seconds += self._gpu_seconds
        self._sample_seconds = 0.0
        self._gpu_seconds = 0.0


class Engine:
    def __init__(self, model_path: str, max_context: Optional[int] = None, dtype="bfloat16", device="cuda:0",
                 options: Optional[EngineOptions] = None, use_cuda_graph: bool = True,
                 kernel_options: Optional[KernelOptions] = None):
        self.options = options or EngineOptions()
        self.options.validate()
        opts = self.options
        probe_context = max_context
        cache_tokens = opts.logical_kv_pages * opts.page_tokens if opts.logical_kv_pages else None
        self.loaded = load_model(model_path, dtype=dtype, device=device, max_context=probe_context,
                                 cache_tokens=cache_tokens, page_tokens=opts.page_tokens,
                                 max_requests=opts.max_active_requests,
                                 max_batched_tokens=opts.max_batched_tokens, use_graphs=use_cuda_graph,
                                 kernel_options=kernel_options)
        self.device = self.loaded.runtime.device
        self.max_context = self.loaded.step.max_context
        # (one slot more than the manager gives out: the storage's spare slot, see CacheStorage)
        self.sampler = Sampler(self.loaded.model.vocab_size, opts.max_active_requests + 1,
                               opts.max_active_requests, self.device)
        self.scheduler = Scheduler(self.loaded.manager, _Runner(self.loaded, self.sampler), opts,
                                   self.max_context, self.loaded.model.vocab_size,
                                   default_eos=self.loaded.spec.eos_token_ids)
        self._lock = threading.RLock()
        self._worker: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._wake = threading.Condition(self._lock)

    # ---------------------------------------------------------- celeg's engine calls
    def submit(self, prompt: Sequence[int], options: Optional[RequestOptions] = None, **kwargs) -> int:
        """``kwargs``: any field of RequestOptions (max_new_tokens, eos_tokens, priority) or of
        SamplingParams (temperature, top_k, top_p, repetition_penalty, seed)."""
        options = _request_options(options, kwargs)
        with self._wake:
            request_id = self.scheduler.submit(prompt, options)
            self._wake.notify_all()
            return request_id

    def step(self) -> bool:
        with torch.cuda.device(self.device), self._lock:
            return self.scheduler.step()

    def poll(self, request_id: int, max_tokens: int = 0) -> PollResult:
        with self._lock:
            return self.scheduler.poll(request_id, max_tokens)

    def status(self, request_id: int) -> RequestStatus:
        with self._lock:
            return self.scheduler.status(request_id)

    def cancel(self, request_id: int) -> bool:
        with self._lock:
            return self.scheduler.cancel(request_id)

    def release(self, request_id: int) -> bool:
        with self._lock:
            return self.scheduler.release(request_id)

    def metrics(self) -> Metrics:
        with self._lock:
            return self.scheduler.metrics

    # ------------------------------------------------------------- worker thread
    def start(self) -> None:
        """Run ``step()`` on a worker thread until :meth:`stop` (celeg src/runtime/concurrency/worker.cpp:48-67)."""
        if self._worker is not None:
            return
        self._stop.clear()

        def loop():
            while not self._stop.is_set():
                if not self.step():
                    with self._wake:
                        if not self.scheduler.has_work():
                            self._wake.wait(timeout=0.01)

        self._worker = threading.Thread(target=loop, name="celeg-b200-engine", daemon=True)
        self._worker.start()

    def stop(self) -> None:
        if self._worker is None:
            return
        self._stop.set()
        with self._wake:
            self._wake.notify_all()
        self._worker.join()
        self._worker = None

    def running(self) -> bool:
        return self._worker is not None

    # ----------------------------------------------------------------- shortcuts
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 options: Optional[RequestOptions] = None, **kwargs):
        """Token ids in, generated token ids out. One prompt gives one list, several give a list of
        lists. Runs ``step()`` on the calling thread until all are terminal."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        batch = [prompts] if single else list(prompts)
        ids = [self.submit(prompt, _request_options(options, dict(kwargs))) for prompt in batch]
        outputs: Dict[int, List[int]] = {i: [] for i in ids}
        pending = set(ids)
        while pending:
            progressed = self.step() if self._worker is None else True
            for request_id in list(pending):
                result = self.poll(request_id)
                outputs[request_id].extend(result.tokens)
                if result.finished:
                    pending.discard(request_id)
                    if result.status is RequestStatus.FAILED:
                        raise RuntimeError(f"request {request_id} failed: {result.error}")
                    self.release(request_id)
            if not progressed and pending:
                raise RuntimeError("the engine made no progress although requests are pending")
        out = [outputs[i] for i in ids]
        return out[0] if single else out

    def forward(self, entries: Iterable[Union[StepEntry, dict]]) -> torch.Tensor:
        """The raw step: logits [wanted, vocab] for a batch of entries, without the scheduler.
        Requests are begun on first use; end them with :meth:`end`."""
        batch = [e if isinstance(e, StepEntry) else StepEntry(e["id"], e["tokens"], e.get("want", ()))
                 for e in entries]
        with torch.cuda.device(self.device), self._lock:
            return self.loaded.step.run(batch, auto_begin=True)

    def end(self, request_id) -> None:
        with self._lock:
            self.loaded.step.end(request_id)


def _request_options(options: Optional[RequestOptions], overrides: dict) -> RequestOptions:
    import dataclasses
    options = options or RequestOptions()
    request_fields = {f.name for f in dataclasses.fields(RequestOptions)} - {"generation"}
    sampling_fields = {f.name for f in dataclasses.fields(SamplingParams)}
    request_kw = {k: v for k, v in overrides.items() if k in request_fields}
    sampling_kw = {k: v for k, v in overrides.items() if k in sampling_fields}
    unknown = set(overrides) - request_fields - sampling_fields
    if unknown:
        raise TypeError(f"unknown request option(s): {', '.join(sorted(unknown))}")
    generation = dataclasses.replace(options.generation, **sampling_kw) if sampling_kw else options.generation
    return dataclasses.replace(options, generation=generation, **request_kw)
