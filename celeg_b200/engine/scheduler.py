"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees. It is host logic over two collaborators, so it runs without a GPU in tests:

* a :class:`~celeg_b200.cache.manager.CacheManager` (slots and pages), and
* a *runner* with ``run(entries, sample_rows) -> list[int]``: runs one step over the entries and
  returns one sampled token per entry that wants one, plus ``reset_request(slot, seed)`` and
  ``save_generator(slot)`` / ``restore_generator(slot, state)`` for per-request sampling state.

Policy, names and defaults follow celeg's CUDA engine
(include/celeg/backend/cuda/concurrency.hpp:18-32; admission
src/backend/cuda/runtime/request_lifecycle.cpp:103-198; prefill budget
src/backend/cuda/runtime/prefill_scheduler.cpp:7-37; decode and page growth
src/backend/cuda/runtime/decode_scheduler.cpp:10-99), with two differences: prompt portions and
decoded tokens go into ONE step, and a pool that cannot serve any live request is resolved by
preempting one request instead of stalling (see :meth:`Scheduler._break_deadlock`).
"""
from __future__ import annotations

import enum
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager, RequestCache
from ..cache.pages import OutOfPages
from ..sampling.params import SamplingParams
from .step import StepEntry


class RequestStatus(enum.Enum):
    QUEUED = "queued"
    PREFILL = "prefill"
    DECODING = "decoding"
    FINISHED = "finished"
    CANCELLED = "cancelled"
    FAILED = "failed"

    @property
    def terminal(self) -> bool:
        return self in (RequestStatus.FINISHED, RequestStatus.CANCELLED, RequestStatus.FAILED)


class SchedulerPolicy(enum.Enum):
    GUARANTEED_NO_EVICT = "guaranteed-no-evict"   # reserve prompt + max_new_tokens at admission
    MAX_UTILIZATION = "max-utilization"           # reserve prompt + one page, grow while decoding


@dataclass
class EngineOptions:
    """celeg's ``ConcurrentEngineOptions`` (same names and defaults) for what this engine keeps."""
    max_active_requests: int = 8
    max_batched_tokens: int = 512
    prefill_chunk_tokens: int = 256
    page_tokens: int = 16
    logical_kv_pages: int = 0                    # 0: ceil(max_context / page_tokens) * max_active_requests
    scheduler_policy: SchedulerPolicy = SchedulerPolicy.GUARANTEED_NO_EVICT
    # enqueue the step after the one whose tokens are being read whenever it does not depend on them (not in celeg)
    run_ahead: bool = True

    def validate(self) -> None:
        for name in ("max_active_requests", "max_batched_tokens", "prefill_chunk_tokens", "page_tokens"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        if self.logical_kv_pages < 0:
            raise ValueError("logical_kv_pages must not be negative")


@dataclass
class RequestOptions:
    """celeg's ``ConcurrentRequestOptions`` (include/celeg/runtime/request_types.hpp:16-22).
    ``eos_tokens=None`` takes the stop ids of the model's configuration."""
    max_new_tokens: int = 128
    eos_tokens: Optional[Sequence[int]] = None
    priority: int = 0
    generation: SamplingParams = field(default_factory=SamplingParams)


@dataclass
class Request:
    id: int
    prompt: List[int]
    options: RequestOptions
    eos_tokens: Tuple[int, ...]
    status: RequestStatus = RequestStatus.QUEUED
    generated: List[int] = field(default_factory=list)
    output: Deque[int] = field(default_factory=deque)       # tokens not polled yet
    prefill_offset: int = 0           # tokens of ``feed`` already in the cache
    feed: List[int] = field(default_factory=list)           # what prefill has to run (prompt, or
    #                                                         prompt + generated after a preemption)
    cache: Optional[RequestCache] = None
    cancel_requested: bool = False
    error: str = ""
    generator_state: Optional[int] = None                   # saved across a preemption
    preemptions: int = 0
    submitted_at: float = 0.0
    first_token_at: Optional[float] = None
    last_token_at: Optional[float] = None


@dataclass
class Metrics:
    """celeg's ``ConcurrentMetrics`` counters that apply here
    (include/celeg/runtime/concurrency/metrics.hpp:8-58)."""
    submitted: int = 0
    completed: int = 0
    cancelled: int = 0
    failed: int = 0
    preempted: int = 0
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    max_step_tokens: int = 0
    max_step_requests: int = 0
    skipped_for_pages: int = 0
    ttft_seconds_sum: float = 0.0
    ttft_count: int = 0
    itl_seconds_sum: float = 0.0
    itl_count: int = 0
    # every sample as well, for percentiles (the first ``SAMPLE_LIMIT`` of each)
    ttft_seconds: List[float] = field(default_factory=list)
    itl_seconds: List[float] = field(default_factory=list)
    active_requests: int = 0
    queued_requests: int = 0
    # cache pages out of the pools (summed over the paged groups): now, in all, and the most at any time
    pages_used: int = 0
    pages_total: int = 0
    pages_high_water: int = 0
    # Where a step's time goes on the host, summed over steps (celeg reports host_prepare_ms,
    # gpu_execute_ms and host_commit_ms per packed step: src/backend/cuda/packed/execution.cu:200-223):
    # plan = cancellations, admission and the batch plan; launch = checking, staging and enqueueing the
    # step and its draw (check / stage / forward / sample are its parts, when the runner reports them);
    # wait = blocked until the step's tokens are on the host; commit = accepting tokens, finishing, freeing.
    host_plan_seconds: float = 0.0
    host_launch_seconds: float = 0.0
    host_check_seconds: float = 0.0
    host_stage_seconds: float = 0.0
    host_forward_seconds: float = 0.0
    host_sample_seconds: float = 0.0
    host_wait_seconds: float = 0.0
    host_commit_seconds: float = 0.0
    gpu_seconds: float = 0.0          # device time of the steps, from events around each (0 if the runner has none)

    SAMPLE_LIMIT = 1 << 20

    def host_ms_per_step(self) -> Dict[str, float]:
        steps = max(1, self.steps)
        return {name: round(1e3 * getattr(self, f"host_{name}_seconds") / steps, 4)
                for name in ("plan", "launch", "check", "stage", "forward", "sample", "wait", "commit")}


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool                     # the step's last token of this entry yields a new token
    is_decode: bool


@dataclass
class Plan:
    entries: List[PlannedEntry] = field(default_factory=list)
    skipped_for_pages: List[Request] = field(default_factory=list)
    # a plan made by ``Scheduler._plan_after``: every entry is one token that the step before leaves on the device.
    # Such a plan says the same as the one after it, so it is used again, and what a launch makes of a plan
    # (the step function's entries, the sampler's rows) is kept with it.
    ahead: bool = False
    source_rows: Optional[List[int]] = None     # which row of the step before holds each entry's token (None: the same row)
    step_entries: Optional[list] = None
    sample_rows: Optional[list] = None


@dataclass
class PollResult:
    status: RequestStatus
    tokens: List[int]
    finished: bool
    error: str = ""


class Scheduler:
    def __init__(self, manager: CacheManager, runner, options: EngineOptions, max_context: int,
                 vocab_size: int, default_eos: Sequence[int] = ()):
        options.validate()
        self.manager = manager
        self.runner = runner
        self.options = options
        self.max_context = max_context
        self.vocab_size = vocab_size
        self.default_eos = tuple(default_eos)
        self.requests: Dict[int, Request] = {}
        self.queue: List[int] = []                  # ids of QUEUED requests
        self.live: List[int] = []                   # ids of PREFILL / DECODING requests
        self.metrics = Metrics()
        self._next_id = 1
        self._hold_admission = False      # set by a preemption: the freed pages go to the others first
        self._inflight = None             # (plan, handle) of a step that was enqueued and not yet collected
        # one step of run-ahead needs a runner that can enqueue without waiting
        self._runs_ahead = options.run_ahead and hasattr(runner, "launch") and hasattr(runner, "collect")
        self._padded_singles = getattr(runner, "padded_singles", None)

    # ------------------------------------------------------------------ public
    def submit(self, prompt: Sequence[int], options: Optional[RequestOptions] = None) -> int:
        """Checks of celeg's submit (src/backend/cuda/runtime/request_lifecycle.cpp:10-32) plus
        the token range (src/backend/cpu/concurrent.cpp:358-362)."""
        options = options or RequestOptions()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("the prompt is empty")
        if len(prompt) > self.max_context:
            raise ValueError(f"the prompt has {len(prompt)} tokens, the context holds {self.max_context}")
        if options.max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        if len(prompt) + options.max_new_tokens > self.max_context:
            raise ValueError(f"prompt ({len(prompt)}) + max_new_tokens ({options.max_new_tokens}) exceeds the "
                             f"context of {self.max_context}")
        for token in prompt:
            if not 0 <= token < self.vocab_size:
                raise ValueError(f"token id {token} is outside the vocabulary of {self.vocab_size}")
        options.generation.validate()
        eos = tuple(options.eos_tokens) if options.eos_tokens is not None else self.default_eos
        request = Request(id=self._next_id, prompt=prompt, options=options, eos_tokens=eos,
                          feed=list(prompt), submitted_at=time.monotonic())
        self._next_id += 1
        self.requests[request.id] = request
        self.queue.append(request.id)
        self.metrics.submitted += 1
        return request.id

    def cancel(self, request_id: int) -> bool:
        request = self.requests.get(request_id)
        if request is None or request.status.terminal:
            return False
        request.cancel_requested = True
        return True

    def status(self, request_id: int) -> RequestStatus:
        return self._get(request_id).status

    def poll(self, request_id: int, max_tokens: int = 0) -> PollResult:
        """Pops tokens that were produced since the last poll; ``finished`` once the request is
        terminal and nothing is left to pop (request_lifecycle.cpp:57-73)."""
        request = self._get(request_id)
        count = len(request.output) if max_tokens <= 0 else min(max_tokens, len(request.output))
        tokens = [request.output.popleft() for _ in range(count)]
        return PollResult(status=request.status, tokens=tokens,
                          finished=request.status.terminal and not request.output, error=request.error)

    def release(self, request_id: int) -> bool:
        """Forget a terminal request (request_lifecycle.cpp:47-55)."""
        request = self.requests.get(request_id)
        if request is None or not request.status.terminal:
            return False
        del self.requests[request_id]
        return True

    def has_work(self) -> bool:
        return bool(self.queue or self.live or self._inflight is not None)

    # -------------------------------------------------------------------- step
    def step(self) -> bool:
        """One engine step: admit, run one batch, accept tokens, admit again. Returns whether
        anything advanced.

        Whenever nothing is in the way (requests waiting, cancellations, pages that may run short), the step
        after is enqueued before this step's tokens are waited for: what it consists of does not depend on
        them. Its decoding rows take their input tokens from the device, where this step's draw left them, its
        prompt portions from the host; a request that reaches ``max_new_tokens`` with this step's token is
        left out. So the GPU does not idle while the host reads tokens, decides and plans. A request that
        ended on an end-of-sequence token of this step has then one more position computed in vain; its
        token of that step is dropped."""
        metrics = self.metrics
        clock = time.perf_counter
        if self._inflight is None:
            started = clock()
            self._honour_cancellations()
            if not self._hold_admission:
                self._admit()
            plan = self.plan()
            metrics.host_plan_seconds += clock() - started
            if not plan.entries:
                self._hold_admission = False
                if self.live and self._break_deadlock():
                    return True
                return False
            if not self._launch(plan, tokens_on_device=False):
                self._hold_admission = False
                return True                                   # the launch failed; its requests have failed
        plan, handle = self._inflight
        self._inflight = None
        started = clock()
        continuing = self._may_run_ahead(plan)
        after = self._plan_after(plan, continuing) if continuing else self._plan_ahead_of_portions(plan)
        metrics.host_plan_seconds += clock() - started
        if after is not None:
            self._launch(after, tokens_on_device=after.ahead)
        progressed = self._collect(plan, handle)
        started = clock()
        self._hold_admission = False
        self._honour_cancellations()
        self._admit()
        self._count_holdings()
        metrics.host_plan_seconds += clock() - started
        return progressed

    def _count_holdings(self) -> None:
        metrics = self.metrics
        metrics.active_requests = len(self.live)
        metrics.queued_requests = len(self.queue)
        pools = [group.pool for group in self.manager.groups]
        metrics.pages_used = sum(pool.used_pages for pool in pools)
        metrics.pages_total = sum(pool.total_pages for pool in pools)
        metrics.pages_high_water = sum(pool.high_water for pool in pools)

    # --------------------------------------------------------------- admission
    def _priority_key(self, request_id: int):
        request = self.requests[request_id]
        return (-request.options.priority, request.id)          # priority desc, then id asc

    def _reservation(self, request: Request) -> int:
        total = len(request.prompt) + request.options.max_new_tokens
        if self.options.scheduler_policy is SchedulerPolicy.GUARANTEED_NO_EVICT:
            return total
        return min(total, len(request.feed) + self.options.page_tokens)

    def _admit(self) -> None:
        while self.queue and len(self.live) < self.options.max_active_requests and self.manager.free_slots > 0:
            request_id = min(self.queue, key=self._priority_key)
            request = self.requests[request_id]
            if request.cancel_requested:
                self.queue.remove(request_id)
                self._finish(request, RequestStatus.CANCELLED)
                continue
            cache = self.manager.open(request.id)
            try:
                self.manager.reserve(cache, self._reservation(request))
            except OutOfPages:
                self.manager.close(request.id)
                break                                            # stays queued; stop admitting
            self.queue.remove(request_id)
            request.cache = cache
            request.status = RequestStatus.PREFILL
            request.prefill_offset = 0
            seed = request.generator_state if request.generator_state is not None \
                else request.options.generation.seed
            self.runner.reset_request(cache.slot, seed)
            self.live.append(request.id)

    # ---------------------------------------------------------------- planning
    def plan(self) -> Plan:
        """Decoding requests first, one token each; what is left of ``max_batched_tokens`` goes to
        prompt portions in priority order, each ``min(remaining, prefill_chunk_tokens, budget)``."""
        plan = Plan()
        ordered = sorted(self.live, key=self._priority_key)
        decoding = [self.requests[i] for i in ordered if self.requests[i].status is RequestStatus.DECODING]
        prefilling = [self.requests[i] for i in ordered if self.requests[i].status is RequestStatus.PREFILL]
        budget = self.options.max_batched_tokens
        free = [group.pool.free_pages for group in self.manager.groups]
        for request in decoding:
            if budget <= 0:
                break
            needed = self.manager.pages_needed(request.cache, request.cache.tokens + 1)
            if any(n > f for n, f in zip(needed, free)):
                plan.skipped_for_pages.append(request)           # retried next step
                continue
            free = [f - n for f, n in zip(free, needed)]
            plan.entries.append(PlannedEntry(request, [request.generated[-1]], samples=True, is_decode=True))
            budget -= 1
        if prefilling and plan.entries and self._padded_singles is not None:
            # the runner pads the decoded tokens of a mixed step to a coarser row count: the portions get what
            # is left of the budget beside those rows, so that the step's rows stay within it
            budget = min(budget, self.options.max_batched_tokens - self._padded_singles(len(plan.entries)))
        for request in prefilling:
            remaining = len(request.feed) - request.prefill_offset
            count = min(remaining, self.options.prefill_chunk_tokens, budget)
            if count <= 0:
                continue
            needed = self.manager.pages_needed(request.cache, request.cache.tokens + count)
            if any(n > f for n, f in zip(needed, free)):
                plan.skipped_for_pages.append(request)
                continue
            free = [f - n for f, n in zip(free, needed)]
            tokens = request.feed[request.prefill_offset:request.prefill_offset + count]
            plan.entries.append(PlannedEntry(request, tokens, samples=(count == remaining), is_decode=False))
            budget -= count
        return plan

    # --------------------------------------------------------------- execution
    def _fail(self, plan: Plan, exc: Exception) -> None:
        """Failure isolation: the requests of this step fail, others live on."""
        for planned in plan.entries:
            if not planned.request.status.terminal:
                planned.request.error = f"{type(exc).__name__}: {exc}"
                self._finish(planned.request, RequestStatus.FAILED)

    def _launch(self, plan: Plan, tokens_on_device: bool) -> bool:
        """Enqueues the plan's step (a runner without ``launch`` runs it to its end here)."""
        started = time.perf_counter()
        if plan.step_entries is None:
            plan.step_entries = [StepEntry(request_id=p.request.id, tokens=p.tokens,
                                           want=[len(p.tokens) - 1] if p.samples else [])
                                 for p in plan.entries]
            plan.sample_rows = [(p.request.cache.slot, p.request.options.generation)
                                for p in plan.entries if p.samples]
        entries, sample_rows = plan.step_entries, plan.sample_rows
        try:
            if self._runs_ahead:
                if plan.source_rows is not None:
                    handle = self.runner.launch(entries, sample_rows, tokens_on_device, source_rows=plan.source_rows)
                else:
                    handle = self.runner.launch(entries, sample_rows, tokens_on_device)
            else:
                handle = self.runner.run(entries, sample_rows)
        except Exception as exc:
            self._fail(plan, exc)
            return False
        finally:
            self.metrics.host_launch_seconds += time.perf_counter() - started
        self._inflight = (plan, handle)
        return True

    def _may_run_ahead(self, plan: Plan) -> Optional[List[PlannedEntry]]:
        """Whether the step after ``plan`` can be enqueued before the tokens of ``plan`` are known, and for
        whom: the requests of ``plan`` that go on decoding whatever those tokens are (an end-of-sequence
        token aside), one token each. A request that reaches its ``max_new_tokens`` with this step's token ends
        for certain and is left out; one that has ended while ``plan`` was in flight likewise. None: not now."""
        if not self._runs_ahead or self.queue or plan.skipped_for_pages:
            return None
        free = None
        max_context = self.max_context
        continuing = []
        alive = 0
        for planned in plan.entries:
            request = planned.request
            cache = request.cache
            if not (planned.is_decode and planned.samples) or request.cancel_requested:
                return None
            if cache is None:
                if request.status.terminal:
                    continue                              # ended while this step was in flight
                return None
            alive += 1
            if len(request.generated) + 2 > request.options.max_new_tokens:
                continue                                  # this step's token is its last
            if cache.tokens + 1 > max_context:
                return None
            if cache.tokens + 1 > cache.capacity:     # (else: room in the pages it holds)
                if free is None:
                    free = [group.pool.free_pages for group in self.manager.groups]
                needed = self.manager.pages_needed(cache, cache.tokens + 1)
                if any(n > f for n, f in zip(needed, free)):
                    return None
                free = [f - n for f, n in zip(free, needed)]
            continuing.append(planned)
        if alive != len(self.live) or not continuing:
            return None                                   # (a live request that this step does not hold)
        return continuing

    @staticmethod
    def _plan_after(plan: Plan, continuing: List[PlannedEntry]) -> Plan:
        if len(continuing) == len(plan.entries):
            if plan.ahead and plan.source_rows is None:
                return plan                              # the same requests, one token each, again
            after = Plan(ahead=True)
            after.entries = [PlannedEntry(p.request, [0], samples=True, is_decode=True) for p in plan.entries]
            return after
        # fewer requests than the step before: row i of this step takes the token of row source_rows[i] of that one
        after = Plan(ahead=True)
        row_of = {id(p): row for row, p in enumerate(plan.entries)}
        after.entries = [PlannedEntry(p.request, [0], samples=True, is_decode=True) for p in continuing]
        after.source_rows = [row_of[id(p)] for p in continuing]
        return after

    def _plan_ahead_of_portions(self, plan: Plan) -> Optional[Plan]:
        """The step after a ``plan`` that holds prompt portions, made before the tokens of ``plan`` are known, so
        that the device does not wait while the host reads them, decides and plans. What the step after looks like
        does not depend on those tokens (an end-of-sequence token aside, see :meth:`step`): a request whose prompt
        ``plan`` completes, or which decodes in it, decodes next, with the token that ``plan`` leaves on the device
        in its row of the draw; one that reaches ``max_new_tokens`` with that token is gone; a prompt goes on
        from where ``plan`` leaves it. The requests are read, not changed: ``plan`` is committed later. None when
        anything is in the way (requests waiting, cancellations, pages that may run short, a decoding request
        that ``plan`` left out): the step after is then planned the usual way, after the tokens."""
        if not self._runs_ahead or self.queue or plan.skipped_for_pages:
            return None
        options = self.options
        decoding_next: Dict[int, int] = {}              # request id -> its row in the draw of ``plan``
        offset_after: Dict[int, int] = {}               # request id -> prefill offset when ``plan`` is done
        planned = set()
        row = 0
        for entry in plan.entries:
            request = entry.request
            if request.cancel_requested:
                return None
            if request.cache is None:
                if request.status.terminal:
                    row += 1 if entry.samples else 0
                    continue                               # ended while this step was in flight
                return None
            planned.add(request.id)
            if entry.samples:
                if len(request.generated) + 2 <= request.options.max_new_tokens:
                    decoding_next[request.id] = row        # (else: this step's token is its last)
                row += 1
            else:
                offset_after[request.id] = request.prefill_offset + len(entry.tokens)
        after = Plan()
        budget = options.max_batched_tokens
        free = [group.pool.free_pages for group in self.manager.groups]

        def takes(cache, count) -> bool:
            nonlocal free
            if cache.tokens + count > self.max_context:
                return False
            if cache.tokens + count > cache.capacity:
                needed = self.manager.pages_needed(cache, cache.tokens + count)
                if any(n > f for n, f in zip(needed, free)):
                    return False
                free = [f - n for f, n in zip(free, needed)]
            return True

        ordered = sorted(self.live, key=self._priority_key)
        source_rows: List[int] = []
        prefilling = []
        for request_id in ordered:
            request = self.requests[request_id]
            if request.cancel_requested or request.cache is None:
                return None
            if request_id in decoding_next:
                if budget <= 0 or not takes(request.cache, 1):
                    return None
                after.entries.append(PlannedEntry(request, [0], samples=True, is_decode=True))
                source_rows.append(decoding_next[request_id])
                budget -= 1
            elif request_id in planned and request_id not in offset_after:
                continue                                   # ends with this step's token
            elif request.status is RequestStatus.DECODING:
                return None                                # decodes, but ``plan`` left it out: its token is on the host
            else:
                prefilling.append(request)
        if prefilling and after.entries and self._padded_singles is not None:
            budget = min(budget, options.max_batched_tokens - self._padded_singles(len(after.entries)))
        for request in prefilling:
            offset = offset_after.get(request.id, request.prefill_offset)
            remaining = len(request.feed) - offset
            count = min(remaining, options.prefill_chunk_tokens, budget)
            if count <= 0:
                continue
            if not takes(request.cache, count):
                return None
            after.entries.append(PlannedEntry(request, request.feed[offset:offset + count],
                                              samples=(count == remaining), is_decode=False))
            budget -= count
        if not after.entries:
            return None
        if source_rows:
            after.ahead = True                             # its leading single tokens are on the device
            after.source_rows = source_rows
        return after

    def _collect(self, plan: Plan, handle) -> bool:
        """Waits for the plan's tokens and accepts them."""
        started = time.perf_counter()
        try:
            tokens = self.runner.collect(handle) if self._runs_ahead else handle
        except Exception as exc:
            self._fail(plan, exc)
            return True
        finally:
            waited = time.perf_counter()
            self.metrics.host_wait_seconds += waited - started
        try:
            return self._commit(plan, tokens)
        finally:
            self.metrics.host_commit_seconds += time.perf_counter() - waited

    def _commit(self, plan: Plan, tokens) -> bool:
        report = getattr(self.runner, "report_times", None)
        if report is not None:
            report(self.metrics)
        now = time.monotonic()
        self.metrics.steps += 1
        self.metrics.skipped_for_pages += len(plan.skipped_for_pages)
        total = sum(len(p.tokens) for p in plan.entries)
        self.metrics.max_step_tokens = max(self.metrics.max_step_tokens, total)
        self.metrics.max_step_requests = max(self.metrics.max_step_requests, len(plan.entries))
        produced = iter(tokens)
        for planned in plan.entries:
            request = planned.request
            token = int(next(produced)) if planned.samples else None
            if request.status.terminal:
                continue                  # ended while this step was in flight: the position was computed in vain
            if planned.is_decode:
                self.metrics.decode_tokens += 1
            else:
                request.prefill_offset += len(planned.tokens)
                self.metrics.prefill_tokens += len(planned.tokens)
            if planned.samples:
                if request.status is RequestStatus.PREFILL:
                    request.status = RequestStatus.DECODING
                self._accept(request, token, now)
        return True

    def _accept(self, request: Request, token: int, now: float) -> None:
        """decode_scheduler.cpp:68-99: the token goes out (an eos token too), then the stop test."""
        request.generated.append(token)
        request.output.append(token)
        if request.first_token_at is None:
            request.first_token_at = now
            self.metrics.ttft_seconds_sum += now - request.submitted_at
            self.metrics.ttft_count += 1
            if len(self.metrics.ttft_seconds) < Metrics.SAMPLE_LIMIT:
                self.metrics.ttft_seconds.append(now - request.submitted_at)
        else:
            self.metrics.itl_seconds_sum += now - request.last_token_at
            self.metrics.itl_count += 1
            if len(self.metrics.itl_seconds) < Metrics.SAMPLE_LIMIT:
                self.metrics.itl_seconds.append(now - request.last_token_at)
        request.last_token_at = now
        if token in request.eos_tokens or len(request.generated) >= request.options.max_new_tokens:
            self._finish(request, RequestStatus.FINISHED)

    def _finish(self, request: Request, status: RequestStatus) -> None:
        """The one place where a request gives back what it holds."""
        if request.cache is not None:
            self.manager.close(request.id)
            request.cache = None
        if request.id in self.live:
            self.live.remove(request.id)
        request.status = status
        if status is RequestStatus.FINISHED:
            self.metrics.completed += 1
        elif status is RequestStatus.CANCELLED:
            self.metrics.cancelled += 1
        elif status is RequestStatus.FAILED:
            self.metrics.failed += 1

    def _honour_cancellations(self) -> None:
        for request_id in list(self.live):
            request = self.requests[request_id]
            if request.cancel_requested:
                self._finish(request, RequestStatus.CANCELLED)
        for request_id in list(self.queue):
            request = self.requests[request_id]
            if request.cancel_requested:
                self.queue.remove(request_id)
                self._finish(request, RequestStatus.CANCELLED)

    # ------------------------------------------------------- when pages run out
    def _break_deadlock(self) -> bool:
        """No live request can advance because the pool is empty (only under MAX_UTILIZATION, or
        with a pool smaller than one request). celeg skips such requests "this step" forever
        (decode_scheduler.cpp:23-66). Here the live request of lowest priority, and among those
        the youngest, is preempted: its pages and slot are given back and it returns to the queue
        with prompt + generated tokens to prefill again, its generator state kept, so its output
        continues as if nothing happened. If it is the only live request, the pool cannot hold
        it at all and it fails with a message that says so."""
        victim = self.requests[max(self.live, key=self._priority_key)]
        if len(self.live) == 1:
            victim.error = (f"out of cache pages: request {victim.id} needs more pages than the pool has "
                            f"({[g.pool.total_pages for g in self.manager.groups]} pages of "
                            f"{self.options.page_tokens} tokens)")
            self._finish(victim, RequestStatus.FAILED)
            return True
        victim.generator_state = self.runner.save_generator(victim.cache.slot)
        self.manager.close(victim.id)
        victim.cache = None
        self.live.remove(victim.id)
        victim.feed = victim.prompt + victim.generated
        victim.prefill_offset = 0
        victim.status = RequestStatus.QUEUED
        victim.preemptions += 1
        self.queue.append(victim.id)
        self.metrics.preempted += 1
        self._hold_admission = True
        return True

    def _get(self, request_id: int) -> Request:
        try:
            return self.requests[request_id]
        except KeyError:
            raise KeyError(f"unknown request id {request_id}") from None
