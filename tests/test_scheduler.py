"""The scheduler's decisions, on the host, with a fake step function: admission order and
out-of-pages at admission, token budget and portions, decode beside prefill, finishing on eos
and on max_new_tokens, cancellation at every stage, failure isolation, and what happens when
pages run out while decoding (skip, then preempt and continue unchanged)."""
from __future__ import annotations

import pytest

from celeg_b200.cache import CacheManager, PagedNeed, StateLayout
from celeg_b200.engine.scheduler import (EngineOptions, RequestOptions, RequestStatus, Scheduler, SchedulerPolicy)
from celeg_b200.sampling import SamplingParams


class FakeRunner:
    """Next token = (sum of every token the request has fed so far + generator state) % 50 + 10; so
    a request's output depends on its whole history and its generator, like a real model's."""

    def __init__(self, manager):
        self.manager = manager
        self.history = {}           # slot -> tokens fed since reset
        self.generator = {}
        self.calls = []
        self.fail_next = False

    def reset_request(self, slot, seed):
        self.history[slot] = []
        self.generator[slot] = seed

    def save_generator(self, slot):
        return self.generator[slot]

    def run(self, entries, sample_rows):
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("injected step failure")
        self.calls.append([(e.request_id, list(e.tokens), list(e.want)) for e in entries])
        out = []
        for entry in entries:
            cache = self.manager.get(entry.request_id)
            self.manager.reserve(cache, cache.tokens + len(entry.tokens))
            self.manager.advance(cache, cache.tokens + len(entry.tokens))
            self.history[cache.slot].extend(entry.tokens)
            if entry.want:
                assert list(entry.want) == [len(entry.tokens) - 1]
                self.generator[cache.slot] += 1
                out.append((sum(self.history[cache.slot]) + self.generator[cache.slot]) % 50 + 10)
        assert len(out) == len(sample_rows)
        return out


def make(pages=64, page_tokens=4, slots=4, **option_overrides):
    options = EngineOptions(max_active_requests=slots, max_batched_tokens=16, prefill_chunk_tokens=8,
                            page_tokens=page_tokens, **option_overrides)
    manager = CacheManager(page_tokens, [pages], [(("kv",), PagedNeed(1, 8, None))], StateLayout(), slots)
    runner = FakeRunner(manager)
    return Scheduler(manager, runner, options, max_context=128, vocab_size=100, default_eos=(7,)), runner, manager


def run_all(scheduler, limit=500):
    steps = 0
    while scheduler.has_work():
        assert scheduler.step(), "no progress"
        scheduler.manager.check_invariants()
        steps += 1
        assert steps < limit
    return steps


def expected_output(prompt, max_new, seed=1, eos=(7,)):
    history, generator, out = list(prompt), seed, []
    for _ in range(max_new):
        generator += 1
        token = (sum(history) + generator) % 50 + 10
        out.append(token)
        history.append(token)
        if token in eos:
            break
    return out


def test_submit_checks():
    scheduler, _, _ = make()
    with pytest.raises(ValueError):
        scheduler.submit([])
    with pytest.raises(ValueError):
        scheduler.submit([1] * 129)
    with pytest.raises(ValueError):
        scheduler.submit([1] * 100, RequestOptions(max_new_tokens=29))
    with pytest.raises(ValueError):
        scheduler.submit([1, 100])
    with pytest.raises(ValueError):
        scheduler.submit([1], RequestOptions(max_new_tokens=0))
    with pytest.raises(ValueError):
        scheduler.submit([1], RequestOptions(generation=SamplingParams(top_k=500)))
    with pytest.raises(ValueError):
        scheduler.submit([1], RequestOptions(generation=SamplingParams(seed=0)))


def test_one_request_prefill_in_portions_then_decode():
    scheduler, runner, manager = make()
    prompt = list(range(1, 20))                                  # 19 tokens, portions of 8
    rid = scheduler.submit(prompt, RequestOptions(max_new_tokens=5, eos_tokens=()))
    run_all(scheduler)
    sizes = [len(call[0][1]) for call in runner.calls]
    assert sizes == [8, 8, 3, 1, 1, 1, 1]
    assert [call[0][2] for call in runner.calls[:3]] == [[], [], [2]]     # logits only at the last portion
    result = scheduler.poll(rid)
    assert result.finished and result.status is RequestStatus.FINISHED
    assert result.tokens == expected_output(prompt, 5, eos=())
    assert manager.groups[0].pool.free_pages == 64 and manager.free_slots == 4
    assert scheduler.release(rid) and not scheduler.release(rid)


def test_decode_rows_come_first_and_budget_is_shared():
    scheduler, runner, _ = make()
    a = scheduler.submit([1, 2, 3], RequestOptions(max_new_tokens=30, eos_tokens=()))
    scheduler.step()                                             # a: whole prompt, first token
    b = scheduler.submit(list(range(1, 41)), RequestOptions(max_new_tokens=2, eos_tokens=()))
    scheduler.step()
    ids = [entry[0] for entry in runner.calls[-1]]
    sizes = [len(entry[1]) for entry in runner.calls[-1]]
    assert ids == [a, b] and sizes == [1, 8]                     # decode token beside a portion of b
    c = scheduler.submit(list(range(1, 41)), RequestOptions(max_new_tokens=2, eos_tokens=()))
    scheduler.step()
    sizes = [len(entry[1]) for entry in runner.calls[-1]]
    assert sizes == [1, 8, 7]                                    # 16-token budget: 1 + 8 + what is left
    run_all(scheduler)
    for rid, prompt, n in ((a, [1, 2, 3], 30), (b, list(range(1, 41)), 2), (c, list(range(1, 41)), 2)):
        assert scheduler.poll(rid).tokens == expected_output(prompt, n, eos=())


def test_priority_then_id_decides_admission():
    scheduler, runner, _ = make(slots=1)
    low = scheduler.submit([1], RequestOptions(max_new_tokens=1, priority=0, eos_tokens=()))
    high = scheduler.submit([2], RequestOptions(max_new_tokens=1, priority=5, eos_tokens=()))
    mid = scheduler.submit([3], RequestOptions(max_new_tokens=1, priority=5, eos_tokens=()))
    run_all(scheduler)
    assert [call[0][0] for call in runner.calls] == [high, mid, low]


def test_eos_is_emitted_and_ends_the_request():
    scheduler, _, _ = make()
    prompt = [3, 4]
    full = expected_output(prompt, 40, eos=())
    stop = full[3]
    rid = scheduler.submit(prompt, RequestOptions(max_new_tokens=40, eos_tokens=(stop,)))
    run_all(scheduler)
    tokens = scheduler.poll(rid).tokens
    assert tokens == full[:full.index(stop) + 1] and tokens[-1] == stop


def test_default_eos_comes_from_the_model():
    scheduler, _, _ = make()
    rid = scheduler.submit([1], RequestOptions(max_new_tokens=4))
    assert scheduler.requests[rid].eos_tokens == (7,)


def test_admission_waits_for_pages_guaranteed_policy():
    scheduler, runner, manager = make(pages=8)                   # 32 positions in all
    a = scheduler.submit([1] * 10, RequestOptions(max_new_tokens=10, eos_tokens=()))    # 5 pages
    b = scheduler.submit([2] * 10, RequestOptions(max_new_tokens=10, eos_tokens=()))    # 5 pages: must wait
    scheduler.step()
    assert scheduler.status(a) is RequestStatus.PREFILL or scheduler.status(a) is RequestStatus.DECODING
    assert scheduler.status(b) is RequestStatus.QUEUED
    run_all(scheduler)
    assert scheduler.status(b) is RequestStatus.FINISHED
    assert scheduler.metrics.preempted == 0 and scheduler.metrics.skipped_for_pages == 0
    assert scheduler.poll(b).tokens == expected_output([2] * 10, 10, eos=())


def test_pages_run_out_while_decoding_skip_then_preempt_and_continue():
    scheduler, runner, manager = make(pages=7, scheduler_policy=SchedulerPolicy.MAX_UTILIZATION)
    prompts = {}
    for value in (1, 2, 3):
        prompt = [value] * 6
        prompts[scheduler.submit(prompt, RequestOptions(max_new_tokens=12, eos_tokens=()))] = prompt
    run_all(scheduler)
    assert scheduler.metrics.skipped_for_pages > 0
    assert scheduler.metrics.preempted > 0
    for rid, prompt in prompts.items():
        assert scheduler.status(rid) is RequestStatus.FINISHED
        assert scheduler.poll(rid).tokens == expected_output(prompt, 12, eos=())   # unchanged by preemption
    assert sum(scheduler.requests[rid].preemptions for rid in prompts) == scheduler.metrics.preempted
    assert scheduler.requests[min(prompts)].preemptions == 0        # the oldest is never the victim
    assert manager.groups[0].pool.free_pages == 7


def test_request_larger_than_the_pool_fails_with_a_message():
    scheduler, _, manager = make(pages=3, scheduler_policy=SchedulerPolicy.MAX_UTILIZATION)
    rid = scheduler.submit([1] * 6, RequestOptions(max_new_tokens=20, eos_tokens=()))
    run_all(scheduler)
    result = scheduler.poll(rid)
    assert result.status is RequestStatus.FAILED and "out of cache pages" in result.error
    assert len(result.tokens) > 0                                # what it produced before is still delivered
    assert manager.groups[0].pool.free_pages == 3 and manager.free_slots == 4


def test_cancel_at_every_stage():
    scheduler, _, manager = make(slots=1)
    running = scheduler.submit([1] * 20, RequestOptions(max_new_tokens=20, eos_tokens=()))
    queued = scheduler.submit([2], RequestOptions(max_new_tokens=3, eos_tokens=()))
    scheduler.step()
    assert scheduler.status(running) is RequestStatus.PREFILL
    assert scheduler.cancel(queued) and scheduler.cancel(running)
    scheduler.step()
    assert scheduler.status(queued) is RequestStatus.CANCELLED
    assert scheduler.status(running) is RequestStatus.CANCELLED
    assert not scheduler.cancel(running)
    assert manager.free_slots == 1 and manager.groups[0].pool.free_pages == 64
    later = scheduler.submit([3], RequestOptions(max_new_tokens=4, eos_tokens=()))
    scheduler.step()
    scheduler.step()
    assert scheduler.status(later) is RequestStatus.DECODING
    scheduler.cancel(later)
    scheduler.step()
    assert scheduler.status(later) is RequestStatus.CANCELLED
    assert scheduler.poll(later).finished is False or scheduler.poll(later).finished   # leftover tokens poll out
    assert scheduler.metrics.cancelled == 3


def test_a_failing_step_fails_only_its_requests():
    scheduler, runner, manager = make(slots=1)
    first = scheduler.submit([1, 2], RequestOptions(max_new_tokens=3, eos_tokens=()))
    second = scheduler.submit([3, 4], RequestOptions(max_new_tokens=3, eos_tokens=()))
    runner.fail_next = True
    run_all(scheduler)
    result = scheduler.poll(first)
    assert result.status is RequestStatus.FAILED and "injected step failure" in result.error
    assert scheduler.poll(second).tokens == expected_output([3, 4], 3, eos=())
    assert manager.free_slots == 1 and manager.groups[0].pool.free_pages == 64


def test_poll_in_pieces_and_metrics():
    scheduler, _, _ = make()
    rid = scheduler.submit([5], RequestOptions(max_new_tokens=6, eos_tokens=()))
    run_all(scheduler)
    part = scheduler.poll(rid, 4)
    assert len(part.tokens) == 4 and not part.finished
    rest = scheduler.poll(rid)
    assert len(rest.tokens) == 2 and rest.finished
    metrics = scheduler.metrics
    assert metrics.submitted == 1 and metrics.completed == 1 and metrics.prefill_tokens == 1
    assert metrics.decode_tokens == 5 and metrics.ttft_count == 1 and metrics.itl_count == 5
    with pytest.raises(KeyError):
        scheduler.poll(999)


# ----------------------------------------------------------------------------------- run-ahead
class AheadRunner(FakeRunner):
    """A runner that can enqueue a step without waiting for it: the step function's host side
    (reserve, advance) happens at launch, the tokens are computed when they are collected, and
    a launch with ``tokens_on_device`` takes its input tokens from the draw of the launch before."""

    def __init__(self, manager):
        super().__init__(manager)
        self.pending = []            # launched, not collected: (entries as lists, slots, from_device)
        self.last_drawn = []         # what the latest collected-or-not launch drew, per row (filled at collect)
        self.log = []

    def launch(self, entries, sample_rows, tokens_on_device=False, source_rows=None):
        if self.fail_next:
            self.fail_next = False
            raise RuntimeError("injected step failure")
        assert len(self.pending) <= 1, "more than two steps in flight"
        assert source_rows is None or (tokens_on_device and len(source_rows) <= len(entries) and
                                       all(len(e.tokens) == 1 for e in entries[:len(source_rows)]))
        rows = []
        for entry in entries:
            cache = self.manager.get(entry.request_id)
            self.manager.reserve(cache, cache.tokens + len(entry.tokens))
            self.manager.advance(cache, cache.tokens + len(entry.tokens))
            rows.append((entry.request_id, cache.slot, list(entry.tokens), list(entry.want)))
        handle = {"rows": rows, "from_device": tokens_on_device, "after": self.pending[-1] if self.pending else None,
                  "source": list(source_rows) if source_rows is not None else None}
        self.pending.append(handle)
        self.log.append(("launch", tokens_on_device, [r[0] for r in rows], [len(r[2]) for r in rows]))
        return handle

    def collect(self, handle):
        assert self.pending and self.pending[0] is handle, "collected out of order"
        self.pending.pop(0)
        self.log.append(("collect", [r[0] for r in handle["rows"]]))
        if handle["from_device"]:
            before = handle["after"]["drawn"]
            source = handle["source"]
            if source is None:
                assert len(before) == len(handle["rows"])
                source = list(range(len(before)))
        out = []
        for index, (request_id, slot, tokens, want) in enumerate(handle["rows"]):
            if handle["from_device"] and index < len(source):
                tokens = [before[source[index]]]
            self.history[slot].extend(tokens)
            if want:
                self.generator[slot] += 1
                out.append((sum(self.history[slot]) + self.generator[slot]) % 50 + 10)
        handle["drawn"] = out
        return out


def make_ahead(pages=64, page_tokens=4, slots=4, **option_overrides):
    options = EngineOptions(max_active_requests=slots, max_batched_tokens=16, prefill_chunk_tokens=8,
                            page_tokens=page_tokens, **option_overrides)
    manager = CacheManager(page_tokens, [pages], [(("kv",), PagedNeed(1, 8, None))], StateLayout(), slots)
    runner = AheadRunner(manager)
    return Scheduler(manager, runner, options, max_context=128, vocab_size=100, default_eos=(7,)), runner, manager


def test_run_ahead_gives_the_same_tokens_and_overlaps_steps():
    scheduler, runner, manager = make_ahead()
    prompts = [[3, 4, 5], [9, 1], [2, 2, 2, 2, 2]]
    ids = [scheduler.submit(p, RequestOptions(max_new_tokens=9, eos_tokens=())) for p in prompts]
    run_all(scheduler)
    for request_id, prompt in zip(ids, prompts):
        assert scheduler.poll(request_id).tokens == expected_output(prompt, 9, eos=())
    # while all three decode, the next step is launched before the tokens of the last are collected
    ahead = [i for i, entry in enumerate(runner.log) if entry[0] == "launch" and entry[1]]
    assert len(ahead) >= 5
    for i in ahead:                                      # each of them was enqueued before the collect of the step before
        assert runner.log[i + 1][0] == "collect"
    assert not runner.pending
    assert manager.free_slots == 4
    manager.check_invariants()


def test_run_ahead_drops_the_token_after_an_end_of_sequence():
    scheduler, runner, manager = make_ahead()
    prompt = [3, 4, 5]
    reference = expected_output(prompt, 30, eos=())
    stop = reference[4]                                  # the fifth token ends the request
    request_id = scheduler.submit(prompt, RequestOptions(max_new_tokens=30, eos_tokens=(stop,)))
    other = scheduler.submit([8, 8], RequestOptions(max_new_tokens=12, eos_tokens=()))
    run_all(scheduler)
    assert scheduler.poll(request_id).tokens == reference[:reference.index(stop) + 1]
    assert scheduler.poll(other).tokens == expected_output([8, 8], 12, eos=())
    assert scheduler.status(request_id) is RequestStatus.FINISHED
    assert not runner.pending and manager.free_slots == 4
    manager.check_invariants()


def test_run_ahead_across_steps_with_prompt_portions():
    """Prompts of several portions beside decoding requests: the step after such a step is enqueued before its
    tokens are read too (the decoding rows take their tokens from the device, the portions theirs from the
    host), a request whose prompt ends in a step decodes in the step after with that step's token, and one that
    ends is left out. Same outputs as without running ahead."""
    prompts = [list(range(1, 30)), [9, 1], list(range(40, 63)), [6, 7, 8], list(range(5, 19))]
    news = [6, 14, 3, 9, 1]
    outputs = {}
    for run_ahead in (False, True):
        scheduler, runner, manager = make_ahead(slots=5, pages=64, run_ahead=run_ahead)
        ids = [scheduler.submit(p, RequestOptions(max_new_tokens=n, eos_tokens=())) for p, n in zip(prompts, news)]
        run_all(scheduler)
        outputs[run_ahead] = [scheduler.poll(i).tokens for i in ids]
        assert not runner.pending and manager.free_slots == 5
        manager.check_invariants()
        if run_ahead:
            # launches that were enqueued while the step before was still uncollected, and held a prompt portion
            waiting, early = 0, 0
            for entry in runner.log:
                if entry[0] == "launch":
                    early += 1 if waiting >= 1 and any(count > 1 for count in entry[3]) else 0
                    waiting += 1
                else:
                    waiting -= 1
            assert early >= 4, runner.log
    for prompt, n, got in zip(prompts, news, outputs[True]):
        assert got == expected_output(prompt, n, eos=())
    assert outputs[True] == outputs[False]


def test_portions_leave_room_for_the_rows_a_runner_pads_decoded_tokens_to():
    """A runner that pads the decoded tokens of a mixed step to a coarser row count says so (``padded_singles``);
    the plan then gives the prompt portions what the budget leaves beside those rows, not beside the tokens."""
    scheduler, runner, manager = make_ahead(slots=4, run_ahead=False)
    runner.padded_singles = lambda count: -(-count // 4) * 4
    scheduler._padded_singles = runner.padded_singles
    first = scheduler.submit([1, 2, 3], RequestOptions(max_new_tokens=20, eos_tokens=()))
    while scheduler.status(first).value != "decoding":
        scheduler.step()
    second = scheduler.submit(list(range(1, 41)), RequestOptions(max_new_tokens=2, eos_tokens=()))
    scheduler._admit()
    plan = scheduler.plan()
    sizes = [len(p.tokens) for p in plan.entries]
    assert sizes[0] == 1 and not plan.entries[1].is_decode
    # budget 16, one decoded token padded to 4 rows: 12 tokens are left, the portion limit is 8
    assert sizes[1] == 8
    scheduler.options.prefill_chunk_tokens = 16
    sizes = [len(p.tokens) for p in scheduler.plan().entries]
    assert sizes == [1, 12]
    run_all(scheduler)
    assert scheduler.poll(first).tokens == expected_output([1, 2, 3], 20, eos=())
    assert scheduler.poll(second).tokens == expected_output(list(range(1, 41)), 2, eos=())


def test_run_ahead_goes_on_with_the_requests_that_do_not_end():
    """Requests that reach their last token at different steps: the step after is still enqueued early, for the
    requests that go on, and takes their tokens from the rows they had in the step before."""
    scheduler, runner, manager = make_ahead()
    prompts = [[3, 4, 5], [9, 1], [2, 2, 2, 2, 2], [6]]
    news = [5, 9, 7, 12]
    ids = [scheduler.submit(p, RequestOptions(max_new_tokens=n, eos_tokens=())) for p, n in zip(prompts, news)]
    run_all(scheduler)
    for request_id, prompt, n in zip(ids, prompts, news):
        assert scheduler.poll(request_id).tokens == expected_output(prompt, n, eos=())
    launches = [entry for entry in runner.log if entry[0] == "launch"]
    shrinking = [i for i in range(1, len(launches))
                 if launches[i][1] and len(launches[i][2]) < len(launches[i - 1][2])]
    assert len(shrinking) >= 2, launches                 # run ahead with fewer rows than the step before
    assert not runner.pending and manager.free_slots == 4
    manager.check_invariants()


def test_no_run_ahead_while_requests_wait_or_prefill_or_are_about_to_end():
    scheduler, runner, manager = make_ahead(slots=1)
    first = scheduler.submit([1, 2, 3], RequestOptions(max_new_tokens=4, eos_tokens=()))
    second = scheduler.submit([4, 5], RequestOptions(max_new_tokens=3, eos_tokens=()))      # waits for the slot
    run_all(scheduler)
    assert scheduler.poll(first).tokens == expected_output([1, 2, 3], 4, eos=())
    assert scheduler.poll(second).tokens == expected_output([4, 5], 3, eos=())
    # with a request queued the scheduler never ran ahead for the first; for the second it may only
    # while two more tokens are certain
    first_launches = [entry for entry in runner.log if entry[0] == "launch" and entry[2] == [first]]
    assert not any(entry[1] for entry in first_launches)
    manager.check_invariants()


def test_run_ahead_with_cancellation_and_failure():
    scheduler, runner, manager = make_ahead()
    a = scheduler.submit([1, 2, 3], RequestOptions(max_new_tokens=20, eos_tokens=()))
    b = scheduler.submit([4, 5, 6], RequestOptions(max_new_tokens=20, eos_tokens=()))
    for _ in range(4):
        scheduler.step()
    scheduler.cancel(a)                                  # a step with a in it is in flight
    for _ in range(3):
        scheduler.step()
    assert scheduler.status(a) is RequestStatus.CANCELLED
    got = scheduler.poll(b).tokens
    assert got == expected_output([4, 5, 6], 20, eos=())[:len(got)] and len(got) >= 5
    runner.fail_next = True
    while scheduler.has_work():
        scheduler.step()
    assert scheduler.status(b) in (RequestStatus.FAILED, RequestStatus.FINISHED)
    assert manager.free_slots == 4
    manager.check_invariants()


def test_run_ahead_can_be_switched_off():
    scheduler, runner, manager = make_ahead(run_ahead=False)
    request_id = scheduler.submit([3, 4, 5], RequestOptions(max_new_tokens=6, eos_tokens=()))
    run_all(scheduler)
    assert scheduler.poll(request_id).tokens == expected_output([3, 4, 5], 6, eos=())
    assert not any(entry[0] == "launch" for entry in runner.log)        # the plain run() path
