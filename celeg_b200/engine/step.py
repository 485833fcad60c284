"""The step function: one batch of (request, its next tokens) through the model, from the
cache that earlier steps left, returning the logits at the wanted places.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere. celeg runs
two passes per engine step, a ragged prefill and a packed decode
(src/backend/cuda/packed/execution.cu:141-224, 234-384; never both in one pass:
src/backend/cuda/runtime/engine_control.cpp:4-23); both already treat a token as a row with its
own position and page table, and here they are one pass.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.manager import CacheManager, NO_PAGE, OutOfPages
from ..cache.storage import CacheStorage
from ..parts import Runtime, StepContext
from .model import Model


class StepInputError(ValueError):
    """The batch is malformed; the message names the request."""


class DeviceCheckError(RuntimeError):
    """A kernel met an index the host should have made impossible."""


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are wanted


def _context_bucket(tokens: int) -> int:
    bucket = 256
    while bucket < tokens:
        bucket *= 2
    return bucket


def _align4(n: int) -> int:
    return (n + 3) // 4 * 4


PROMPT_TOKEN_STEP = 128       # a padded prompt step's portions are filled up to a multiple of this many tokens
PADDING_TOKENS = PROMPT_TOKEN_STEP + 32   # most rows a step may be padded by (portions + spare single tokens)
# A prompt step's shape is captured in a CUDA graph when it comes for this many times (a capture costs about three
# launches from the host: it pays from the coming after that on, and a shape that comes twice never pays)
CAPTURE_AT_COMING = 3
PADDING_SPANS = 40             # most spans it may be padded by (spare single tokens and the spare portion)


@dataclass
class _PaddedPrompt:
    """The launch shape of a padded prompt step (see ``StepFunction._padded_prompt_shape``)."""
    key: tuple
    singles: int             # single tokens the step really brings
    single_rows: int         # ... and how many rows they take
    portions: int
    padded_tokens: int       # tokens of the portions and of the spare portion together
    spare_tokens: int
    spans: int
    logit_rows: int


class StepFunction:
    def __init__(self, model: Model, manager: CacheManager, storage: CacheStorage, rt: Runtime,
                 max_tokens: int, max_spans: int, max_context: int, use_graphs: bool = False):
        self.model = model
        self.manager = manager
        self.storage = storage
        self.rt = rt
        self.max_tokens = max_tokens
        self.max_spans = max_spans
        self.max_context = max_context
        self.page_tokens = manager.page_tokens
        self.max_pages = (max_context + self.page_tokens - 1) // self.page_tokens
        self.groups = len(manager.groups)
        # (the runtime's buffers hold more rows than a step may bring: room for the rows a step is padded by)
        self.buffer_tokens = max(max_tokens, rt.max_tokens)
        # (and more spans than a step may bring: a step padded to a launch shape has spare single tokens, up to
        # the next row count of _graph_rows, and a spare portion)
        self.span_capacity = max_spans + PADDING_SPANS
        capacity = (3 * _align4(self.buffer_tokens) + _align4(self.span_capacity + 1) + _align4(self.span_capacity)
                    + _align4(self.buffer_tokens) + self.groups * _align4(self.span_capacity * self.max_pages)
                    + _align4(self.buffer_tokens))       # (the last: source rows of a step's tokens, see run)
        # a ring of pinned staging buffers: a buffer is refilled only after the copy that read it
        # last has finished on the device
        self._ring = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * len(self._ring)
        self._ring_next = 0
        self._ring_np = [buffer.numpy() for buffer in self._ring]
        self._host = self._ring[0]
        self._host_np = self._ring_np[0]
        self._dev = torch.zeros(capacity, dtype=torch.int32, device=rt.device)
        self.error_flag = rt.error_flag
        self._decode_logits = torch.empty((self.span_capacity, model.vocab_size), dtype=torch.float32,
                                          device=rt.device)
        self._wide_logits: Optional[torch.Tensor] = None
        self.use_graphs = use_graphs
        self._graphs: Dict[tuple, torch.cuda.CUDAGraph] = {}
        self._graph_launches: Dict[tuple, int] = {}
        self._prompt_seen: Dict[tuple, int] = {}
        self.max_prompt_graphs = 24
        self.max_padded_graphs = 96
        self.steps_run = 0
        self.kernel_steps_graphed = 0
        self.last_step: Optional[StepContext] = None
        self.before_forward = None                # see set_before_forward
        # host seconds spent in run(), by phase: checking the batch and reserving pages, filling and
        # sending the step's metadata, enqueueing the model's kernels (or replaying their graph)
        self.host_seconds = {"check": 0.0, "stage": 0.0, "forward": 0.0}

    # ------------------------------------------------------------------ requests
    def begin(self, request_id: Hashable):
        return self.manager.open(request_id)

    def end(self, request_id: Hashable) -> None:
        self.manager.close(request_id)

    def position_of(self, request_id: Hashable) -> int:
        return self.manager.get(request_id).tokens

    # ---------------------------------------------------------------------- step
    def run(self, entries: Sequence[StepEntry], auto_begin: bool = False,
            token_source: Optional[torch.Tensor] = None, source_rows: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Returns float32 logits [wanted, vocab] in the order of the entries and of ``want``.
        The tensor is a view of a buffer that the next call overwrites. ``token_source`` (int32, on the device):
        without ``source_rows`` the entries' tokens are placeholders and token i of the step is ``token_source[i]``;
        with them the single tokens at the head of the step are placeholders, token i < len(source_rows) is
        ``token_source[source_rows[i]]``, and the other entries carry their tokens."""
        started = time.perf_counter()
        vocab = self.model.vocab_size
        if not entries:
            return self._decode_logits[:0]
        if len(entries) > self.max_spans:
            raise StepInputError(f"{len(entries)} requests in one step, the limit is {self.max_spans}")
        checked_entries = self._check_single_tokens(entries, auto_begin) if len(entries) >= 8 else None
        opened: List[Hashable] = []               # requests that this step begins: ended again if it is refused
        try:
            if checked_entries is not None:
                caches, wanted = checked_entries
                total = len(entries)
                counts = [1] * total
            else:
                caches, counts, total, wanted = self._check_entries(entries, auto_begin, opened)
            if total > self.max_tokens:
                raise StepInputError(f"{total} tokens in one step, the limit is {self.max_tokens}")
            # pages for the whole batch, all or nothing
            need = self.manager.pages_needed_each(caches, counts)
            for g, group in enumerate(self.manager.groups):
                if need[g] > group.pool.free_pages:
                    raise OutOfPages(f"the step needs {need[g]} more page(s) of group {group.key}, "
                                     f"{group.pool.free_pages} free")
        except (StepInputError, OutOfPages):
            for request_id in opened:
                self.manager.close(request_id)
            raise
        self.manager.reserve_each(caches, counts)

        spans = len(entries)
        all_decode = total == spans
        max_ctx = max(cache.tokens + count for cache, count in zip(caches, counts))
        mixed = None if all_decode else self._padded_prompt_shape(entries, wanted, max_ctx)
        if all_decode or mixed is not None:
            prompt_key = mixed.key if mixed is not None else None
        else:
            prompt_key = self._prompt_graph_key(entries, total, wanted, max_ctx)
        if (all_decode and self.use_graphs) or prompt_key is not None:
            stride = self.max_pages                         # fixed, so the captured addresses hold
        else:
            stride = (max_ctx + self.page_tokens - 1) // self.page_tokens
        slot = self._ring_next
        self._ring_next = (slot + 1) % len(self._ring)
        if self._ring_events[slot] is not None:
            self._ring_events[slot].synchronize()
        self._host = self._ring[slot]
        self._host_np = self._ring_np[slot]
        checked = time.perf_counter()
        # a decoding step that will be replayed from a graph takes a launch shape from a short list, so that
        # a batch that shrinks request by request does not capture a graph for every size
        padded = self._graph_rows(spans) if (all_decode and self.use_graphs and wanted <= self.max_spans) else spans
        n_logits = wanted
        if mixed is not None:
            step, logit_rows, n_words = self._stage_padded_prompt(entries, caches, mixed, stride, max_ctx)
            n_logits = mixed.logit_rows
        else:
            if padded > spans and wanted == spans:
                # every request wants its row: the spare rows' logits are computed too (nobody reads them), so
                # that the launch shape depends on the padded row count alone
                n_logits = padded
            step, logit_rows, n_words = self._stage(entries, caches, total, spans, n_logits, stride, max_ctx, padded)
        tokens_from = None
        sent = n_words
        if token_source is not None and source_rows is not None:
            if n_words + len(source_rows) > self._host_np.shape[0]:
                raise StepInputError("too many source rows for the staging buffer")
            self._host_np[n_words:n_words + len(source_rows)] = source_rows
            sent = n_words + len(source_rows)
        self._dev[:sent].copy_(self._host[:sent], non_blocking=True)
        if token_source is not None:
            # the tokens of this step are on the device already (what the step before drew): token i of
            # the step is token_source[i]; the entries carry placeholders
            if token_source.dtype != torch.int32 or (source_rows is None and token_source.numel() < total):
                raise StepInputError("a token source must hold one int32 token for every token of the step")
            if source_rows is None:
                if token_source.numel() < step.tokens:
                    raise StepInputError("a token source must hold one int32 token for every row of the step")
                tokens_from = token_source              # copied by _forward: inside the step's graph, if it has one
            else:
                # the first len(source_rows) tokens of the step (single tokens at its head) come from the device,
                # the others are what the entries carry
                count = len(source_rows)
                if (count > total or min(source_rows) < 0 or max(source_rows) >= token_source.numel()
                        or any(len(entry.tokens) != 1 for entry in entries[:count])):
                    raise StepInputError("source rows must name a row of the token source for each of the single "
                                         "tokens at the head of the step")
                # (the rows travel behind the step's metadata in the same pinned buffer and the same copy)
                torch.index_select(token_source, 0, self._dev[n_words:n_words + count], out=step.token_ids[:count])
        event = torch.cuda.Event()
        event.record()
        self._ring_events[slot] = event
        self.last_step = step
        staged = time.perf_counter()

        if wanted <= self.max_spans:
            logits = self._decode_logits
        else:
            if self._wide_logits is None or self._wide_logits.shape[0] < wanted:
                self._wide_logits = torch.empty((wanted, vocab), dtype=torch.float32, device=self.rt.device)
            logits = self._wide_logits

        if all_decode and self.use_graphs and wanted <= self.max_spans:
            graph_key = (padded, n_logits, _context_bucket(max_ctx))
        else:
            graph_key = prompt_key
        if graph_key is not None:
            if tokens_from is not None:
                graph_key = graph_key + ("tokens on the device", tokens_from.data_ptr())
            self._run_graphed(graph_key, step, logit_rows, n_logits, logits, tokens_from)
        else:
            self._forward(step, logit_rows, n_logits, logits, tokens_from)
        self.manager.advance_each(caches, counts)
        self.steps_run += 1
        done = time.perf_counter()
        self.host_seconds["check"] += checked - started
        self.host_seconds["stage"] += staged - checked
        self.host_seconds["forward"] += done - staged
        return logits[:wanted]

    def padded_single_rows(self, singles: int) -> int:
        """How many rows the ``singles`` single tokens at the head of a step of prompt portions take when the step
        is padded to a launch shape: 16, 32, 64, then multiples of 32 (a coarser grid than a decoding step's:
        beside prompt portions a few spare single tokens cost nothing, and every row count less is a graph less
        to capture). A scheduler that wants the step's rows to stay within its token budget counts these."""
        if singles <= 0 or not self.use_graphs:
            return max(0, singles)
        rows = next((n for n in (16, 32, 64) if n >= singles), (singles + 31) // 32 * 32)
        return rows if rows <= self.max_spans else self._graph_rows(singles)

    def _check_entries(self, entries, auto_begin: bool, opened: list):
        """The checks of :meth:`run`, request by request. Returns (caches, counts, total, wanted); a request that
        ``auto_begin`` opens here is added to ``opened``."""
        vocab = self.model.vocab_size
        seen_ids = set()
        total = 0
        wanted = 0
        caches = []
        counts = []
        find = self.manager.find
        for entry in entries:
            request_id = entry.request_id
            if request_id in seen_ids:
                raise StepInputError(f"request {request_id!r} appears twice in one step")
            seen_ids.add(request_id)
            tokens = entry.tokens
            count = len(tokens)
            if count == 1:
                low = high = int(tokens[0])
            elif count == 0:
                raise StepInputError(f"request {request_id!r} brings no tokens")
            else:
                if not isinstance(tokens, np.ndarray):
                    tokens = entry.tokens = np.asarray(tokens, dtype=np.int64)
                low, high = int(tokens.min()), int(tokens.max())
            if low < 0 or high >= vocab:
                bad = low if low < 0 else high
                raise StepInputError(f"request {request_id!r}: token id {bad} is outside the "
                                     f"vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= int(place) < count:
                    raise StepInputError(f"request {request_id!r}: wanted place {place} is outside its "
                                         f"{count} tokens")
            cache = find(request_id)
            if cache is None:
                if not auto_begin:
                    raise StepInputError(f"request {request_id!r} was not begun") from None
                cache = self.manager.open(request_id)
                opened.append(request_id)
            if cache.tokens + count > self.max_context:
                raise StepInputError(f"request {request_id!r} would reach {cache.tokens + count} positions, "
                                     f"the context limit is {self.max_context}")
            caches.append(cache)
            counts.append(count)
            total += count
            wanted += len(entry.want)
        return caches, counts, total, wanted

    def _check_single_tokens(self, entries, auto_begin: bool):
        """The checks of :meth:`run` for a step in which every request brings one token, over whole lists
        instead of request by request (a step of hundreds of decoding requests spends more time in a loop of
        checks than in anything else on the host). Returns (caches, wanted), or None when the step is of
        another kind or something is wrong with it: the general loop then finds out what and says so."""
        try:
            if any(len(entry.tokens) != 1 for entry in entries):
                return None
            ids = [entry.request_id for entry in entries]
            if len(set(ids)) != len(ids):
                return None
            tokens = np.asarray([entry.tokens[0] for entry in entries], dtype=np.int64)
            if int(tokens.min()) < 0 or int(tokens.max()) >= self.model.vocab_size:
                return None
            wanted = 0
            for entry in entries:
                want = entry.want
                if want:
                    if len(want) != 1 or int(want[0]) != 0:
                        return None
                    wanted += 1
            find = self.manager.find
            caches = [find(request_id) for request_id in ids]
            if any(cache is None for cache in caches):
                return None
            if max(cache.tokens for cache in caches) + 1 > self.max_context:
                return None
            return caches, wanted
        except (TypeError, ValueError):
            return None

    def _padded_prompt_shape(self, entries, wanted: int, max_ctx: int):
        """A step of the form the scheduler plans under load (single decoded tokens first, then prompt portions)
        rarely has the shape of an earlier one: the number of decoding requests and the portions' lengths change
        from step to step, and launching it kernel by kernel from the host costs more than a small step takes on
        the device. Such a step can take a launch shape from a coarse grid instead: spare single tokens up to a
        row count of :meth:`_graph_rows`, and one spare portion that fills the portions' tokens up to a multiple
        of ``PROMPT_TOKEN_STEP``. Spare rows carry token 0 at positions 0.. of the storage's spare pages and
        slot; the kernels take their bounds (attention tiles, longest span) from the grid, not from the step.
        Returns the shape (with its graph key) once it has come ``CAPTURE_AT_COMING`` times, else None."""
        if not self.use_graphs or wanted > self.max_spans:
            return None
        lengths = [len(e.tokens) for e in entries]
        singles = next((i for i, n in enumerate(lengths) if n != 1), len(lengths))
        portions = lengths[singles:]
        if not portions or any(n == 1 for n in portions):
            return None                                   # all single tokens, or a single token after a portion
        single_rows = self.padded_single_rows(singles)
        portion_tokens = sum(portions)
        # the step's rows together are a multiple of PROMPT_TOKEN_STEP: the products work in tiles of 128 rows, and a
        # tile more (2,112 rows where 2,048 would do) is a wave more of their blocks
        padded_tokens = -(-(single_rows + portion_tokens) // PROMPT_TOKEN_STEP) * PROMPT_TOKEN_STEP - single_rows
        spare = padded_tokens - portion_tokens
        spans = single_rows + len(portions) + (1 if spare else 0)
        logit_rows = max(1, wanted, single_rows + len(portions))    # (a scheduler's step wants one row a span at most)
        # (the spare portion lives in the storage's spare pages, and its table row holds max_pages entries)
        spare_room = min(self.storage.scratch_page_count, self.max_pages) * self.page_tokens
        if (single_rows + padded_tokens > self.buffer_tokens or spans > self.span_capacity
                or logit_rows > self.span_capacity
                or single_rows - singles > PADDING_TOKENS - PROMPT_TOKEN_STEP
                or spare > spare_room):
            return None
        key = ("padded prompt", single_rows, len(portions), padded_tokens, logit_rows, _context_bucket(max_ctx))
        if key not in self._graphs:
            if len(self._prompt_seen) > 4096:
                self._prompt_seen.clear()
            seen = self._prompt_seen.get(key, 0) + 1
            self._prompt_seen[key] = seen
            if seen < CAPTURE_AT_COMING:
                return None
            kept = [k for k in self._graphs if k and k[0] == "padded prompt"]
            if len(kept) >= self.max_padded_graphs:          # the oldest goes (dicts keep insertion order)
                del self._graphs[kept[0]]
                del self._graph_launches[kept[0]]
        return _PaddedPrompt(key, singles, single_rows, len(portions), padded_tokens, spare, spans, logit_rows)

    def _stage_padded_prompt(self, entries, caches, shape: "_PaddedPrompt", stride: int, max_ctx: int):
        """:meth:`_stage` for a step padded to ``shape``: rows are [the single tokens | spare single tokens | the
        portions | the spare portion]; the logit rows are the wanted ones followed by repeats of row 0."""
        host = self._host_np
        total, spans = shape.single_rows + shape.padded_tokens, shape.spans
        offsets = {}
        cursor = 0
        for name, size in (("token_ids", total), ("positions", total), ("token_span", total),
                           ("span_begin", spans + 1), ("span_slot", spans), ("logit_rows", shape.logit_rows)):
            offsets[name] = cursor
            cursor += _align4(size)
        table_offsets = []
        for _ in range(self.groups):
            table_offsets.append(cursor)
            cursor += _align4(spans * stride)
        token_ids = host[offsets["token_ids"]:offsets["token_ids"] + total]
        positions = host[offsets["positions"]:offsets["positions"] + total]
        token_span = host[offsets["token_span"]:offsets["token_span"] + total]
        span_begin = host[offsets["span_begin"]:offsets["span_begin"] + spans + 1]
        span_slot = host[offsets["span_slot"]:offsets["span_slot"] + spans]
        logit_rows_host = host[offsets["logit_rows"]:offsets["logit_rows"] + shape.logit_rows]
        tables = [host[o:o + spans * stride].reshape(spans, stride) for o in table_offsets]
        for grid in tables:
            grid.fill(NO_PAGE)
        scratch_slot = self.storage.scratch_slot
        row = 0
        span = 0
        out = 0
        lengths = []

        def real(entry, cache):
            nonlocal row, span, out
            count = len(entry.tokens)
            token_ids[row:row + count] = entry.tokens
            positions[row:row + count] = np.arange(cache.tokens, cache.tokens + count, dtype=np.int32)
            token_span[row:row + count] = span
            span_begin[span] = row
            span_slot[span] = cache.slot
            for place in entry.want:
                logit_rows_host[out] = row + int(place)
                out += 1
            for g in range(self.groups):
                table = cache.table_array(g)
                used = min(table.shape[0], stride)
                tables[g][span, :used] = table[:used]
            lengths.append(count)
            row += count
            span += 1

        def spare(count):
            nonlocal row, span
            token_ids[row:row + count] = 0
            positions[row:row + count] = np.arange(count, dtype=np.int32)
            token_span[row:row + count] = span
            span_begin[span] = row
            span_slot[span] = scratch_slot
            pages = -(-count // self.page_tokens)
            for g in range(self.groups):
                first = self.storage.scratch_pages[g]
                tables[g][span, :pages] = np.arange(first, first + pages, dtype=np.int32)
            lengths.append(count)
            row += count
            span += 1

        for entry, cache in zip(entries[:shape.singles], caches[:shape.singles]):
            real(entry, cache)
        for _ in range(shape.single_rows - shape.singles):
            spare(1)
        for entry, cache in zip(entries[shape.singles:], caches[shape.singles:]):
            real(entry, cache)
        if shape.spare_tokens:
            spare(shape.spare_tokens)
        assert row == total and span == spans and out <= shape.logit_rows
        span_begin[spans] = row
        logit_rows_host[out:] = 0
        dev = self._dev

        def view(name, size):
            return dev[offsets[name]:offsets[name] + size]

        step = StepContext(
            tokens=total, spans=spans,
            token_ids=view("token_ids", total), positions=view("positions", total),
            token_span=view("token_span", total), span_begin=view("span_begin", spans + 1),
            span_slot=view("span_slot", spans),
            block_tables=[dev[o:o + spans * stride].view(spans, stride) for o in table_offsets],
            error_flag=self.error_flag, max_span=shape.padded_tokens, max_context=max_ctx,
            context_bucket=_context_bucket(max_ctx), host_span_lengths=lengths,
            leading_single_tokens=shape.single_rows,
            prompt_tile_bound=-(-shape.padded_tokens // PROMPT_TOKEN_STEP) + shape.portions + 1,
            logits_of_all_rows=False)
        return step, view("logit_rows", shape.logit_rows), cursor

    def _prompt_graph_key(self, entries, total: int, wanted: int, max_ctx: int):
        """Steps with prompt portions are launched from the host kernel by kernel, which takes longer than the
        GPU needs for portions of a few hundred tokens. Every launch shape of such a step follows from the
        lengths of its portions, the number of wanted rows and whether those are all rows in order, so a step
        whose shape has come before (a long prompt cut into equal portions) is captured in a CUDA graph at
        its third coming (``CAPTURE_AT_COMING``) and replayed from then on. None: run it kernel by kernel."""
        if not self.use_graphs or wanted > self.max_spans:
            return None
        all_rows = wanted == total and all(tuple(e.want) == tuple(range(len(e.tokens))) for e in entries)
        # (single tokens at the head of the step go to the decode attention, whose launch follows the context)
        bucket = _context_bucket(max_ctx) if len(entries[0].tokens) == 1 else 0
        key = ("prompt", tuple(len(e.tokens) for e in entries), wanted, all_rows, bucket)
        if key in self._graphs:
            return key
        if len(self._prompt_seen) > 4096:
            self._prompt_seen.clear()
        seen = self._prompt_seen.get(key, 0) + 1
        self._prompt_seen[key] = seen
        if seen < CAPTURE_AT_COMING:
            return None
        prompt_graphs = [k for k in self._graphs if k and k[0] == "prompt"]
        if len(prompt_graphs) >= self.max_prompt_graphs:     # the oldest goes (dicts keep insertion order)
            del self._graphs[prompt_graphs[0]]
            del self._graph_launches[prompt_graphs[0]]
        return key

    def set_before_forward(self, hook) -> None:
        """``hook(step)`` is called with every step's description before the model runs, on the step's stream and
        inside its graph if it has one (a sampler marks the step's tokens as seen there). Graphs captured without
        it are dropped."""
        self.before_forward = hook
        self._graphs.clear()
        self._graph_launches.clear()

    def _forward(self, step, logit_rows, wanted, logits, tokens_from) -> None:
        """What a step enqueues on the device after its metadata: its tokens from the device (when the step
        before drew them: every row of the step takes the token of the same row there; rows past the step's
        requests get whatever lies there, they are spare), the hook, the model."""
        if tokens_from is not None:
            step.token_ids[:step.tokens].copy_(tokens_from[:step.tokens], non_blocking=True)
        if self.before_forward is not None:
            self.before_forward(step)
        self.model.forward(step, logit_rows, wanted, logits)

    def _run_graphed(self, key, step, logit_rows, wanted, logits, tokens_from=None) -> None:
        graph = self._graphs.get(key)
        if graph is None:
            # Warm up outside capture (library handles, lazy allocations), then capture. The
            # warm-up advances the fixed-size state once and the replay below would advance it
            # again, so the state from before the warm-up is put back in between (cache pages
            # are written with the same values both times).
            saved = self.storage.state.clone()
            self._forward(step, logit_rows, wanted, logits, tokens_from)
            torch.cuda.current_stream().synchronize()
            graph = torch.cuda.CUDAGraph()
            before = kernels.LAUNCHES
            with torch.cuda.graph(graph):
                self._forward(step, logit_rows, wanted, logits, tokens_from)
            self._graph_launches[key] = kernels.LAUNCHES - before
            self.storage.state.copy_(saved)
            self._graphs[key] = graph
        graph.replay()
        kernels.LAUNCHES += self._graph_launches[key]      # kernels of this package inside the graph
        self.kernel_steps_graphed += 1

    def _graph_rows(self, spans: int) -> int:
        """The number of rows a graphed decoding step of ``spans`` requests is launched with: 1, 2, 4, 8, 12 or
        16 (the small-batch kernels work on 8 or 16 rows whatever the number), then the next multiple of 8,
        beyond 64 of 32."""
        if spans <= 16:
            rows = next(n for n in (1, 2, 4, 8, 12, 16) if n >= spans)
        else:
            rows = (spans + 7) // 8 * 8 if spans <= 64 else (spans + 31) // 32 * 32
        return rows if rows <= self.max_spans else spans

    def _stage(self, entries, caches, total, spans, wanted, stride, max_ctx, padded=None):
        """Fill the pinned staging buffer; returns the StepContext, the logit-row tensor and the
        number of int32 words to copy. The layout depends only on (T, R, F, stride), so steps of
        the same shape use the same device addresses. ``padded`` > spans (decoding steps only): rows are
        added up to that number; they carry token 0 at position 0 of the storage's spare page and slot;
        ``wanted`` then counts their logit rows too if the caller has them computed (nobody reads them)."""
        real_spans = spans
        if padded is not None and padded > spans:
            total = spans = padded
        host = self._host_np
        offsets = {}
        cursor = 0
        for name, size in (("token_ids", total), ("positions", total), ("token_span", total),
                           ("span_begin", spans + 1), ("span_slot", spans), ("logit_rows", max(wanted, 1))):
            offsets[name] = cursor
            cursor += _align4(size)
        table_offsets = []
        for _ in range(self.groups):
            table_offsets.append(cursor)
            cursor += _align4(spans * stride)
        token_ids = host[offsets["token_ids"]:offsets["token_ids"] + total]
        positions = host[offsets["positions"]:offsets["positions"] + total]
        token_span = host[offsets["token_span"]:offsets["token_span"] + total]
        span_begin = host[offsets["span_begin"]:offsets["span_begin"] + spans + 1]
        span_slot = host[offsets["span_slot"]:offsets["span_slot"] + spans]
        logit_rows_host = host[offsets["logit_rows"]:offsets["logit_rows"] + max(wanted, 1)]
        tables = [host[o:o + spans * stride].reshape(spans, stride) for o in table_offsets]
        row = 0
        out = 0
        lengths = []
        if total == spans:
            # every request brings one token (a decode step): fill whole arrays at once
            token_ids[:real_spans] = [entry.tokens[0] for entry in entries]
            positions[:real_spans] = [cache.tokens for cache in caches]
            token_span[:] = range(spans)
            span_begin[:spans] = range(spans)
            span_slot[:real_spans] = [cache.slot for cache in caches]
            if real_spans < spans:
                token_ids[real_spans:] = 0
                positions[real_spans:] = 0
                span_slot[real_spans:] = self.storage.scratch_slot
            for index, entry in enumerate(entries):
                if entry.want:
                    logit_rows_host[out] = index
                    out += 1
            if wanted > out:                       # (the spare rows of a padded step, see run)
                logit_rows_host[out:wanted] = range(real_spans, real_spans + wanted - out)
            mirrors = self.manager.table_mirrors
            slots = span_slot[:real_spans] if mirrors is not None else None
            for g in range(self.groups):
                grid = tables[g]
                if mirrors is not None and mirrors[g].shape[1] >= stride:
                    # the tables of all slots lie in one array: the rows of this step's requests in one gather
                    np.take(mirrors[g][:, :stride], slots, axis=0, out=grid[:real_spans])
                    if real_spans < spans:
                        grid[real_spans:].fill(NO_PAGE)
                else:
                    grid.fill(NO_PAGE)
                    for index, cache in enumerate(caches):
                        table = cache.table_array(g)
                        used = min(table.shape[0], stride)
                        grid[index, :used] = table[:used]
                if real_spans < spans:
                    grid[real_spans:, 0] = self.storage.scratch_pages[g]
            lengths = [1] * spans
            row = spans
        else:
            for index, (entry, cache) in enumerate(zip(entries, caches)):
                count = len(entry.tokens)
                token_ids[row:row + count] = entry.tokens
                positions[row:row + count] = np.arange(cache.tokens, cache.tokens + count, dtype=np.int32)
                token_span[row:row + count] = index
                span_begin[index] = row
                span_slot[index] = cache.slot
                for place in entry.want:
                    logit_rows_host[out] = row + int(place)
                    out += 1
                for g in range(self.groups):
                    table = cache.table_array(g)
                    used = min(table.shape[0], stride)
                    tables[g][index, :used] = table[:used]
                    tables[g][index, used:] = NO_PAGE
                lengths.append(count)
                row += count
        span_begin[spans] = row
        dev = self._dev

        def view(name, size):
            return dev[offsets[name]:offsets[name] + size]

        step = StepContext(
            tokens=total, spans=spans,
            token_ids=view("token_ids", total), positions=view("positions", total),
            token_span=view("token_span", total), span_begin=view("span_begin", spans + 1),
            span_slot=view("span_slot", spans),
            block_tables=[dev[o:o + spans * stride].view(spans, stride) for o in table_offsets],
            error_flag=self.error_flag, max_span=max(lengths), max_context=max_ctx,
            context_bucket=_context_bucket(max_ctx), host_span_lengths=lengths,
            leading_single_tokens=next((i for i, n in enumerate(lengths) if n != 1), spans),
            logits_of_all_rows=(wanted == total and
                                all(int(logit_rows_host[i]) == i for i in range(wanted))))
        return step, view("logit_rows", max(wanted, 1)), cursor

    # -------------------------------------------------------------------- checks
    def raise_on_device_error(self) -> None:
        """Synchronises and raises if any kernel flagged an impossible index."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise DeviceCheckError(device_error_text(code))


def device_error_text(code: int) -> str:
    return (f"a kernel reported error code {code} (1: cache write without a page, 2: attention read without "
            f"a page, 3: more key splits than the launch has blocks for, 11-24 and 61-65: a bounded wait of "
            f"a tcgen05 kernel ran out)")
