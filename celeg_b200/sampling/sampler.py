"""Device-side sampling state and the call that draws one token per wanted row.

Each request's generator state and seen-table live in arrays indexed by the request's state
slot, so what a request draws does not depend on the batch it is in (celeg keeps the same per
lane: src/backend/cuda/packed/metadata.cu:20-24)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import kernels
from .params import SamplingParams


class Sampler:
    def __init__(self, vocab_size: int, slots: int, max_rows: int, device: torch.device):
        self.vocab_size = vocab_size
        self.device = device
        self.max_rows = max_rows
        self.seen = torch.zeros((slots, vocab_size), dtype=torch.uint8, device=device)
        self.rng = torch.ones(slots, dtype=torch.int64, device=device)
        # staging: [slot | top_k] int32 and [temperature | top_p | penalty] float32, one copy each
        self._host_i = torch.empty(2 * max_rows, dtype=torch.int32).pin_memory()
        self._host_f = torch.empty(3 * max_rows, dtype=torch.float32).pin_memory()
        self._stage_ring = [(self._host_i, self._host_f, None)] + [
            (torch.empty(2 * max_rows, dtype=torch.int32).pin_memory(),
             torch.empty(3 * max_rows, dtype=torch.float32).pin_memory(), None) for _ in range(3)]
        self._stage_next = 0
        self._dev_i = torch.zeros(2 * max_rows, dtype=torch.int32, device=device)
        self._dev_f = torch.zeros(3 * max_rows, dtype=torch.float32, device=device)
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._partial_score = torch.zeros(max_rows * 64, dtype=torch.float32, device=device)
        self._partial_token = torch.zeros(max_rows * 64, dtype=torch.int32, device=device)
        self._pieces = kernels.sample_scratch(device)        # lets a small batch's rows be cut over several blocks
        self._out_host = torch.zeros(max_rows, dtype=torch.int32).pin_memory()
        self._out_hosts = [self._out_host, torch.zeros(max_rows, dtype=torch.int32).pin_memory()]
        self._flip = 0
        # the drawn tokens go to the host on a stream of their own: on the stream of the kernels the copy would
        # stand between this step's draw and the next step's first kernel
        self._copy_stream = torch.cuda.Stream(device=device)
        self._copied: Optional[torch.cuda.Event] = None      # the last copy out of ``out`` has finished
        self._staged = None
        self._staged_rows = None
        self._all_greedy = False

    def reset_slot(self, slot: int, seed: int) -> None:
        """A new request takes the slot: nothing seen, generator at its seed."""
        self.seen[slot].zero_()
        self.set_rng(slot, seed)

    def set_rng(self, slot: int, state: int) -> None:
        self.rng[slot] = state - (1 << 64) if state >= (1 << 63) else state

    def get_rng(self, slot: int) -> int:
        value = int(self.rng[slot].item())
        return value + (1 << 64) if value < 0 else value

    def mark_step(self, step) -> None:
        """The tokens a step fed count as seen by their requests."""
        kernels.mark_seen(self.seen, step.token_ids, step.token_span, step.span_slot, step.tokens)

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[int, SamplingParams]]) -> List[int]:
        """One token per row of ``logits``; ``rows[i]`` = (state slot, options). Synchronises."""
        return self.read(self.launch(logits, rows))

    def read(self, handle) -> List[int]:
        """Waits for a launched draw (only for it, not for what was enqueued later) and returns its tokens."""
        event, host, count = handle
        if event is not None:
            event.synchronize()
        if count == 0:
            return []
        return host[:count].tolist()

    def launch(self, logits: torch.Tensor, rows: Sequence[Tuple[int, SamplingParams]], also_copy=None):
        """Enqueues the draw and the copy of the tokens to pinned host memory; :meth:`read` returns
        them. ``self.out[:len(rows)]`` holds them on the device until the next launch (a following step
        may take its input tokens from there). At most two launches may be unread at a time; the rows and
        their options may change from launch to launch. ``also_copy`` = (pinned host tensor, device
        tensor): copied along with the tokens (a step's error flag), there when :meth:`read` returns."""
        count = len(rows)
        if count == 0:
            if also_copy is not None:
                also_copy[0].copy_(also_copy[1], non_blocking=True)
                event = torch.cuda.Event()
                event.record()
                return event, None, 0
            return None, None, 0
        if count > self.max_rows:
            raise ValueError(f"{count} rows to sample, the sampler was sized for {self.max_rows}")
        m = self.max_rows
        # (the very list of the launch before: a scheduler that decodes the same requests again hands it over
        # unchanged, and comparing hundreds of rows field by field would cost more than the launch)
        signature = self._staged if rows is self._staged_rows else tuple((slot, params) for slot, params in rows)
        self._staged_rows = rows
        if signature is not self._staged and signature != self._staged:
            # the rows or their options changed: stage them again. Launches are not waited for one by one (a
            # scheduler enqueues a step before it reads the one before), so the pinned buffers form a ring: one
            # is written again only when the copy that read it last has left.
            index = self._stage_next
            self._stage_next = (index + 1) % len(self._stage_ring)
            host_i, host_f, copied = self._stage_ring[index]
            if copied is not None:
                copied.synchronize()
            hi, hf = host_i.numpy(), host_f.numpy()
            for i, (slot, params) in enumerate(rows):
                hi[i] = slot
                hi[m + i] = params.top_k
                hf[i] = params.temperature
                hf[m + i] = params.top_p
                hf[2 * m + i] = params.repetition_penalty
            self._dev_i.copy_(host_i, non_blocking=True)
            self._dev_f.copy_(host_f, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record()
            self._stage_ring[index] = (host_i, host_f, copied)
            self._staged = signature
            self._all_greedy = all(params.greedy for _, params in rows)
        if self._copied is not None:
            # ``out`` is written again: not before its last copy has left (long done by now; the order is formal)
            torch.cuda.current_stream().wait_event(self._copied)
            self._copied = None
        if self._all_greedy:
            kernels.sample_greedy(logits, count, self._dev_i[:m], self.seen, self._dev_f[2 * m:], self.out,
                                  self._partial_score, self._partial_token)
        else:
            kernels.sample(logits, count, self._dev_i[:m], self.seen, self.rng, self._dev_f[:m], self._dev_i[m:],
                           self._dev_f[m:2 * m], self._dev_f[2 * m:], self.out, scratch=self._pieces)
        host = self._out_hosts[self._flip]
        self._flip ^= 1
        main = torch.cuda.current_stream()
        drawn = torch.cuda.Event()
        drawn.record(main)
        side = self._copy_stream
        side.wait_event(drawn)
        with torch.cuda.stream(side):
            host.copy_(self.out, non_blocking=True)
            if also_copy is not None:
                also_copy[0].copy_(also_copy[1], non_blocking=True)
            event = torch.cuda.Event()
            event.record(side)
        self._copied = event
        return event, host, count
