"""Mixer parts. Interface of a mixer:

    Mixer(params, weights, parts, rt)       parts: built nested parts (e.g. {"position": ...})
    cache_need() -> PagedNeed | StateNeed | None
    bind_cache(binding)                     PagedBinding or StateBinding from the cache storage
    forward(x, out, step)                   x: normed activations [T, hidden]; writes the
                                            mixer's output (to be added to the residual) to out
    takes_split_norm(step) -> bool          optional: True if forward() hands x to the runtime's products
                                            only, which can apply a row scale that x still lacks (then x
                                            may be a kernels.SplitNorm instead of a tensor)
    ends_with_product = True                optional: the last thing forward() does to ``out`` is
                                            rt.linear(..., out, ...); the runtime may then add that product
                                            to the residual stream itself and leave ``out`` unwritten

A mixer does not know which model or layer it is in; everything it needs about the step is
in the StepContext, everything about its cache in the binding.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping, Optional

import torch

from .. import kernels
from ..cache.manager import PagedNeed, StateNeed
from .registry import register_part
from .runtime import Runtime, StepContext


@dataclass
class PagedBinding:
    """Where a paged mixer's keys and values live: one layer of a group's storage,
    [pages, kv_heads, page_tokens, head_dim] each; ``owner`` False = read only (the cache
    belongs to an earlier layer of the run order)."""
    group: int
    k: torch.Tensor
    v: torch.Tensor
    page_tokens: int
    owner: bool = True


@dataclass
class StateBinding:
    """Where a fixed-state mixer's state lives: ``state`` is a view [slots, elements] of the
    slot slab; ``slot_stride`` floats separate one slot from the next."""
    state: torch.Tensor
    slot_stride: int
    owner: bool = True


# Blocks of the decode attention that a B200 holds at a time at a head size of 64 (148 SMs x 5): what the times
# of its launches at 1 to 256 requests and 2 k to 130 k keys fit (see decode_split). A mixer asks the kernel
# library for the number of its own head size on its own device.
DECODE_RESIDENT_BLOCKS = 740


def decode_split(tokens: int, kv_heads: int, context_bucket: int, window: Optional[int], max_context: int,
                 resident_blocks: int = DECODE_RESIDENT_BLOCKS):
    """How the decode attention splits the keys of a step of ``tokens`` requests: (chunk, max_splits,
    cap_splits). Every request's keys are cut into chunks of ``chunk`` (a multiple of 64); ``max_splits`` chunks
    cover the step's context bucket and ``cap_splits`` >= max_splits is what the scratch is sized for, a
    number that depends only on the longest context the runtime allows.

    Few requests with short contexts: enough splits for about one and a half blocks per SM, chunks of at most
    1,024 keys. Where that limit binds (many requests or long contexts) the chunk grows up to 4,096 keys: fewer
    blocks start and fewer partial results are merged. The launch's blocks (requests x kv heads x splits) run
    in rounds of ``resident_blocks``. If one round can hold them, about half a round is asked for: the
    times fall off sharply just above a whole round (2 requests at 65 k keys: 60 us with 720 blocks, 75 us with
    816) and are flat or a little better towards half of one (1 request at 130 k: 70 us with 712 blocks, 63 us
    with 368; at 65 k 41 us with 360 to 408). Otherwise, of 1,024 / 2,048 / 4,096 keys the largest chunk within a
    twentieth of the most even filling of the rounds is taken (a count like 1,024 blocks, 1.4 rounds, was the
    slowest choice wherever it was measured). Measured on B200, 32 query heads on 8 kv heads of 64, microseconds
    a layer at chunks of 1,024 / 2,048 / 4,096 keys: 64 requests at 8 k keys 173 / 168 / 196, 16 at 32 k
    179 / 171 / 194, 8 at 65 k 188 / 175 / 200, 32 at 65 k 654 / 636 / 631, 8 at 130 k 360 / 337 / 326."""
    bucket = context_bucket
    if window:
        bucket = min(bucket, 1 << max(8, (window - 1).bit_length()))
    longest = max_context if not window else min(max_context, 2 * window)
    cap_splits = max(32, -(-longest // 1024) * 2)
    blocks_wanted = 224
    items = max(1, tokens * kv_heads)
    splits = max(1, min(bucket // 128, -(-blocks_wanted // items), cap_splits))
    chunk = min(-(-bucket // splits), 1024)
    chunk = (chunk + 63) // 64 * 64
    if chunk == 1024:
        if items * -(-bucket // 4096) < resident_blocks:
            # one round holds the launch: about half a round of blocks, in chunks of 1,024 to 4,096 keys
            splits = max(1, resident_blocks // 2 // items)
            chunk = min(max((-(-bucket // splits) + 63) // 64 * 64, 1024), 4096)
        else:
            def evenness(candidate: int) -> float:
                blocks = items * -(-bucket // candidate)
                rounds = -(-blocks // resident_blocks)
                return blocks / (rounds * resident_blocks)
            candidates = (1024, 2048, 4096)
            best = max(evenness(c) for c in candidates)
            chunk = max(c for c in candidates if evenness(c) >= best - 0.05)
    max_splits = -(-bucket // chunk)
    if max_splits > cap_splits:             # a bucket beyond the longest context: cannot come from a valid step
        raise ValueError(f"a context bucket of {context_bucket} keys needs {max_splits} splits, the scratch holds "
                         f"{cap_splits} (longest context {max_context})")
    return chunk, max_splits, cap_splits


@register_part("mixer", "attention")
class AttentionMixer:
    """Causal grouped-query attention over the paged cache with optional per-head q/k RMSNorm,
    a position encoding, an optional window, and softmax scale given by the configuration.
    Order of operations as in celeg (src/backend/cpu/operators/attention_token.cpp:151-204;
    src/backend/cuda/packed/operators.cu:66-99, 101-246, 494-529): fused q|k|v projection,
    norm, rotation, cache write, attention, output projection."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        self.scale = float(params.get("softmax_scale", self.head_dim ** -0.5))
        self.eps = float(params.get("qk_norm_eps", 1e-6))
        self.reads_only = bool(params.get("reads_cache_only", False))
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are not a multiple of {self.kv_heads} kv heads")
        self.position = parts.get("position")
        q_width = self.heads * self.head_dim
        kv_width = self.kv_heads * self.head_dim
        if self.reads_only:
            self.stored_kv_heads = 0
            fused = weights["q_proj"]
        else:
            self.stored_kv_heads = self.kv_heads
            fused = torch.cat([weights["q_proj"], weights["k_proj"], weights["v_proj"]], dim=0)
        self.qkv_width = q_width + 2 * self.stored_kv_heads * self.head_dim
        self.w_qkv = rt.matrix(fused)
        self.w_out = rt.matrix(weights["out_proj"])
        self.q_norm = rt.vector(weights["q_norm"]) if "q_norm" in weights else None
        self.k_norm = rt.vector(weights["k_norm"]) if "k_norm" in weights else None
        self.binding: Optional[PagedBinding] = None
        self._resident_blocks: Optional[int] = None      # (asked of the kernel library at the first decode step)
        self.qkv = rt.scratch("attention.qkv", self.qkv_width)
        self.attended = rt.scratch("attention.out", q_width)
        assert kv_width >= 0

    def cache_need(self):
        return PagedNeed(kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def bind_cache(self, binding: PagedBinding) -> None:
        if binding.owner and self.reads_only:
            raise ValueError("an attention mixer without k/v projections cannot own a cache")
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_qkv)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, b, t = self.rt, self.binding, step.tokens
        rt.linear(x, self.w_qkv, self.qkv, t)
        table = step.block_tables[b.group]
        fused = self.position.fused() if self.position is not None else {"inv_freq": None, "rotary_dim": 0}
        store = b.owner and not self.reads_only
        if (fused is not None and store and rt.fuse_decode_qk and self._decodes(step)):
            # one token per request: norm, rotation and cache write happen inside the attention kernel
            chunk, max_splits, partial_o, partial_ml, counters = self._decode_split(step)
            kernels.attention_decode_fused(self.qkv, self.qkv_width, self.attended, b.k, b.v, step.positions,
                                           step.token_span, table, t, self.heads, self.kv_heads, self.head_dim,
                                           b.page_tokens, self.window, self.scale, chunk, max_splits, partial_o,
                                           partial_ml, counters, step.error_flag, self.q_norm, self.k_norm,
                                           fused["inv_freq"], fused["rotary_dim"], self.eps)
            rt.linear(self.attended, self.w_out, out, t)
            return
        if fused is not None:
            kernels.qk_norm_rope_store(self.qkv, self.q_norm, self.k_norm, fused["inv_freq"], step.positions,
                                       step.token_span, table, b.k, b.v, t, self.heads, self.stored_kv_heads,
                                       self.head_dim, fused["rotary_dim"], b.page_tokens, self.eps, store,
                                       step.error_flag)
        else:
            # unfused: normalise in place, let the position part rewrite q and k, then store
            kernels.qk_norm_rope_store(self.qkv, self.q_norm, self.k_norm, None, step.positions, step.token_span,
                                       table, b.k, b.v, t, self.heads, self.stored_kv_heads, self.head_dim, 0,
                                       b.page_tokens, self.eps, 2 if self.stored_kv_heads else 0, step.error_flag)
            rows = self.qkv[:t]
            q_width = self.heads * self.head_dim
            kv_width = self.stored_kv_heads * self.head_dim
            q_view = rows[:, :q_width].unflatten(1, (self.heads, self.head_dim))
            k_view = rows[:, q_width:q_width + kv_width].unflatten(1, (self.stored_kv_heads, self.head_dim))
            self.position.apply(q_view, k_view, step.positions[:t], t)
            if store:
                kernels.qk_norm_rope_store(self.qkv, None, None, None, step.positions, step.token_span, table,
                                           b.k, b.v, t, self.heads, self.stored_kv_heads, self.head_dim, 0,
                                           b.page_tokens, self.eps, True, step.error_flag)
        self.attend(step, table)
        rt.linear(self.attended, self.w_out, out, t)

    def _decode_split(self, step: StepContext, tokens: Optional[int] = None):
        """One query token per request: how the keys are split so that few requests still fill the GPU,
        and the scratch of the split (chunk, max_splits, partial outputs, maxima and sums, counters)."""
        rt = self.rt
        if self._resident_blocks is None:
            self._resident_blocks = kernels.attention_decode_resident_blocks(self.head_dim) or DECODE_RESIDENT_BLOCKS
        chunk, max_splits, cap_splits = decode_split(tokens or step.tokens, self.kv_heads, step.context_bucket,
                                                     self.window, rt.max_context, self._resident_blocks)
        rows = rt.max_requests * self.heads * cap_splits
        partial_o = rt.flat_scratch("attention.partial_o", rows * self.head_dim, torch.float32)
        partial_ml = rt.flat_scratch("attention.partial_ml", rows * 2, torch.float32)
        counters = rt.flat_scratch("attention.counters", rt.max_requests * self.kv_heads, torch.int32, zero=True)
        return chunk, max_splits, partial_o, partial_ml, counters

    def _decodes(self, step: StepContext) -> bool:
        """Whether the step goes to the split-key decode kernel (one query token per request)."""
        rt = self.rt
        return (step.max_span == 1 and step.tokens <= rt.max_requests and
                kernels.attention_decode_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype))

    def attend(self, step: StepContext, table: torch.Tensor) -> None:
        """Attention of the step's queries (normalised, rotated, in ``self.qkv``) over the cache, which holds the
        step's own keys and values already. A step that is all single tokens goes to the split-key decode
        kernel. A step that begins with single-token spans and goes on with prompt portions (the order the
        scheduler plans: decoding requests first) is served by both: the decode kernel shares a request's keys
        among the query heads of a group and splits long contexts, where a prompt kernel would walk the whole
        context once per query head for one row of a 128-row tile."""
        b = self.binding
        rt = self.rt
        if self._decodes(step):
            self._attend_single_tokens(step, table, step.tokens)
            return
        single = step.leading_single_tokens
        if (0 < single < step.tokens and single <= rt.max_requests and step.host_span_lengths is not None
                and kernels.attention_decode_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype)):
            self._attend_single_tokens(step, table, single)
            self._attend_portions(step, table, single)
            return
        self._attend_portions(step, table, 0)

    def _attend_single_tokens(self, step: StepContext, table: torch.Tensor, count: int) -> None:
        """The first ``count`` tokens of the step, each the only token of its span."""
        b = self.binding
        chunk, max_splits, partial_o, partial_ml, counters = self._decode_split(step, count)
        kernels.attention_decode(self.qkv, self.qkv_width, self.attended, b.k, b.v, step.positions,
                                 step.token_span, table, count, self.heads, self.kv_heads,
                                 self.head_dim, b.page_tokens, self.window, self.scale, chunk, max_splits,
                                 partial_o, partial_ml, counters, step.error_flag)

    def _attend_portions(self, step: StepContext, table: torch.Tensor, skip: int) -> None:
        """The spans from ``skip`` on (the spans before it have one token each, so span ``skip`` begins at token
        ``skip``). The kernels take token indices from ``span_begin`` and table rows by span, so a later part of
        both arrays addresses the same buffers."""
        b = self.binding
        rt = self.rt
        spans = step.spans - skip
        span_begin = step.span_begin[skip:]
        span_table = table[skip:]
        lengths = step.host_span_lengths[skip:] if step.host_span_lengths is not None else None
        if (lengths is not None and rt.tcgen05_attention and kernels.attention_prefill_tcgen05_supported(
                self.heads, self.kv_heads, self.head_dim, b.page_tokens, rt.act_dtype)):
            # head size 64: S and O' in tensor memory, Q/K/V by TMA
            tiles = step.prompt_tile_bound or sum((length + 127) // 128 for length in lengths)
            kernels.attention_prefill_tcgen05(self.qkv, self.qkv_width, self.attended, b.k, b.v, step.positions,
                                              span_begin, span_table, step.tokens, spans, tiles, self.heads,
                                              self.kv_heads, self.head_dim, b.page_tokens, self.window, self.scale,
                                              step.error_flag)
            return
        if kernels.attention_prefill_supported(self.heads, self.kv_heads, self.head_dim, rt.act_dtype):
            kernels.attention_prefill(self.qkv, self.qkv_width, self.attended, b.k, b.v, step.positions,
                                      span_begin, span_table, step.tokens, spans, self.heads, self.kv_heads,
                                      self.head_dim, b.page_tokens, self.window, self.scale, step.error_flag)
            return
        kernels.attention_generic(self.qkv[skip:], self.qkv_width, self.attended[skip:], b.k, b.v,
                                  step.positions[skip:], step.token_span[skip:], table, step.tokens - skip,
                                  self.heads, self.kv_heads, self.head_dim, b.page_tokens, self.window, self.scale,
                                  step.error_flag)


@register_part("mixer", "short_conv")
class ShortConvMixer:
    """Gated short convolution: [B|C|X] = in_proj(x); conv over B*X with a depthwise causal
    kernel of ``taps`` taps; out_proj(C * conv). Per-request state: the last taps-1 values of
    B*X per channel, float32 (celeg src/backend/cpu/kernels/convolution.cpp:7-28;
    src/backend/cuda/packed/operators.cu:31-62)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.taps = int(params["taps"])
        self.w_in = rt.matrix(weights["in_proj"])
        self.w_out = rt.matrix(weights["out_proj"])
        self.kernel = rt.vector(weights["conv"].reshape(self.hidden, self.taps))
        self.binding: Optional[StateBinding] = None
        self.projected = rt.scratch("short_conv.proj", 3 * self.hidden)
        self.gated = rt.scratch("short_conv.out", self.hidden)

    def cache_need(self):
        return StateNeed(elements=(self.taps - 1) * self.hidden)

    def bind_cache(self, binding: StateBinding) -> None:
        self.binding = binding

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_in)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        if not rt.linear_short_conv(x, self.w_in, self.kernel, self.taps, self.binding, self.gated, step):
            rt.linear(x, self.w_in, self.projected, t)
            kernels.short_conv(self.projected, self.kernel, self.binding.state, self.binding.slot_stride,
                               self.gated, step.token_span, step.span_begin, step.span_slot, t, step.spans,
                               self.hidden, self.taps, step.max_span)
        rt.linear(self.gated, self.w_out, out, t)
