"""The two ends of a model as parts: what turns a step's token ids into rows of the residual stream
("input") and what turns the stream's wanted rows into logits ("output"). A model description that
names neither gets the two below, built from its embedding table, final norm, head and scale factors;
one that needs something else at an end (a norm after the embedding, capped logits, several heads)
names a kind of its own, registered like any other part.

An input part has ``run(stream, step, first)``: write ``stream.residual[:step.tokens]``; ``first`` is
None or ``(norm weight, SplitNorm)`` of the first block's norm, which the part may prepare (and then sets
``stream.prepared``). ``vocab_size`` is the number of token ids it takes.
An output part has ``next_norm(step, n_logits)``: the norm it applies first if it takes it split over the
last block's closing product and its own (else None), and ``run(stream, step, logit_rows, n_logits,
logits)``: float32 logits of the stream's rows ``logit_rows[:n_logits]`` (all rows in order when
``step.logits_of_all_rows``) into ``logits[:n_logits]``.

celeg's counterparts: the embedding gather and the tied or untied LM head of the packed executor
(src/backend/cuda/packed/operators.cu:19-64, src/backend/cuda/packed/logits.cu:12-77).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("input", "embedding")
class EmbeddingInput:
    """rows = multiplier * table[token ids] in float32; the first half of the first block's norm when asked."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.table = rt.matrix(weights["table"])
        self.vocab_size = int(self.table.shape[0])
        self.multiplier = float(params.get("multiplier", 1.0))

    def run(self, stream, step: StepContext, first=None) -> None:
        tokens = step.token_ids[:step.tokens]
        if first is not None:
            norm, (weight, split) = first
            kernels.embedding(self.table, tokens, stream.residual, self.multiplier, prepare=split, next_weight=weight)
            stream.prepared = (norm, split)
        else:
            kernels.embedding(self.table, tokens, stream.residual, self.multiplier)


@register_part("output", "norm_head")
class NormHeadOutput:
    """logits = multiplier * (norm(stream rows) @ head^T): the nested part ``norm``, then the head matrix
    (the embedding table itself when the description ties them: the runtime places a tensor once)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.norm = parts["norm"]
        self.head = rt.matrix(weights["head"])
        self.multiplier = float(params.get("multiplier", 1.0))
        self.normed = rt.scratch("model.final_normed", int(self.head.shape[1]))

    def next_norm(self, step: StepContext, n_logits: int):
        if n_logits > 0 and step.logits_of_all_rows and self.rt.takes_split_norm(n_logits, self.head):
            return self.norm
        return None

    def run(self, stream, step: StepContext, logit_rows: torch.Tensor, n_logits: int, logits: torch.Tensor) -> None:
        if step.logits_of_all_rows:
            normed = stream.normed(self.norm, self.normed, n_logits)
        else:
            normed = stream.normed(self.norm, self.normed, n_logits, gather=logit_rows)
        self.rt.linear(normed, self.head, logits, n_logits)
        if self.multiplier != 1.0:
            logits[:n_logits].mul_(self.multiplier)
