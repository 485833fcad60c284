"""Feed-forward parts. Interface:

    FeedForward(params, weights, parts, rt)
    forward(x, out, step)     x: normed activations [T, hidden]; writes the output to out
    takes_split_norm(step)    optional, as for mixers
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("feed_forward", "swiglu")
class SwiGluFeedForward:
    """down(silu(gate(x)) * up(x)); gate and up are one fused projection [2I, H] (gate rows
    first), as celeg concatenates w1 and w3 (src/backend/cpu/weights_loader.cpp:93-99;
    src/backend/cuda/packed/operators.cu:531-596)."""

    def __init__(self, params: Mapping, weights: Mapping[str, torch.Tensor], parts: Mapping, rt: Runtime):
        self.rt = rt
        self.hidden = int(params["hidden_size"])
        self.inner = int(params["intermediate_size"])
        self.w_gate_up = rt.matrix(torch.cat([weights["gate"], weights["up"]], dim=0))
        self.w_down = rt.matrix(weights["down"])
        self.gate_up = rt.scratch("swiglu.gate_up", 2 * self.inner)
        self.activated = rt.scratch("swiglu.act", self.inner)

    ends_with_product = True      # forward() writes `out` last, with rt.linear

    def takes_split_norm(self, step: StepContext) -> bool:
        return self.rt.takes_split_norm(step.tokens, self.w_gate_up)

    def forward(self, x: torch.Tensor, out: torch.Tensor, step: StepContext) -> None:
        rt, t = self.rt, step.tokens
        rt.linear_swiglu(x, self.w_gate_up, self.gate_up, self.activated, t, self.inner)
        rt.linear(self.activated, self.w_down, out, t)
