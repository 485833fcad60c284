"""Block arrangements: how a layer's norms, mixer and feed-forward sit around the residual
stream. Interface:

    Arrangement(layer_parts, rt)     layer_parts: dict with mixer_norm, mixer, feed_forward_norm,
                                     feed_forward (the last two may be None)
    run(residual, pending, step) -> pending
        residual: float32 [T, hidden], the residual stream, updated in place
        pending:  an activation-type [T, hidden] output of the previous sub-layer that has NOT
                  been added to the residual yet, or None; the returned tensor has the same
                  meaning for the next block. Carrying it lets the add fuse with the next norm.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .registry import register_part
from .runtime import Runtime, StepContext


@register_part("arrangement", "prenorm_residual")
class PreNormResidual:
    """h = x + Mixer(Norm(x)); y = h + FeedForward(Norm(h))
    (celeg src/backend/cpu/model_forward_token.cpp:89-176; src/backend/cuda/packed/layer_executor.cu:101-216)."""

    def __init__(self, layer_parts: Mapping, rt: Runtime):
        self.rt = rt
        self.mixer_norm = layer_parts["mixer_norm"]
        self.mixer = layer_parts["mixer"]
        self.ffn_norm = layer_parts.get("feed_forward_norm")
        self.ffn = layer_parts.get("feed_forward")
        hidden = self.mixer_norm.width
        self.normed = rt.scratch("block.normed", hidden)
        self.delta_a = rt.scratch("block.delta_a", hidden)
        self.delta_b = rt.scratch("block.delta_b", hidden)

    def run(self, residual: torch.Tensor, pending: Optional[torch.Tensor], step: StepContext,
            mixer=None) -> torch.Tensor:
        mixer = mixer or self.mixer
        t = step.tokens
        self.mixer_norm.add_norm(residual, pending, self.normed, t)
        mixer.forward(self.normed, self.delta_a, step)
        if self.ffn is None:
            return self.delta_a
        self.ffn_norm.add_norm(residual, self.delta_a, self.normed, t)
        self.ffn.forward(self.normed, self.delta_b, step)
        return self.delta_b
