"""Block arrangements: how a layer's norms, mixer and feed-forward sit around the residual
stream. Interface:

    Arrangement(layer_parts, rt)     layer_parts: dict with mixer_norm, mixer, feed_forward_norm,
                                     feed_forward (the last two may be None)
    run(stream, step)                stream: the step's ResidualStream, updated in place;
                                     stream.after_layer is the norm that will read the stream after this
                                     layer if its reader takes a split norm (see ResidualStream), else None
    first_norm(step)                 optional: the norm that reads the stream first, under the same condition

A part's ``forward(x, out, step)`` gets the normed activations and a buffer for its output; the
arrangement hands that buffer to the residual stream, which adds it inside the next norm kernel.
"""
from __future__ import annotations

from typing import Mapping

from .registry import register_part
from .runtime import ResidualStream, Runtime, StepContext


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

    def _sublayer(self, norm, part, delta, upcoming, stream: ResidualStream, step: StepContext) -> None:
        x = stream.normed(norm, self.normed, step.tokens)
        stream.expect(delta, upcoming if getattr(part, "ends_with_product", False) else None, step.tokens)
        part.forward(x, delta, step)
        stream.add_later(delta)

    def first_norm(self, step: StepContext):
        """The norm that reads the stream first, if its reader takes a split norm (else None)."""
        takes = getattr(self.mixer, "takes_split_norm", None)
        return self.mixer_norm if takes is not None and takes(step) else None

    def run(self, stream: ResidualStream, step: StepContext) -> None:
        after = stream.after_layer
        if self.ffn is None:
            self._sublayer(self.mixer_norm, self.mixer, self.delta_a, after, stream, step)
            return
        takes = getattr(self.ffn, "takes_split_norm", None)
        between = self.ffn_norm if takes is not None and takes(step) else None
        self._sublayer(self.mixer_norm, self.mixer, self.delta_a, between, stream, step)
        self._sublayer(self.ffn_norm, self.ffn, self.delta_b, after, stream, step)
