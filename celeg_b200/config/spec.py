"""Data that describes a model as an arrangement of parts.

An architecture builder turns its typed configuration into a :class:`ModelSpec`;
nothing below that level knows which architecture it serves. The shape follows
celeg's semantic graph (include/celeg/model/graph.hpp:414-469: a layer is
``{mixer_norm, mixer, feed_forward_norm, feed_forward, residual}``), with the
difference that every part is an open ``kind`` string resolved through the part
registries, so a new mixer or feed-forward needs no change here.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class TensorRef:
    """A checkpoint tensor a part needs: its name and the shape it must have.

    ``alt_shapes`` lists other stored shapes that are accepted and reshaped to
    ``shape`` (celeg accepts the conv kernel as [H,1,L] or [H,L]:
    src/model/inference/support.cpp:14-21).
    """
    name: str
    shape: Tuple[int, ...]
    alt_shapes: Tuple[Tuple[int, ...], ...] = ()
    integer: bool = False


@dataclass(frozen=True)
class PartSpec:
    """One part (norm, mixer, feed-forward, position encoding): registry kind,
    its sizes and constants, the tensors it owns, and parts nested in it.

    ``category`` names the registry the kind is looked up in ("norm", "mixer", "feed_forward",
    "position", ...). The four named parts of a :class:`LayerSpec` need none (their place says it); a
    nested part or an extra part of a layer states it, or carries a name that is itself a category."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    tensors: Mapping[str, TensorRef] = field(default_factory=dict)
    parts: Mapping[str, "PartSpec"] = field(default_factory=dict)
    category: Optional[str] = None

    def all_tensors(self) -> List[TensorRef]:
        out = list(self.tensors.values())
        for child in self.parts.values():
            out.extend(child.all_tensors())
        return out


@dataclass(frozen=True)
class LayerSpec:
    """One block: how the parts are arranged (``arrangement`` is a registry kind
    too) and which parts they are."""
    name: str
    arrangement: str
    mixer_norm: PartSpec
    mixer: PartSpec
    feed_forward_norm: Optional[PartSpec]
    feed_forward: Optional[PartSpec]
    # Further parts by name, each with its ``category``: norms after the mixer or the feed-forward, a second
    # mixer, a gate. The arrangement finds them under their names beside the four above; a part among them
    # that asks for a cache gets one of its own.
    extra_parts: Mapping[str, PartSpec] = field(default_factory=dict)

    def all_tensors(self) -> List[TensorRef]:
        out: List[TensorRef] = []
        for part in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward,
                     *self.extra_parts.values()):
            if part is not None:
                out.extend(part.all_tensors())
        return out


@dataclass(frozen=True)
class ExecutionEntry:
    """One position of the run order: which layer runs there, and whose cache its
    mixer uses. ``cache_of`` is the index of an EARLIER entry of the order whose
    cache this entry reads instead of owning one; ``None`` means it owns its own.
    A layer named at two positions runs twice with the same weights and, unless
    ``cache_of`` says otherwise, two caches."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_context: int
    embedding: TensorRef
    layers: Tuple[LayerSpec, ...]
    order: Tuple[ExecutionEntry, ...]
    final_norm: PartSpec
    lm_head: Optional[TensorRef]          # None: tied to the embedding table
    eos_token_ids: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None
    embedding_multiplier: float = 1.0
    logits_multiplier: float = 1.0
    optional_tensors: Tuple[TensorRef, ...] = ()
    # The two ends of the model as parts of the categories "input" (token ids -> rows of the residual stream) and
    # "output" (rows -> logits). None: the built-in ones, made of the fields above (embedding table and its
    # multiplier; final norm, tied or untied head and the logits' multiplier). A description that names its own
    # lists every tensor they need in them; ``embedding`` still names the table (its rows are the vocabulary).
    input: Optional[PartSpec] = None
    output: Optional[PartSpec] = None

    def input_part(self) -> PartSpec:
        if self.input is not None:
            return self.input
        return PartSpec("embedding", params={"multiplier": self.embedding_multiplier},
                        tensors={"table": self.embedding}, category="input")

    def output_part(self) -> PartSpec:
        if self.output is not None:
            return self.output
        return PartSpec("norm_head", params={"multiplier": self.logits_multiplier},
                        tensors={"head": self.lm_head if self.lm_head is not None else self.embedding},
                        parts={"norm": self.final_norm}, category="output")

    def all_tensors(self) -> List[TensorRef]:
        out: List[TensorRef] = []
        seen = set()
        refs = list(self.input_part().all_tensors())
        for layer in self.layers:
            refs.extend(layer.all_tensors())
        refs.extend(self.output_part().all_tensors())
        for ref in refs:                       # (a tied head names the embedding table a second time)
            if ref.name not in seen:
                seen.add(ref.name)
                out.append(ref)
        return out

    def validate(self) -> None:
        from .errors import ConfigError
        for position, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"run order position {position} names layer {entry.layer}, "
                                  f"the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < position:
                    raise ConfigError(f"run order position {position} reads the cache of position "
                                      f"{entry.cache_of}, which does not run before it")
                if self.order[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"run order position {position} reads the cache of position "
                                      f"{entry.cache_of}, which owns none itself")
