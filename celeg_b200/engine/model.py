"""A model built from a description: parts looked up in the registries, weights handed to
them by name, caches bound per position of the run order."""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Tuple

import torch

from .. import kernels
from ..cache.manager import PagedNeed, StateLayout, StateNeed
from ..cache.storage import CacheStorage
from ..config.spec import LayerSpec, ModelSpec, PartSpec
from ..parts import PagedBinding, Runtime, StateBinding, StepContext, part_factory
from ..parts.runtime import ResidualStream


def _weights_of(part: PartSpec, tensors: Mapping[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {role: tensors[ref.name] for role, ref in part.tensors.items()}


def build_part(category: str, part: Optional[PartSpec], tensors: Mapping[str, torch.Tensor], rt: Runtime):
    """The part a description names, from the registry of its category. Norms are built from
    ``(params, weights, rt)``, position encodings from ``(params, rt)``, every other category from
    ``(params, weights, nested parts, rt)``; a nested part's category is what its description states, else
    its name if that is a category."""
    if part is None:
        return None
    factory = part_factory(category, part.kind)
    if category == "norm":
        return factory(part.params, _weights_of(part, tensors), rt)
    if category == "position":
        return factory(part.params, rt)
    children = {name: build_part(child.category or name, child, tensors, rt) for name, child in part.parts.items()}
    return factory(part.params, _weights_of(part, tensors), children, rt)


class Layer:
    """The parts of one block, built: the four named ones and whatever else the description lists, all under
    their names in ``parts`` (what the arrangement gets). ``cache_parts`` are those that ask for a cache."""

    def __init__(self, spec: LayerSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime):
        self.name = spec.name
        self.parts = {
            "mixer_norm": build_part("norm", spec.mixer_norm, tensors, rt),
            "mixer": build_part("mixer", spec.mixer, tensors, rt),
            "feed_forward_norm": build_part("norm", spec.feed_forward_norm, tensors, rt),
            "feed_forward": build_part("feed_forward", spec.feed_forward, tensors, rt),
        }
        for name, part in spec.extra_parts.items():
            if name in self.parts:
                raise ValueError(f"layer {spec.name}: the extra part '{name}' has the name of a standard part")
            if not part.category:
                raise ValueError(f"layer {spec.name}: the extra part '{name}' does not state its category")
            self.parts[name] = build_part(part.category, part, tensors, rt)
        self.mixer = self.parts["mixer"]
        self.cache_parts = {name: part for name, part in self.parts.items()
                            if part is not None and hasattr(part, "cache_need")}
        self.block = part_factory("arrangement", spec.arrangement)(self.parts, rt)


class Model:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.vocab_size = spec.vocab_size
        self.hidden_size = spec.hidden_size
        self.layers = [Layer(layer, tensors, rt) for layer in spec.layers]
        self.order = list(spec.order)
        # the two ends (parts of the categories "input" and "output"; the built-in ones unless the description
        # names others)
        self.input = build_part("input", spec.input_part(), tensors, rt)
        self.output = build_part("output", spec.output_part(), tensors, rt)
        rt.release_sources()
        self.stream = ResidualStream(rt, spec.hidden_size)
        self.residual = self.stream.residual
        # per position of the run order: {part name: binding} for the parts of its layer that hold a cache
        self.bindings: List[Dict[str, object]] = [{} for _ in self.order]
        self._rebind = len({entry.layer for entry in self.order}) != len(self.order)
        self._plan_caches()

    # ------------------------------------------------------------------ caches
    def _plan_caches(self) -> None:
        """Group the needs of every cache-holding part: one paged group per distinct need, one slot layout.
        A place in a cache is named by (position of the run order, name of the part in its layer)."""
        self.group_keys: List[tuple] = []
        self.group_needs: List[PagedNeed] = []
        self.group_members: List[List[tuple]] = []      # (position, part name) places that OWN a layer of the group
        self.state_layout = StateLayout()
        self.position_group: Dict[tuple, Tuple[int, int]] = {}   # place -> (group, layer index in group)
        for position, entry in enumerate(self.order):
            for name, part in self.layers[entry.layer].cache_parts.items():
                need = part.cache_need()
                if entry.cache_of is not None:
                    source = self.layers[self.order[entry.cache_of].layer].cache_parts.get(name)
                    source_need = source.cache_need() if source is not None else None
                    if type(need) is not type(source_need) or need != source_need:
                        raise ValueError(f"run order position {position} reads the cache of position "
                                         f"{entry.cache_of}, whose need {source_need} for '{name}' differs from "
                                         f"its own {need}")
                    continue
                if need is None:
                    continue
                place = (position, name)
                if isinstance(need, PagedNeed):
                    key = need.group_key()
                    if key not in self.group_keys:
                        self.group_keys.append(key)
                        self.group_needs.append(need)
                        self.group_members.append([])
                    group = self.group_keys.index(key)
                    self.position_group[place] = (group, len(self.group_members[group]))
                    self.group_members[group].append(place)
                elif isinstance(need, StateNeed):
                    self.state_layout.add(place, need.elements)
                else:
                    raise TypeError(f"part '{name}' of layer {entry.layer} asks for an unknown cache need {need!r}")

    def attach(self, storage: CacheStorage) -> None:
        """Give every cache-holding part at every position of the run order the place its cache lives in."""
        for position, entry in enumerate(self.order):
            for name, part in self.layers[entry.layer].cache_parts.items():
                need = part.cache_need()
                if need is None:
                    continue
                source = (position if entry.cache_of is None else entry.cache_of, name)
                owner = entry.cache_of is None
                if isinstance(need, PagedNeed):
                    group, index = self.position_group[source]
                    self.bindings[position][name] = PagedBinding(group=group, k=storage.k[group][index],
                                                                 v=storage.v[group][index],
                                                                 page_tokens=storage.page_tokens, owner=owner)
                else:
                    offset = self.state_layout.offsets[source]
                    self.bindings[position][name] = StateBinding(state=storage.state[:, offset:],
                                                                 slot_stride=storage.state.stride(0), owner=owner)
        if not self._rebind:
            for position, entry in enumerate(self.order):
                self._bind(position)

    def _bind(self, position: int) -> None:
        parts = self.layers[self.order[position].layer].cache_parts
        for name, binding in self.bindings[position].items():
            parts[name].bind_cache(binding)

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once: what the parts put on the device, and the head (a tied
        head is the embedding table, counted once; of an untied table a step gathers a few rows only)."""
        total = self.rt.weight_bytes
        table, head = getattr(self.input, "table", None), getattr(self.output, "head", None)
        if table is not None and head is not table:
            total -= table.numel() * table.element_size()
        return total

    def weight_tensors(self) -> List[torch.Tensor]:
        """Every tensor that a part of the model holds (the ends' and the layers'), each once."""
        found, seen = [], set()
        holders = [self.input, self.output, getattr(self.output, "norm", None)]
        for layer in self.layers:
            holders.extend(layer.parts.values())
        for holder in holders:
            if holder is None:
                continue
            for value in vars(holder).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    found.append(value)
        return found

    # ----------------------------------------------------------------- forward
    def forward(self, step: StepContext, logit_rows: torch.Tensor, n_logits: int, logits: torch.Tensor) -> None:
        """Run the step's tokens through every position of the run order and write the logits
        of the wanted rows into ``logits[:n_logits]`` (float32)."""
        rt = self.rt
        stream = self.stream
        stream.begin()
        blocks = [self.layers[entry.layer].block for entry in self.order]
        firsts = [block.first_norm(step) if hasattr(block, "first_norm") else None for block in blocks]
        head_norm = self.output.next_norm(step, n_logits) if hasattr(self.output, "next_norm") else None
        first = None
        if firsts and firsts[0] is not None and rt.small_batch(step.tokens):
            halves = stream.split(firsts[0], 1)
            first = (firsts[0], halves) if halves is not None else None
        self.input.run(stream, step, first)
        for position, entry in enumerate(self.order):
            layer = self.layers[entry.layer]
            if self._rebind:
                self._bind(position)
            stream.after_layer = firsts[position + 1] if position + 1 < len(blocks) else head_norm
            layer.block.run(stream, step)
        stream.after_layer = None
        if n_logits == 0:
            stream.prepared = None
            return
        self.output.run(stream, step, logit_rows, n_logits, logits)
