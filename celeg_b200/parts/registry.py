"""Registries of part kinds. A model description names parts by ``kind``; the class behind a
kind is looked up here when the model is built, so a new mixer, feed-forward, norm, position
encoding, block arrangement or end of the model (what makes rows of token ids, what makes logits of rows)
is added by registering a class, with no change to the engine.

celeg dispatches over closed variants (``std::visit`` in src/backend/cuda/packed/layer_executor.cu:131-191);
the open registry is this engine's own choice.
"""
from __future__ import annotations

from typing import Callable, Dict

CATEGORIES = ("norm", "mixer", "feed_forward", "position", "arrangement", "input", "output")
_REGISTRY: Dict[str, Dict[str, Callable]] = {category: {} for category in CATEGORIES}


def register_part(category: str, kind: str, factory: Callable = None, *, replace: bool = False):
    """Register ``factory`` for ``kind``; usable as a decorator."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category '{category}'; categories: {', '.join(CATEGORIES)}")

    def _register(cls):
        if kind in _REGISTRY[category] and not replace:
            raise KeyError(f"{category} kind '{kind}' is already registered")
        _REGISTRY[category][kind] = cls
        return cls

    return _register(factory) if factory is not None else _register


def part_factory(category: str, kind: str) -> Callable:
    try:
        return _REGISTRY[category][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "none"
        raise KeyError(f"no {category} is registered under kind '{kind}'; known: {known}") from None


def registered(category: str):
    return sorted(_REGISTRY[category])
