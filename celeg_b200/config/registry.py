"""One registry from an architecture's name (config.json ``model_type``) to its
typed configuration and its model builder.

celeg keeps an ``ArchitectureCatalog`` that is filled at start-up and then
consulted for every checkpoint (src/model/architecture.cpp:31-80); an unknown
checkpoint is an error that lists what is known. The same contract holds here,
keyed by ``model_type``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

from .errors import ConfigError, UnknownArchitectureError
from .spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Mapping[str, Any]], Any]          # raw dict -> typed config
    resolve_config: Callable[[Any, Mapping[str, Any]], Any]   # (config, tensor shapes) -> config
    build_spec: Callable[[Any], ModelSpec]                    # typed config -> ModelSpec
    random_init: Callable[[Any, str, tuple], str]             # (config, tensor name, shape) -> distribution id


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(architecture: Architecture, *, replace: bool = False) -> None:
    if architecture.name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{architecture.name}' is already registered")
    _ARCHITECTURES[architecture.name] = architecture


def known_architectures() -> list:
    return sorted(_ARCHITECTURES)


def architecture_named(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitectureError(
            f"no architecture is registered for model_type '{name}'; known: "
            f"{', '.join(known_architectures()) or 'none'}") from None


def architecture_of(raw_config: Mapping[str, Any]) -> Architecture:
    model_type = raw_config.get("model_type")
    if not isinstance(model_type, str) or not model_type:
        raise UnknownArchitectureError(
            "config.json has no 'model_type'; known: " + (", ".join(known_architectures()) or "none"))
    return architecture_named(model_type)


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as handle:
            raw = json.load(handle)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return merge_generation_config(raw, model_dir)


def merge_generation_config(raw: dict, model_dir: str) -> dict:
    """``generation_config.json`` beside config.json names the token ids that generation really uses; where
    it gives ``bos_token_id`` or ``eos_token_id`` (a number, or a list of numbers) they replace config.json's,
    as in celeg (src/checkpoint/catalog.cpp:95-123). A file that cannot be read as JSON is ignored there, and
    here."""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.isfile(path):
        return raw
    try:
        with open(path, "r", encoding="utf-8") as handle:
            generation = json.load(handle)
    except (OSError, ValueError):
        return raw
    if not isinstance(generation, dict):
        return raw
    merged = dict(raw)
    for key in ("bos_token_id", "eos_token_id"):
        value = generation.get(key)
        if isinstance(value, bool):
            continue
        if isinstance(value, (int, float)):
            merged[key] = int(value)
        elif isinstance(value, list):
            ids = [int(item) for item in value if isinstance(item, (int, float)) and not isinstance(item, bool)]
            if ids:
                merged[key] = ids
    return merged
