"""Typed configuration, the model description data, and the architecture registry."""
from .errors import ConfigError, UnknownArchitectureError
from .spec import ExecutionEntry, LayerSpec, ModelSpec, PartSpec, TensorRef
from .registry import (Architecture, architecture_named, architecture_of, known_architectures,
                       read_config_json, register_architecture)
from .lfm2 import CONV, FULL_ATTENTION, Lfm2Config
from . import lfm2_arch as _lfm2_arch  # registers "lfm2"
from .lfm2_arch import build_lfm2_spec

__all__ = [
    "Architecture", "ConfigError", "UnknownArchitectureError", "ExecutionEntry", "LayerSpec",
    "ModelSpec", "PartSpec", "TensorRef", "architecture_named", "architecture_of",
    "known_architectures", "read_config_json", "register_architecture", "CONV",
    "FULL_ATTENTION", "Lfm2Config", "build_lfm2_spec",
]
