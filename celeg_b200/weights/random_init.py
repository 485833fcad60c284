"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed. celeg has no such mode; its tests build name-and-shape-only
repositories (tests/automatic_inference_test.cpp:147-177). Distributions: matrices
N(0, 0.02), norm weights 1 + N(0, 0.05), conv kernels N(0, 0.1). Every tensor has its
own generator keyed by (seed, tensor name), so a tensor's values do not depend on which
other tensors exist."""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Dict, Mapping, Optional

import torch

from ..config.registry import Architecture, architecture_of
from .safetensors_io import write_safetensors

_DISTRIBUTIONS = {"linear": (0.0, 0.02), "norm": (1.0, 0.05), "conv": (0.0, 0.1)}


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    generator = torch.Generator(device="cpu")
    generator.manual_seed(int.from_bytes(digest[:8], "little") >> 1)
    return generator


def random_tensors(architecture: Architecture, config: Any, seed: int,
                   dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    spec = architecture.build_spec(config)
    tensors: Dict[str, torch.Tensor] = {}
    for ref in spec.all_tensors():
        if ref.name in tensors:
            continue
        mean, std = _DISTRIBUTIONS[architecture.random_init(config, ref.name, ref.shape)]
        shape = ref.alt_shapes[0] if ref.alt_shapes else ref.shape   # stored layout of the checkpoint
        values = torch.empty(shape, dtype=torch.float32).normal_(0.0, std, generator=_generator(seed, ref.name))
        tensors[ref.name] = (values + mean).to(dtype)
    return tensors


def write_random_model(model_dir: str, raw_config: Mapping[str, Any], seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Create ``model_dir`` with config.json and model.safetensors; returns the folder."""
    architecture = architecture_of(raw_config)
    config = architecture.parse_config(raw_config)
    tensors = random_tensors(architecture, config, seed, dtype)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(dict(raw_config), handle, indent=1)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "random_seed": str(seed)})
    return model_dir
