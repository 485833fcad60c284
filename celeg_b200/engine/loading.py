"""From a model folder to a step function: config.json picks the architecture, the checkpoint is
checked against the model description, caches are sized, parts are built."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.fingerprint import model_fingerprint
from ..config.registry import architecture_of, read_config_json
from ..parts import Runtime
from ..parts.options import KernelOptions
from ..weights.loader import load_tensors
from ..weights.safetensors_io import TensorRepository
from .model import Model
from .step import PADDING_TOKENS, StepFunction

DEFAULT_PAGE_TOKENS = 16        # celeg's CUDA engine default (include/celeg/backend/cuda/concurrency.hpp:23)


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        dtype = name
    else:
        table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
                 "fp32": torch.float32, "f32": torch.float32}
        if str(name).lower() not in table:
            raise ValueError(f"dtype must be bfloat16 or float32, got {name!r}")
        dtype = table[str(name).lower()]
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype}")
    return dtype


@dataclass
class LoadedModel:
    config: object
    spec: object
    model: Model
    runtime: Runtime
    manager: CacheManager
    storage: CacheStorage
    step: StepFunction
    fingerprint: str = ""            # hash of the resolved configuration and every tensor's name, shape and type


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0", *, max_context: Optional[int] = None,
               cache_tokens: Optional[int] = None, page_tokens: int = DEFAULT_PAGE_TOKENS,
               max_requests: int = 8, max_batched_tokens: int = 512, use_graphs: bool = False,
               kernel_options: Optional[KernelOptions] = None) -> LoadedModel:
    """``cache_tokens``: how many positions all live requests may hold together (each request
    rounded up to whole pages); default ``max_requests * max_context``. ``kernel_options``: the
    switches of the kernel path (defaults: what measured best)."""
    dtype = parse_dtype(dtype)
    device = torch.device(device)
    raw = read_config_json(model_dir)
    architecture = architecture_of(raw)
    repository = TensorRepository(model_dir)
    try:
        shapes = repository.shapes()
        config = architecture.resolve_config(architecture.parse_config(raw), shapes)
        spec = architecture.build_spec(config)
        tensors = load_tensors(repository, spec)
        fingerprint = fingerprint_of(config, raw, repository)
    finally:
        repository.close()
    context = min(max_context or spec.max_context, spec.max_context) if max_context else spec.max_context
    # (buffers hold the rows a step may be padded by when it takes its launch shape from a grid, see StepFunction)
    rt = Runtime(device, dtype, max_batched_tokens + (PADDING_TOKENS if use_graphs else 0), max_requests=max_requests,
                 max_context=context, options=kernel_options)
    with torch.cuda.device(device):
        model = Model(spec, tensors, rt)
        del tensors
        if cache_tokens is None:
            cache_tokens = max_requests * context
        pages = (cache_tokens + page_tokens - 1) // page_tokens
        group_pages = [pages for _ in model.group_keys]
        storage = CacheStorage([(need, len(members)) for need, members in
                                zip(model.group_needs, model.group_members)],
                               group_pages, page_tokens, model.state_layout, max_requests, dtype, device)
        manager = CacheManager(page_tokens, group_pages, list(zip(model.group_keys, model.group_needs)),
                               model.state_layout, max_requests, clear_slot=storage.clear_slot,
                               table_capacity=(context + page_tokens - 1) // page_tokens)
        for group, members in zip(manager.groups, model.group_members):
            group.members = list(members)
        model.attach(storage)
        step = StepFunction(model, manager, storage, rt, max_batched_tokens, max_requests, context,
                            use_graphs=use_graphs)
    return LoadedModel(config=config, spec=spec, model=model, runtime=rt, manager=manager, storage=storage,
                       step=step, fingerprint=fingerprint)


def fingerprint_of(config, raw: dict, repository: TensorRepository) -> str:
    """The model's fingerprint from its resolved configuration (``to_dict()`` where the architecture's
    configuration has one, else config.json as read) and the checkpoint's tensor table."""
    as_dict = config.to_dict() if hasattr(config, "to_dict") else dict(raw)
    shapes = repository.shapes()
    return model_fingerprint(as_dict, shapes, {name: repository.stored_dtype(name) for name in shapes})
