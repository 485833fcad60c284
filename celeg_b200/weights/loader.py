"""Weights by tensor name: what a model description asks for against what the
folder holds, reported in ONE error.

celeg binds each role to a tensor name and fails on a missing role, an ambiguous
binding or a wrong shape (src/model/inference/support.cpp:23-55); tensors nobody
asked for are reported here as well. Kept precision: a tensor stored in bfloat16
stays bfloat16, a tensor stored in 32-bit floating point stays float32, float16
is widened to float32 (exact), integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Mapping, Sequence, Tuple

import torch

from ..config.spec import ModelSpec, TensorRef
from .safetensors_io import TensorRepository


class WeightsError(ValueError):
    """The checkpoint does not fit the model. ``missing``, ``unexpected`` and
    ``wrong_shape`` carry the lists that the message prints."""

    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, tuple, tuple]], wrong_dtype: Sequence[Tuple[str, str]] = ()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        lines = ["checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{name} is {list(found)}, expected {list(expected)}" for name, found, expected in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{name} is {found}" for name, found in self.wrong_dtype))
        super().__init__("\n".join(lines))


_FLOAT = {"BF16", "F16", "F32", "F64"}
_INTEGER = {"I8", "U8", "I16", "I32", "I64"}


def check_tensors(expected: Iterable[TensorRef], shapes: Mapping[str, tuple],
                  dtypes: Mapping[str, str] = None, optional: Iterable[str] = ()) -> None:
    """Raise one :class:`WeightsError` naming every mismatch, or return."""
    wanted: Dict[str, TensorRef] = {}
    for ref in expected:
        wanted.setdefault(ref.name, ref)
    missing = [name for name in wanted if name not in shapes]
    allowed = set(wanted) | set(optional)
    unexpected = sorted(name for name in shapes if name not in allowed)
    wrong_shape = []
    wrong_dtype = []
    for name, ref in wanted.items():
        if name not in shapes:
            continue
        found = tuple(shapes[name])
        if found != tuple(ref.shape) and found not in ref.alt_shapes:
            wrong_shape.append((name, found, tuple(ref.shape)))
        if dtypes is not None:
            stored = dtypes[name]
            if (stored not in _INTEGER) if ref.integer else (stored not in _FLOAT):
                wrong_dtype.append((name, stored))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype)


def kept_precision(tensor: torch.Tensor) -> torch.Tensor:
    if tensor.dtype == torch.bfloat16 or tensor.dtype == torch.float32:
        return tensor
    if tensor.dtype in (torch.float16,):
        return tensor.to(torch.float32)
    if tensor.dtype == torch.float64:
        return tensor.to(torch.float32)
    if tensor.dtype in (torch.int8, torch.uint8, torch.int16, torch.int32):
        return tensor.to(torch.int32)
    if tensor.dtype == torch.int64:
        if tensor.numel() and (tensor.max() > 2**31 - 1 or tensor.min() < -2**31):
            raise ValueError("an int64 table holds values outside the int32 range")
        return tensor.to(torch.int32)
    raise ValueError(f"unsupported stored dtype {tensor.dtype}")


def load_tensors(repository: TensorRepository, spec: ModelSpec) -> Dict[str, torch.Tensor]:
    """CPU tensors for every tensor the description names, reshaped to the shape it states."""
    refs = spec.all_tensors()
    shapes = repository.shapes()
    dtypes = {name: repository.stored_dtype(name) for name in shapes}
    check_tensors(refs, shapes, dtypes, optional=[ref.name for ref in spec.optional_tensors])
    out: Dict[str, torch.Tensor] = {}
    for ref in refs:
        if ref.name in out:
            continue
        out[ref.name] = kept_precision(repository.tensor(ref.name)).reshape(ref.shape)
    return out
