"""Reading and writing the safetensors container, without any helper library.

Layout: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``,
then the data area. The checks are the ones celeg's reader makes
(src/checkpoint/formats/safetensors.cpp:155-239): header inside the file, JSON
object, offsets ordered and in range, byte count equal to shape x element size,
no duplicate and no overlapping tensors; every message names the tensor.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch


class CheckpointFormatError(ValueError):
    """The file is not a well-formed safetensors container."""


_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "I16": (torch.int16, 2), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int          # offsets inside the data area
    end: int
    path: str


class SafetensorsFile:
    """One mapped file; tensors are materialised on request."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError:
            raise CheckpointFormatError(f"{path}: cannot be opened") from None
        if size < 8:
            raise CheckpointFormatError(f"{path}: shorter than the 8-byte header length")
        self._handle = open(path, "rb")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > _MAX_HEADER or 8 + header_len > size:
            raise CheckpointFormatError(f"{path}: header length {header_len} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise CheckpointFormatError(f"{path}: header is not valid JSON: {exc}") from None
        if not isinstance(header, dict):
            raise CheckpointFormatError(f"{path}: header must be a JSON object")
        self.data_start = 8 + header_len
        data_size = size - self.data_start
        self.metadata = header.get("__metadata__") or {}
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(info, dict):
                raise CheckpointFormatError(f"{path}: entry of tensor '{name}' is not an object")
            dtype = info.get("dtype")
            shape = info.get("shape")
            offsets = info.get("data_offsets")
            if dtype not in _DTYPES:
                raise CheckpointFormatError(f"{path}: tensor '{name}' has unsupported dtype {dtype!r}")
            if not isinstance(shape, list) or not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0
                                                      for d in shape):
                raise CheckpointFormatError(f"{path}: tensor '{name}' has a malformed shape {shape!r}")
            if (not isinstance(offsets, list) or len(offsets) != 2 or
                    not all(isinstance(o, int) and not isinstance(o, bool) for o in offsets)):
                raise CheckpointFormatError(f"{path}: tensor '{name}' has malformed data_offsets {offsets!r}")
            begin, end = offsets
            if begin < 0 or end < begin or end > data_size:
                raise CheckpointFormatError(
                    f"{path}: tensor '{name}' lies at [{begin}, {end}) outside the data area of {data_size} bytes")
            count = 1
            for dim in shape:
                count *= dim
            if end - begin != count * _DTYPES[dtype][1]:
                raise CheckpointFormatError(
                    f"{path}: tensor '{name}' holds {end - begin} bytes, shape {shape} of {dtype} needs "
                    f"{count * _DTYPES[dtype][1]}")
            self.entries[name] = TensorEntry(name, dtype, tuple(shape), begin, end, path)
        ordered = sorted((e for e in self.entries.values() if e.end > e.begin), key=lambda e: e.begin)
        for left, right in zip(ordered, ordered[1:]):
            if right.begin < left.end:
                raise CheckpointFormatError(
                    f"{path}: tensors '{left.name}' and '{right.name}' overlap in the data area")

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor with a copy of the stored values, in the stored dtype."""
        entry = self.entries[name]
        dtype, _ = _DTYPES[entry.dtype]
        raw = bytearray(self._map[self.data_start + entry.begin:self.data_start + entry.end])
        if not raw:
            return torch.empty(entry.shape, dtype=dtype)
        return torch.frombuffer(raw, dtype=dtype).reshape(entry.shape)

    def close(self) -> None:
        try:
            self._map.close()
        finally:
            self._handle.close()


class TensorRepository:
    """All tensors of a model folder: ``model.safetensors``, or the shards named by
    ``model.safetensors.index.json`` (celeg src/checkpoint/repositories/safetensors.cpp)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        paths: List[str] = []
        if os.path.isfile(single):
            paths = [single]
        elif os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as handle:
                    weight_map = json.load(handle)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as exc:
                raise CheckpointFormatError(f"{index}: no readable 'weight_map': {exc}") from None
            paths = [os.path.join(model_dir, shard) for shard in sorted(set(weight_map.values()))]
        else:
            raise CheckpointFormatError(
                f"{model_dir}: neither model.safetensors nor model.safetensors.index.json exists")
        self.files = [SafetensorsFile(path) for path in paths]
        self._owner: Dict[str, SafetensorsFile] = {}
        for handle in self.files:
            for name in handle.entries:
                if name in self._owner:
                    raise CheckpointFormatError(
                        f"tensor '{name}' is stored twice: in {self._owner[name].path} and {handle.path}")
                self._owner[name] = handle

    def names(self) -> List[str]:
        return sorted(self._owner)

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return {name: handle.entries[name].shape for name, handle in self._owner.items()}

    def stored_dtype(self, name: str) -> str:
        return self._owner[name].entries[name].dtype

    def tensor(self, name: str) -> torch.Tensor:
        return self._owner[name].tensor(name)

    def close(self) -> None:
        for handle in self.files:
            handle.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """Write CPU tensors in name order; the data area starts on an 8-byte boundary."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    ordered: List[Tuple[str, torch.Tensor]] = []
    for name in sorted(tensors):
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise CheckpointFormatError(f"tensor '{name}' has dtype {tensor.dtype}, which safetensors cannot hold")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
        ordered.append((name, tensor))
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in ordered:
            if tensor.numel():
                handle.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
