"""Reading and writing the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header that maps each
tensor name to ``{"dtype", "shape", "data_offsets"}``, then the raw bytes. It
takes the place of the reference's GGUF reader (app/gguf/reader.py:46-66,
app/gguf/loader.py:33-50): tensors are fetched by name, one at a time, so a
large model never sits in host memory twice.
"""

from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Iterable

import numpy as np
import torch


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors container."""


_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {dtype: name for name, (dtype, _) in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "path", "data_start")

    def __init__(self, name, dtype, shape, begin, end, path, data_start):
        self.name = name
        self.dtype = dtype
        self.shape = tuple(shape)
        self.begin = begin
        self.end = end
        self.path = path
        self.data_start = data_start


def _read_header(path: Path) -> tuple[dict, int]:
    size = path.stat().st_size
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise SafetensorsError(f"{path}: shorter than a safetensors header")
        (length,) = struct.unpack("<Q", prefix)
        if length > _MAX_HEADER or 8 + length > size:
            raise SafetensorsError(f"{path}: header length {length} does not fit the file")
        try:
            header = json.loads(handle.read(length).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise SafetensorsError(f"{path}: header is not JSON ({exc})") from exc
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    return header, 8 + length


class SafetensorsFile:
    """The tensors of one file, by name."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        header, data_start = _read_header(self.path)
        size = self.path.stat().st_size
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype_name, shape = info["dtype"], info["shape"]
                begin, end = info["data_offsets"]
            except (KeyError, TypeError, ValueError) as exc:
                raise SafetensorsError(f"{self.path}: malformed entry for {name!r}") from exc
            if dtype_name not in _DTYPES:
                raise SafetensorsError(f"{self.path}: {name!r} has unsupported dtype {dtype_name}")
            dtype, width = _DTYPES[dtype_name]
            count = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
            if end - begin != count * width or begin < 0 or data_start + end > size:
                raise SafetensorsError(
                    f"{self.path}: {name!r} claims bytes [{begin}, {end}) for shape {shape} "
                    f"{dtype_name}, which does not fit")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, self.path, data_start)

    def names(self) -> list[str]:
        return list(self.entries)


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """The tensor's values in its stored dtype, in host memory this call owns."""
    count = entry.end - entry.begin
    with open(entry.path, "rb") as handle:
        handle.seek(entry.data_start + entry.begin)
        raw = np.fromfile(handle, dtype=np.uint8, count=count)
    if raw.size != count:
        raise SafetensorsError(f"{entry.path}: {entry.name!r} is truncated")
    if count == 0:
        return torch.empty(entry.shape, dtype=entry.dtype)
    return torch.from_numpy(raw).view(entry.dtype).reshape(entry.shape)


class ModelFiles:
    """All tensors of a model folder: ``model.safetensors`` or an index over shards."""

    def __init__(self, model_dir: str | Path) -> None:
        self.model_dir = Path(model_dir)
        single = self.model_dir / "model.safetensors"
        index = self.model_dir / "model.safetensors.index.json"
        self.entries: dict[str, TensorEntry] = {}
        if single.is_file():
            self.entries.update(SafetensorsFile(single).entries)
        elif index.is_file():
            with open(index, "r", encoding="utf-8") as handle:
                weight_map = json.load(handle).get("weight_map", {})
            for shard in sorted(set(weight_map.values())):
                shard_file = SafetensorsFile(self.model_dir / shard)
                for name, entry in shard_file.entries.items():
                    if weight_map.get(name) == shard:
                        self.entries[name] = entry
        else:
            raise SafetensorsError(
                f"{self.model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name].shape

    def dtype(self, name: str) -> torch.dtype:
        return self.entries[name].dtype

    def read(self, name: str) -> torch.Tensor:
        return read_tensor(self.entries[name])


def write_safetensors(path: str | Path, tensors: Iterable[tuple[str, torch.Tensor]],
                      metadata: dict[str, str] | None = None) -> None:
    """Writes tensors in the order given. ``tensors`` may be a generator: each tensor is
    needed twice (once for the header, once for its bytes), so it is held until written."""
    items = [(name, t.detach().cpu().contiguous()) for name, t in tensors]
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, tensor in items:
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store {name!r} of dtype {tensor.dtype}")
        nbytes = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in items:
            if tensor.numel():
                handle.write(tensor.view(torch.uint8).numpy().tobytes()
                             if tensor.dim() else tensor.reshape(1).view(torch.uint8).numpy().tobytes())
