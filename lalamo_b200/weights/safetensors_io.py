"""Reading and writing safetensors files.

The format (``lalamo/safetensors.py:69-106``): an 8-byte little-endian header length, a JSON
header mapping tensor names to ``{"dtype", "shape", "data_offsets"}`` (offsets relative to the
end of the header), then the raw little-endian data.  Tensors are read lazily from a
copy-on-write memory map, one by one, when asked for.
"""

from __future__ import annotations

import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterator, Mapping

import numpy as np
import torch

__all__ = ["SafetensorsFile", "TensorInfo", "open_checkpoint", "write_safetensors"]

_TORCH_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {dtype: name for name, dtype in _TORCH_DTYPES.items()}


class SafetensorsFormatError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: tuple[int, ...]
    start: int
    end: int


class SafetensorsFile:
    """One ``.safetensors`` file, opened lazily."""

    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        size = self.path.stat().st_size
        with open(self.path, "rb") as stream:
            prefix = stream.read(8)
            if len(prefix) != 8:
                raise SafetensorsFormatError(f"{self.path}: shorter than its 8-byte header length")
            (header_size,) = struct.unpack("<Q", prefix)
            if header_size > size - 8:
                raise SafetensorsFormatError(f"{self.path}: header length {header_size} exceeds the file size")
            try:
                header = json.loads(stream.read(header_size))
            except (UnicodeDecodeError, json.JSONDecodeError) as error:
                raise SafetensorsFormatError(f"{self.path}: header is not JSON ({error})") from error
        self.metadata: dict[str, str] = header.pop("__metadata__", None) or {}
        self._data_start = 8 + header_size
        self._infos: dict[str, TensorInfo] = {}
        for name, entry in header.items():
            dtype = entry["dtype"]
            if dtype not in _TORCH_DTYPES:
                raise SafetensorsFormatError(f"{self.path}: tensor {name!r} has unsupported dtype {dtype}")
            start, end = entry["data_offsets"]
            shape = tuple(int(extent) for extent in entry["shape"])
            expected = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=_TORCH_DTYPES[dtype]).element_size()
            if end - start != expected or self._data_start + end > size:
                raise SafetensorsFormatError(f"{self.path}: tensor {name!r} has inconsistent offsets")
            self._infos[name] = TensorInfo(dtype, shape, start, end)
        self._map: np.memmap | None = None

    def names(self) -> list[str]:
        return list(self._infos)

    def info(self, name: str) -> TensorInfo:
        return self._infos[name]

    def read(self, name: str) -> torch.Tensor:
        info = self._infos[name]
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="c")
        raw = self._map[self._data_start + info.start : self._data_start + info.end]
        dtype = _TORCH_DTYPES[info.dtype]
        if raw.size == 0:
            return torch.empty(info.shape, dtype=dtype)
        return torch.from_numpy(raw).view(dtype).reshape(info.shape)


class Checkpoint(Mapping[str, TensorInfo]):
    """All the ``*.safetensors`` files of a model folder, seen as one name space
    (the reference chains its shards the same way, ``lalamo/model_import/common.py:194-213``)."""

    def __init__(self, files: list[SafetensorsFile]) -> None:
        self._owner: dict[str, SafetensorsFile] = {}
        for file in files:
            for name in file.names():
                self._owner[name] = file

    def __getitem__(self, name: str) -> TensorInfo:
        return self._owner[name].info(name)

    def __iter__(self) -> Iterator[str]:
        return iter(self._owner)

    def __len__(self) -> int:
        return len(self._owner)

    def read(self, name: str) -> torch.Tensor:
        return self._owner[name].read(name)


def open_checkpoint(model_dir: str | Path) -> Checkpoint:
    paths = sorted(Path(model_dir).glob("*.safetensors"))
    if not paths:
        raise FileNotFoundError(f"{model_dir} holds no .safetensors file")
    return Checkpoint([SafetensorsFile(path) for path in paths])


def write_safetensors(path: str | Path, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _NAMES:
            raise ValueError(f"cannot store dtype {tensor.dtype} of tensor {name!r}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + size]}
        offset += size
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-len(encoded) % 8)
    with open(path, "wb") as stream:
        stream.write(struct.pack("<Q", len(encoded)))
        stream.write(encoded)
        for name in order:
            tensor = tensors[name].detach().cpu().contiguous()
            stream.write(tensor.reshape(-1).view(torch.uint8).numpy().tobytes())
