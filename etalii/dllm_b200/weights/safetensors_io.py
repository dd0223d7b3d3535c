"""A small safetensors reader and writer: an 8-byte little-endian header length, a JSON header of
name -> {dtype, shape, data_offsets}, then the tensors' bytes.

Checks follow the reference's reader (src/etalii_dllm/importing/safetensors.py:71-146): header within the file,
offsets inside the data section and matching shape times item size, no overlap. Sharded checkpoints
(`model.safetensors.index.json`) and plain `*.safetensors` folders are found as there (safetensors.py:149-170).
Tensors come back as torch CPU tensors in their stored dtype; nothing is converted here.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Iterable, Mapping

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "F64": (torch.float64, 8),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str) -> None:
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors file")
        self._handle = open(path, "rb")
        (header_size,) = struct.unpack("<Q", self._handle.read(8))
        if header_size > size - 8:
            raise SafetensorsError(f"{path}: the header runs past the end of the file")
        try:
            header = json.loads(self._handle.read(header_size).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as error:
            raise SafetensorsError(f"{path}: the header is not JSON ({error})") from error
        header.pop("__metadata__", None)
        self._data_start = 8 + header_size
        data_size = size - self._data_start
        self.entries: dict[str, tuple[str, tuple[int, ...], int, int]] = {}
        spans = []
        for name, entry in header.items():
            dtype, shape = entry.get("dtype"), tuple(int(d) for d in entry.get("shape", ()))
            begin, end = (int(v) for v in entry.get("data_offsets", (0, -1)))
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            count = 1
            for d in shape:
                count *= d
            if not (0 <= begin <= end <= data_size) or end - begin != count * _DTYPES[dtype][1]:
                raise SafetensorsError(f"{path}: tensor {name!r} has bad offsets {begin}..{end} for shape {shape}")
            self.entries[name] = (dtype, shape, begin, end)
            if end > begin:
                spans.append((begin, end, name))
        spans.sort()
        for (_, end, a), (begin, _, b) in zip(spans, spans[1:]):
            if begin < end:
                raise SafetensorsError(f"{path}: tensors {a!r} and {b!r} overlap")
        self._map = mmap.mmap(self._handle.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A copy of the tensor in its stored dtype (the file can be closed afterwards)."""
        dtype, shape, begin, end = self.entries[name]
        torch_dtype, _ = _DTYPES[dtype]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin, offset=self._data_start + begin)
        return torch.from_numpy(raw.copy()).view(torch_dtype).reshape(shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._handle.close()


def checkpoint_files(folder: str) -> list[str]:
    """The safetensors files of a model folder: those of the shard index, else model.safetensors, else every
    *.safetensors."""
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, encoding="utf-8") as handle:
            files = sorted(set(json.load(handle).get("weight_map", {}).values()))
        return [os.path.join(folder, f) for f in files]
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise SafetensorsError(f"{folder}: no safetensors file")  # safetensors.py:161-162
    return files


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]]) -> None:
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: dict[str, dict] = {}
    offset = 0
    for name, tensor in items:
        if tensor.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r} has unsupported dtype {tensor.dtype}")
        size = tensor.numel() * tensor.element_size()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape),
                        "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in items:
            flat = tensor.detach().contiguous().cpu().reshape(-1)
            handle.write(flat.view(torch.uint8).numpy().tobytes())
