"""Reading and writing the safetensors container, by tensor name.

The format: an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (plus an optional
``__metadata__`` entry), then one byte buffer that the offsets index.

berniehans/titan reads GGUF instead (engine/engine-io/src/reader.rs,
loader.rs:104-193): header, tensor infos, then one blob that ``tensor(name)``
slices.  The guards are the same in kind: bad header length, offsets outside
the file, sizes that do not match the shape (engine-io/src/error.rs:6-66).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


# storage dtype -> (torch dtype, bytes per element)
_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 << 20


class SafetensorsFile:
    """A memory-mapped safetensors file; ``tensor(name)`` returns a CPU tensor
    that aliases the mapping (copy it or move it to a device before closing)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors header")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > _MAX_HEADER or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file of {size} bytes")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: the header is not a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self._base = 8 + n
        self._data_len = size - self._base
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            try:
                dtype, shape, (b, end) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for '{name}'") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has the unsupported dtype {dtype}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype][1] if shape else _DTYPES[dtype][1]
            if not (0 <= b <= end <= self._data_len) or end - b != want:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' ({dtype} {list(shape)}) claims bytes [{b}, {end}) of a "
                    f"{self._data_len}-byte buffer; its shape needs {want} bytes")
            self.entries[name] = (dtype, shape, int(b), int(end))
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, b, end = self.entries[name]
        tdtype, _ = _DTYPES[dtype]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=end - b, offset=self._base + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")        # the mapping is read-only; nobody writes to these tensors
            return torch.from_numpy(buf).view(tdtype).reshape(shape)

    def close(self) -> None:
        # tensors handed out alias the mapping; it is released with the last of them
        self._f.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """``model.safetensors``, or the shards that ``model.safetensors.index.json`` names."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    if os.path.isfile(index):
        with open(index) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(model_dir, s)) for s in shards]
    raise SafetensorsError(f"no model.safetensors (or index) in {model_dir}")


def write_safetensors(path: str, tensors: Iterable[Tuple[str, Tuple[int, ...], torch.dtype]],
                      produce, metadata: Dict[str, str] = None) -> None:
    """Write a file whose header is known up front and whose tensors are made one
    at a time: ``tensors`` lists (name, shape, dtype) in file order and
    ``produce(name)`` returns that tensor.  Nothing larger than one tensor is held."""
    tensors = list(tensors)
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    for name, shape, dtype in tensors:
        n = int(np.prod(shape, dtype=np.int64)) * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype in tensors:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"tensor '{name}' was announced as {dtype} {shape}, produced {t.dtype} {tuple(t.shape)}")
            t = t.detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
