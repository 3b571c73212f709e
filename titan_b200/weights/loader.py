"""Binding tensors of a model folder to the parts that own them, by name.

Every part declares the tensors it owns as ``WeightSpec``s.  The loader checks
the whole folder against the whole declaration first and raises ONE
``WeightError`` that lists every missing tensor, every unexpected tensor and
every wrong shape; only then does it hand tensors out.

Precision policy.  A ``matrix`` (anything that enters a matrix product, the
embedding table included) is kept in the engine's compute dtype: bfloat16 for
serving, float32 for the true 32-bit path (a bfloat16 file upcasts exactly).
A ``vector`` (norm weights and the like) is held in float32 whatever the file
stores, which is exact for bfloat16 files and keeps 32-bit tensors 32-bit.
An ``int_table`` is held as int32.

berniehans/titan binds GGUF tensors by name one at a time and fails on the
first problem (engine/engine-core/src/forward_driver.rs:315-358, 620-647).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files


class WeightError(ValueError):
    """The folder's tensors do not match what the model declares."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        self.wrong_dtype = sorted(wrong_dtype)
        lines = ["the weights do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, the model needs {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is stored as {got}")
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class WeightSpec:
    name: str                         # full tensor name in the file
    shape: Tuple[int, ...]
    role: str = "matrix"              # "matrix" | "vector" | "int_table"
    init: Tuple[str, float] = ("normal", 0.02)   # ("normal", std) | ("one_plus_normal", std)


def check_names(declared: Iterable[WeightSpec], found: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
                ignorable: Iterable[str] = ()) -> None:
    """Raise one WeightError for everything that is wrong, or return."""
    declared = list(declared)
    want = {w.name: w for w in declared}
    ignorable = set(ignorable)
    missing = [n for n in want if n not in found]
    unexpected = [n for n in found if n not in want and n not in ignorable]
    wrong_shape, wrong_dtype = [], []
    for n, w in want.items():
        if n in found:
            shape, dtype = found[n]
            if tuple(shape) != tuple(w.shape):
                wrong_shape.append((n, tuple(shape), tuple(w.shape)))
            floating = dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64)
            if (w.role == "int_table") == floating:
                wrong_dtype.append((n, str(dtype).replace("torch.", "")))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)


def held_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "vector":
        return torch.float32
    if role == "int_table":
        return torch.int32
    return compute_dtype


class WeightSource:
    """Where a model's tensors come from: ``get(spec) -> tensor`` on the device,
    in the dtype the policy above gives."""

    def get(self, spec: WeightSpec) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError


class FolderWeights(WeightSource):
    def __init__(self, model_dir: str, declared: Iterable[WeightSpec], compute_dtype: torch.dtype,
                 device, ignorable: Iterable[str] = ()):
        self.files: List[SafetensorsFile] = open_model_files(model_dir)
        self.where: Dict[str, SafetensorsFile] = {}
        found = {}
        for f in self.files:
            for n in f.names():
                self.where[n] = f
                found[n] = (f.shape(n), f.dtype(n))
        check_names(declared, found, ignorable)
        self.compute_dtype, self.device = compute_dtype, device

    def get(self, spec: WeightSpec) -> torch.Tensor:
        t = self.where[spec.name].tensor(spec.name)
        return t.to(device=self.device, dtype=held_dtype(spec.role, self.compute_dtype)).contiguous()


class DictWeights(WeightSource):
    """Tensors already in memory (tests, and random weights made on the device)."""

    def __init__(self, tensors: Dict[str, torch.Tensor], declared: Iterable[WeightSpec],
                 compute_dtype: torch.dtype, device, ignorable: Iterable[str] = ()):
        check_names(declared, {n: (tuple(t.shape), t.dtype) for n, t in tensors.items()}, ignorable)
        self.tensors, self.compute_dtype, self.device = tensors, compute_dtype, device

    def get(self, spec: WeightSpec) -> torch.Tensor:
        t = self.tensors[spec.name]
        return t.to(device=self.device, dtype=held_dtype(spec.role, self.compute_dtype)).contiguous()
