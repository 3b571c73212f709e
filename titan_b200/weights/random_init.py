"""Random weights from a configuration and a seed.

``write_model_folder`` writes ``config.json`` and ``model.safetensors``; the
folder then loads like any other.  ``RandomWeights`` makes the same kind of
tensors directly on a device, for sizes that should not pass through a file.

Distributions: matrices and the embedding ~ N(0, 0.02); norm weights
1 + N(0, 0.1), so that a forgotten or doubled norm weight shows.  Each tensor
has its own generator, keyed by (seed, tensor name), so a tensor's values do
not depend on which other tensors the model has.

berniehans/titan has no random-weights mode; its one generator is the
deterministic pattern of tools/build_synthetic_gguf.py:129-203.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import List

import torch

from .loader import WeightSource, WeightSpec, held_dtype
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def make_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, spec.name))
    kind, std = spec.init
    if spec.role == "int_table":
        return torch.randint(0, 1 << 15, spec.shape, generator=g, device=device, dtype=torch.int32)
    t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * std
    if kind == "one_plus_normal":
        t = t + 1.0
    elif kind != "normal":
        raise ValueError(f"unknown init '{kind}' for {spec.name}")
    return t.to(dtype)


class RandomWeights(WeightSource):
    def __init__(self, seed: int, compute_dtype: torch.dtype, device, store_dtype: torch.dtype = None):
        self.seed, self.compute_dtype, self.device = seed, compute_dtype, device
        # values are rounded to store_dtype first, as a file of that dtype would hold them
        self.store_dtype = store_dtype or compute_dtype

    def get(self, spec: WeightSpec) -> torch.Tensor:
        t = make_tensor(spec, self.seed, self.store_dtype if spec.role != "int_table" else torch.int32, self.device)
        return t.to(held_dtype(spec.role, self.compute_dtype)).contiguous()


def write_model_folder(folder: str, config, seed: int, dtype: torch.dtype = torch.bfloat16) -> str:
    """``config``: a typed configuration with to_dict() and to_model_spec()."""
    from ..parts import declare_weights
    os.makedirs(folder, exist_ok=True)
    declared: List[WeightSpec] = declare_weights(config.to_model_spec())
    with open(os.path.join(folder, "config.json"), "w") as f:
        d = config.to_dict()
        d["torch_dtype"] = str(dtype).replace("torch.", "")
        json.dump(d, f, indent=1)
    by_name = {w.name: w for w in declared}
    listing = [(w.name, tuple(w.shape), torch.int32 if w.role == "int_table" else dtype) for w in declared]
    write_safetensors(os.path.join(folder, "model.safetensors"), listing,
                      lambda n: make_tensor(by_name[n], seed, torch.int32 if by_name[n].role == "int_table" else dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
