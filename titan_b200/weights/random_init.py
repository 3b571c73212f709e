"""Random weights from a configuration and a seed.

``write_model_folder`` writes ``config.json`` and ``model.safetensors``; the
folder then loads like any other.  ``RandomWeights`` makes the same tensors
directly on a device, for sizes that should not pass through a file.

Distributions: matrices and the embedding ~ N(0, 0.02); norm weights
1 + N(0, 0.1), so that a forgotten or doubled norm weight shows.

The generator is counter based: element ``i`` of a tensor is a pure function of
(seed, tensor name, i).  It is written twice, here in numpy and as a CUDA kernel
(csrc/random_fill.cu), out of integer arithmetic and single IEEE-754 double
operations only (no library logarithm or cosine, whose last bits differ between
libraries), so both give the same bits: a model made on the device with a seed
can be made again on the CPU, whole or any slice of any tensor, and a tensor's
values do not depend on which other tensors the model has.

berniehans/titan has no random-weights mode; its one generator is the
deterministic pattern of tools/build_synthetic_gguf.py:129-203.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import List

import numpy as np
import torch

from .loader import WeightSource, WeightSpec, held_dtype
from .safetensors_io import write_safetensors

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_LN2, _HALF_PI = 0.6931471805599453094, 1.5707963267948966192


def tensor_key(seed: int, name: str) -> int:
    """64 bits from (seed, tensor name)."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix64(z: np.ndarray) -> np.ndarray:
    """The finaliser of splitmix64 on uint64 arrays (products wrap modulo 2^64)."""
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _bits(key: int, start: int, count: int) -> np.ndarray:
    i = np.arange(start + 1, start + count + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _mix64(np.uint64(key) + i * _GOLDEN)


def standard_normal(key: int, start: int, count: int) -> np.ndarray:
    """Elements ``start .. start + count`` of the standard-normal stream of ``key`` (float64): Box-Muller on two
    24-bit uniforms, with the logarithm as (e - 24) ln 2 + 2 atanh((m - 1)/(m + 1)) in eleven terms and the
    cosine by quadrant and Taylor polynomial.  Operation for operation what csrc/random_fill.cu does."""
    z = _bits(key, start, count)
    n = ((z >> np.uint64(40)) + np.uint64(1)).astype(np.float64)          # 1 .. 2^24, exact
    k2 = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.int64)
    mant, exp = np.frexp(n)                                              # n = mant 2^exp, mant in [0.5, 1)
    m, e = mant * 2.0, exp - 1
    t = (m - 1.0) / (m + 1.0)
    t2 = t * t
    s = np.full(count, 1.0 / 21.0)
    for j in range(9, -1, -1):
        s = s * t2 + (1.0 / float(2 * j + 1))
    ln_u = (e - 24).astype(np.float64) * _LN2 + (2.0 * t) * s
    r = np.sqrt(-2.0 * ln_u)
    quadrant = k2 >> 22
    phi = ((k2 & 0x3FFFFF).astype(np.float64) * (1.0 / 4194304.0)) * _HALF_PI
    p2 = phi * phi
    c, sn = np.zeros(count), np.zeros(count)
    fc, fs = 6402373705728000.0, 121645100408832000.0                    # 18!, 19!
    for j in range(9, -1, -1):
        sign = -1.0 if j & 1 else 1.0
        c = c * p2 + sign / fc
        sn = sn * p2 + sign / fs
        if j > 0:
            fc, fs = fc / float((2 * j) * (2 * j - 1)), fs / float((2 * j + 1) * (2 * j))
    sn = sn * phi
    trig = np.where(quadrant == 0, c, np.where(quadrant == 1, -sn, np.where(quadrant == 2, -c, sn)))
    return r * trig


def values(key: int, start: int, count: int, std: float, mean: float) -> np.ndarray:
    """float32 values ``normal * std + mean`` of a slice of a tensor's stream."""
    return standard_normal(key, start, count).astype(np.float32) * np.float32(std) + np.float32(mean)


def _parameters(spec: WeightSpec):
    kind, std = spec.init
    if kind not in ("normal", "one_plus_normal"):
        raise ValueError(f"unknown init '{kind}' for {spec.name}")
    return float(std), (1.0 if kind == "one_plus_normal" else 0.0)


def make_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The tensor ``spec`` of the model with this seed, in ``dtype`` (values are made in float32 and rounded
    once); on a CUDA device by the fill kernel, else by numpy, with the same bits."""
    key = tensor_key(seed, spec.name)
    count = 1
    for d in spec.shape:
        count *= int(d)
    if torch.device(device).type == "cuda":
        from .. import kernels as K
        if spec.role == "int_table":
            out = torch.empty(spec.shape, dtype=torch.int32, device=device)
            K.fill_random(out, key, 0.0, 0.0)
            return out
        std, mean = _parameters(spec)
        out = torch.empty(spec.shape, dtype=dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32, device=device)
        K.fill_random(out, key, std, mean)
        return out.to(dtype)
    if spec.role == "int_table":
        return torch.from_numpy((_bits(key, 0, count) >> np.uint64(49)).astype(np.int32).reshape(spec.shape))
    std, mean = _parameters(spec)
    pieces = [values(key, at, min(1 << 22, count - at), std, mean) for at in range(0, count, 1 << 22)]
    return torch.from_numpy(np.concatenate(pieces).reshape(spec.shape)).to(dtype)


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
