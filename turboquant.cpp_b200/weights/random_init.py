"""Random weights: a source of seeded tensors, and a writer of model folders.

``RandomSource`` produces the tensors of a plan from a seed: matrices and
biases N(0, std), norm weights 1 + N(0, std).  Every element is a pure
function of (seed, tensor name, index in the tensor): a 64-bit counter-based
hash gives 40 random bits, 16 of them choose one of 65,536 equally probable
intervals of the standard normal distribution and 24 a place inside it.  The
arithmetic is integer operations, one table lookup and one IEEE float32
multiplication and addition, so the same bits come out on the CPU and on a
GPU: a model drawn on the device (tens of gigabytes in a second) is the model
that ``write_random_model`` writes to a folder from the same configuration and
seed, and a test can compare an engine that never saw a file with an
implementation that only reads files.

``write_random_model`` writes config.json and model.safetensors for a
configuration, so that everything downstream — the loader, the engine, trace
replay — reads a random model exactly as it reads a real one.  The reference
has no such mode; its tests fill weights by hand with std::mt19937
(tests/test_ops.cpp:908-914).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from .loader import WeightSource, WeightSpec
from .safetensors_io import SafetensorsWriter

_MASK64 = (1 << 64) - 1
_INTERVALS = 1 << 16
_CHUNK = 1 << 24            # elements drawn at a time (bounds the int64 temporaries)


def _tensor_key(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little")


def _signed(v: int) -> int:
    """A 64-bit pattern as the int64 torch holds it."""
    v &= _MASK64
    return v - (1 << 64) if v >= (1 << 63) else v


_knots: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
_knots_on: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}


def normal_knots(device="cpu") -> Tuple[torch.Tensor, torch.Tensor]:
    """(left end, width) in float32 of each of the 65,536 intervals: the ends are the quantiles
    (j + 1/2) / 65,537 for j = 0 … 65,536 (all finite; the outermost are about -+4.3)."""
    global _knots
    if _knots is None:
        j = torch.arange(_INTERVALS // 2, dtype=torch.float64)
        half = torch.special.ndtri((j + 0.5) / (_INTERVALS + 1))               # float64, on the CPU
        k = torch.cat([half, torch.zeros(1, dtype=torch.float64), -half.flip(0)]).to(torch.float32)   # symmetric
        _knots = (k[:-1].contiguous(), (k[1:] - k[:-1]).contiguous())
    key = str(torch.device(device))
    if key not in _knots_on:
        _knots_on[key] = tuple(t.to(device) for t in _knots)
    return _knots_on[key]


def standard_normal(key: int, first: int, count: int, device) -> torch.Tensor:
    """Elements first … first+count-1 of the stream of a 64-bit key, float32 on `device`."""
    left, width = normal_knots(device)
    i = torch.arange(first, first + count, dtype=torch.int64, device=device)
    # splitmix64 of key + (index + 1) * golden ratio; int64 arithmetic wraps, shifts are made logical by masks
    z = i * _signed(0x9E3779B97F4A7C15) + _signed(key + 0x9E3779B97F4A7C15)
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _signed(0xBF58476D1CE4E5B9)
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _signed(0x94D049BB133111EB)
    z = z ^ ((z >> 31) & ((1 << 33) - 1))
    interval = (z >> 48) & 0xFFFF
    frac = ((z >> 24) & 0xFFFFFF).to(torch.float32) * (1.0 / (1 << 24))          # exact in float32
    step = frac * width[interval]                  # one rounding
    return left[interval] + step                   # one rounding (two operations: never contracted to an FMA)


class RandomSource(WeightSource):
    """Seeded tensors for a plan; the same values on every device."""

    def __init__(self, plan: Sequence[WeightSpec], seed: int, std: float = 0.02,
                 dtype: torch.dtype = torch.bfloat16, fp32_names: Sequence[str] = ()):
        self.plan = {s.name: s for s in plan}
        self.seed = int(seed)
        self.std = float(std)
        self.dtype = dtype
        self.fp32_names = set(fp32_names)

    def stored_dtype(self, spec: WeightSpec) -> torch.dtype:
        if spec.integer:
            return torch.int32
        return torch.float32 if spec.name in self.fp32_names else self.dtype

    def index(self):
        return {n: (self.stored_dtype(s), tuple(s.shape)) for n, s in self.plan.items()}

    def read(self, name, device):
        spec = self.plan[name]
        device = torch.device(device)
        shape = tuple(spec.shape)
        n = 1
        for d in shape:
            n *= int(d)
        if spec.init == "zeros":
            return torch.zeros(shape, dtype=self.stored_dtype(spec), device=device)
        if spec.init == "ones":
            return torch.ones(shape, dtype=self.stored_dtype(spec), device=device)
        if spec.init == "int_range":
            return torch.arange(n, dtype=torch.int32, device=device).reshape(shape)
        if spec.init not in ("normal", "one_plus_normal"):
            raise ValueError(f"tensor '{name}': unknown init '{spec.init}'")
        out = torch.empty(n, dtype=self.stored_dtype(spec), device=device)
        key = _tensor_key(self.seed, name)
        std = torch.tensor(self.std, dtype=torch.float32, device=device)
        for first in range(0, n, _CHUNK):
            count = min(_CHUNK, n - first)
            t = standard_normal(key, first, count, device) * std
            if spec.init == "one_plus_normal":
                t = t + 1.0
            out[first:first + count] = t           # rounds to the stored dtype
        return out.reshape(shape)


def write_random_model(folder: str, config_dict: Dict, plan: Sequence[WeightSpec], seed: int,
                       std: float = 0.02, dtype: torch.dtype = torch.bfloat16,
                       fp32_names: Sequence[str] = (), device="cpu") -> None:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``.  `device`: where the values are drawn
    before they are written (the same values everywhere; a GPU draws a large model much faster)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1, sort_keys=True)
    src = RandomSource(plan, seed, std, dtype, fp32_names)
    seen, ordered = set(), []
    for s in plan:                       # tied tensors appear once
        if s.name not in seen:
            seen.add(s.name)
            ordered.append(s)
    writer = SafetensorsWriter(os.path.join(folder, "model.safetensors"),
                               [(s.name, src.stored_dtype(s), s.shape) for s in ordered],
                               metadata={"format": "pt", "seed": str(seed)})
    for s in ordered:
        writer.write(s.name, src.read(s.name, device).cpu())
    writer.close()
