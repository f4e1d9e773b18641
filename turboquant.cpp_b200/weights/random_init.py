"""Random weights: a source of seeded tensors, and a writer of model folders.

``RandomSource`` produces the tensors of a plan from a seed: matrices and
biases N(0, std), norm weights 1 + N(0, std).  Each tensor's values depend on
(seed, tensor name) only.  ``write_random_model`` writes config.json and
model.safetensors for a configuration, so that everything downstream — the
loader, the engine, trace replay — reads a random model exactly as it reads a
real one.  The reference has no such mode; its tests fill weights by hand
with std::mt19937 (tests/test_ops.cpp:908-914).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from .loader import WeightSource, WeightSpec
from .safetensors_io import SafetensorsWriter


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 62) - 1)


class RandomSource(WeightSource):
    """Seeded tensors for a plan.  On a CUDA device the values are drawn on the
    device (a model of tens of gigabytes cannot come through the host in
    reasonable time); values drawn on the CPU and on a GPU differ."""

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
        gen = torch.Generator(device=device)
        gen.manual_seed(_tensor_seed(self.seed, name))
        shape = tuple(spec.shape)
        if spec.init == "zeros":
            t = torch.zeros(shape, dtype=torch.float32, device=device)
        elif spec.init == "ones":
            t = torch.ones(shape, dtype=torch.float32, device=device)
        elif spec.init == "int_range":
            return torch.arange(int(torch.tensor(shape).prod()) if shape else 1, dtype=torch.int32,
                                device=device).reshape(shape)
        elif spec.init in ("normal", "one_plus_normal"):
            t = torch.empty(shape, dtype=torch.float32, device=device)
            t.normal_(0.0, self.std, generator=gen)
            if spec.init == "one_plus_normal":
                t += 1.0
        else:
            raise ValueError(f"tensor '{name}': unknown init '{spec.init}'")
        return t.to(self.stored_dtype(spec))


def write_random_model(folder: str, config_dict: Dict, plan: Sequence[WeightSpec], seed: int,
                       std: float = 0.02, dtype: torch.dtype = torch.bfloat16,
                       fp32_names: Sequence[str] = ()) -> None:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``."""
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
        writer.write(s.name, src.read(s.name, "cpu"))
    writer.close()
