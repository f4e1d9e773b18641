"""Weights by tensor name.

A model lists the tensors it needs as ``WeightSpec``s (name, shape, how to
initialise it at random).  ``check_plan`` compares that list with what a
source holds and raises ONE ``WeightError`` naming every missing tensor,
every unexpected tensor and every wrong shape.  ``WeightStore`` then hands
tensors to the parts on the device, in the dtype the run keeps them in:

* bfloat16 runs keep floating tensors in bfloat16, except that a tensor
  stored in 32-bit (or 64-bit) stays 32-bit; integer tables become int32;
* float32 runs widen every floating tensor to float32.

The reference looks tensors up by name with a linear scan and prefix
fallbacks (src/engine/tq_model.c:324-360), converts BF16/F16 to F32
(:367-412) and lets missing per-layer tensors become NULL, which skips the
layer at run time (src/engine/tq_transformer.c:2525-2552) — the silent
failure its own loader warns about (src/engine/tq_model.c:3818-3821).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, find_shards, DTYPES


class WeightError(ValueError):
    """Tensors of a source do not match the model's plan; lists all faults."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


@dataclass(frozen=True)
class WeightSpec:
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"        # 'normal' | 'one_plus_normal' | 'zeros' | 'ones' | 'int_range'
    integer: bool = False        # an integer table (kept as int32)


def run_dtype_of(name: str) -> torch.dtype:
    table = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
    if name not in table:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{name}'")
    return table[name]


def kept_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    """The dtype a tensor is kept in on the device (see the module's header)."""
    if not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class WeightSource:
    """Something that holds named tensors: a model folder or a random generator."""

    def index(self) -> Dict[str, Tuple[torch.dtype, Tuple[int, ...]]]:
        raise NotImplementedError

    def read(self, name: str, device: torch.device) -> torch.Tensor:
        """The tensor as stored, on ``device``."""
        raise NotImplementedError

    def close(self) -> None:
        pass


class SafetensorsSource(WeightSource):
    def __init__(self, folder: str):
        self.folder = folder
        self.files = [SafetensorsFile(p) for p in find_shards(folder)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.entries:
                if name in self._where:
                    raise WeightError(f"tensor '{name}' appears in two shards of '{folder}'")
                self._where[name] = f

    def index(self):
        return {n: (DTYPES[f.entries[n][0]][0], f.entries[n][1]) for n, f in self._where.items()}

    def read(self, name, device):
        return self._where[name].read(name).to(device)

    def close(self):
        for f in self.files:
            f.close()


def check_plan(index: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]], plan: Sequence[WeightSpec],
               where: str = "weights") -> None:
    """Raises one WeightError that lists everything wrong, or returns."""
    wanted = {}
    for s in plan:
        if s.name in wanted and wanted[s.name].shape != tuple(s.shape):
            raise ValueError(f"plan lists tensor '{s.name}' twice with different shapes")
        wanted[s.name] = s
    missing = sorted(n for n in wanted if n not in index)
    unexpected = sorted(n for n in index if n not in wanted)
    wrong_shape, wrong_dtype = [], []
    for n, s in wanted.items():
        if n in index:
            dtype, shape = index[n]
            if tuple(shape) != tuple(s.shape):
                wrong_shape.append((n, tuple(s.shape), tuple(shape)))
            if s.integer == dtype.is_floating_point or dtype == torch.bool:
                wrong_dtype.append((n, "integer" if s.integer else "floating", str(dtype)))
    if not (missing or unexpected or wrong_shape or wrong_dtype):
        return
    lines = [f"{where}: tensors do not match the model "
             f"({len(missing)} missing, {len(unexpected)} unexpected, {len(wrong_shape)} wrong shape, "
             f"{len(wrong_dtype)} wrong dtype)"]

    def some(items, fmt, limit=20):
        out = [fmt(i) for i in items[:limit]]
        if len(items) > limit:
            out.append(f"    … and {len(items) - limit} more")
        return out

    if missing:
        lines.append("  missing:")
        lines += some(missing, lambda n: f"    {n} {list(wanted[n].shape)}")
    if unexpected:
        lines.append("  unexpected:")
        lines += some(unexpected, lambda n: f"    {n} {list(index[n][1])}")
    if wrong_shape:
        lines.append("  wrong shape:")
        lines += some(wrong_shape, lambda t: f"    {t[0]}: expected {list(t[1])}, found {list(t[2])}")
    if wrong_dtype:
        lines.append("  wrong dtype:")
        lines += some(wrong_dtype, lambda t: f"    {t[0]}: expected {t[1]}, found {t[2]}")
    raise WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_dtype)


class WeightStore:
    """Hands a checked plan's tensors to the parts, on the device, in the kept dtype."""

    def __init__(self, source: WeightSource, plan: Sequence[WeightSpec], device, run_dtype: torch.dtype,
                 where: str = "weights"):
        self.source = source
        self.device = torch.device(device)
        self.run_dtype = run_dtype
        self._index = source.index()
        check_plan(self._index, plan, where)
        self._plan = {s.name: s for s in plan}
        self._cache: Dict[str, torch.Tensor] = {}

    def get(self, name: str) -> torch.Tensor:
        """Each call returns the same tensor for a name, so tied weights share storage."""
        if name in self._cache:
            return self._cache[name]
        if name not in self._plan:
            raise KeyError(f"tensor '{name}' is not in the model's plan")
        t = self.source.read(name, self.device)
        t = t.to(kept_dtype(t.dtype, self.run_dtype)).contiguous()
        self._cache[name] = t
        return t

    def kept_dtype_of(self, name: str) -> torch.dtype:
        """The dtype get(name) will return, without reading the tensor."""
        return kept_dtype(self._index[name][0], self.run_dtype)

    def take(self, name: str) -> torch.Tensor:
        """Like get, but forgets the tensor: for parts that copy it into a stacked buffer."""
        t = self.get(name)
        del self._cache[name]
        return t

    def release(self) -> None:
        self._cache.clear()
