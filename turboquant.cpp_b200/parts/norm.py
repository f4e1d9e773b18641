"""RMSNorm: ss = sum(x^2)/n + eps; y = x * (1/sqrt(ss)) * w, the weight used as it is
(src/engine/tq_ops.c:1373-1410).  Reads the fp32 residual stream; statistics in fp32."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import elementwise as K
from ..weights.loader import WeightSpec, WeightStore
from .base import Norm, register_norm


class RMSNorm(Norm):
    def __init__(self, name: str, size: int, eps: float):
        if size < 1 or not eps > 0.0:
            raise ValueError(f"RMSNorm '{name}': size {size} and eps {eps} must be positive")
        self.name, self.size, self.eps = name, int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), init="one_plus_normal")]

    def bind(self, store: WeightStore) -> None:
        self.weight = store.get(self.name)

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def forward(self, x, out_dtype, rows=None, add=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype, device=x.device)
        return K.rmsnorm(x, self.weight, self.eps, out, add=add, rows=rows)

    def add_forward(self, x, y, out_dtype):
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        return K.rmsnorm(x, self.weight, self.eps, out, add=y)


register_norm("rmsnorm", RMSNorm)
