"""Dense matrix products y = x W^T.

The reference's dense projections go through one routine that calls the platform's BLAS where
there is one (src/engine/tq_ops.c:296-343, Accelerate at :297-306); here they go through cuBLAS
(torch.mm).  The float32 path never uses a reduced-precision matrix mode: TF32 is switched off
for the call and the process's setting restored after it.  Expert products do not come through here (kernels/moe.py).
"""
from __future__ import annotations

from typing import Optional

import torch

from ._call import KernelError


class _FullPrecision:
    """No TF32 and no reduced-precision bfloat16 reductions for the products inside; the process's own settings
    come back afterwards (a host program's choice for its other work is not this library's to change)."""

    def __enter__(self):
        m = torch.backends.cuda.matmul
        self.saved = (m.allow_tf32, m.allow_bf16_reduced_precision_reduction)
        if self.saved[0]:
            m.allow_tf32 = False
        if self.saved[1]:
            m.allow_bf16_reduced_precision_reduction = False

    def __exit__(self, *exc):
        m = torch.backends.cuda.matmul
        if m.allow_tf32 != self.saved[0]:
            m.allow_tf32 = self.saved[0]
        if m.allow_bf16_reduced_precision_reduction != self.saved[1]:
            m.allow_bf16_reduced_precision_reduction = self.saved[1]


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [T, K] times weight [N, K] transposed -> [T, N].  A float32 weight makes the product a
    true float32 one whatever x is; a bfloat16 weight takes bfloat16 x and accumulates in float32."""
    if not x.is_cuda:
        raise KernelError("linear: CUDA tensors only; there is no CPU path")
    with _FullPrecision():
        if weight.dtype == torch.float32:
            y = torch.mm(x if x.dtype == torch.float32 else x.float(), weight.t())
        elif weight.dtype == torch.bfloat16:
            xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
            if out_dtype == torch.float32:
                return torch.mm(xb, weight.t(), out_dtype=torch.float32)
            y = torch.mm(xb, weight.t())
        else:
            raise KernelError(f"linear: weight dtype {weight.dtype} not supported")
    if out_dtype is not None and y.dtype != out_dtype:
        y = y.to(out_dtype)
    return y
