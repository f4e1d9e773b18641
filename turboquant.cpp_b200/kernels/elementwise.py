"""Row-wise kernels (csrc/elementwise.cu): embedding rows, RMSNorm, SiLU*up, row gather."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import check, code, ptr, stream, want_f32, want_int32

_LIB = "elementwise"


def embed_rows(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32.  tokens int32 [T]; table [V, H]; out float32 [T, H]."""
    want_int32(tokens, "tokens")
    want_f32(out, "the residual stream")
    T, H = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_embed_rows(ptr(tokens), ptr(table), c_int(code(table.dtype)), ptr(out),
                                  c_int(T), c_int(H), c_int(table.shape[0]), stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            add: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of rows of the float32 residual stream x [T, H] into out [R, H].

    add:  the norm is taken of x + add (summed in float32).
    rows: out[r] = norm of row rows[r] and x is left alone; without rows, R = T and the sum
          x + add is written back into x."""
    want_f32(x, "the residual stream")
    R, H = out.shape
    if rows is not None:
        want_int32(rows, "rows")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_rmsnorm(ptr(x), ptr(add), c_int(code(add.dtype) if add is not None else 0), ptr(rows),
                               ptr(weight), c_int(code(weight.dtype)), ptr(out), c_int(code(out.dtype)),
                               c_int(R), c_int(H), c_float(eps), stream()))
    return out


def residual_add(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x += y with x float32."""
    want_f32(x, "the residual stream")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_residual_add(ptr(x), ptr(y), c_int(code(y.dtype)), c_longlong(x.numel()), stream()))
    return x


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[t, :] += bias, in place, summed in float32.  x [T, N]; bias [N] (any of the two dtypes)."""
    T, N = x.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_add_bias(ptr(x), c_int(code(x.dtype)), ptr(bias), c_int(code(bias.dtype)), c_int(T), c_int(N),
                                stream()))
    return x


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    T, I = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_silu_mul(ptr(gate_up), c_int(code(gate_up.dtype)), ptr(out), c_int(code(out.dtype)),
                                c_int(T), c_int(I), stream()))
    return out


def gather_rows(src: torch.Tensor, index: torch.Tensor, divisor: int, out: torch.Tensor) -> torch.Tensor:
    """out[r] = src[index[r] // divisor]."""
    want_int32(index, "index")
    R, H = out.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gather_rows(ptr(src), ptr(index), c_int(divisor), ptr(out), c_int(code(out.dtype)),
                                   c_int(R), c_int(H), c_int(src.shape[0]), stream()))
    return out
