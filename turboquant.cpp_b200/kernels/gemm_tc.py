"""Grouped bf16 GEMM on tcgen05 tensor cores (csrc/gemm_tc.cu): the experts' products."""
from __future__ import annotations

from ctypes import c_int
from typing import Dict, Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream
from .moe import ExpertLayout

_LIB = "gemm_tc"
TOKEN_TILES = (16, 32, 64, 128)
_status: Dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that a kernel sets when one of its bounded waits ran out."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device=None) -> None:
    """Raises if a tensor-core kernel gave up on a wait since the last check (synchronises)."""
    for idx, t in _status.items():
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        if int(t.item()) != 0:
            t.zero_()
            raise KernelError("gemm_tc: a wait inside a tensor-core kernel ran out; its output is not valid")


def usable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """The tensor-core kernel takes bfloat16 operands whose rows are a multiple of 16 bytes."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def token_tile_for(rows: int, groups: int) -> int:
    """Token-tile width for `rows` rows spread over `groups` groups (mean rows per group decides)."""
    mean = rows / max(1, groups)
    for bn in TOKEN_TILES:
        if mean <= bn * 0.75:
            return bn
    return TOKEN_TILES[-1]


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, layout: Optional[ExpertLayout], swiglu: bool,
            token_tile: int) -> torch.Tensor:
    """x [R, K] bf16; w [G, Nw, K] bf16 (Nw = N, or 2N with swiglu: gate rows then up rows); out [R, N]
    bf16 or fp32.  layout: expert-sorted tiles of `token_tile` rows (None: one group)."""
    if not usable(x, w):
        raise KernelError("gemm_tc: needs bfloat16 operands with K a multiple of 8 and 16-byte aligned storage")
    R, K = x.shape
    N = out.shape[1]
    if w.dim() == 2:
        w = w.unsqueeze(0)
    G = w.shape[0]
    if w.shape[2] != K or w.shape[1] != (2 * N if swiglu else N):
        raise KernelError(f"gemm_tc: weight {tuple(w.shape)} does not fit x {tuple(x.shape)} -> out {tuple(out.shape)}")
    if layout is not None and layout.tile_rows != token_tile:
        raise KernelError(f"gemm_tc: the layout has tiles of {layout.tile_rows} rows, the kernel was asked for {token_tile}")
    if layout is None and G != 1:
        raise KernelError("gemm_tc: several groups need a layout")
    lib = load_kernel(_LIB)
    lo = layout
    check(_LIB, lib.tq_gemm_tc(
        ptr(x), ptr(w), ptr(out), c_int(code(out.dtype)),
        ptr(lo.tile_expert) if lo else None, ptr(lo.tile_row0) if lo else None, ptr(lo.tile_count) if lo else None,
        ptr(lo.n_tiles) if lo else None, c_int(lo.max_tiles if lo else 0), c_int(token_tile),
        c_int(R), c_int(N), c_int(K), c_int(G), c_int(1 if swiglu else 0), ptr(status_word(x.device)), stream()))
    return out
