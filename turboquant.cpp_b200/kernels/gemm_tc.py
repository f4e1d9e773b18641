"""Grouped bf16 GEMM on tcgen05 tensor cores (csrc/gemm_tc.cu): the experts' products."""
from __future__ import annotations

import os
from ctypes import c_int
from typing import Dict, Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream
from .moe import ExpertLayout

_LIB = "gemm_tc"
TOKEN_TILES = (16, 32, 64, 128, 256)
_status: Dict[int, torch.Tensor] = {}


GAVE_UP = "a wait inside a tensor-core kernel ran out; its output is not valid"


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 that a tensor-core kernel sets when one of its bounded waits ran out, for launches that name
    no word of their own (one per device).  An engine passes its own word, so that a fault is seen by the
    engine whose step it spoiled."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device=None, word: Optional[torch.Tensor] = None) -> None:
    """Raises if a tensor-core kernel gave up on a wait since the last check (synchronises).  `word`: a status
    word of the caller's; without it, the per-device words."""
    words = [word] if word is not None else [t for idx, t in _status.items()
                                             if device is None or torch.device(device).index in (None, idx)]
    for t in words:
        if int(t.item()) != 0:
            t.zero_()
            raise KernelError("gemm_tc: " + GAVE_UP)


BLOCK_ROWS, BLOCK_K = 128, 64


class PackedWeights:
    """Weights [G, Nw, K] re-laid for the tensor-core kernel: [G * tiles, ceil(K/64), 128, 64] bf16, every
    [128 x 64] block contiguous and zero-padded.  Plain: a block holds 128 rows.  With swiglu a block holds
    the gate rows and the up rows of 64 output columns, interleaved in runs of 16: block row 32q+i is the gate
    and 32q+16+i the up of column 64*tile + 16q + i (q < 4, i < 16)."""

    def __init__(self, data: torch.Tensor, groups: int, n: int, k: int, swiglu: bool):
        self.data, self.groups, self.n, self.k, self.swiglu = data, groups, n, k, swiglu

    @property
    def dtype(self):
        return self.data.dtype

    def nbytes(self) -> int:
        return self.data.numel() * self.data.element_size()


def packable(w: torch.Tensor) -> bool:
    """bfloat16 weights whose K gives the activations 16-byte rows."""
    return w.dtype == torch.bfloat16 and w.shape[-1] % 8 == 0


def pack_weights(w: torch.Tensor, swiglu: bool) -> PackedWeights:
    """w [G, Nw, K] (or [Nw, K]) bf16 with Nw = N, or 2N with swiglu (gate rows, then up rows)."""
    if w.dim() == 2:
        w = w.unsqueeze(0)
    if not packable(w):
        raise KernelError("gemm_tc: weights must be bfloat16 with K a multiple of 8")
    G, Nw, K = w.shape
    N = Nw // 2 if swiglu else Nw
    cols = BLOCK_ROWS // 2 if swiglu else BLOCK_ROWS            # output columns of a block
    n_t, n_k = -(-N // cols), -(-K // BLOCK_K)
    rows = torch.zeros((G, n_t, BLOCK_ROWS, n_k * BLOCK_K), dtype=w.dtype, device=w.device)
    if swiglu:
        both = torch.zeros((G, 2, n_t * cols, K), dtype=w.dtype, device=w.device)
        both[:, 0, :N] = w[:, :N]
        both[:, 1, :N] = w[:, N:]
        # [G, half, tile, q, i, K] -> [G, tile, q, half, i, K]
        rows.view(G, n_t, 4, 2, 16, n_k * BLOCK_K)[..., :K] = both.view(G, 2, n_t, 4, 16, K).permute(0, 2, 3, 1, 4, 5)
        del both
    else:
        rows.view(G, n_t * BLOCK_ROWS, n_k * BLOCK_K)[:, :N, :K] = w
    out = rows.view(G, n_t, BLOCK_ROWS, n_k, BLOCK_K).permute(0, 1, 3, 2, 4).contiguous()
    del rows
    return PackedWeights(out.view(G * n_t, n_k, BLOCK_ROWS, BLOCK_K), G, N, K, swiglu)


def usable(x: torch.Tensor, w) -> bool:
    """The tensor-core kernel takes bfloat16 activations with 16-byte rows and packed weights."""
    return (isinstance(w, PackedWeights) and x.dtype == torch.bfloat16 and x.shape[-1] == w.k
            and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0)


def token_tile_for(rows: int, groups: int) -> int:
    """Token-tile width for `rows` rows spread over `groups` groups (mean rows per group decides)."""
    mean = rows / max(1, groups)
    for bn in TOKEN_TILES:
        if mean <= bn * 0.75:
            return bn
    return TOKEN_TILES[-1]


def k_splits_for(rows: int, n: int, k: int, token_tile: int, resident: int = 296) -> int:
    """Into how many shares the K of a plain one-group product is cut: a product of few tokens whose output is
    narrow has few tiles (rows of 128 output columns), so without this a handful of SMs would stream all its
    weights; with it about `resident` units of work do.  1 where the tiles fill the GPU anyway, where K is short,
    or where the partial sums (rows x n floats per share) would weigh against the weights they save time on."""
    tiles = -(-n // BLOCK_ROWS) * -(-rows // max(1, token_tile))
    num_kb = -(-k // BLOCK_K)
    if tiles * 2 > resident or num_kb < 16 or token_tile > 64:       # the kernel shares K out for narrow token tiles only
        return 1
    want = min(resident // tiles, num_kb // 8, 32)
    while want > 1 and want * rows * n * 4 * 2 > n * k * 2 // 2:        # partial sums written and read vs. weight bytes
        want -= 1
    if want <= 1:
        return 1
    per = -(-num_kb // want)
    return -(-num_kb // per)


PAIR_MIN_TILE = 128      # token tiles from this width on run on pairs of CTAs (cta_group::2)
_NO_PAIRS = os.environ.get("TQ_NO_PAIRS", "") not in ("", "0")


def gemm_tc(x: torch.Tensor, w: PackedWeights, out: torch.Tensor, layout: Optional[ExpertLayout],
            token_tile: int, pair: Optional[bool] = None, status: Optional[torch.Tensor] = None,
            sm_share: int = 0, k_splits: int = 1, early_weights: bool = False) -> torch.Tensor:
    """x [R, K] bf16; w: packed weights of G groups; out [R, N] bf16 or fp32 (with w.swiglu:
    silu(x.Wg) * (x.Wu)).  layout: expert-sorted tiles of `token_tile` rows (None: one group).
    pair: run on pairs of CTAs (default: for wide token tiles, unless TQ_NO_PAIRS=1).  status: the int32 the
    kernel sets if a bounded wait runs out (default: the device's word).  sm_share: 1..99 = the launch takes only
    that percentage of the CTAs the GPU runs at once and leaves the rest to a launch on another stream.
    k_splits > 1: out is [k_splits, R, N] float32; slice s holds the partial sums over the s-th share of K (see
    k_splits_for) and the caller adds the slices up in order.  early_weights: the caller vouches that the weights
    and the layout were final before the kernel ahead of this one in the stream started (a down projection behind
    its gate/up product); the kernel then starts streaming weights while that kernel still runs."""
    if pair is None:
        pair = token_tile >= PAIR_MIN_TILE and not _NO_PAIRS
    if not usable(x, w):
        raise KernelError("gemm_tc: needs bfloat16 activations with K a multiple of 8 and weights packed for this K")
    R, K = x.shape
    N = out.shape[-1]
    if k_splits > 1 and (out.dim() != 3 or out.shape[0] != k_splits or out.shape[1] != R or out.dtype != torch.float32 or w.swiglu):
        raise KernelError("gemm_tc: with K shared out, out must be [k_splits, R, N] float32 and the product plain")
    if N != w.n:
        raise KernelError(f"gemm_tc: weights give {w.n} columns, out has {N}")
    if layout is not None and layout.tile_rows != token_tile:
        raise KernelError(f"gemm_tc: the layout has tiles of {layout.tile_rows} rows, the kernel was asked for {token_tile}")
    if layout is None and w.groups != 1:
        raise KernelError("gemm_tc: several groups need a layout")
    lib = load_kernel(_LIB)
    lo = layout
    check(_LIB, lib.tq_gemm_tc(
        ptr(x), ptr(w.data), ptr(out), c_int(code(out.dtype)),
        ptr(lo.tile_expert) if lo else None, ptr(lo.tile_row0) if lo else None, ptr(lo.tile_count) if lo else None,
        ptr(lo.n_tiles) if lo else None, c_int(lo.max_tiles if lo else 0), c_int(token_tile),
        c_int(R), c_int(N), c_int(K), c_int(w.groups), c_int(1 if w.swiglu else 0), c_int(1 if pair else 0),
        ptr(status if status is not None else status_word(x.device)), c_int(int(sm_share)), c_int(int(k_splits)),
        c_int(1 if early_weights else 0), stream()))
    return out


DUAL_CALLS = 0       # launches of two products so far (tests read it)


def gemm_tc_dual(x: torch.Tensor, w: PackedWeights, out: torch.Tensor, layout: ExpertLayout,
                 x2: torch.Tensor, w2: PackedWeights, out2: torch.Tensor, token_tile: int,
                 status: Optional[torch.Tensor] = None, second_first: bool = False) -> None:
    """Two products in one launch on pairs of CTAs: out = x . w over the layout's groups (as gemm_tc), and
    out2 = x2 . w2 over one group with token tiles of `token_tile` (128 or 256) consecutive rows.  Both SwiGLU (bf16
    results) or both plain (float32 results).  The persistent CTAs walk both products' tiles in one sequence, the
    second product's spread evenly among the first's (or first, with second_first): a product bound by the tensor
    cores beside one bound by its weight stream, where two launches would run one after the other.  The results
    are those of two separate launches with the same token tile, bit for bit."""
    if not (usable(x, w) and usable(x2, w2)):
        raise KernelError("gemm_tc_dual: needs bfloat16 activations with K a multiple of 8 and weights packed for this K")
    if w.swiglu != w2.swiglu or out.dtype != out2.dtype:
        raise KernelError("gemm_tc_dual: both products are SwiGLU or both plain, with one output type")
    if out.shape != (x.shape[0], w.n) or out2.shape != (x2.shape[0], w2.n) or w2.groups != 1:
        raise KernelError(f"gemm_tc_dual: outputs {tuple(out.shape)}, {tuple(out2.shape)} do not fit {x.shape[0]} x {w.n} "
                          f"and {x2.shape[0]} x {w2.n} (one group)")
    if layout.tile_rows != token_tile:
        raise KernelError(f"gemm_tc_dual: the layout has tiles of {layout.tile_rows} rows, the kernel was asked for {token_tile}")
    global DUAL_CALLS
    DUAL_CALLS += 1
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gemm_tc_dual(
        ptr(x), ptr(w.data), ptr(out), ptr(layout.tile_expert), ptr(layout.tile_row0), ptr(layout.tile_count),
        ptr(layout.n_tiles), c_int(layout.max_tiles), c_int(x.shape[0]), c_int(w.n), c_int(w.k), c_int(w.groups),
        ptr(x2), ptr(w2.data), ptr(out2), c_int(x2.shape[0]), c_int(w2.n), c_int(w2.k), c_int(code(out.dtype)),
        c_int(token_tile), c_int(1 if w.swiglu else 0),
        ptr(status if status is not None else status_word(x.device)), c_int(1 if second_first else 0), stream()))
