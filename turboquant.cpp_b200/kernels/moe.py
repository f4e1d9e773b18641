"""Mixture-of-experts kernels (csrc/moe.cu): router, expert-sorted layout, grouped GEMM, combine."""
from __future__ import annotations

from ctypes import c_int
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import check, code, ptr, stream, want_f32, want_int32

_LIB = "moe"
TILE_ROWS = 64     # rows of a tile of the exact grouped GEMM


def align_chunk(n_pairs: int) -> int:
    """Pairs per block of the layout kernels: 512 or more, and 256 chunks at most."""
    return max(512, 256 * -(-n_pairs // (256 * 256)))


def router_topk(x: torch.Tensor, w_router: torch.Tensor, w_shared_gate: Optional[torch.Tensor], top_k: int,
                renorm: bool, ids: torch.Tensor, weights: torch.Tensor,
                shared_scale: Optional[torch.Tensor]) -> None:
    """ids/weights [T, k] of the k most probable experts of each token; shared_scale [T] =
    sigmoid(w_shared_gate . x) when a shared gate is given."""
    T, H = x.shape
    E = w_router.shape[0]
    want_int32(ids, "expert ids")
    want_f32(weights, "expert weights")
    if w_shared_gate is not None and w_shared_gate.dtype != w_router.dtype:
        w_shared_gate = w_shared_gate.to(w_router.dtype)
    logits = torch.empty((T, E + 1), dtype=torch.float32, device=x.device)      # scratch of the two-kernel router
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_router_topk(ptr(x), c_int(code(x.dtype)), ptr(w_router), ptr(w_shared_gate),
                                   c_int(code(w_router.dtype)), ptr(logits), ptr(ids), ptr(weights), ptr(shared_scale),
                                   c_int(T), c_int(H), c_int(E), c_int(top_k), c_int(1 if renorm else 0), stream()),
          kernels=2)


def router_select(logits: torch.Tensor, top_k: int, renorm: bool, ids: torch.Tensor, weights: torch.Tensor,
                  shared_scale: Optional[torch.Tensor]) -> None:
    """The selection step alone, on float32 logits [T, E + 1] (column E: the shared gate's logit).
    The chosen entries of `logits` are overwritten."""
    want_f32(logits, "router logits")
    want_int32(ids, "expert ids")
    T, E1 = logits.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_router_select(ptr(logits), ptr(ids), ptr(weights), ptr(shared_scale), c_int(T), c_int(E1 - 1),
                                     c_int(top_k), c_int(1 if renorm else 0), stream()))


def max_tiles(n_pairs: int, n_experts: int, tile_rows: int) -> int:
    """Upper bound of the number of row tiles for any routing of n_pairs pairs."""
    return min(n_pairs, n_pairs // tile_rows + n_experts)


class ExpertLayout:
    """Buffers of the expert-sorted layout for up to n_pairs (token, choice) pairs."""

    def __init__(self, n_pairs: int, n_experts: int, tile_rows: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.n_pairs, self.n_experts, self.tile_rows = n_pairs, n_experts, tile_rows
        self.max_tiles = max(1, max_tiles(n_pairs, n_experts, tile_rows))
        self.counts = torch.empty(n_experts, **i32)
        self.sorted_pair = torch.empty(max(1, n_pairs), **i32)
        self.row_of_pair = torch.empty(max(1, n_pairs), **i32)
        self.expert_offset = torch.empty(n_experts + 1, **i32)
        self.tile_expert = torch.empty(self.max_tiles, **i32)
        self.tile_row0 = torch.empty(self.max_tiles, **i32)
        self.tile_count = torch.empty(self.max_tiles, **i32)
        self.n_tiles = torch.empty(1, **i32)
        self.chunk_hist = torch.empty(-(-max(1, n_pairs) // align_chunk(n_pairs)) * n_experts, **i32)     # scratch of moe_align


SMALL_MAX_PAIRS, SMALL_MAX_EXPERTS = 512, 1023      # what the kernel accepts
SMALL_PAIRS_WORTH_IT = 128                           # beyond this one block is slower than the separate kernels


def router_small_usable(n_tokens: int, top_k: int, n_experts: int, hidden: int) -> bool:
    return (n_tokens * top_k <= SMALL_MAX_PAIRS and n_experts <= SMALL_MAX_EXPERTS
            and (hidden + n_experts + 1) * 4 <= 27 * 1024)


def router_small_pays(n_tokens: int, top_k: int, n_experts: int, hidden: int) -> bool:
    """Measured on B200: at 256 pairs (batch 64, top-4) the single block costs more than it saves."""
    return n_tokens * top_k <= SMALL_PAIRS_WORTH_IT and router_small_usable(n_tokens, top_k, n_experts, hidden)


_counters = {}


def _counter(device: torch.device) -> torch.Tensor:
    """One int32 per device that the last block of router_small finds its turn with; zero between launches."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _counters:
        _counters[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _counters[idx]


def router_small(x: torch.Tensor, w_router: torch.Tensor, w_shared_gate: Optional[torch.Tensor], top_k: int,
                 renorm: bool, ids: torch.Tensor, weights: torch.Tensor, shared_scale: Optional[torch.Tensor],
                 layout: ExpertLayout, x_rows: torch.Tensor) -> None:
    """For steps of few tokens: router, expert-sorted layout and the sorted copies of the token rows
    (x_rows[row] = x[token of that row]) in one launch.  Launches on one device must not overlap (they share
    the counter that tells the last block its turn)."""
    T, H = x.shape
    E = w_router.shape[0]
    want_int32(ids, "expert ids")
    want_f32(weights, "expert weights")
    if w_shared_gate is not None and w_shared_gate.dtype != w_router.dtype:
        w_shared_gate = w_shared_gate.to(w_router.dtype)
    lib = load_kernel(_LIB)
    lo = layout
    check(_LIB, lib.tq_router_small(
        ptr(x), c_int(code(x.dtype)), ptr(w_router), ptr(w_shared_gate), c_int(code(w_router.dtype)),
        ptr(ids), ptr(weights), ptr(shared_scale), c_int(lo.tile_rows), ptr(lo.counts), ptr(lo.sorted_pair),
        ptr(lo.row_of_pair), ptr(lo.expert_offset), ptr(lo.tile_expert), ptr(lo.tile_row0), ptr(lo.tile_count),
        ptr(lo.n_tiles), ptr(x_rows), ptr(_counter(x.device)), c_int(T), c_int(H), c_int(E), c_int(top_k),
        c_int(1 if renorm else 0), stream()))


def moe_align(ids: torch.Tensor, layout: ExpertLayout) -> None:
    want_int32(ids, "expert ids")
    P = ids.numel()
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_moe_align(ptr(ids), c_int(P), c_int(layout.n_experts), c_int(layout.tile_rows),
                                 c_int(align_chunk(layout.n_pairs)), ptr(layout.chunk_hist), ptr(layout.counts), ptr(layout.sorted_pair), ptr(layout.row_of_pair),
                                 ptr(layout.expert_offset), ptr(layout.tile_expert), ptr(layout.tile_row0),
                                 ptr(layout.tile_count), ptr(layout.n_tiles), stream()), kernels=2)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, layout: Optional[ExpertLayout],
                 swiglu: bool, few_rows: bool = False) -> torch.Tensor:
    """Exact (CUDA-core, fp32 accumulation) grouped product.  a [R, K]; w [G, Nw, K] with Nw = N,
    or 2N when swiglu (gate rows, then up rows); out [R, N].  layout None: one group (G = 1).
    few_rows: the tiles hold a few rows each (a decode step): the kernel that streams the weights once per eight
    rows of a tile instead of the tiled one (any number of rows is right, many are slow)."""
    R, K = a.shape
    N = out.shape[1]
    if w.dim() == 2:
        w = w.unsqueeze(0)
    assert w.shape[2] == K and w.shape[1] == (2 * N if swiglu else N), (tuple(w.shape), N, K, swiglu)
    assert layout is not None or w.shape[0] == 1
    lib = load_kernel(_LIB)
    lo = layout
    check(_LIB, lib.tq_grouped_gemm(
        ptr(a), c_int(code(a.dtype)), ptr(w), c_int(code(w.dtype)), ptr(out), c_int(code(out.dtype)),
        ptr(lo.tile_expert) if lo else None, ptr(lo.tile_row0) if lo else None,
        ptr(lo.tile_count) if lo else None, ptr(lo.n_tiles) if lo else None,
        c_int(lo.max_tiles if lo else 0), c_int(R), c_int(N), c_int(K), c_int(1 if swiglu else 0),
        c_int(1 if few_rows else 0), stream()))
    return out


def moe_combine(y_rows: torch.Tensor, row_of_pair: torch.Tensor, weights: torch.Tensor,
                y_shared: Optional[torch.Tensor], shared_scale: Optional[torch.Tensor],
                out: torch.Tensor, top_k: int) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * y_rows[row_of_pair[t*k + j]] + shared_scale[t] * y_shared[t]; y_shared may be
    [parts, T, H]: partial sums that are added up in order first."""
    want_f32(y_rows, "expert outputs")
    want_f32(out, "combined output")
    T, H = out.shape
    parts = 1
    if y_shared is not None:
        want_f32(y_shared, "shared expert output")
        parts = y_shared.shape[0] if y_shared.dim() == 3 else 1
        if y_shared.numel() != parts * T * H:
            raise ValueError(f"moe_combine: shared expert output of shape {tuple(y_shared.shape)} for {T} x {H}")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_moe_combine(ptr(y_rows), ptr(row_of_pair), ptr(weights), ptr(y_shared), ptr(shared_scale),
                                   ptr(out), c_int(T), c_int(H), c_int(top_k), c_int(y_rows.shape[0]), c_int(parts), stream()))
    return out
