"""Attention kernels over the paged cache (csrc/attention.cu)."""
from __future__ import annotations

import os
from ctypes import c_float, c_int
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32

_LIB = "attention"
MAX_HEAD_DIM = 256
PAIRING = {"half": 0, "interleaved": 1}


def check_head_dim(head_dim: int) -> None:
    if head_dim % 16 or not 16 <= head_dim <= MAX_HEAD_DIM:
        raise KernelError(f"attention kernels take head sizes 16, 32, …, {MAX_HEAD_DIM}; got {head_dim}")


def qkv_rope_cache(qkv: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                   sin: Optional[torch.Tensor], pairing: str, positions: torch.Tensor,
                   seq_of_token: torch.Tensor, page_table: torch.Tensor, page_size: int,
                   q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
                   n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Bias and rotary encoding on the fused projection qkv [T, (nh+2nkv)*hd]; queries to q_out
    [T, nh, hd]; keys and values into cache_layer [pages, 2, nkv, page_size, hd] (None: the layer
    reads another layer's cache, so only the queries are produced)."""
    T = qkv.shape[0]
    if cos is not None:
        want_f32(cos, "cos table")
        want_f32(sin, "sin table")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_qkv_rope_cache(
        ptr(qkv), c_int(code(qkv.dtype)), ptr(bias), c_int(code(bias.dtype) if bias is not None else 0),
        ptr(cos), ptr(sin), c_int(PAIRING[pairing]), ptr(positions), ptr(seq_of_token), ptr(page_table),
        c_int(page_table.shape[1]), c_int(page_size), ptr(q_out), ptr(cache_layer),
        c_int(0 if cache_layer is None else 1), c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
        c_int(page_table.shape[0]), c_int(0 if cache_layer is None else cache_layer.shape[0]), stream()))


def attention(q: torch.Tensor, cache_layer: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
              page_table: torch.Tensor, page_size: int, window: int, scale: float, out: torch.Tensor,
              n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Exact attention of every token's queries over its sequence's cache (causal; window > 0
    limits a query to the last `window` positions, itself included)."""
    T = q.shape[0]
    want_int32(positions, "positions")
    want_int32(page_table, "page table")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_attention(ptr(q), ptr(cache_layer), c_int(code(q.dtype)), ptr(positions),
                                 ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1]), c_int(page_size),
                                 c_int(window), c_float(scale), ptr(out), c_int(T), c_int(n_heads),
                                 c_int(n_kv_heads), c_int(head_dim), c_int(page_table.shape[0]),
                                 c_int(cache_layer.shape[0]), stream()))
    return out


SPLIT_HEAD_DIMS = (16, 32, 64, 128, 256)


def split_usable(n_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Any number of query heads per KV head: a CTA keeps up to eight in registers, more are shared out."""
    return head_dim in SPLIT_HEAD_DIMS and page_size % 16 == 0


def head_chunks(n_heads: int, n_kv_heads: int) -> int:
    """CTAs that share the query heads of one KV head (a CTA keeps up to 8 of them in registers)."""
    return -(-(n_heads // n_kv_heads) // 8)


RESIDENT_CTAS = 592      # CTAs of the split kernel a B200 runs at once (148 SMs x 4, register-limited)
_resident = {}


def resident_ctas(device=None) -> int:
    """CTAs of the split kernel the device runs at once: four per SM (the register form's limit), from the
    device's own SM count."""
    if not torch.cuda.is_available():
        return RESIDENT_CTAS
    idx = torch.device(device).index if device is not None and torch.device(device).index is not None \
        else torch.cuda.current_device()
    if idx not in _resident:
        _resident[idx] = 4 * torch.cuda.get_device_properties(idx).multi_processor_count
    return _resident[idx]


def gqa_mma_usable(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether the split attention runs its tensor-core form: bfloat16, head size 64 or 128 and 3 to 16 query
    heads per KV head (the launcher decides the same way; TQ_NO_GQA_MMA=1 switches it off)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 3 <= n_heads // n_kv_heads <= 16
            and os.environ.get("TQ_NO_GQA_MMA", "0") in ("", "0"))


def split_resident(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, device=None) -> int:
    """CTAs of the split attention the device runs at once for this shape: four per SM in the register form, three
    in the tensor-core form (64 KiB of shared memory each)."""
    r = resident_ctas(device)
    return r * 3 // 4 if gqa_mma_usable(dtype, n_heads, n_kv_heads, head_dim) else r


EARLY_KEYS = os.environ.get("TQ_EARLY_KEYS", "1") not in ("", "0")     # decode steps ask for old keys before the wait on the kernel ahead
GQA_MAX_SPLITS = 8       # measured on B200 (7 heads per KV head, 2,048 keys): 1, 2 and 8 tokens all run fastest with 8 ranges
#                          (18-20 us; 16 ranges 20, 32 ranges 30: the last CTA's merge grows with the ranges x heads)


def splits_for(n_tokens: int, n_kv_heads: int, resident: int = RESIDENT_CTAS) -> int:
    """Ranges the keys of one (token, KV head) are cut into.  All CTAs do equal work, so what matters is
    how full the last wave is: with few rows the CTAs should fit one wave; with many, the count that
    leaves the smallest tail.  (Measured on B200 at context 2,048: 8 tokens x 16 heads, 4 ranges 40 us,
    5 ranges 50 us; 64 x 16, 4 ranges 191 us against 197 us for 1 or 2.)"""
    rows = max(1, n_tokens * n_kv_heads)
    if rows <= resident:
        return max(1, min(16, resident // rows))
    if rows >= 4 * resident:               # many waves anyway: the tail is small, more ranges only add merging
        return 1

    def fill(s: int) -> float:
        ctas = rows * s
        return ctas / (-(-ctas // resident) * resident)
    return max(range(1, 9), key=lambda s: (round(fill(s), 3), -s))


TICKET_ROWS = 1 << 16
_tickets = {}


def tickets(device: torch.device) -> torch.Tensor:
    """TICKET_ROWS int32 per device, zero between launches: with them the split kernel's CTAs find out which of a
    row's ranges finishes last (that one merges).  Launches that use them must not overlap on the device."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _tickets:
        _tickets[idx] = torch.zeros(TICKET_ROWS, dtype=torch.int32, device=device)
    return _tickets[idx]


def attention_split(q: torch.Tensor, cache_layer: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                    page_table: torch.Tensor, page_size: int, window: int, scale: float, out: torch.Tensor,
                    n_heads: int, n_kv_heads: int, head_dim: int, n_splits: int,
                    partial: Optional[torch.Tensor], early_keys: bool = False) -> torch.Tensor:
    """Attention with the keys of each (token, KV head) cut into n_splits ranges and merged, in one launch;
    `partial` holds T * n_heads * n_splits * (head_dim + 2) floats of scratch (not needed with one range).
    early_keys: the caller vouches that the kernel ahead of this one in the stream wrote nothing this launch reads
    but the queries and the keys and values at the tokens' own positions (a decode step: one new token per
    sequence); the kernel then asks for older keys before it waits for that kernel."""
    T = q.shape[0]
    want_int32(positions, "positions")
    want_int32(page_table, "page table")
    arrived = None
    if n_splits > 1:
        want_f32(partial, "partial states")
        if partial.numel() < T * n_heads * n_splits * (head_dim + 2):
            raise KernelError("attention_split: the scratch for partial states is too small")
        if T * n_heads > TICKET_ROWS:
            raise KernelError(f"attention_split: {T * n_heads} (token, head) rows with several ranges exceed "
                              f"the {TICKET_ROWS} tickets; use one range")
        arrived = tickets(q.device)
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_attention_split(ptr(q), ptr(cache_layer), c_int(code(q.dtype)), ptr(positions),
                                       ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1]),
                                       c_int(page_size), c_int(window), c_float(scale),
                                       ptr(partial) if n_splits > 1 else None, c_int(n_splits), ptr(arrived),
                                       ptr(out), c_int(T), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                                       c_int(page_table.shape[0]), c_int(cache_layer.shape[0]),
                                       c_int(1 if early_keys else 0), stream()),
          kernels=2 if n_splits > 1 and (T * head_chunks(n_heads, n_kv_heads) * n_kv_heads * n_splits
                                         > 2 * resident_ctas(q.device) or os.environ.get("TQ_SPLIT_RING", "0") not in ("", "0"))
          else 1)      # many short CTAs: the launcher adds a merge launch of its own
    return out


def attention_tiled(q: torch.Tensor, cache_layer: torch.Tensor, cu_seqlens: torch.Tensor, seq_start: torch.Tensor,
                    page_table: torch.Tensor, page_size: int, window: int, scale: float, out: torch.Tensor,
                    n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Causal attention of whole runs of new tokens in exact fp32 arithmetic on CUDA cores: 32 queries share every
    tile of keys and values through shared memory.  For float32 runs and for head sizes the tensor-core prompt
    kernel does not take.  Rows as in attention_prefill."""
    T = q.shape[0]
    want_int32(cu_seqlens, "cu_seqlens")
    want_int32(seq_start, "seq_start")
    want_int32(page_table, "page table")
    if head_dim % 4:
        raise KernelError(f"attention_tiled: head size {head_dim} must be a multiple of 4")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_attention_tiled(ptr(q), ptr(cache_layer), c_int(code(q.dtype)), ptr(cu_seqlens), ptr(seq_start),
                                       ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), c_int(window),
                                       c_float(scale), ptr(out), c_int(T), c_int(n_seqs), c_int(n_heads),
                                       c_int(n_kv_heads), c_int(head_dim), c_int(cache_layer.shape[0]), stream()))
    return out


def prefill_usable(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """The tensor-core prompt kernel takes bfloat16, head sizes 64 and 128 and pages of 64 tokens."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def attention_prefill(q: torch.Tensor, cache_layer: torch.Tensor, cu_seqlens: torch.Tensor, seq_start: torch.Tensor,
                      page_table: torch.Tensor, page_size: int, window: int, scale: float, out: torch.Tensor,
                      n_seqs: int, max_q_len: int, n_heads: int, n_kv_heads: int, head_dim: int,
                      status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of whole runs of new tokens (prompts, or pieces of them) on tcgen05 tensor
    cores (csrc/attention_prefill.cu).  Row t of q belongs to the sequence whose [cu_seqlens[i],
    cu_seqlens[i+1]) holds t and sits at position seq_start[i] + (t - cu_seqlens[i]); the step's keys
    and values are already in the cache."""
    from .gemm_tc import status_word
    T = q.shape[0]
    want_int32(cu_seqlens, "cu_seqlens")
    want_int32(seq_start, "seq_start")
    want_int32(page_table, "page table")
    if not prefill_usable(q.dtype, head_dim, page_size) or cache_layer.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: needs bfloat16, head size 64 or 128 and pages of 64 tokens")
    lib = load_kernel("attention_prefill")
    check("attention_prefill", lib.tq_attention_prefill(
        ptr(q), ptr(cache_layer), ptr(cu_seqlens), ptr(seq_start), ptr(page_table), c_int(page_table.shape[1]),
        c_int(page_size), c_int(cache_layer.shape[0]), c_int(window), c_float(scale), ptr(out), c_int(T), c_int(n_seqs),
        c_int(max_q_len), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
        ptr(status if status is not None else status_word(q.device)), stream()))
    return out
