"""Dense projections of one to four tokens as weight streams (csrc/gemv.cu)."""
from __future__ import annotations

from ctypes import c_int
from typing import Optional

import torch

from ..csrc.build import load_kernel
from ._call import KernelError, check, code, ptr, stream, want_f32, want_int32

_LIB = "gemv"
MAX_TOKENS = 4
_NO_GEMV = __import__("os").environ.get("TQ_NO_GEMV", "0") not in ("", "0")


# Where the stream beats the library product (measured on B200 inside CUDA graphs, microseconds, ours / library):
#   2,048 x 2,048 (an output projection): 3.8 / 8.3 with 1 token, 4.0 / 7.0 with 2, 5.3 / 8.2 with 4
#   6,144 x 2,048 fused with bias, rotation and cache write (the library product needs a 3.4 us kernel behind it):
#   6.5 / 6.9 + 3.4 with 1 token, 8.6 / 6.9 + 3.4 with 2, 11.3 / 6.8 + 3.4 with 4
PLAIN_MAX_TOKENS, PLAIN_MAX_ROWS = 4, 4096
FUSED_MAX_TOKENS = 2


def usable(x: torch.Tensor, weight: torch.Tensor, max_tokens: int = MAX_TOKENS) -> bool:
    """bfloat16 rows of up to four tokens against bfloat16 weights with 16-byte rows that fit shared memory."""
    return (not _NO_GEMV and x.dim() == 2 and 1 <= x.shape[0] <= min(MAX_TOKENS, max_tokens) and x.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[0] * x.shape[1] * 2 <= 48 * 1024
            and x.is_contiguous() and weight.is_contiguous() and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


def pays(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """The plain product is usable here and faster than the library's."""
    return usable(x, weight, PLAIN_MAX_TOKENS) and weight.shape[0] <= PLAIN_MAX_ROWS


def fused_pays(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return usable(x, weight, FUSED_MAX_TOKENS)


def gemv(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, n] = sum_k x[t, k] weight[n, k] in float32.  x [T <= 4, K] bf16; weight [N, K] bf16; out [T, N] float32."""
    if not usable(x, weight):
        raise KernelError("gemv: needs 1 to 4 bfloat16 rows, bfloat16 weights and K a multiple of 8")
    want_f32(out, "gemv output")
    T, K = x.shape
    N = weight.shape[0]
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_gemv(ptr(x), ptr(weight), ptr(out), c_int(T), c_int(N), c_int(K), stream()))
    return out


def qkv_gemv_rope(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
                  page_table: torch.Tensor, page_size: int, q_out: torch.Tensor, cache_layer: Optional[torch.Tensor],
                  n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """The fused query/key/value projection of up to four tokens with bias, rotary encoding (half pairing), queries
    to q_out [T, nh, hd] and keys and values into cache_layer [pages, 2, nkv, page_size, hd], in one launch.
    The product is rounded to bfloat16 before the bias, as the library product it stands in for hands it on."""
    if not usable(x, weight):
        raise KernelError("qkv_gemv_rope: needs 1 to 4 bfloat16 rows, bfloat16 weights and K a multiple of 8")
    want_int32(positions, "positions")
    want_int32(page_table, "page table")
    if cos is not None:
        want_f32(cos, "cos table")
        want_f32(sin, "sin table")
    T, K = x.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_qkv_gemv_rope(
        ptr(x), ptr(weight), ptr(bias), c_int(code(bias.dtype) if bias is not None else 0), ptr(cos), ptr(sin),
        ptr(positions), ptr(seq_of_token), ptr(page_table), c_int(page_table.shape[1]), c_int(page_size), ptr(q_out),
        ptr(cache_layer), c_int(0 if cache_layer is None else 1), c_int(T), c_int(K), c_int(n_heads), c_int(n_kv_heads),
        c_int(head_dim), c_int(page_table.shape[0]), c_int(0 if cache_layer is None else cache_layer.shape[0]), stream()))
