"""Sampling kernels (csrc/sampling.cu): argmax, temperature with a nucleus, repetition penalty."""
from __future__ import annotations

from ctypes import c_float, c_int

import torch

from ..csrc.build import load_kernel
from ._call import check, ptr, stream, want_f32, want_int32

_LIB = "sampling"


def argmax_rows(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = index of the first maximum of logits[r]."""
    want_f32(logits, "logits")
    want_int32(out, "tokens")
    R, V = logits.shape
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_argmax_rows(ptr(logits), c_int(R), c_int(V), ptr(out), stream()))
    return out


def sample_rows(logits: torch.Tensor, temperature: float, top_p: float, uniforms: torch.Tensor,
                work: torch.Tensor, out: torch.Tensor, scratch_in_global: bool = False) -> torch.Tensor:
    """Temperature / top-p draw per row from uniforms [R] in [0, 1).  work holds R*V floats of scratch, used when
    a row's share per CTA does not fit shared memory (beyond 360,448 columns) or when scratch_in_global asks."""
    want_f32(logits, "logits")
    want_f32(uniforms, "uniforms")
    want_f32(work, "work")
    want_int32(out, "tokens")
    R, V = logits.shape
    assert work.numel() >= R * V
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_sample_rows(ptr(logits), c_int(R), c_int(V), c_float(temperature), c_float(top_p),
                                   ptr(uniforms), ptr(work), c_int(int(scratch_in_global)), ptr(out), stream()))
    return out


def rep_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: float) -> torch.Tensor:
    """In place: for each entry of recent [R, W] (a token id, or -1) the logit of that token in its row is divided
    by the penalty if positive and multiplied by it otherwise, once per occurrence."""
    want_f32(logits, "logits")
    want_int32(recent, "recent tokens")
    R, V = logits.shape
    if recent.dim() != 2 or recent.shape[0] != R or not recent.is_contiguous() or not logits.is_contiguous():
        raise ValueError("rep_penalty: recent must be a contiguous [rows, window] table and logits contiguous")
    lib = load_kernel(_LIB)
    check(_LIB, lib.tq_rep_penalty(ptr(logits), c_int(R), c_int(V), ptr(recent), c_int(recent.shape[1]),
                                   c_float(penalty), stream()))
    return logits
