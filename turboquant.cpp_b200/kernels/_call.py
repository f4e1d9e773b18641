"""Glue between torch tensors and the C launchers of the kernel libraries."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_kernel

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    """A launcher refused its arguments or the launch failed; the message is the launcher's."""


def code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def ptr(t: Optional[torch.Tensor]) -> Optional[ctypes.c_void_p]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels take CUDA tensors; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError("kernels take contiguous tensors")
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def stream() -> ctypes.c_void_p:
    """The current stream of the current device as the launchers take it.  Every launch asks, so this goes to
    torch's C entry points where this build of torch has them (a tenth of the cost of building a Stream object)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


LAUNCHES = 0     # kernels of this library launched so far (counted by the wrappers)


def check(lib_name: str, rc: int, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if rc != 0:
        lib = load_kernel(lib_name)
        raise KernelError(lib.tq_last_error().decode("utf-8", "replace") or f"{lib_name}: error {rc}")


def want_int32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")


def want_f32(t: torch.Tensor, what: str) -> None:
    if t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
