"""The allocation-free attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they call it (a host program that
gave all device memory to its own pool at start-up, a plug-in inside one, a path where cudaMalloc's
implicit synchronisation is not acceptable).  `tq_attention_split_static` keeps its scratch in a
fixed array inside the library for them.  This test calls it twice in a row with different inputs —
the second call finds the first call's leftovers in the shared array — and compares each result with
the ordinary entry point's, which gets a fresh scratch buffer from the caller.  It also checks that a
request beyond the array's size is refused with a clear message and launches nothing.

The file sorts last, so a run that stops at the first failure has already run every other test; it
passes alone in a fresh process as well as after the others.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_FLOATS = 2 * 1024 * 1024


def _inputs(seed, T, nh, nkv, hd, page, n_pages, dtype):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    q = torch.randn((T, nh, hd), generator=g, device=DEV).to(dtype)
    cache = torch.randn((n_pages, 2, nkv, page, hd), generator=g, device=DEV).to(dtype)
    lens = np.random.default_rng(seed).integers(1, n_pages * page // T, size=T)
    width = int(-(-lens.max() // page))
    table = np.full((T, width), -1, dtype=np.int32)
    perm = np.random.default_rng(seed + 1).permutation(n_pages)
    used = 0
    for i, L in enumerate(lens):
        n = -(-int(L) // page)
        table[i, :n] = perm[used:used + n]
        used += n
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    return q, cache, i32(lens - 1), i32(np.arange(T)), i32(table)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-6)])
def test_static_scratch_entry_point_matches_on_two_calls_in_a_row(dtype, tol):
    from turboquant_cpp_b200.csrc.build import load_kernel
    from turboquant_cpp_b200.kernels import attention as KA
    lib = load_kernel("attention")
    fn = lib.tq_attention_split_static          # the exported C symbol itself
    fn.restype = ctypes.c_int
    nh, nkv, hd, page, n_pages = 8, 2, 128, 64, 96
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (seed, T, n_splits, window) in enumerate([(1, 6, 7, 0), (2, 9, 3, 50)]):
        q, cache, pos, seq_of, table = _inputs(seed, T, nh, nkv, hd, page, n_pages, dtype)
        want = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
        partial = torch.empty(T * nh * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
        KA.attention_split(q, cache, pos, seq_of, table, page, window, 1 / math.sqrt(hd), want, nh, nkv, hd,
                           n_splits, partial)
        got = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
        rc = fn(vp(q), vp(cache), ctypes.c_int(0 if dtype == torch.float32 else 1), vp(pos), vp(seq_of), vp(table),
                ctypes.c_int(table.shape[1]), ctypes.c_int(page), ctypes.c_int(window), ctypes.c_float(1 / math.sqrt(hd)),
                ctypes.c_int(n_splits), vp(got), ctypes.c_int(T), ctypes.c_int(nh), ctypes.c_int(nkv), ctypes.c_int(hd),
                stream)
        assert rc == 0, lib.tq_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        err = (got.float() - want.float()).abs().max().item() / want.float().abs().max().item()
        assert err <= tol, f"call {call}: static-scratch result differs from the ordinary one by {err:.2e}"


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from turboquant_cpp_b200.csrc.build import load_kernel
    lib = load_kernel("attention")
    fn = lib.tq_attention_split_static
    fn.restype = ctypes.c_int
    T, nh, hd, n_splits = 4096, 16, 128, 8                         # 4096*16*8*130 floats > the array
    assert T * nh * n_splits * (hd + 2) > STATIC_FLOATS
    out = torch.zeros(8, device=DEV)
    before = out.clone()
    null = ctypes.c_void_p(0)
    rc = fn(null, null, ctypes.c_int(1), null, null, null, ctypes.c_int(1), ctypes.c_int(64), ctypes.c_int(0),
            ctypes.c_float(1.0), ctypes.c_int(n_splits), ctypes.c_void_p(out.data_ptr()), ctypes.c_int(T),
            ctypes.c_int(nh), ctypes.c_int(nh), ctypes.c_int(hd), ctypes.c_void_p(0))
    assert rc != 0
    msg = lib.tq_last_error().decode()
    assert "scratch" in msg and str(STATIC_FLOATS) in msg
    torch.cuda.synchronize()
    assert torch.equal(out, before)                                 # nothing ran
