"""The tensor-core grouped GEMM against numpy and against the exact CUDA-core kernel."""
import math

import numpy as np
import pytest
import torch

from plain import qwen2_moe_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def rel(got, want):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    return np.abs(got - want).max() / max(1e-30, np.abs(want).max())


@pytest.mark.parametrize("R,N,K,G", [(1, 128, 64, 1), (5, 128, 256, 3), (40, 200, 136, 6), (300, 1408, 2048, 8),
                                      (77, 96, 72, 5), (1000, 256, 512, 4)])
@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("bn,pair", [(16, False), (32, False), (64, False), (128, False), (256, False), (128, True), (256, True)])
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_grouped(R, N, K, G, swiglu, bn, pair, odtype):
    from turboquant_cpp_b200.kernels import gemm_tc as KT, moe as KM
    rng = np.random.default_rng(R * 7 + N + bn)
    a = P.round_bf16(rng.normal(size=(R, K)))
    w = P.round_bf16(rng.normal(size=(G, 2 * N if swiglu else N, K)) / math.sqrt(K))
    ids = rng.integers(0, G, size=(R, 1)).astype(np.int32)
    if G > 2:
        ids[ids == 1] = 2                                   # a group without rows
    lay = KM.ExpertLayout(R, G, bn, DEV)
    KM.moe_align(dev(ids, torch.int32), lay)
    order = lay.sorted_pair.cpu().numpy()[:R]
    a_sorted = a[order]
    out = torch.full((R, N), float("nan"), dtype=odtype, device=DEV)
    KT.gemm_tc(dev(a_sorted, torch.bfloat16), KT.pack_weights(dev(w, torch.bfloat16), swiglu), out, lay, bn, pair)
    KT.check_status()
    want = np.zeros((R, N))
    for g in range(G):
        sel = np.nonzero(ids[order, 0] == g)[0]
        if len(sel):
            x = a_sorted[sel]
            want[sel] = P.silu(x @ w[g, :N].T) * (x @ w[g, N:].T) if swiglu else x @ w[g].T
    tol = 2e-5 if odtype == torch.float32 else 6e-3         # fp32 accumulation; one bfloat16 rounding of the result
    assert rel(out, want) < tol
    # the exact kernel on the same data
    ref = torch.empty((R, N), dtype=torch.float32, device=DEV)
    lay64 = KM.ExpertLayout(R, G, 64, DEV)
    KM.moe_align(dev(ids, torch.int32), lay64)
    KM.grouped_gemm(dev(a_sorted, torch.bfloat16), dev(w, torch.bfloat16), ref, lay64, swiglu)
    assert rel(out, ref.double().cpu().numpy()) < tol


@pytest.mark.parametrize("R,N,K", [(3, 5632, 2048), (130, 300, 1408), (2048, 384, 256)])
@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("pair", [False, True])
def test_one_group(R, N, K, swiglu, pair):
    from turboquant_cpp_b200.kernels import gemm_tc as KT
    rng = np.random.default_rng(R + N)
    a = P.round_bf16(rng.normal(size=(R, K)))
    w = P.round_bf16(rng.normal(size=(1, 2 * N if swiglu else N, K)) / math.sqrt(K))
    bn = max(128, KT.token_tile_for(R, 1)) if pair else KT.token_tile_for(R, 1)
    out = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
    KT.gemm_tc(dev(a, torch.bfloat16), KT.pack_weights(dev(w, torch.bfloat16), swiglu), out, None, bn, pair)
    KT.check_status()
    # with a share of the GPU only (fewer persistent CTAs walk the same tiles): the same bits
    part = torch.full((R, N), float("nan"), dtype=torch.float32, device=DEV)
    KT.gemm_tc(dev(a, torch.bfloat16), KT.pack_weights(dev(w, torch.bfloat16), swiglu), part, None, bn, pair, sm_share=3)
    KT.check_status()
    assert torch.equal(part, out)
    want = P.silu(a @ w[0, :N].T) * (a @ w[0, N:].T) if swiglu else a @ w[0].T
    assert rel(out, want) < 2e-5


def test_refuses_what_it_cannot_do():
    from turboquant_cpp_b200.kernels import KernelError, gemm_tc as KT
    w = torch.zeros((1, 16, 20), dtype=torch.bfloat16, device=DEV)    # K not a multiple of 8
    assert not KT.packable(w)
    with pytest.raises(KernelError):
        KT.pack_weights(w, False)
    out = torch.zeros((4, 16), dtype=torch.float32, device=DEV)
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device=DEV)
    pw = KT.pack_weights(torch.zeros((1, 16, 64), dtype=torch.bfloat16, device=DEV), False)
    with pytest.raises(KernelError):
        KT.gemm_tc(x, pw, out, None, 48)                               # not a token tile the kernel has
    with pytest.raises(KernelError):
        KT.gemm_tc(x, pw, out, None, 64, True)                         # pairs of CTAs want wide token tiles
    with pytest.raises(KernelError):
        KT.gemm_tc(x.float(), pw, out, None, 16)                       # activations must be bfloat16
    with pytest.raises(KernelError):
        KT.gemm_tc(x[:, :32].contiguous(), pw, out, None, 16)          # packed for another K
    with pytest.raises(KernelError):
        KT.gemm_tc(x, pw, torch.zeros((4, 24), dtype=torch.float32, device=DEV), None, 16)


def test_packing_layout():
    from turboquant_cpp_b200.kernels import gemm_tc as KT
    w = torch.arange(2 * 2 * 130 * 72, dtype=torch.float32, device=DEV).reshape(2, 260, 72).to(torch.bfloat16)
    pw = KT.pack_weights(w, True)                                      # N = 130 -> 3 tiles of 64 columns, K = 72 -> 2 k-blocks
    assert pw.data.shape == (2 * 3, 2, 128, 64) and pw.n == 130 and pw.k == 72 and pw.groups == 2
    d = pw.data.view(2, 3, 2, 128, 64)                                  # group, tile, k-block, row, col
    # column 129 = tile 2, column 1 of the tile = quarter 0, i = 1: gate at row 1, up at row 17
    assert torch.equal(d[1, 2, 1, 1, :8], w[1, 129, 64:72])
    assert torch.equal(d[1, 2, 0, 17, :], w[1, 130 + 129, :64])
    # column 64 + 37 = tile 1, quarter 2, i = 5: gate at row 69, up at row 85
    assert torch.equal(d[0, 1, 0, 69, :], w[0, 101, :64])
    assert torch.equal(d[0, 1, 0, 85, :], w[0, 130 + 101, :64])
    assert float(d[0, 2, 0, 2:16, :].abs().sum()) == 0.0                # columns beyond N are zero (gate ...
    assert float(d[0, 2, 0, 18:, :].abs().sum()) == 0.0                 # ... and up)
    assert float(d[0, 0, 1, :, 8:].abs().sum()) == 0.0                  # elements beyond K are zero
    pp = KT.pack_weights(w, False)                                      # plain: 260 rows -> 3 tiles of 128
    assert pp.data.shape == (2 * 3, 2, 128, 64)
    assert torch.equal(pp.data.view(2, 3, 2, 128, 64)[1, 2, 1, 3, :8], w[1, 259, 64:72])


@pytest.mark.parametrize("R,N,K,bn,pair", [(1, 2048, 5632, 16, False), (8, 300, 1408, 16, False), (64, 3584, 2048, 64, False),
                                           (40, 256, 4096, 64, False)])
def test_k_shared_out_over_the_gpu(R, N, K, bn, pair):
    """A product with few tiles and a long K, its K cut into shares that write partial sums to slices of their own:
    the slices add up to the product, every share holds at least one k-block, and the result does not depend on
    the launch (fixed shares, no atomics)."""
    from turboquant_cpp_b200.kernels import gemm_tc as KT
    rng = np.random.default_rng(R + N + K)
    a = P.round_bf16(rng.normal(size=(R, K)))
    w = P.round_bf16(rng.normal(size=(1, N, K)) / math.sqrt(K))
    pw = KT.pack_weights(dev(w, torch.bfloat16), False)
    want = a @ w[0].T
    for ks in sorted({2, 3, KT.k_splits_for(R, N, K, bn), (K + 63) // 64}):
        if ks < 2:
            continue
        per = -(-((K + 63) // 64) // ks)
        if (ks - 1) * per >= (K + 63) // 64:
            with pytest.raises(KT.KernelError, match="empty"):
                KT.gemm_tc(dev(a, torch.bfloat16), pw, torch.empty((ks, R, N), dtype=torch.float32, device=DEV), None, bn, pair, k_splits=ks)
            continue
        out = torch.full((ks, R, N), float("nan"), dtype=torch.float32, device=DEV)
        KT.gemm_tc(dev(a, torch.bfloat16), pw, out, None, bn, pair, k_splits=ks)
        KT.check_status()
        assert rel(out.sum(dim=0), want) < 2e-5
        again = torch.empty_like(out)
        KT.gemm_tc(dev(a, torch.bfloat16), pw, again, None, bn, pair, k_splits=ks)
        assert torch.equal(out, again)
    assert KT.k_splits_for(8, 2048, 5632, 16) > 4 and KT.k_splits_for(2048, 2048, 5632, 256) == 1
    assert KT.k_splits_for(8, 2048, 512, 16) == 1                       # a short K is not cut
    with pytest.raises(KT.KernelError, match="single CTAs"):             # wide token tiles (pairs of CTAs) are never shared out
        KT.gemm_tc(dev(a, torch.bfloat16), pw, torch.empty((2, R, N), dtype=torch.float32, device=DEV), None, 128, True, k_splits=2)
    with pytest.raises(KT.KernelError):                                  # the SwiGLU epilogue needs the whole sum
        KT.gemm_tc(dev(a, torch.bfloat16), KT.pack_weights(dev(w[:, :N // 2 * 2], torch.bfloat16), True),
                   torch.empty((2, R, N // 2), dtype=torch.float32, device=DEV), None, bn, pair, k_splits=2)


@pytest.mark.parametrize("R,N,K,G,R2,N2,K2", [(300, 200, 136, 6, 130, 328, 136), (1100, 1408, 512, 8, 700, 1000, 256),
                                               (40, 96, 72, 5, 513, 64, 2048), (600, 704, 256, 3, 1, 130, 64)])
@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("second_first", [False, True])
def test_two_products_in_one_launch(R, N, K, G, R2, N2, K2, swiglu, bn, second_first):
    """The grouped product and a one-group product of other sizes walked by the same persistent CTAs: each output
    has the bits of its own separate launch, and every element was written."""
    from turboquant_cpp_b200.kernels import gemm_tc as KT, moe as KM
    rng = np.random.default_rng(R + N2 + bn)
    odtype = torch.bfloat16 if swiglu else torch.float32
    a = dev(P.round_bf16(rng.normal(size=(R, K))), torch.bfloat16)
    w = KT.pack_weights(dev(P.round_bf16(rng.normal(size=(G, 2 * N if swiglu else N, K)) / math.sqrt(K)), torch.bfloat16), swiglu)
    a2 = dev(P.round_bf16(rng.normal(size=(R2, K2))), torch.bfloat16)
    w2 = KT.pack_weights(dev(P.round_bf16(rng.normal(size=(1, 2 * N2 if swiglu else N2, K2)) / math.sqrt(K2)), torch.bfloat16), swiglu)
    ids = np.sort(rng.integers(0, G, size=(R, 1)).astype(np.int32), axis=0)
    if G > 2:
        ids[ids == 1] = 2                                   # a group without rows
    lay = KM.ExpertLayout(R, G, bn, DEV)
    KM.moe_align(dev(ids, torch.int32), lay)
    alone = torch.full((R, N), float("nan"), dtype=odtype, device=DEV)
    alone2 = torch.full((R2, N2), float("nan"), dtype=odtype, device=DEV)
    KT.gemm_tc(a, w, alone, lay, bn, True)
    KT.gemm_tc(a2, w2, alone2, None, bn, True)
    both = torch.full((R, N), float("nan"), dtype=odtype, device=DEV)
    both2 = torch.full((R2, N2), float("nan"), dtype=odtype, device=DEV)
    for _ in range(3):                                      # the same launch again: nothing left behind
        KT.gemm_tc_dual(a, w, both, lay, a2, w2, both2, bn, second_first=second_first)
    KT.check_status()
    assert not torch.isnan(alone.float()).any() and not torch.isnan(alone2.float()).any()
    assert torch.equal(both, alone) and torch.equal(both2, alone2)


def test_two_products_refuse_what_they_cannot_do():
    from turboquant_cpp_b200.kernels import gemm_tc as KT, moe as KM
    from turboquant_cpp_b200.kernels._call import KernelError
    a = torch.zeros((64, 64), dtype=torch.bfloat16, device=DEV)
    w = KT.pack_weights(torch.zeros((2, 128, 64), dtype=torch.bfloat16, device=DEV), False)
    ws = KT.pack_weights(torch.zeros((1, 256, 64), dtype=torch.bfloat16, device=DEV), True)
    w1 = KT.pack_weights(torch.zeros((1, 128, 64), dtype=torch.bfloat16, device=DEV), False)
    out = torch.zeros((64, 128), dtype=torch.float32, device=DEV)
    lay = KM.ExpertLayout(64, 2, 64, DEV)
    KM.moe_align(torch.zeros((64, 1), dtype=torch.int32, device=DEV), lay)
    with pytest.raises(KernelError, match="128 or 256"):
        KT.gemm_tc_dual(a, w, out, lay, a, w1, out.clone(), 64)
    lay = KM.ExpertLayout(64, 2, 128, DEV)
    KM.moe_align(torch.zeros((64, 1), dtype=torch.int32, device=DEV), lay)
    with pytest.raises(KernelError, match="both plain"):
        KT.gemm_tc_dual(a, w, out, lay, a, ws, out.clone(), 128)
    with pytest.raises(KernelError, match="float32"):
        KT.gemm_tc_dual(a, w, out.bfloat16(), lay, a, w1, out.bfloat16(), 128)
