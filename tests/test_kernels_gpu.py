"""Each kernel alone against the plain implementation's function for the same part, at sizes other
than the engine's tiny models (odd widths, head sizes in steps of 16, one or many KV heads)."""
import math

import numpy as np
import pytest
import torch

from plain import qwen2_moe_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.tensor(np.asarray(a), dtype=dtype, device=DEV).contiguous()


def bf16_values(a):
    """Round a float64 array to bfloat16 values, so that both sides start from the same numbers."""
    return P.round_bf16(a)


def close(got, want, tol):
    got = got.detach().float().cpu().numpy().astype(np.float64)
    err = np.abs(got - want).max() / max(1e-30, np.abs(want).max())
    assert err < tol, f"relative error {err:.3e} exceeds {tol:.1e}"


DTYPES = [(torch.float32, 3e-6), (torch.bfloat16, 6e-3)]   # fp32 sums; one bfloat16 rounding of the result


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
def test_embed_rows(wdtype):
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(0)
    table = bf16_values(rng.normal(size=(37, 50)))
    toks = rng.integers(0, 37, size=23)
    out = torch.empty((23, 50), dtype=torch.float32, device=DEV)
    K.embed_rows(dev(toks, torch.int32), dev(table, wdtype), out)
    close(out, P.embedding(table, toks), 1e-7)


@pytest.mark.parametrize("H", [50, 192, 2048, 3000])
@pytest.mark.parametrize("R", [7, 700])                   # few rows: a block per row; many: a warp per row
@pytest.mark.parametrize("odtype,tol", DTYPES)
def test_rmsnorm(H, R, odtype, tol):
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(1)
    x = rng.normal(size=(R, H)) * 3
    w = bf16_values(1 + 0.1 * rng.normal(size=H))
    y = rng.normal(size=(R, H))
    eps = 1e-5
    # plain norm
    out = torch.empty((R, H), dtype=odtype, device=DEV)
    xd = dev(x)
    K.rmsnorm(xd, dev(w, torch.bfloat16), eps, out)
    close(out, P.rmsnorm(x.astype(np.float32).astype(np.float64), w, eps), tol)
    close(xd, x, 1e-7)                                    # x untouched
    # residual sum fused in: x += y, then the norm
    yd = dev(y)
    K.rmsnorm(xd, dev(w), eps, out, add=yd)
    xs = x.astype(np.float32).astype(np.float64) + y.astype(np.float32).astype(np.float64)
    close(out, P.rmsnorm(xs, w, eps), tol)
    close(xd, xs, 1e-6)                                   # the sum was written back
    # gather of rows, with a pending sum that is not written back
    rows = np.array([5, 0, 5, 3]) if R < 512 else rng.integers(0, R, size=600)
    out2 = torch.empty((len(rows), H), dtype=odtype, device=DEV)
    before = xd.clone()
    K.rmsnorm(xd, dev(w), eps, out2, add=yd, rows=dev(rows, torch.int32))
    close(out2, P.rmsnorm((xs + y.astype(np.float32))[rows], w, eps), tol)
    assert torch.equal(before, xd)


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_silu_mul(dtype, tol):
    from turboquant_cpp_b200.kernels import elementwise as K
    rng = np.random.default_rng(2)
    gu = bf16_values(rng.normal(size=(5, 2 * 70)) * 4)
    out = torch.empty((5, 70), dtype=dtype, device=DEV)
    K.silu_mul(dev(gu, dtype), out)
    close(out, P.silu(gu[:, :70]) * gu[:, 70:], tol)


# ---------------------------------------------------------------------------------------------
def paged_inputs(rng, seq_lens, q_lens, nkv, hd, page_size, dtype, n_pages=64):
    """A batch whose sequences already hold (seq_len - q_len) tokens: K/V of all positions, shuffled
    pages, and the packed description of the step's new tokens."""
    B = len(seq_lens)
    perm = rng.permutation(n_pages)
    tables, used = [], 0
    for L in seq_lens:
        n = -(-L // page_size)
        tables.append(perm[used:used + n])
        used += n
    width = max(len(t) for t in tables)
    table = np.full((B, width), -1, dtype=np.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = t
    k_all = [bf16_values(rng.normal(size=(L, nkv, hd))) for L in seq_lens]
    v_all = [bf16_values(rng.normal(size=(L, nkv, hd))) for L in seq_lens]
    cache = np.zeros((n_pages, 2, nkv, page_size, hd))
    for i, L in enumerate(seq_lens):
        for p in range(L):
            pg = table[i, p // page_size]
            cache[pg, 0, :, p % page_size] = k_all[i][p]
            cache[pg, 1, :, p % page_size] = v_all[i][p]
    positions = np.concatenate([np.arange(L - q, L) for L, q in zip(seq_lens, q_lens)])
    seq_of = np.concatenate([np.full(q, i) for i, q in enumerate(q_lens)])
    cache[np.setdiff1d(np.arange(n_pages), perm[:used])] = 1e30     # pages of no sequence: never to be read
    # the slots of a sequence's last page beyond its length hold what an earlier owner of the page left there:
    # large finite values here (the engine's cache starts as zeros and only ever holds what its kernels wrote, so
    # stale slots are finite; a kernel may load them but must give them no weight)
    for i, L in enumerate(seq_lens):
        if L % page_size:
            cache[table[i, L // page_size], :, :, L % page_size:] = 1e30
    return dict(table=table, k=k_all, v=v_all, cache=cache, positions=positions, seq_of=seq_of)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 4, 16), (6, 2, 32), (5, 1, 48), (8, 2, 128), (3, 3, 80), (2, 1, 256)])
@pytest.mark.parametrize("window", [0, 7])
@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_attention(nh, nkv, hd, window, dtype, tol):
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(nh * 100 + hd + window)
    seq_lens, q_lens, page = [70, 1, 130, 9], [70, 1, 3, 1], 64
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype)
    T = sum(q_lens)
    q = bf16_values(rng.normal(size=(T, nh, hd)))
    out = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    KA.attention(dev(q, dtype), dev(d["cache"], dtype), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
                 dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd), out, nh, nkv, hd)
    want = np.zeros((T, nh * hd))
    t0 = 0
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        qfull = np.zeros((L, nh, hd))
        qfull[L - ql:] = q[t0:t0 + ql]
        want[t0:t0 + ql] = P.attention(qfull, d["k"][i], d["v"][i], window)[L - ql:]
        t0 += ql
    close(out, want, tol)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 4, 16), (6, 2, 32), (8, 1, 64), (16, 16, 128), (14, 2, 128), (3, 1, 256),
                                       (5, 5, 64), (12, 1, 64), (28, 4, 128), (17, 1, 32)])
@pytest.mark.parametrize("window", [0, 7, 70])
@pytest.mark.parametrize("n_splits", [1, 3, 16])
@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_attention_split(nh, nkv, hd, window, n_splits, dtype, tol):
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(nh * 100 + hd + window + n_splits)
    seq_lens, q_lens, page = [70, 1, 130, 9, 300], [70, 1, 3, 1, 1], 64
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype)
    T = sum(q_lens)
    q = bf16_values(rng.normal(size=(T, nh, hd)))
    out = torch.empty((T, nh * hd), dtype=dtype, device=DEV)
    partial = torch.full((T * nh * n_splits * (hd + 2),), float("nan"), dtype=torch.float32, device=DEV)
    assert KA.split_usable(nh, nkv, hd, page)
    KA.attention_split(dev(q, dtype), dev(d["cache"], dtype), dev(d["positions"], torch.int32),
                       dev(d["seq_of"], torch.int32), dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd),
                       out, nh, nkv, hd, n_splits, partial)
    want = np.zeros((T, nh * hd))
    t0 = 0
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        qfull = np.zeros((L, nh, hd))
        qfull[L - ql:] = q[t0:t0 + ql]
        want[t0:t0 + ql] = P.attention(qfull, d["k"][i], d["v"][i], window)[L - ql:]
        t0 += ql
    close(out, want, tol)
    assert int(KA.tickets(torch.device(DEV)).abs().sum()) == 0       # every row's last range put its ticket back


def test_attention_split_merges_in_range_order_whoever_comes_last():
    """The range that finishes last merges; which one that is differs from launch to launch, the result does not."""
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(5)
    nh, nkv, hd, page, n_splits = 8, 2, 128, 64, 9
    seq_lens, q_lens = [700, 40, 1300, 64], [2, 1, 1, 1]
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, torch.bfloat16)
    T = sum(q_lens)
    q = dev(bf16_values(rng.normal(size=(T, nh, hd))), torch.bfloat16)
    args = (dev(d["cache"], torch.bfloat16), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
            dev(d["table"], torch.int32), page, 0, 1 / math.sqrt(hd))
    outs = []
    for _ in range(20):
        out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(T * nh * n_splits * (hd + 2), dtype=torch.float32, device=DEV)
        KA.attention_split(q, *args, out, nh, nkv, hd, n_splits, partial)
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    assert int(KA.tickets(torch.device(DEV)).abs().sum()) == 0


@pytest.mark.parametrize("nh,nkv,hd,n_splits,ring", [(16, 16, 128, 4, "0"), (16, 16, 128, 3, "1"), (28, 4, 128, 8, "0"),
                                                       (4, 2, 64, 1, "0"), (6, 1, 32, 16, "0")])
def test_attention_split_asks_for_old_keys_before_the_wait_and_still_sees_the_new_ones(nh, nkv, hd, n_splits, ring, monkeypatch):
    """A decode step: the kernel ahead writes each token's key and value at its own position, the attention kernel
    behind it (launched early, its first groups of old keys asked for before it waits) must see them.  Twenty rounds
    with fresh keys, values and queries each; the newest key is made the one that decides the result (its score
    stands out), so a launch that missed it would differ; both ways of launching give the same bits."""
    from turboquant_cpp_b200.kernels import attention as KA
    monkeypatch.setenv("TQ_SPLIT_RING", ring)
    rng = np.random.default_rng(nh + hd + n_splits)
    seq_lens, page = [300, 17, 1, 130, 64, 2048, 9, 65], 64           # lengths after the step: the new token is the last
    q_lens = [1] * len(seq_lens)
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, torch.bfloat16, n_pages=80)
    T = len(seq_lens)
    pos, seq_of, table = (dev(d[k], torch.int32) for k in ("positions", "seq_of", "table"))
    cache = dev(d["cache"], torch.bfloat16)
    width = (nh + 2 * nkv) * hd
    for r in range(20):
        qkv = bf16_values(rng.normal(size=(T, width)))
        G = nh // nkv
        qkv[:, nh * hd:(nh + nkv) * hd] = bf16_values(3.0 * qkv[:, :nh * hd].reshape(T, nkv, G, hd)[:, :, 0]).reshape(T, -1)   # the new key points along its group's first query
        q = torch.empty((T, nh, hd), dtype=torch.bfloat16, device=DEV)
        outs = []
        for early in (True, False):
            KA.qkv_rope_cache(dev(qkv, torch.bfloat16), None, None, None, "half", pos, seq_of, table, page, q, cache, nh, nkv, hd)
            out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
            partial = torch.empty(T * nh * n_splits * (hd + 2), dtype=torch.float32, device=DEV) if n_splits > 1 else None
            KA.attention_split(q, cache, pos, seq_of, table, page, 0, 1 / math.sqrt(hd), out, nh, nkv, hd, n_splits, partial,
                               early_keys=early)
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), f"round {r}"
        # the new value carries weight in the result of the first head of each KV head: without it the output differs
        v_new = torch.tensor(qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd), dtype=torch.float32, device=DEV)
        got = outs[0].float().view(T, nkv, nh // nkv, hd)[:, :, 0]
        assert (torch.nn.functional.cosine_similarity(got, v_new, dim=-1) > 0.5).all(), f"round {r}: the new key was not seen"


@pytest.mark.parametrize("nh,hd", [(3, 128), (1, 128)])
@pytest.mark.parametrize("window,n_splits", [(0, 1), (0, 4), (900, 7)])
def test_attention_split_ring_equals_registers(nh, hd, window, n_splits, monkeypatch):
    """With one query head per KV head of size 128 in bfloat16, large launches bring keys and values in through a
    ring of cp.async copies in shared memory; the arithmetic is that of the register form, so both give the same
    bits, also where a range of keys is shorter than the ring is deep, ends inside a group of eight, or starts at a
    window's edge."""
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(nh + hd + window)
    seq_lens, q_lens, page = [2000, 1, 9, 37, 1333], [1, 1, 2, 1, 3], 64
    d = paged_inputs(rng, seq_lens, q_lens, nh, hd, page, torch.bfloat16)
    T = sum(q_lens)
    q = dev(bf16_values(rng.normal(size=(T, nh, hd))), torch.bfloat16)
    outs = []
    for ring in ("1", "0"):
        monkeypatch.setenv("TQ_SPLIT_RING", ring)
        out = torch.empty((T, nh * hd), dtype=torch.bfloat16, device=DEV)
        partial = torch.full((T * nh * n_splits * (hd + 2),), float("nan"), dtype=torch.float32, device=DEV)
        KA.attention_split(q, dev(d["cache"], torch.bfloat16), dev(d["positions"], torch.int32),
                           dev(d["seq_of"], torch.int32), dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd),
                           out, nh, nh, hd, n_splits, partial)
        outs.append((out, partial))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1].nan_to_num(nan=-7.0), outs[1][1].nan_to_num(nan=-7.0))


@pytest.mark.parametrize("nh,nkv,hd", [(2, 2, 128), (6, 2, 32), (5, 1, 48), (3, 3, 80), (2, 1, 256), (7, 1, 16)])
@pytest.mark.parametrize("window", [0, 40, 200])
@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_attention_tiled(nh, nkv, hd, window, dtype, tol):
    """Runs of new tokens of unequal lengths, some behind earlier tokens of their sequence (so a run starts in the
    middle of a page and of a key tile), against the plain attention; and against the one-query-at-a-time kernel,
    which computes the same sums in another order."""
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(nh * 10 + hd + window)
    seq_lens, q_lens, page = [300, 130, 64, 1, 513, 33], [300, 70, 64, 1, 257, 32], 64
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype, n_pages=40)
    T = sum(q_lens)
    q = bf16_values(rng.normal(size=(T, nh, hd)))
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    start = np.array(seq_lens) - np.array(q_lens)
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    args = (dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd))
    KA.attention_tiled(dev(q, dtype), dev(d["cache"], dtype), dev(cu, torch.int32), dev(start, torch.int32), *args,
                       out, len(seq_lens), nh, nkv, hd)
    want = np.zeros((T, nh * hd))
    t0 = 0
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        qfull = np.zeros((L, nh, hd))
        qfull[L - ql:] = q[t0:t0 + ql]
        want[t0:t0 + ql] = P.attention(qfull, d["k"][i], d["v"][i], window)[L - ql:]
        t0 += ql
    close(out, want, tol)
    one = torch.empty_like(out)
    KA.attention(dev(q, dtype), dev(d["cache"], dtype), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
                 *args, one, nh, nkv, hd)
    assert (out.float() - one.float()).abs().max().item() <= (1e-6 if dtype == torch.float32 else 2 ** -7) * one.float().abs().max().item()


def test_attention_tiled_time_at_a_2048_token_prompt():
    """One 2,048-token prompt, 16 heads of 128, float32: the tiled kernel against one CTA per query (prints both)."""
    from turboquant_cpp_b200.kernels import attention as KA
    T, nh, hd, page = 2048, 16, 128, 64
    g = torch.Generator(device=DEV).manual_seed(0)
    q = torch.randn((T, nh, hd), generator=g, device=DEV)
    cache = torch.randn((T // page, 2, nh, page, hd), generator=g, device=DEV)
    table = torch.arange(T // page, dtype=torch.int32, device=DEV).reshape(1, -1)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    tiled, one = torch.empty((T, nh * hd), device=DEV), torch.empty((T, nh * hd), device=DEV)
    run_tiled = lambda: KA.attention_tiled(q, cache, i32([0, T]), i32([0]), table, page, 0, 1 / math.sqrt(hd), tiled, 1, nh, nh, hd)
    run_one = lambda: KA.attention_split(q, cache, torch.arange(T, dtype=torch.int32, device=DEV), torch.zeros(T, dtype=torch.int32, device=DEV),
                                         table, page, 0, 1 / math.sqrt(hd), one, nh, nh, hd, 1, None)
    # the two kernels in turn, the best of five rounds each: the GPU's clocks move with what ran before this test,
    # and a round in turn meets the same clocks with both
    times = [1e9, 1e9]
    run_tiled(), run_one()
    for _ in range(5):
        for i, fn in enumerate((run_tiled, run_one)):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(3):
                fn()
            b.record()
            torch.cuda.synchronize()
            times[i] = min(times[i], a.elapsed_time(b) / 3)
    assert (tiled - one).abs().max().item() <= 1e-6 * one.abs().max().item() * 4
    flops = 4.0 * nh * hd * T * (T + 1) / 2
    print(f"\n[tiled fp32 attention, 2048 tokens x 16 heads x 128] {times[0]:.3f} ms ({flops / times[0] / 1e9:.1f} TFLOP/s) "
          f"against {times[1]:.3f} ms with one CTA per query")
    assert times[0] < times[1]


@pytest.mark.parametrize("nh,nkv,hd", [(2, 2, 128), (6, 2, 128), (4, 1, 64), (3, 3, 64)])
@pytest.mark.parametrize("window", [0, 40, 200])
def test_attention_prefill(nh, nkv, hd, window):
    """Runs of new tokens of unequal lengths; some sequences already hold earlier tokens."""
    from turboquant_cpp_b200.kernels import attention as KA, gemm_tc as KT
    rng = np.random.default_rng(nh * 10 + hd + window)
    seq_lens, q_lens, page = [300, 130, 64, 1, 513], [300, 70, 64, 1, 257], 64
    dtype = torch.bfloat16
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype, n_pages=40)
    T = sum(q_lens)
    q = bf16_values(rng.normal(size=(T, nh, hd)))
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    starts = np.array(seq_lens) - np.array(q_lens)
    KA.attention_prefill(dev(q, dtype), dev(d["cache"], dtype), dev(cu, torch.int32), dev(starts, torch.int32),
                         dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd), out, len(seq_lens), max(q_lens),
                         nh, nkv, hd)
    KT.check_status()
    want = np.zeros((T, nh * hd))
    t0 = 0
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        qfull = np.zeros((L, nh, hd))
        qfull[L - ql:] = q[t0:t0 + ql]
        want[t0:t0 + ql] = P.attention(qfull, d["k"][i], d["v"][i], window)[L - ql:]
        t0 += ql
    close(out, want, 1e-2)      # P is rounded to bfloat16 before the second product, and so is the result


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 64, 0), (16, 4, 128, 0), (16, 16, 128, 300)])
def test_attention_prefill_many_units_per_cta(nh, nkv, hd, window):
    """More (query tile, sequence, head) units than SMs, some of them empty (short sequences): every persistent
    CTA walks several units, reloading Q and alternating between its two accumulators."""
    from turboquant_cpp_b200.kernels import attention as KA, gemm_tc as KT
    rng = np.random.default_rng(nh + hd + window)
    seq_lens, q_lens, page = [700, 130, 64, 1, 513, 333], [700, 70, 64, 1, 257, 333], 64
    dtype = torch.bfloat16
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype, n_pages=48)
    T = sum(q_lens)
    n_units = -(-max(q_lens) // 128) * len(seq_lens) * nh
    assert n_units > 2 * torch.cuda.get_device_properties(0).multi_processor_count or nh == 8
    q = bf16_values(rng.normal(size=(T, nh, hd)))
    out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=DEV)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    starts = np.array(seq_lens) - np.array(q_lens)
    KA.attention_prefill(dev(q, dtype), dev(d["cache"], dtype), dev(cu, torch.int32), dev(starts, torch.int32),
                         dev(d["table"], torch.int32), page, window, 1 / math.sqrt(hd), out, len(seq_lens), max(q_lens),
                         nh, nkv, hd)
    KT.check_status()
    want = np.zeros((T, nh * hd))
    t0 = 0
    for i, (L, ql) in enumerate(zip(seq_lens, q_lens)):
        qfull = np.zeros((L, nh, hd))
        qfull[L - ql:] = q[t0:t0 + ql]
        want[t0:t0 + ql] = P.attention(qfull, d["k"][i], d["v"][i], window)[L - ql:]
        t0 += ql
    close(out, want, 1e-2)


def test_attention_prefill_far_key_and_window_edge():
    """A key 600 positions back carries a huge score: every later query's output is that key's value;
    a window that ends one short of it hides it, a window that just reaches it shows it again."""
    from turboquant_cpp_b200.kernels import attention as KA, gemm_tc as KT
    rng = np.random.default_rng(11)
    nh = nkv = 2
    hd, page, L, far = 128, 64, 700, 37
    dtype = torch.bfloat16
    d = paged_inputs(rng, [L], [L], nkv, hd, page, dtype, n_pages=16)
    q = bf16_values(rng.normal(size=(L, nh, hd)))
    k = d["k"][0]
    k[far] = 0
    k[far, :, 0] = 40.0
    q[:, :, 0] = 40.0
    d["cache"][d["table"][0, far // page], 0, :, far % page] = k[far]
    args = lambda w, out: KA.attention_prefill(
        dev(q, dtype), dev(d["cache"], dtype), dev([0, L], torch.int32), dev([0], torch.int32),
        dev(d["table"], torch.int32), page, w, 1 / math.sqrt(hd), out, 1, L, nh, nkv, hd)
    out = torch.empty((L, nh * hd), dtype=dtype, device=DEV)
    args(0, out)
    KT.check_status()
    close(out, P.attention(q, k, d["v"][0], 0), 1e-2)
    close(out[far:], np.tile(d["v"][0][far].reshape(1, -1), (L - far, 1)), 1e-2)
    w = 100
    args(w, out)
    want = P.attention(q, k, d["v"][0], w)
    close(out, want, 1e-2)
    got = out.float().cpu().numpy()
    edge = far + w - 1                                       # the last query that still sees the far key
    assert np.abs(got[edge] - np.tile(d["v"][0][far].reshape(-1), 1)).max() < 0.05
    assert np.abs(got[edge + 1] - d["v"][0][far].reshape(-1)).max() > 0.5


def test_attention_prefill_rising_scores_rescale_the_accumulator():
    """Scores that grow with the key's position: the running maximum rises in every key tile, by more than
    2^8 per tile for some query rows (the accumulator in tensor memory must be rescaled there) and by less
    for others (their exponentials are taken against an older maximum and exceed 1)."""
    from turboquant_cpp_b200.kernels import attention as KA, gemm_tc as KT
    rng = np.random.default_rng(23)
    nh = nkv = 2
    hd, page, L = 128, 64, 640
    dtype = torch.bfloat16
    d = paged_inputs(rng, [L], [L], nkv, hd, page, dtype, n_pages=16)
    q = bf16_values(rng.normal(size=(L, nh, hd)))
    k = d["k"][0]
    k[:, :, 0] = bf16_values(np.arange(L) / 16.0)[:, None]          # rises by 4 per tile of 64 keys
    # per tile the score rises by 4 * q0 / sqrt(hd) nats: q0 = 2..60 gives 1..30 bits per tile
    q[:, :, 0] = bf16_values(2.0 + 58.0 * rng.random(size=(L, nh)))
    for p in range(L):
        d["cache"][d["table"][0, p // page], 0, :, p % page] = k[p]
    out = torch.empty((L, nh * hd), dtype=dtype, device=DEV)
    KA.attention_prefill(dev(q, dtype), dev(d["cache"], dtype), dev([0, L], torch.int32), dev([0], torch.int32),
                         dev(d["table"], torch.int32), page, 0, 1 / math.sqrt(hd), out, 1, L, nh, nkv, hd)
    KT.check_status()
    close(out, P.attention(q, k, d["v"][0], 0), 1e-2)
    w = 150                                                          # and with a window that drops the early keys
    KA.attention_prefill(dev(q, dtype), dev(d["cache"], dtype), dev([0, L], torch.int32), dev([0], torch.int32),
                         dev(d["table"], torch.int32), page, w, 1 / math.sqrt(hd), out, 1, L, nh, nkv, hd)
    KT.check_status()
    close(out, P.attention(q, k, d["v"][0], w), 1e-2)


def test_attention_far_key_stands_out():
    """One key far back gets a large score: the output must be (almost) that key's value, which a
    kernel that skips or misplaces distant pages would miss."""
    from turboquant_cpp_b200.kernels import attention as KA
    rng = np.random.default_rng(5)
    nh = nkv = 2
    hd, page, L, far = 32, 64, 700, 3
    d = paged_inputs(rng, [L], [1], nkv, hd, page, torch.float32)
    q = rng.normal(size=(1, nh, hd))
    k = d["k"][0]
    k[far] = 0
    k[far, :, 0] = 40.0
    q[0, :, 0] = 40.0
    pg = d["table"][0, far // page]
    d["cache"][pg, 0, :, far % page] = k[far]
    out = torch.empty((1, nh * hd), dtype=torch.float32, device=DEV)
    KA.attention(dev(q), dev(d["cache"]), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
                 dev(d["table"], torch.int32), page, 0, 1 / math.sqrt(hd), out, nh, nkv, hd)
    qfull = np.zeros((L, nh, hd))
    qfull[-1] = q[0]
    want = P.attention(qfull, k, d["v"][0], 0)[-1:]
    close(out, want, 3e-6)
    close(out, d["v"][0][far].reshape(1, -1), 1e-3)      # it is that value
    # with a window that excludes it, the far key must not be seen
    KA.attention(dev(q), dev(d["cache"]), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
                 dev(d["table"], torch.int32), page, L - far - 1, 1 / math.sqrt(hd), out, nh, nkv, hd)
    close(out, P.attention(qfull, k, d["v"][0], L - far - 1)[-1:], 3e-6)
    KA.attention(dev(q), dev(d["cache"]), dev(d["positions"], torch.int32), dev(d["seq_of"], torch.int32),
                 dev(d["table"], torch.int32), page, L - far, 1 / math.sqrt(hd), out, nh, nkv, hd)
    close(out, d["v"][0][far].reshape(1, -1), 1e-3)      # the window's edge includes it again


@pytest.mark.parametrize("nh,nkv,hd", [(4, 4, 16), (6, 2, 32), (5, 1, 48), (2, 2, 128)])
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_qkv_rope_cache(nh, nkv, hd, pairing, dtype, tol):
    from turboquant_cpp_b200.kernels import attention as KA
    from turboquant_cpp_b200.parts.rotary import RotaryEncoding
    rng = np.random.default_rng(7)
    seq_lens, q_lens, page = [70, 130, 5], [70, 2, 1], 64
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, dtype)
    T = sum(q_lens)
    width = (nh + 2 * nkv) * hd
    qkv = bf16_values(rng.normal(size=(T, width)))
    bias = bf16_values(rng.normal(size=width))
    theta = 12345.0
    rot = RotaryEncoding(hd, theta, 256, pairing)
    rot.prepare(DEV)
    cos, sin, _ = rot.tables()
    cache = torch.zeros((64, 2, nkv, page, hd), dtype=dtype, device=DEV)
    q_out = torch.empty((T, nh, hd), dtype=dtype, device=DEV)
    KA.qkv_rope_cache(dev(qkv, dtype), dev(bias, dtype), cos, sin, pairing, dev(d["positions"], torch.int32),
                      dev(d["seq_of"], torch.int32), dev(d["table"], torch.int32), page, q_out, cache, nh, nkv, hd)
    x = qkv + bias
    pos = d["positions"]
    q = P.rotary(x[:, :nh * hd].reshape(T, nh, hd), pos, theta, pairing)
    k = P.rotary(x[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd), pos, theta, pairing)
    v = x[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    close(q_out, q, tol)
    c = cache.float().cpu().numpy()
    for t in range(T):
        pg = d["table"][d["seq_of"][t], pos[t] // page]
        np.testing.assert_allclose(c[pg, 0, :, pos[t] % page], k[t], atol=tol * 8, rtol=0)
        np.testing.assert_allclose(c[pg, 1, :, pos[t] % page], v[t], atol=tol * 8, rtol=0)
    # nothing else was written
    written = np.zeros(c.shape, dtype=bool)
    for t in range(T):
        written[d["table"][d["seq_of"][t], pos[t] // page], :, :, pos[t] % page] = True
    assert np.all(c[~written] == 0)


@pytest.mark.parametrize("T,N,K", [(1, 2048, 2048), (2, 50, 40), (3, 133, 264), (4, 4096, 3584), (1, 7, 8)])
def test_gemv(T, N, K):
    """One to four tokens against bfloat16 weights: widths that are no multiple of the rows a warp or a block takes,
    a K shorter than one pass of a warp."""
    from turboquant_cpp_b200.kernels import gemv as KG
    rng = np.random.default_rng(T + N + K)
    x, w = bf16_values(rng.normal(size=(T, K))), bf16_values(rng.normal(size=(N, K)) / math.sqrt(K))
    out = torch.full((T, N), float("nan"), dtype=torch.float32, device=DEV)
    KG.gemv(dev(x, torch.bfloat16), dev(w, torch.bfloat16), out)
    close(out, x @ w.T, 3e-6)
    assert not KG.usable(torch.zeros((5, K), dtype=torch.bfloat16, device=DEV), dev(w, torch.bfloat16))       # five tokens
    assert not KG.usable(dev(x, torch.float32), dev(w, torch.bfloat16))                                        # float32 rows
    with pytest.raises(KG.KernelError):
        KG.gemv(dev(x, torch.float32), dev(w, torch.bfloat16), out)


@pytest.mark.parametrize("nh,nkv,hd,H", [(4, 4, 16, 64), (6, 2, 32, 192), (5, 1, 48, 120), (16, 16, 128, 2048), (28, 4, 128, 3584)])
@pytest.mark.parametrize("T", [1, 3, 4])
@pytest.mark.parametrize("with_bias,with_rope,bias_dtype", [(True, True, torch.bfloat16), (True, True, torch.float32),
                                                            (False, True, None), (True, False, torch.bfloat16)])
def test_qkv_gemv_rope(nh, nkv, hd, H, T, with_bias, with_rope, bias_dtype):
    """The fused projection of up to four tokens: product (rounded to bfloat16 as the library product's result is),
    bias, rotation, queries out, keys and values at their positions' places in the pages and nowhere else; also
    without a cache (a layer that reads another's)."""
    from turboquant_cpp_b200.kernels import gemv as KG
    from turboquant_cpp_b200.parts.rotary import RotaryEncoding
    rng = np.random.default_rng(nh * 10 + hd + T)
    seq_lens, q_lens, page = ([70, 130, 5, 64][:T] if T < 4 else [70, 130, 5, 64]), [1] * T, 64
    if T == 3:
        seq_lens, q_lens = [70, 131], [1, 2]                      # two tokens of one sequence in the step
    d = paged_inputs(rng, seq_lens, q_lens, nkv, hd, page, torch.bfloat16)
    width = (nh + 2 * nkv) * hd
    x = bf16_values(rng.normal(size=(T, H)))
    w = bf16_values(rng.normal(size=(width, H)) / math.sqrt(H))
    bias = bf16_values(rng.normal(size=width)) if with_bias else None
    theta = 12345.0
    rot = RotaryEncoding(hd, theta, 256, "half")
    rot.prepare(DEV)
    cos, sin, _ = rot.tables() if with_rope else (None, None, None)
    cache = torch.zeros((64, 2, nkv, page, hd), dtype=torch.bfloat16, device=DEV)
    q_out = torch.full((T, nh, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    pos = d["positions"]
    args = (dev(x, torch.bfloat16), dev(w, torch.bfloat16), None if bias is None else dev(bias, bias_dtype), cos, sin,
            dev(pos, torch.int32), dev(d["seq_of"], torch.int32), dev(d["table"], torch.int32), page)
    KG.qkv_gemv_rope(*args, q_out, cache, nh, nkv, hd)
    y = P.round_bf16(x @ w.T) + (bias if bias is not None else 0.0)
    turn = (lambda a: P.rotary(a, pos, theta, "half")) if with_rope else (lambda a: a)
    q = turn(y[:, :nh * hd].reshape(T, nh, hd))
    k = turn(y[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd))
    v = y[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
    tol = 6e-3
    close(q_out, q, tol)
    c = cache.float().cpu().numpy()
    written = np.zeros(c.shape, dtype=bool)
    for t in range(T):
        pg = d["table"][d["seq_of"][t], pos[t] // page]
        np.testing.assert_allclose(c[pg, 0, :, pos[t] % page], k[t], atol=tol * 8, rtol=0)
        np.testing.assert_allclose(c[pg, 1, :, pos[t] % page], v[t], atol=tol * 8, rtol=0)
        written[pg, :, :, pos[t] % page] = True
    assert np.all(c[~written] == 0)
    q_only = torch.full((T, nh, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    KG.qkv_gemv_rope(*args, q_only, None, nh, nkv, hd)
    assert torch.equal(q_only, q_out)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,k,H,renorm,shared", [(8, 2, 64, False, True), (6, 3, 192, True, True), (5, 1, 120, False, False),
                                                  (60, 4, 200, False, True), (130, 8, 96, True, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_router(E, k, H, renorm, shared, dtype):
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(E + 1000)
    T = 33
    x = bf16_values(rng.normal(size=(T, H)))
    wr = bf16_values(rng.normal(size=(E, H)) * 0.3)
    wsg = bf16_values(rng.normal(size=(1, H)) * 0.3)
    ids = torch.empty((T, k), dtype=torch.int32, device=DEV)
    wts = torch.empty((T, k), dtype=torch.float32, device=DEV)
    sc = torch.empty((T,), dtype=torch.float32, device=DEV) if shared else None
    KM.router_topk(dev(x, dtype), dev(wr, dtype), dev(wsg, dtype) if shared else None, k, renorm, ids, wts, sc)
    rid, rw, margin = P.router(x, wr, k, renorm)
    assert margin.min() > 1e-4, "test data has a near-tie"      # in units of the logits' spread
    assert np.array_equal(ids.cpu().numpy(), rid)
    close(wts, rw, 1e-5)
    if shared:
        close(sc, 1 / (1 + np.exp(-(x @ wsg.T)[:, 0])), 1e-5)


def test_router_ties_go_to_the_lowest_index():
    from turboquant_cpp_b200.kernels import moe as KM
    x = np.ones((1, 16))
    wr = np.zeros((7, 16))
    wr[2] = wr[5] = 0.25          # two equal maxima, the rest equal and lower
    ids = torch.empty((1, 3), dtype=torch.int32, device=DEV)
    wts = torch.empty((1, 3), dtype=torch.float32, device=DEV)
    KM.router_topk(dev(x), dev(wr), None, 3, False, ids, wts, None)
    assert ids.cpu().tolist() == [[2, 5, 0]]


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (50, 6, 3), (300, 5, 1), (1000, 60, 4), (7, 64, 8),
                                   (2048, 60, 4), (5000, 130, 5), (4097, 3, 1), (700, 1500, 6)])   # several chunks, a ragged last one
def test_moe_align(T, E, k):
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(T)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    if T > 10:
        ids[ids == 1] = 0 if E > 2 and k == 1 else ids[ids == 1]     # may leave expert 1 without rows
    lay = KM.ExpertLayout(T * k, E, 64, DEV)
    KM.moe_align(dev(ids, torch.int32), lay)
    flat = ids.reshape(-1)
    counts = np.bincount(flat, minlength=E)
    assert np.array_equal(lay.counts.cpu().numpy(), counts)
    off = np.concatenate([[0], np.cumsum(counts)])
    assert np.array_equal(lay.expert_offset.cpu().numpy(), off)
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(lay.sorted_pair.cpu().numpy()[:T * k], order)
    inv = np.empty(T * k, dtype=np.int64)
    inv[order] = np.arange(T * k)
    assert np.array_equal(lay.row_of_pair.cpu().numpy()[:T * k], inv)
    n = int(lay.n_tiles.item())
    assert n == sum(-(-c // 64) for c in counts) <= lay.max_tiles
    te, t0, tc = (a.cpu().numpy()[:n] for a in (lay.tile_expert, lay.tile_row0, lay.tile_count))
    covered = np.zeros(T * k, dtype=int)
    for e, r0, c in zip(te, t0, tc):
        assert 1 <= c <= 64 and off[e] <= r0 and r0 + c <= off[e + 1]
        covered[r0:r0 + c] += 1
    assert np.all(covered == 1)


@pytest.mark.parametrize("R,N,K,G", [(1, 32, 64, 8), (130, 48, 192, 6), (77, 100, 50, 3), (200, 70, 130, 5), (9, 24, 4100, 2)])
@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("few_rows", [False, True])
def test_grouped_gemm(R, N, K, G, swiglu, dtype, tol, few_rows):
    """few_rows: the kernel of decode steps (a stream of the weights for up to eight rows of a tile at a time); it
    takes any number of rows per tile, so the same cases hold for it."""
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(R + N)
    a = bf16_values(rng.normal(size=(R, K)))
    w = bf16_values(rng.normal(size=(G, 2 * N if swiglu else N, K)) / math.sqrt(K))
    ids = rng.integers(0, G, size=(R, 1)).astype(np.int32)
    if G > 2:
        ids[ids == 1] = 2                      # an expert without rows
    lay = KM.ExpertLayout(R, G, 64, DEV)
    KM.moe_align(dev(ids, torch.int32), lay)
    order = lay.sorted_pair.cpu().numpy()[:R]
    a_sorted = a[order]
    out = torch.full((R, N), float("nan"), dtype=dtype, device=DEV)
    KM.grouped_gemm(dev(a_sorted, dtype), dev(w, dtype), out, lay, swiglu, few_rows=few_rows)
    want = np.zeros((R, N))
    for r in range(R):
        e = ids[order[r], 0]
        if swiglu:
            want[r] = P.silu(w[e, :N] @ a_sorted[r]) * (w[e, N:] @ a_sorted[r])
        else:
            want[r] = w[e] @ a_sorted[r]
    close(out, want, tol)
    # one group, no layout (the shared expert's products)
    out1 = torch.full((R, N), float("nan"), dtype=dtype, device=DEV)
    KM.grouped_gemm(dev(a, dtype), dev(w[:1], dtype), out1, None, swiglu, few_rows=few_rows)
    w0 = w[0]
    want1 = P.silu(a @ w0[:N].T) * (a @ w0[N:].T) if swiglu else a @ w0.T
    close(out1, want1, tol)


def test_moe_combine():
    from turboquant_cpp_b200.kernels import moe as KM
    rng = np.random.default_rng(9)
    T, k, H = 21, 3, 70
    Y = rng.normal(size=(T * k, H))
    Ys = rng.normal(size=(T, H))
    inv = rng.permutation(T * k).astype(np.int32)
    w = rng.random(size=(T, k))
    s = rng.random(size=T)
    out = torch.empty((T, H), dtype=torch.float32, device=DEV)
    KM.moe_combine(dev(Y), dev(inv, torch.int32), dev(w), dev(Ys), dev(s), out, k)
    want = np.einsum("tk,tkh->th", w, Y[inv].reshape(T, k, H)) + s[:, None] * Ys
    close(out, want, 2e-6)
    KM.moe_combine(dev(Y), dev(inv, torch.int32), dev(w), None, None, out, k)
    close(out, np.einsum("tk,tkh->th", w, Y[inv].reshape(T, k, H)), 2e-6)
    # the shared expert's output as partial sums (slices [T, H]) that are added up first; both row widths
    for H2 in (70, 72):
        Y2, parts = rng.normal(size=(T * k, H2)), rng.normal(size=(5, T, H2))
        out2 = torch.empty((T, H2), dtype=torch.float32, device=DEV)
        KM.moe_combine(dev(Y2), dev(inv, torch.int32), dev(w), dev(parts), dev(s), out2, k)
        close(out2, np.einsum("tk,tkh->th", w, Y2[inv].reshape(T, k, H2)) + s[:, None] * parts.sum(axis=0), 2e-6)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("V", [257, 5000, 151936])
def test_argmax_first_maximum(V):
    from turboquant_cpp_b200.kernels import sampling as KS
    rng = np.random.default_rng(V)
    l = rng.normal(size=(5, V)).astype(np.float32)
    l[1, [V - 1, 7, V // 2]] = 9.0          # equal maxima: the first wins
    l[2, 0] = 9.0
    l[3, V - 1] = 9.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    KS.argmax_rows(dev(l), out)
    assert out.cpu().tolist() == [P.sample_argmax(r) for r in l]
    assert out.cpu().tolist()[1] == 7


@pytest.mark.parametrize("in_global", [False, True])
@pytest.mark.parametrize("V,temp,top_p", [(257, 0.8, 1.0), (320, 0.7, 0.9), (5000, 1.5, 0.5), (20011, 1.0, 0.8),
                                          (151936, 0.8, 0.95)])
def test_sample_rows_matches_plain(V, temp, top_p, in_global):
    """Rows shared by 1, 1, 2, 4 and 8 CTAs; the scratch in shared memory and in global memory."""
    from turboquant_cpp_b200.kernels import sampling as KS
    rng = np.random.default_rng(V)
    R = 24
    l = (rng.normal(size=(R, V)) * 2).astype(np.float32)
    u = rng.random(size=R).astype(np.float32)
    u[0], u[1] = 0.0, 0.99999994
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    work = torch.empty(R * V, dtype=torch.float32, device=DEV)
    KS.sample_rows(dev(l), temp, top_p, dev(u), work, out, scratch_in_global=in_global)
    want = [P.sample_top_p(l[r], temp, top_p, float(u[r])) for r in range(R)]
    got = out.cpu().tolist()
    # a draw within float rounding of a boundary of the cumulative sum may fall either side
    same = sum(g == w for g, w in zip(got, want))
    assert same >= R - 1, (got, want)
    # u = 0 takes the first maximum; the largest u ends the walk at the last candidate even when the sums, added
    # in different orders, disagree in their last bit about whether the target was reached
    assert got[0] == want[0] == int(np.argmax(l[0])) and got[1] == want[1]


@pytest.mark.parametrize("V", [700, 9001, 20000, 151936])
def test_sample_rows_among_equal_values_goes_by_index(V):
    """All logits equal: every p is 1, the sum is V exactly, and the draw u picks token ceil(u * V) - 1.  With a
    row cut over several CTAs this is the hand-over of the count of equal values from one slice to the next."""
    from turboquant_cpp_b200.kernels import sampling as KS
    slices = min(8, 1 << ((-(-V // 4096)).bit_length() - 1))
    edge = -(-V // slices)
    u = [0.0, 0.5, 0.99999994, 1.0 / V, 0.25, 0.75]
    for s in range(1, slices):                                # the last token of a slice and the first of the next
        u += [(s * edge - 0.5) / V, (s * edge + 0.5) / V]
    u = np.asarray(u, dtype=np.float32)
    R = len(u)
    l = np.full((R, V), -3.25, dtype=np.float32)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    work = torch.empty(R * V, dtype=torch.float32, device=DEV)
    KS.sample_rows(dev(l), 1.0, 1.0, dev(u), work, out)
    want = [max(1, int(np.ceil(np.float32(x) * np.float32(V)))) - 1 for x in u]
    assert out.cpu().tolist() == want
    clear = [r for r in range(R) if 0.25 < (float(u[r]) * V) % 1.0 < 0.75]      # not within rounding of a boundary
    assert len(clear) >= 2 * (slices - 1)
    assert [P.sample_top_p(l[r], 1.0, 1.0, float(u[r])) for r in clear] == [want[r] for r in clear]


def test_sample_rows_distribution():
    """Four equal logits: each token near a quarter of many draws (the reference's own check,
    tests/test_ops.cpp:528-571, asks for 10-50 % of 1000 draws)."""
    from turboquant_cpp_b200.kernels import sampling as KS
    R, V = 2000, 4
    l = np.zeros((R, V), dtype=np.float32)
    u = np.random.default_rng(3).random(size=R).astype(np.float32)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    work = torch.empty(R * V, dtype=torch.float32, device=DEV)
    KS.sample_rows(dev(l), 1.0, 1.0, dev(u), work, out)
    counts = np.bincount(out.cpu().numpy(), minlength=V)
    assert counts.min() > 0.2 * R and counts.max() < 0.3 * R


@pytest.mark.parametrize("T,E,k,H,renorm,shared", [(1, 8, 2, 64, False, True), (8, 60, 4, 2048, False, True),
                                                    (64, 64, 8, 200, True, False), (33, 5, 1, 120, False, False),
                                                    (3, 1023, 40, 96, True, True), (128, 300, 4, 64, False, False),
                                                    (5, 17, 3, 100, True, True), (7, 60, 4, 2048, False, True),
                                                    (1, 60, 4, 2048, False, True), (2, 60, 4, 2048, True, True),
                                                    (4, 64, 8, 3584, False, True), (3, 6, 3, 192, True, False),
                                                    (4, 200, 16, 520, False, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cluster", [True, False])
def test_router_small_equals_the_separate_kernels(T, E, k, H, renorm, shared, dtype, cluster, monkeypatch):
    """The one-launch decode path gives exactly what the separate kernels give, call after call: a block per
    token for logits and selection; then, with up to 8 tokens, the blocks are a cluster that passes the choices
    round in shared memory and every block writes its own rows, else the block that finishes last (a counter)
    does the layout and the gathered rows.  One to four bfloat16 tokens take a single block that lays the pairs out
    by counting (with `cluster` off here, that form is switched off too, so the others see these sizes as well)."""
    from turboquant_cpp_b200.kernels import elementwise as KE, moe as KM
    if not cluster:
        if T > 8:
            pytest.skip("more than 8 tokens never form a cluster")
        monkeypatch.setenv("TQ_ROUTER_NO_CLUSTER", "1")
        monkeypatch.setenv("TQ_ROUTER_NO_TINY", "1")
    else:
        monkeypatch.setenv("TQ_ROUTER_NO_TINY", "0")      # "0": the single-block form wherever it can run, not only at one token
    rng = np.random.default_rng(T + E)
    x = dev(bf16_values(rng.normal(size=(T, H))), dtype)
    if T > 1:
        x[1] = x[0]                          # two tokens with the same choices: their pairs share experts
    wr = dev(bf16_values(rng.normal(size=(E, H)) * 0.3), dtype)
    wsg = dev(bf16_values(rng.normal(size=(1, H)) * 0.3), dtype) if shared else None
    assert KM.router_small_usable(T, k, E, H)

    def buffers():
        return (torch.empty((T, k), dtype=torch.int32, device=DEV), torch.empty((T, k), dtype=torch.float32, device=DEV),
                torch.empty((T,), dtype=torch.float32, device=DEV) if shared else None, KM.ExpertLayout(T * k, E, 16, DEV),
                torch.empty((T * k, H), dtype=dtype, device=DEV))
    ids1, w1, s1, lay1, rows1 = buffers()
    KM.router_topk(x, wr, wsg, k, renorm, ids1, w1, s1)
    KM.moe_align(ids1, lay1)
    KE.gather_rows(x, lay1.sorted_pair, k, rows1)
    for _ in range(3):                      # the counter that finds the last block is left ready for the next launch
        ids2, w2, s2, lay2, rows2 = buffers()
        rows2.fill_(float("nan"))
        KM.router_small(x, wr, wsg, k, renorm, ids2, w2, s2, lay2, rows2)
    assert torch.equal(ids1, ids2) and torch.equal(w1, w2) and torch.equal(rows1, rows2)
    if shared:
        assert torch.equal(s1, s2)
    n = int(lay1.n_tiles.item())
    assert n == int(lay2.n_tiles.item())
    for a, b in ((lay1.counts, lay2.counts), (lay1.expert_offset, lay2.expert_offset),
                 (lay1.sorted_pair[:T * k], lay2.sorted_pair[:T * k]), (lay1.row_of_pair[:T * k], lay2.row_of_pair[:T * k]),
                 (lay1.tile_expert[:n], lay2.tile_expert[:n]), (lay1.tile_row0[:n], lay2.tile_row0[:n]),
                 (lay1.tile_count[:n], lay2.tile_count[:n])):
        assert torch.equal(a, b)


@pytest.mark.parametrize("R,V,W", [(1, 7, 1), (5, 1000, 32), (70, 151, 128)])
def test_rep_penalty(R, V, W):
    """In place, once per occurrence, positive logits divided and the others multiplied; -1 and ids beyond the
    vocabulary are skipped; rows do not touch one another."""
    from turboquant_cpp_b200.kernels import sampling as KS
    rng = np.random.default_rng(R + V)
    logits = rng.normal(size=(R, V)).astype(np.float32)
    logits[:, 0] = 0.0
    recent = rng.integers(-1, min(V, 12) + 2, size=(R, W)).astype(np.int32)      # few ids: many repeats; some -1, some >= V
    recent[recent >= min(V, 12)] = V + 3
    got = KS.rep_penalty(dev(logits, torch.float32), dev(recent, torch.int32), 1.3)
    want = np.stack([P.repetition_penalty(logits[r], recent[r].tolist(), 1.3) for r in range(R)])
    assert np.allclose(got.cpu().numpy(), want, rtol=1e-6, atol=0)
