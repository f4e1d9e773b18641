"""The plain implementation against the reference's own CPU code, once, on a tiny random model.

tests/golden/logits.bin was written by tests/golden/make_golden.sh, which compiles the reference's
C sources and runs tests/golden/ref_driver.c (7 tokens through tq_forward).  The weights are not
stored: the driver draws them from a xorshift generator in creation order, and this test draws the
same numbers.  The reference rotates interleaved pairs, always renormalises the chosen experts'
weights, and uses a fast exp in the experts' SiLU and the shared gate's sigmoid
(src/engine/tq_ops.c:1418-1448, src/engine/tq_moe.c:659-678, :42-48); with those three switches set
the same way the plain model reproduces its logits to float32 rounding.  With the exact exp, which
is the library's formula, the difference is the approximation's error (about 1e-2 of the logits).

tests/golden/samples.bin, from tests/golden/ref_sampler.c, holds what the reference's samplers picked on
drawn logits; the plain samplers pick the same tokens from the same uniform numbers (1 of 1,944 draws
falls on the other side of a float32 rounding).
"""
import os
import types

import numpy as np

from plain import qwen2_moe_plain as P

HERE = os.path.dirname(os.path.abspath(__file__))


class XorShift:
    def __init__(self):
        self.s = 88172645463325252

    def draw(self, n):
        out = np.empty(n, dtype=np.float32)
        s, M = self.s, (1 << 64) - 1
        for i in range(n):
            s ^= (s << 13) & M
            s ^= s >> 7
            s ^= (s << 17) & M
            out[i] = s >> 40
        self.s = s
        return (out / np.float32(1 << 24) - np.float32(0.5)) * np.float32(0.2)

    def fill(self, *shape):
        return self.draw(int(np.prod(shape))).reshape(shape).astype(np.float64)

    def ones(self, n):
        return (np.float32(1.0) + self.draw(n) * np.float32(0.1)).astype(np.float64)


def reference_fast_exp(x):
    """exp as the reference's experts approximate it (src/engine/tq_moe.c:42-48)."""
    x = np.asarray(x, dtype=np.float32)
    bits = (np.float32(12102203.0) * x + np.float32(1065353216.0)).astype(np.int32)
    y = bits.view(np.float32).astype(np.float64)
    y = np.where(x < -20.0, 0.0, y)
    return np.where(x > 20.0, np.exp(x.astype(np.float64)), y)


def build_model():
    L, D, NH, NKV, HD, E, K, I, S, V = 2, 64, 4, 2, 16, 8, 2, 32, 64, 256
    g = XorShift()
    w = {"model.embed_tokens.weight": g.fill(V, D), "lm_head.weight": g.fill(V, D), "model.norm.weight": g.ones(D)}
    for l in range(L):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = g.ones(D)
        w[p + "post_attention_layernorm.weight"] = g.ones(D)
        w[p + "self_attn.q_proj.weight"] = g.fill(NH * HD, D)
        w[p + "self_attn.k_proj.weight"] = g.fill(NKV * HD, D)
        w[p + "self_attn.v_proj.weight"] = g.fill(NKV * HD, D)
        w[p + "self_attn.o_proj.weight"] = g.fill(D, NH * HD)
        w[p + "self_attn.q_proj.bias"] = g.fill(NH * HD)
        w[p + "self_attn.k_proj.bias"] = g.fill(NKV * HD)
        w[p + "self_attn.v_proj.bias"] = g.fill(NKV * HD)
        w[p + "mlp.gate.weight"] = g.fill(E, D)
        for e in range(E):
            q = f"{p}mlp.experts.{e}."
            w[q + "gate_proj.weight"] = g.fill(I, D)
            w[q + "up_proj.weight"] = g.fill(I, D)
            w[q + "down_proj.weight"] = g.fill(D, I)
        w[p + "mlp.shared_expert.gate_proj.weight"] = g.fill(S, D)
        w[p + "mlp.shared_expert.up_proj.weight"] = g.fill(S, D)
        w[p + "mlp.shared_expert.down_proj.weight"] = g.fill(D, S)
        w[p + "mlp.shared_expert_gate.weight"] = g.fill(1, D)
    return types.SimpleNamespace(
        w=w, L=L, H=D, nh=NH, nkv=NKV, hd=HD, eps=1e-6, theta=10000.0, E=E, k=K, norm_topk=True, tied=False,
        cfg={"shared_expert_intermediate_size": S}, layer_is_sparse=lambda l: True, layer_window=lambda l: 0)


def test_plain_model_reproduces_the_reference_build():
    ref = np.fromfile(os.path.join(HERE, "golden", "logits.bin"), dtype="<f4").reshape(7, 256).astype(np.float64)
    m = build_model()
    toks = [3, 17, 200, 42, 9, 77, 255]
    scale = np.abs(ref).max()
    P.MOE_EXP = reference_fast_exp
    try:
        same = P.forward(m, toks, pairing="interleaved")
    finally:
        P.MOE_EXP = np.exp
    assert np.abs(same - ref).max() / scale < 5e-6          # the reference's computation, to float32 rounding
    exact = P.forward(m, toks, pairing="interleaved")
    err = np.abs(exact - ref).max() / scale
    assert 1e-4 < err < 3e-2                                  # the fast exp's own error, nothing else
    other = P.forward(m, toks, pairing="half")
    assert np.abs(other - ref).max() / scale > 3e-2           # the pairing matters and is not the reference's
    # the half-split pairing (x[i], x[i+hd/2]) is the reference's rotation on the same pairs stored in another
    # order: with the rows of every head of the query and key projections (and biases) reordered from
    # (0, 1, 2, 3, …) to (0, 2, 4, …, 1, 3, 5, …), pair i sits at (i, i + hd/2), each head's dot products are
    # unchanged, and the half-split model must give the reference's logits
    hd = m.hd
    order = np.concatenate([np.arange(0, hd, 2), np.arange(1, hd, 2)])
    halved = types.SimpleNamespace(**m.__dict__)
    halved.w = dict(m.w)
    for name, a in m.w.items():
        if ".self_attn.q_proj." in name or ".self_attn.k_proj." in name:
            heads = a.shape[0] // hd
            halved.w[name] = a.reshape((heads, hd) + a.shape[1:])[:, order].reshape(a.shape)
    P.MOE_EXP = reference_fast_exp
    try:
        half = P.forward(halved, toks, pairing="half")
    finally:
        P.MOE_EXP = np.exp
    assert np.abs(half - ref).max() / scale < 5e-6


def build_model_with_a_dense_layer_and_a_tied_head():
    """The model of tests/golden/ref_driver2.c: layer 0 with experts, layer 1 dense, the head is the embedding."""
    L, D, NH, NKV, HD, E, K, I, S, ID, V = 2, 64, 4, 2, 16, 8, 2, 32, 64, 80, 256
    g = XorShift()
    w = {"model.embed_tokens.weight": g.fill(V, D), "model.norm.weight": g.ones(D)}
    for l in range(L):
        p = f"model.layers.{l}."
        w[p + "input_layernorm.weight"] = g.ones(D)
        w[p + "post_attention_layernorm.weight"] = g.ones(D)
        w[p + "self_attn.q_proj.weight"] = g.fill(NH * HD, D)
        w[p + "self_attn.k_proj.weight"] = g.fill(NKV * HD, D)
        w[p + "self_attn.v_proj.weight"] = g.fill(NKV * HD, D)
        w[p + "self_attn.o_proj.weight"] = g.fill(D, NH * HD)
        w[p + "self_attn.q_proj.bias"] = g.fill(NH * HD)
        w[p + "self_attn.k_proj.bias"] = g.fill(NKV * HD)
        w[p + "self_attn.v_proj.bias"] = g.fill(NKV * HD)
        if l == 1:
            w[p + "mlp.gate_proj.weight"] = g.fill(ID, D)
            w[p + "mlp.up_proj.weight"] = g.fill(ID, D)
            w[p + "mlp.down_proj.weight"] = g.fill(D, ID)
            continue
        w[p + "mlp.gate.weight"] = g.fill(E, D)
        for e in range(E):
            q = f"{p}mlp.experts.{e}."
            w[q + "gate_proj.weight"] = g.fill(I, D)
            w[q + "up_proj.weight"] = g.fill(I, D)
            w[q + "down_proj.weight"] = g.fill(D, I)
        w[p + "mlp.shared_expert.gate_proj.weight"] = g.fill(S, D)
        w[p + "mlp.shared_expert.up_proj.weight"] = g.fill(S, D)
        w[p + "mlp.shared_expert.down_proj.weight"] = g.fill(D, S)
        w[p + "mlp.shared_expert_gate.weight"] = g.fill(1, D)
    m = types.SimpleNamespace(
        w=w, L=L, H=D, nh=NH, nkv=NKV, hd=HD, eps=1e-6, theta=10000.0, E=E, k=K, norm_topk=True, tied=True,
        cfg={"shared_expert_intermediate_size": S}, layer_is_sparse=lambda l: l == 0, layer_window=lambda l: 0)
    return m, g


def test_dense_layer_tied_head_and_router_against_the_reference_build():
    """tests/golden/ref_driver2.c: a dense SwiGLU layer (exact exp there, src/engine/tq_ops.c:1454-1478) behind a
    layer with experts, logits through the embedding table, and tq_moe_route alone."""
    ref = np.fromfile(os.path.join(HERE, "golden", "logits2.bin"), dtype="<f4").reshape(7, 256).astype(np.float64)
    m, g = build_model_with_a_dense_layer_and_a_tied_head()
    toks = [3, 17, 200, 42, 9, 77, 255]
    scale = np.abs(ref).max()
    P.MOE_EXP = reference_fast_exp
    try:
        same = P.forward(m, toks, pairing="interleaved")
    finally:
        P.MOE_EXP = np.exp
    assert np.abs(same - ref).max() / scale < 5e-6
    untied = types.SimpleNamespace(**{**m.__dict__, "tied": False})
    untied.w = dict(m.w, **{"lm_head.weight": m.w["model.embed_tokens.weight"][::-1].copy()})
    assert np.abs(P.forward(untied, toks, pairing="interleaved") - ref).max() / scale > 1e-2     # the head matters
    # the router alone: the reference's ids and weights of the 3 largest of 8 logits are this library's formula with
    # renormalisation (softmax over all, the 3 most probable, divided by their sum)
    raw = np.fromfile(os.path.join(HERE, "golden", "route.bin"), dtype="<i4")
    ids_ref = raw[:18].reshape(6, 3)
    wts_ref = raw[18:].view("<f4").reshape(6, 3).astype(np.float64)
    wr, hid = g.fill(8, 64), g.fill(6, 64)
    ids, wts, margin = P.router(hid, wr, 3, True)
    assert margin.min() > 1e-4                                   # no near-tie decides this comparison
    assert np.array_equal(ids, ids_ref)
    assert np.abs(wts - wts_ref).max() < 2e-6
    loose, _, _ = P.router(hid, wr, 3, False)[1], None, None     # without renormalisation the weights are smaller
    assert np.all(loose.sum(axis=1) < 1.0) and np.allclose(loose / loose.sum(axis=1, keepdims=True), wts_ref, atol=2e-6)


def reference_uniforms(state, n):
    """n numbers of the reference's generator from one state (xorshift64*, src/engine/tq_generate.c:53-58):
    the top 31 bits of state * 0x2545F4914F6CDD1D as a float32 over 2^31."""
    M, out = (1 << 64) - 1, []
    for _ in range(n):
        state ^= state >> 12
        state ^= (state << 25) & M
        state ^= state >> 27
        out.append(np.float32(((state * 0x2545F4914F6CDD1D) & M) >> 33) / np.float32(1 << 31))
    return out


def test_plain_samplers_pick_the_reference_builds_tokens():
    """tests/golden/samples.bin holds what the reference's tq_sample_argmax and tq_sample_topp picked on 81 cases
    (3 vocabularies x 3 spreads of logits x 3 temperatures x 3 values of top-p), 24 draws each
    (tests/golden/ref_sampler.c).  The plain samplers, given the same logits and the same uniform numbers, pick the
    same tokens, except where a draw lands within float32 rounding of a boundary of the cumulative sum."""
    ref = np.fromfile(os.path.join(HERE, "golden", "samples.bin"), dtype="<i4")
    DRAWS = 24
    g = XorShift()
    case, at, differ, total = 0, 0, 0, 0
    for V in (256, 1000, 5003):
        for spread in (4.0, 10.0, 25.0):
            raw = g.draw(V) / np.float32(0.2)                   # the generator's number in [-0.5, 0.5)
            logits = (raw * np.float32(spread)).astype(np.float32)
            for T in (0.7, 1.0, 0.3):
                for top_p in (0.9, 1.0, 0.5):
                    assert P.sample_argmax(logits) == ref[at]
                    us = reference_uniforms(1000 + case, DRAWS)
                    for d in range(DRAWS):
                        got = P.sample_top_p(logits, float(np.float32(T)), float(np.float32(top_p)), float(us[d]))
                        differ += int(got != ref[at + 1 + d])
                        total += 1
                    at += 1 + DRAWS
                    case += 1
    assert at == ref.size and case == 81
    assert differ <= total // 200, f"{differ} of {total} draws differ"
