"""Helpers of the replay tests: build step schedules from requests, run them through the engine,
and compare every wanted position with the plain implementation.

Routing is discontinuous: when two experts' router logits are closer than the arithmetic's error,
either choice is right, and a different choice changes the logits by far more than rounding.  So
the comparison has two parts: (1) the engine's expert choices must equal the plain model's, except
where the plain model's own margin (gap between the k-th and the next router logit, in units of the
spread of that token's logits) is below `flip_margin` — and such places must be rare; (2) the
logits must agree with the plain model run *with the engine's choices*, to the tolerance of the dtype.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

from plain.qwen2_moe_plain import PlainModel, forward as plain_forward, no_round, round_bf16

# (logit tolerance relative to the largest logit, margin below which a different expert is accepted)
#  float32: fp32 sums of up to a few thousand terms in another order than float64: a few 1e-6 of the
#            logits' scale, and 1e-5 of the spread of a token's router logits.
#  bfloat16: the plain model rounds activations where the engine stores bfloat16, so what is left is
#            summation order plus 1-ulp (2^-8) flips of single activations that spread through the
#            layers (and P rounded to bfloat16 inside the prompt attention kernel): a few 1e-3 of the
#            logits' scale; a token's router logits move by up to about 1e-2 of their spread.
TOL = {"float32": (2e-5, 1e-5), "bfloat16": (1.5e-2, 2.5e-2)}


def whole(rid: str, tokens: Sequence[int], keep=None):
    """The request alone, whole, logits everywhere (or at the positions `keep` holds)."""
    want = [p for p in range(len(tokens)) if keep is None or p in keep]
    return [[(rid, list(tokens), want)]], {0: [rid]}


def with_tail(rid: str, tokens: Sequence[int], tail: int = 32, keep=None):
    """All but the last `tail` tokens in one step, then the rest one by one (logits of the first step
    everywhere, or at the positions `keep` holds)."""
    n = len(tokens)
    head = max(1, n - tail)
    steps = [[(rid, list(tokens[:head]), [p for p in range(head) if keep is None or p in keep])]]
    for i in range(head, n):
        steps.append([(rid, [tokens[i]], [0])])
    return steps, {len(steps) - 1: [rid]}


def batched(requests: Dict[str, Sequence[int]], prompt_lens: Dict[str, int], keep=None):
    """Requests start together with prompts of unequal lengths, then go on one token each; a
    request leaves when its tokens are used up.  Logits are wanted everywhere (of the prompts: at the
    positions `keep` holds, if given)."""
    steps, ends = [], {}
    steps.append([(r, list(t[:prompt_lens[r]]), [p for p in range(prompt_lens[r]) if keep is None or p in keep])
                  for r, t in requests.items()])
    done = {r: prompt_lens[r] for r in requests}
    for r in requests:
        if done[r] == len(requests[r]):
            ends.setdefault(0, []).append(r)
    while any(done[r] < len(requests[r]) for r in requests):
        step = []
        for r, t in requests.items():
            if done[r] < len(t):
                step.append((r, [t[done[r]]], [0]))
                done[r] += 1
                if done[r] == len(t):
                    ends.setdefault(len(steps), []).append(r)
        steps.append(step)
    return steps, ends


def run_schedule(engine, steps, ends):
    """Runs steps through the engine.  Returns per request: logits {position: row} and expert
    choices per sparse layer {layer_index_in_sparse_order: {position: ids}}."""
    import turboquant_cpp_b200 as tq
    live, logits, routing = {}, {}, {}
    pos = {}
    for si, step in enumerate(steps):
        entries, order = [], []
        for rid, toks, want in step:
            if rid not in live:
                live[rid] = engine.open()
                pos[rid] = 0
            entries.append(tq.StepEntry(live[rid], toks, want))
            order.append((rid, len(toks), want))
        engine.debug = {}
        out = engine.step(entries)
        out = None if out is None else out.float().cpu().numpy()
        ids = [a.cpu().numpy() for a in engine.debug.get("router_ids", [])]
        engine.debug = None
        row, t0 = 0, 0
        for rid, n, want in order:
            for w in want:
                logits.setdefault(rid, {})[pos[rid] + w] = out[row]
                row += 1
            for li, a in enumerate(ids):
                for j in range(n):
                    routing.setdefault(rid, {}).setdefault(li, {})[pos[rid] + j] = a[t0 + j]
            pos[rid] += n
            t0 += n
        for rid in ends.get(si, []):
            engine.close(live.pop(rid))
    assert not live, f"requests never ended: {sorted(live)}"
    return logits, routing


_plain_runs: Dict[tuple, tuple] = {}      # (plain model, tokens, dtype, rows) -> (record, logits of the plain model's own choices)


def check_against_plain(plain: PlainModel, tokens: Sequence[int], logits: Dict[int, np.ndarray],
                        routing: Dict[int, Dict[int, np.ndarray]], dtype: str, what: str = "", report: dict = None):
    """report: a dict that receives the worst logit error and the smallest router margin seen."""
    tol, flip_margin = TOL[dtype]
    rnd = round_bf16 if dtype == "bfloat16" else no_round
    sparse = [l for l in range(plain.L) if plain.layer_is_sparse(l)]
    n = len(tokens)
    forced = {}
    for li, l in enumerate(sparse):
        assert sorted(routing[li]) == list(range(n)), f"{what}: layer {l} did not see every position exactly once"
        forced[l] = np.stack([routing[li][p] for p in range(n)])
    rows = sorted(logits)
    key = (id(plain), tuple(tokens), dtype, tuple(rows))
    if key not in _plain_runs:                # the same request comes back under several schedules
        rec = {}
        own = plain_forward(plain, tokens, rnd, record=rec, rows=rows)
        _plain_runs[key] = (rec, own)
    rec, own = _plain_runs[key]
    n_diff = 0
    for l in sparse:
        differ = np.nonzero(np.any(np.sort(rec["ids"][l], axis=1) != np.sort(forced[l], axis=1), axis=1))[0]
        for p in differ:
            assert rec["margin"][l][p] < flip_margin, (
                f"{what}: layer {l} position {p}: engine chose experts {forced[l][p].tolist()}, plain "
                f"{rec['ids'][l][p].tolist()} with margin {rec['margin'][l][p]:.3e}")
        n_diff += len(differ)
    # near-ties are a few per cent of all choices (the gap to the next expert is a fraction of the spread
    # divided by the number of experts); more than that would be a fault, not rounding
    assert n_diff <= max(2, (n * len(sparse)) // 20), f"{what}: {n_diff} expert choices differ"
    ref = own if n_diff == 0 else plain_forward(plain, tokens, rnd, forced_ids=forced, rows=rows)
    scale = np.abs(ref).max()
    worst, worst_p = 0.0, -1
    for i, p in enumerate(rows):
        e = np.abs(logits[p] - ref[i]).max() / scale
        if e > worst:
            worst, worst_p = e, p
    assert worst < tol, f"{what}: logits at position {worst_p} differ by {worst:.3e} of scale (tolerance {tol:.1e})"
    if report is not None:
        report["worst"] = max(report.get("worst", 0.0), worst)
        if sparse:
            report["margin"] = min(report.get("margin", np.inf), min(float(rec["margin"][l].min()) for l in sparse))
        report["flips"] = report.get("flips", 0) + n_diff
    return worst
