"""bin/trace_run as a user runs it: a subprocess fed with JSON steps, logits read back from files.
The same requests whole, with the last 32 tokens one by one, and in batches of unequal lengths."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY
from plain import qwen2_moe_plain as P
from replay_util import TOL, batched, whole, with_tail

pytestmark = pytest.mark.gpu


def replay(folder, dtype, steps, ends, out_dir, max_tokens=1024):
    lines = []
    for i, step in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in step],
                                 "end": ends.get(i, [])}))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                        "--out", out_dir, "--max-tokens", str(max_tokens)],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    V = None
    logits, pos = {}, {}
    for i, step in enumerate(steps):
        n_want = sum(len(w) for _, _, w in step)
        path = os.path.join(out_dir, f"{i}.f32")
        if n_want == 0:
            assert not os.path.exists(path)
            for rid, toks, _ in step:
                pos[rid] = pos.get(rid, 0) + len(toks)
            continue
        a = np.fromfile(path, dtype="<f4")
        V = a.size // n_want
        a = a.reshape(n_want, V)
        row = 0
        for rid, toks, want in step:
            for w in want:
                logits.setdefault(rid, {})[pos.get(rid, 0) + w] = a[row]
                row += 1
            pos[rid] = pos.get(rid, 0) + len(toks)
    return logits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_replay_modes_agree_with_each_other_and_with_plain(tiny_folders, plain_models, tmp_path, name, dtype):
    V = TINY[name][0]["vocab_size"]
    rng = np.random.default_rng(50)
    reqs = {"a": rng.integers(0, V, size=45).tolist(), "b": rng.integers(0, V, size=100).tolist(),
            "c": rng.integers(0, V, size=71).tolist()}
    folder = tiny_folders[name]
    # each request alone and whole, one after another (slots are used again)
    steps, ends = [], {}
    for rid, toks in reqs.items():
        s, e = whole(rid, toks)
        ends.update({k + len(steps): v for k, v in e.items()})
        steps += s
    alone = replay(folder, dtype, steps, ends, str(tmp_path / "alone"))
    # the last 32 tokens one by one
    steps, ends = [], {}
    for rid, toks in reqs.items():
        s, e = with_tail(rid, toks, 32)
        ends.update({k + len(steps): v for k, v in e.items()})
        steps += s
    tail = replay(folder, dtype, steps, ends, str(tmp_path / "tail"))
    # one batch of unequal lengths, shorter requests end earlier; --max-tokens as small as the rule allows
    s, e = batched(reqs, {"a": 13, "b": 68, "c": 39})
    need = sum(-(-len(t) // 64) * 64 for t in reqs.values())
    both = replay(folder, dtype, s, e, str(tmp_path / "batch"), max_tokens=need)
    tol = TOL[dtype][0]
    rnd = P.round_bf16 if dtype == "bfloat16" else P.no_round
    for rid, toks in reqs.items():
        ref = P.forward(plain_models[name], toks, rnd)
        scale = np.abs(ref).max()
        for mode, got in (("alone", alone), ("tail", tail), ("batched", both)):
            assert sorted(got[rid]) == list(range(len(toks))), mode
            errs = np.array([np.abs(got[rid][p] - ref[p]).max() / scale for p in range(len(toks))])
            if dtype == "float32":
                assert errs.max() < tol, f"{mode} {rid}: position {errs.argmax()} differs by {errs.max():.2e}"
            else:
                # without the engine's expert choices at hand, a near-tie in a router may fall the other
                # way for a few positions; all others must agree
                assert np.mean(errs < tol) > 0.9, f"{mode} {rid}: {np.mean(errs < tol):.2f} of positions agree"
        if dtype == "float32":
            for p in range(len(toks)):
                assert np.abs(alone[rid][p] - tail[rid][p]).max() / scale < tol
                assert np.abs(alone[rid][p] - both[rid][p]).max() / scale < tol


def test_nothing_wanted_writes_nothing_and_cache_full_is_an_error(tiny_folders, tmp_path):
    folder = tiny_folders["A"]
    got = replay(folder, "float32", [[("a", [1, 2, 3], [])], [("a", [4], [0])]], {1: ["a"]}, str(tmp_path / "o"))
    assert sorted(got["a"]) == [3]
    lines = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": list(range(100)), "want": []}], "end": []})
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(tmp_path / "o2"), "--max-tokens", "64"], input=lines + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode != 0 and "CacheFull" in r.stderr
