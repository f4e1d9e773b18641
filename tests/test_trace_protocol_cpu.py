"""The replay program's protocol with a stand-in engine (CPU): steps from standard input, `done <step>` after each,
a file only for steps in which something is wanted, requests opened at their first step and given back at `end`."""
import io
import json
import types

import numpy as np
import pytest
import torch

import turboquant_cpp_b200.engine as engine_pkg
from turboquant_cpp_b200.engine import trace


class StandInEngine:
    """logits of the token at place p of a request = [request's running sum up to p, place, 0, ...] (vocab 5)."""
    made = []

    def __init__(self, model, max_tokens, device="cuda:0"):
        self.max_tokens, self.open_now, self.closed, self.sums, self.n = max_tokens, set(), [], {}, 0
        StandInEngine.made.append(self)

    def open(self):
        self.n += 1
        self.open_now.add(self.n)
        self.sums[self.n] = (0, 0)
        return self.n

    def close(self, seq):
        self.open_now.remove(seq)
        self.closed.append(seq)

    def step(self, entries):
        rows = []
        for e in entries:
            assert e.seq in self.open_now and len(e.tokens) > 0
            s, length = self.sums[e.seq]
            sums = np.cumsum(e.tokens) + s
            for w in e.want:
                rows.append([float(sums[w]), float(length + w), 0.0, 0.0, 0.0])
            self.sums[e.seq] = (int(sums[-1]), length + len(e.tokens))
        return torch.tensor(rows, dtype=torch.float32) if rows else None

    def check_kernels(self):
        pass


def run(monkeypatch, capsys, tmp_path, steps):
    StandInEngine.made.clear()
    monkeypatch.setattr(engine_pkg, "Engine", StandInEngine)
    monkeypatch.setattr(engine_pkg, "load_model", lambda folder, dtype, device: types.SimpleNamespace())
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps) + "\n"))
    rc = trace.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(tmp_path / "out"), "--max-tokens", "192"])
    return rc, capsys.readouterr().out.split("\n"), StandInEngine.made[-1]


def test_steps_files_and_ends(monkeypatch, capsys, tmp_path):
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}, {"id": "b", "tokens": [1], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": [2], "want": []}, {"id": "b", "tokens": [4], "want": []}], "end": ["b"]},
        {"step": 7, "entries": [{"id": "a", "tokens": [1], "want": [0]}], "end": ["a"]},
        {"step": 8, "entries": [{"id": "b", "tokens": [9, 9], "want": [1]}], "end": ["b", "never-seen"]},
    ]
    rc, lines, eng = run(monkeypatch, capsys, tmp_path, steps)
    assert rc == 0 and [l for l in lines if l] == ["done 0", "done 1", "done 7", "done 8"]
    out = tmp_path / "out"
    assert sorted(p.name for p in out.iterdir()) == ["0.f32", "7.f32", "8.f32"]          # step 1 wanted nothing
    a0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, 5)
    assert a0.tolist() == [[5, 0, 0, 0, 0], [25, 2, 0, 0, 0]]                             # entries' and want's order
    assert np.fromfile(out / "7.f32", dtype="<f4").reshape(-1, 5).tolist() == [[28, 4, 0, 0, 0]]   # on top of steps 0 and 1
    assert np.fromfile(out / "8.f32", dtype="<f4").reshape(-1, 5).tolist() == [[18, 1, 0, 0, 0]]   # "b" again: a new request
    assert eng.max_tokens == 192 and not eng.open_now and len(eng.closed) == 3


def test_without_a_device_it_says_so(monkeypatch, capsys, tmp_path):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    monkeypatch.setattr("sys.stdin", io.StringIO(""))
    rc = trace.main(["--model", str(tmp_path), "--dtype", "bfloat16", "--out", str(tmp_path / "o"), "--max-tokens", "64"])
    assert rc == 2 and "no CUDA device" in capsys.readouterr().err
    with pytest.raises(SystemExit):
        trace.main(["--model", str(tmp_path), "--dtype", "float16", "--out", "x", "--max-tokens", "64"])
