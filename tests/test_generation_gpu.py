"""Generation through the Python entry point and the command line, against the plain implementation."""
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, TINY
from plain import qwen2_moe_plain as P

pytestmark = pytest.mark.gpu


def prompts_for(name, lens, seed):
    V = TINY[name][0]["vocab_size"]
    rng = np.random.default_rng(seed)
    return [rng.integers(0, V, size=n).tolist() for n in lens]


def greedy_with_margin(plain, prompt, n, rnd=P.no_round, rep_penalty=1.0, rep_window=32):
    """Plain greedy continuation, and for every generated token the gap between the two largest
    logits (a tiny gap may legitimately resolve the other way under another summation order)."""
    toks, out, gaps = list(prompt), [], []
    for _ in range(n):
        l = P.forward(plain, toks, rnd)[-1]
        if rep_penalty > 1.0:
            l = P.repetition_penalty(l, P.recent_tokens(prompt, out, rep_window), rep_penalty)
        top = np.sort(l)[-2:]
        gaps.append(top[1] - top[0])
        t = int(np.argmax(l))
        out.append(t)
        toks.append(t)
    return out, gaps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lens,n_new", [("A", [5, 11, 17], 8), ("B", [1, 9, 40, 70], 16)])
def test_greedy_generation_through_the_entry_point(tiny_folders, plain_models, name, lens, n_new, dtype):
    import turboquant_cpp_b200 as tq
    prompts = prompts_for(name, lens, 40)
    with tq.Model(tiny_folders[name], temperature=0.0, max_tokens=n_new, dtype=dtype, max_batch=4,
                  context_length=128) as m:
        outs = m.generate_batch(prompts)
        assert m.last_stats.batches == 1 and m.last_stats.generated_tokens == n_new * len(prompts)
        again = m.generate_batch(prompts[::-1])[::-1]          # another order in the batch, slots used again
        assert again == outs
        alone = [m.ask(p) for p in prompts]                     # each alone
        assert alone == outs
        m.engine.cache.book.check_invariants()
        assert m.engine.cache.book.slots.n_held == 0
    rnd = P.round_bf16 if dtype == "bfloat16" else P.no_round
    gap_floor = 1e-5 if dtype == "float32" else 5e-3
    for p, o in zip(prompts, outs):
        want, gaps = greedy_with_margin(plain_models[name], p, n_new, rnd)
        for i, (a, b) in enumerate(zip(o, want)):
            if a != b:
                assert gaps[i] < gap_floor, f"token {i}: engine {a}, plain {b}, gap {gaps[i]:.3e}"
                break                                            # after a near-tie the texts part ways
        else:
            assert o == want


@pytest.mark.parametrize("name,lens,n_new", [("B", [1, 9, 40, 70], 16)])
def test_seeded_sampling_matches_the_plain_sampler(tiny_folders, plain_models, name, lens, n_new):
    """Temperature 0.8 with a seed: every request draws from its own stream, so the batch, the
    request alone and the plain loop give the same tokens (float32)."""
    import turboquant_cpp_b200 as tq
    prompts = prompts_for(name, lens, 41)
    with tq.Model(tiny_folders[name], temperature=0.8, top_p=1.0, max_tokens=n_new, seed=7, dtype="float32",
                  max_batch=4, context_length=128) as m:
        outs = m.generate_batch(prompts)
        assert m.generate_batch(prompts) == outs                 # seeded
        assert m.generate_batch(prompts, seed=8) != outs
        nucleus = m.generate_batch(prompts, top_p=0.5)
        assert nucleus != outs
    for i, (p, o) in enumerate(zip(prompts, outs)):
        want = P.generate(plain_models[name], p, n_new, temperature=0.8, top_p=1.0, seed=7, sequence=i)
        assert o == want, f"request {i}"
    i = 2
    want = P.generate(plain_models[name], prompts[i], n_new, temperature=0.8, top_p=0.5, seed=7, sequence=i)
    assert nucleus[i] == want


def test_stop_tokens_and_streaming(tiny_folders, plain_models):
    import turboquant_cpp_b200 as tq
    p = prompts_for("A", [7], 42)[0]
    want, _ = greedy_with_margin(plain_models["A"], p, 12)
    stop = want[4]
    first = want.index(stop)
    with tq.Model(tiny_folders["A"], temperature=0.0, max_tokens=12, dtype="float32", max_batch=2,
                  context_length=64) as m:
        assert m.warm_up() == [1, 2] and m.warm_up() == []       # the decode steps of both batch sizes, captured once
        out = m.ask(p, stop_token_ids=[stop])
        assert out == want[:first + 1] and m.last_results[0].finish_reason == "stop"
        assert list(m.generate(p)) == want                       # the iterator yields the same tokens
    with pytest.raises(FileNotFoundError):
        tq.Model("/nonexistent/model/folder")


def test_command_line(tiny_folders, plain_models):
    p = prompts_for("A", [5, 9], 43)
    want = [greedy_with_margin(plain_models["A"], q, 6)[0] for q in p]
    cmd = [sys.executable, os.path.join(ROOT, "bin", "quant"), tiny_folders["A"], "-n", "6", "-T", "0", "--dtype", "float32",
           "-p", ",".join(map(str, p[0])), "-p", " ".join(map(str, p[1]))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.strip().splitlines() if l.strip()]
    assert [[int(t) for t in l.split()] for l in lines] == want
    assert "tokens in" in r.stderr and "tok/s" in r.stderr
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "quant"), tiny_folders["A"], "--info"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "Qwen2MoeForCausalLM" in r.stdout and "num_experts: 8" in r.stdout


def test_command_line_random_weights_tokens_file_profile_and_layer_sums(tiny_folders, tmp_path):
    """--random CONFIG --seed-weights N runs the model that write_random_folder writes for the same configuration
    and seed (the folder of Tiny A was written with seed 0); --tokens-file gives the prompts; --profile prints the
    reference's bucket line and the buckets' rates; TQ_DEBUG_LAYERS prints per-layer sums of the residual stream."""
    import json
    from conftest import TINY_A
    p = prompts_for("A", [7, 4], 45)
    quant = [sys.executable, os.path.join(ROOT, "bin", "quant")]
    common = ["-n", "5", "-T", "0", "--dtype", "float32"]
    cfg_file, tok_file = str(tmp_path / "cfg.json"), str(tmp_path / "prompts.txt")
    json.dump(TINY_A, open(cfg_file, "w"))
    open(tok_file, "w").write("# two prompts\n" + "\n".join(" ".join(map(str, q)) for q in p) + "\n\n")
    a = subprocess.run(quant + [tiny_folders["A"]] + common + ["--tokens-file", tok_file], capture_output=True, text=True, timeout=600)
    b = subprocess.run(quant + ["--random", cfg_file, "--seed-weights", "0"] + common + ["--tokens-file", tok_file, "--profile"],
                       capture_output=True, text=True, timeout=600, env=dict(os.environ, TQ_DEBUG_LAYERS="1"))
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    assert a.stdout == b.stdout and len(a.stdout.strip().splitlines()) == 2
    line = [l for l in b.stderr.splitlines() if l.startswith("[Profile 10 tok]")]
    assert len(line) == 1 and all(k in line[0] for k in ("matmul=", "moe=", "attn=", "other=", "per-tok:"))
    rates = [l for l in b.stderr.splitlines() if l.startswith("[Profile] ")]
    assert {l.split()[1].rstrip(":") for l in rates} >= {"matmul", "moe", "attn"} and all("GB/s" in l and "TFLOP/s" in l for l in rates)
    sums = [l for l in b.stderr.splitlines() if l.startswith("[fwd]   L")]
    assert any("L0 pos=0 final x sum=" in l for l in sums) and any("L1 pos=1 " in l for l in sums)
    c = subprocess.run(quant + ["--random", cfg_file, "--seed-weights", "1"] + common + ["--tokens-file", tok_file],
                       capture_output=True, text=True, timeout=600)
    assert c.returncode == 0 and c.stdout != a.stdout                       # another seed, another model
    assert subprocess.run(quant + common, capture_output=True, text=True).returncode != 0       # neither folder nor --random


def test_command_line_measurements(tiny_folders):
    """--bench-prefill and --bench-memory print the reference's machine-readable lines (tools/quant.c:788, 848):
    prompt length, milliseconds and tokens a second; context and decoded tokens a second, for every context that
    leaves room for the 20 decoded tokens."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "quant"), tiny_folders["A"], "--dtype", "float32",
           "--bench-prefill", "--bench-memory"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    pre = [l for l in r.stderr.splitlines() if l.startswith("PREFILL_CSV:")]
    mem = [l for l in r.stderr.splitlines() if l.startswith("BENCH_CSV:")]
    assert len(pre) == 1
    n, ms, rate = pre[0].split(":")[1].split(",")
    assert int(n) == 128 and float(ms) > 0 and float(rate) > 0            # Tiny A holds 128 positions
    assert [int(l.split(":")[1].split(",")[0]) for l in mem] == [16, 64]   # 256 + 20 is beyond them
    assert all(float(l.split(",")[1]) > 0 for l in mem)



def test_repetition_penalty_through_the_entry_point(tiny_folders, plain_models):
    """With a repetition penalty the greedy continuation is the plain loop's with the same penalty (the last
    `window` tokens of prompt and output lower their logits before every draw); it differs from the
    continuation without one, does not depend on the batch, and a window of 3 differs from one of 32."""
    import turboquant_cpp_b200 as tq
    prompts = prompts_for("A", [5, 11, 17], 44)
    n_new = 10
    with tq.Model(tiny_folders["A"], temperature=0.0, max_tokens=n_new, dtype="float32", max_batch=4,
                  context_length=128, rep_penalty=3.0) as m:
        outs = m.generate_batch(prompts)
        assert [m.ask(p) for p in prompts] == outs
        plain_outs = m.generate_batch(prompts, rep_penalty=1.0)
        short = m.generate_batch(prompts, rep_window=3)
    assert outs != plain_outs and short != outs
    for window, got in ((32, outs), (3, short), (32, plain_outs)):
        pen = 1.0 if got is plain_outs else 3.0
        for p, o in zip(prompts, got):
            want, gaps = greedy_with_margin(plain_models["A"], p, n_new, rep_penalty=pen, rep_window=window)
            for i, (a, b) in enumerate(zip(o, want)):
                if a != b:
                    assert gaps[i] < 1e-5, f"token {i}: engine {a}, plain {b}, gap {gaps[i]:.3e}"
                    break
            else:
                assert o == want
