"""bench.py's arithmetic and the parts of its contract that need no GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_byte_and_flop_counts_of_the_headline_model():
    """Counted by hand for the Qwen1.5-MoE-A2.7B sizes: 24 layers, hidden 2048, 16 x 128 heads, 60 experts of 1408
    (top-4), a shared expert of 5632, vocabulary 151,936."""
    _, cfg = bench.MODELS["a2.7b"]
    n = bench.model_numbers(cfg, 24)
    assert n["expert"] == 3 * 2048 * 1408                               # gate, up, down of one expert: 8.65 M weights
    assert n["attn"] == 4 * 2048 * 2048 + 3 * 2048                      # q, k, v, o and the three biases
    assert n["shared"] == 3 * 2048 * 5632 + 2048 and n["router"] == 60 * 2048
    assert n["kv_per_token"] == 24 * 2 * 16 * 128                       # values per cached token: 192 Ki bytes in bfloat16
    # a decode step of 8 sequences with 25 distinct experts in every layer and 16,500 cached tokens: 16.6 GB
    by = bench.decode_bytes(n, [25] * 24, 8, 16500)
    weights = 24 * (n["attn"] + n["shared"] + n["router"] + n["norms"]) + 24 * 25 * n["expert"] + n["head"]
    assert abs(by - (2 * weights + 16500 * n["kv_per_token"] * 2)) < 1e6
    assert 16.0e9 < by < 17.2e9
    assert bench.decode_bytes(n, [25] * 24, 8, 16500, el=4) == 2 * by   # float32: every byte twice
    # a prompt of 2,048 tokens: 8.9 TFLOP (the products of 4 experts and the shared one per token, causal attention)
    fl = bench.prefill_flops(n, 2048)
    assert 8.7e12 < fl < 9.0e12
    _, big = bench.MODELS["57b"]
    nb = bench.model_numbers(big, 28)
    assert nb["expert"] == 3 * 3584 * 2560 and nb["kv_per_token"] == 28 * 2 * 4 * 128


def run_bench(*args):
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    return p.returncode, lines


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_2():
    rc, lines = run_bench("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 2 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["n_gpus"] == 2 and "one GPU" in d["error"]


def test_the_reference_arm_says_why_it_is_unavailable():
    rc, lines = run_bench("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert rc == 0 and len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and len(d["unavailable"]) > 20 and "\n" not in d["unavailable"]


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    pk = bench.peaks()
    assert pk["source"] in ("measured", "fallback") and pk["hbm_gbs"] > 1000 and pk["bf16_tflops"] > 100
    if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")):
        assert pk["source"] == "measured"
        assert pk["hbm_gbs"] == json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
