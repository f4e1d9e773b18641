"""Weights: the container, the by-name plan with its one error, random folders (CPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import turboquant_cpp_b200 as tq
from turboquant_cpp_b200.weights import (SafetensorsError, SafetensorsFile, SafetensorsSource, WeightError, WeightSpec,
                                         WeightStore, check_plan, kept_dtype, save_file, RandomSource)
from conftest import TINY_A, TINY_B


def test_container_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2, 2),
         "e": torch.empty(0, 4)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.entries) == set(t)
    for n in t:
        assert torch.equal(f.read(n), t[n])
    f.close()
    # the same bytes as the reference library of the format writes
    from safetensors.torch import load_file
    back = load_file(p)
    for n in t:
        assert torch.equal(back[n], t[n])


def test_truncated_and_corrupt_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    save_file({"a": torch.randn(64, 64)}, p)
    blob = open(p, "rb").read()
    open(p, "wb").write(blob[:-100])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(blob[:5])
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10 ** 9) + blob[8:])
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"nope" + blob[12:])
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    plan = [WeightSpec("a", (2, 3)), WeightSpec("b", (4,)), WeightSpec("c", (5, 5)), WeightSpec("t", (3,), integer=True)]
    index = {"a": (torch.bfloat16, (2, 3)), "c": (torch.bfloat16, (5, 6)), "x": (torch.float32, (1,)),
             "t": (torch.float32, (3,))}
    with pytest.raises(WeightError) as e:
        check_plan(index, plan, "folder")
    err = e.value
    assert err.missing == ["b"] and err.unexpected == ["x"]
    assert err.wrong_shape == [("c", (5, 5), (5, 6))] and err.wrong_dtype[0][0] == "t"
    msg = str(err)
    for needle in ("folder", "missing", "b [4]", "unexpected", "x [1]", "wrong shape", "c: expected [5, 5], found [5, 6]"):
        assert needle in msg
    check_plan({"a": (torch.float32, (2, 3))}, [WeightSpec("a", (2, 3))])


def test_kept_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert kept_dtype(torch.bfloat16, bf) == bf and kept_dtype(torch.float16, bf) == bf
    assert kept_dtype(torch.float32, bf) == f32          # a tensor stored in 32-bit stays so
    assert kept_dtype(torch.int64, bf) == torch.int32 and kept_dtype(torch.int32, f32) == torch.int32
    assert kept_dtype(torch.bfloat16, f32) == f32 and kept_dtype(torch.float16, f32) == f32


def test_random_folder_is_seeded_and_complete(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    tq.write_random_folder(a, TINY_B, seed=1)
    tq.write_random_folder(b, TINY_B, seed=1)
    tq.write_random_folder(c, TINY_B, seed=2)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert fa.entries == fb.entries == fc.entries
    assert "lm_head.weight" not in fa.entries                      # tied
    assert fa.entries["model.layers.1.mlp.gate_proj.weight"] == ("BF16", (160, 192))      # the dense layer
    assert fa.entries["model.layers.0.mlp.experts.5.down_proj.weight"] == ("BF16", (192, 48))
    assert fa.entries["model.layers.2.mlp.shared_expert_gate.weight"] == ("BF16", (1, 192))
    assert fa.entries["model.layers.0.self_attn.k_proj.bias"] == ("BF16", (64,))
    n = "model.layers.0.self_attn.q_proj.weight"
    assert torch.equal(fa.read(n), fb.read(n)) and not torch.equal(fa.read(n), fc.read(n))
    w = fa.read(n).float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    g = fa.read("model.norm.weight").float()
    assert abs(g.mean().item() - 1.0) < 0.01                       # norm weights are 1 + N(0, std)
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["Qwen2MoeForCausalLM"] and cfg["sliding_window"] == 32


def test_store_checks_the_folder_against_the_model(tmp_path):
    d = str(tmp_path / "m")
    tq.write_random_folder(d, TINY_A, seed=0)
    model = tq.build_model(TINY_A, "float32")
    src = SafetensorsSource(d)
    store = WeightStore(src, model.weight_specs(), "cpu", torch.float32)
    t = store.get("model.embed_tokens.weight")
    assert t.dtype == torch.float32 and store.get("model.embed_tokens.weight") is t
    src.close()
    # the same folder does not fit another configuration: everything wrong is listed at once
    other = tq.build_model(TINY_B, "float32")
    src = SafetensorsSource(d)
    with pytest.raises(WeightError) as e:
        WeightStore(src, other.weight_specs(), "cpu", torch.float32, where=d)
    assert e.value.missing and e.value.unexpected and e.value.wrong_shape
    assert "lm_head.weight" in e.value.unexpected
    src.close()


def test_fp32_stored_tensors_stay_fp32_in_a_bfloat16_run():
    specs = [WeightSpec("r", (4, 8)), WeightSpec("m", (4, 8))]
    src = RandomSource(specs, 3, fp32_names=["r"])
    store = WeightStore(src, specs, "cpu", torch.bfloat16)
    assert store.get("r").dtype == torch.float32 and store.get("m").dtype == torch.bfloat16


def test_random_values_are_a_pure_function_of_seed_name_and_index():
    """An element's value does not depend on how the tensor is cut or where it is drawn: recomputed here with
    plain Python integers and numpy float32 from the documented recipe."""
    from turboquant_cpp_b200.weights.random_init import _tensor_key, normal_knots, standard_normal
    left, width = (t.numpy() for t in normal_knots("cpu"))
    assert np.all(width > 0) and left[32768] == 0.0 and np.allclose(left[1:32768], -(left + width)[65534:32767:-1], atol=1e-6)
    M = (1 << 64) - 1
    key = _tensor_key(7, "some.tensor")

    def element(i):
        z = (key + (i + 1) * 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z ^= z >> 31
        j, frac = (z >> 48) & 0xFFFF, np.float32(((z >> 24) & 0xFFFFFF) / float(1 << 24))
        return np.float32(left[j] + np.float32(frac * width[j]))
    whole = standard_normal(key, 0, 5000, "cpu").numpy()
    for i in (0, 1, 2, 77, 4999):
        assert whole[i] == element(i)
    piece = standard_normal(key, 4000, 1000, "cpu").numpy()
    assert np.array_equal(piece, whole[4000:])
    far = standard_normal(key, (1 << 35) + 3, 2, "cpu").numpy()           # indices beyond 32 bits
    assert far[0] == element((1 << 35) + 3) and far[1] == element((1 << 35) + 4)
    # through the source: the tensor is the stream of its name, scaled, rounded to the stored dtype
    spec = WeightSpec("some.tensor", (50, 100))
    t = RandomSource([spec], 7, std=0.5, dtype=torch.float32).read("some.tensor", "cpu").numpy()
    assert np.array_equal(t.reshape(-1), whole * np.float32(0.5))
    big = standard_normal(key, 0, 1 << 20, "cpu")
    assert abs(big.mean().item()) < 5e-3 and abs(big.std().item() - 1.0) < 5e-3
    assert abs(((big - big.mean()) ** 4).mean().item() / big.var().item() ** 2 - 3.0) < 0.05     # normal, not uniform sums
