"""The engine against the plain implementation on the GPU: whole requests, the last tokens one by
one, batches of unequal lengths with slots used again — in float32 and in bfloat16."""
import numpy as np
import pytest
import torch

from conftest import TINY
from plain.qwen2_moe_plain import forward as plain_forward, round_bf16, no_round

pytestmark = pytest.mark.gpu

# Tolerances, fixed from the arithmetic and not from what passes:
#  float32: the engine sums in fp32 in another order than the float64 plain model; logits are O(1),
#           sums run over <= a few hundred terms -> a few 1e-6 absolute at most.
#  bfloat16: the plain model rounds activations to bfloat16 where the engine stores them, so what
#           remains is fp32 summation order plus occasional 1-ulp flips of a bfloat16 value
#           (2^-8 relative) that spread through later layers: a few 1e-3 of the logits' scale.
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(1e-30, np.abs(b).max()))


@pytest.fixture(scope="module")
def engines(tiny_folders):
    import turboquant_cpp_b200 as tq
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            model = tq.load_model(tiny_folders[name], dtype, "cuda:0")
            cache[(name, dtype)] = tq.Engine(model, max_tokens=2048)
        return cache[(name, dtype)]
    return get


def tokens_for(name, n, seed):
    V = TINY[name][0]["vocab_size"]
    return np.random.default_rng(seed).integers(0, V, size=n).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_request(engines, plain_models, name, dtype):
    import turboquant_cpp_b200 as tq
    eng = engines(name, dtype)
    n = min(100, TINY[name][0]["max_position_embeddings"])
    toks = tokens_for(name, n, 10)
    seq = eng.open()
    logits = eng.step([tq.StepEntry(seq, toks, list(range(n)))]).cpu().numpy()
    eng.close(seq)
    ref = plain_forward(plain_models[name], toks, rnd=round_bf16 if dtype == "bfloat16" else no_round)
    assert logits.shape == ref.shape
    assert rel_err(logits, ref) < TOL[dtype]
