"""The engine at the layer widths of the two real models of this architecture, against the plain implementation:

  A  Qwen1.5-MoE-A2.7B widths: hidden 2048, 16 heads = 16 KV heads x 128, 60 experts top-4 of 1408, shared
     expert 5632, vocabulary 151,936, two layers;
  B  Qwen2-57B-A14B widths: hidden 3584, 28 heads on 4 KV heads x 128 (7 query heads per KV head), 64 experts
     top-8 of 2560, shared expert 20480, one layer (the vocabulary is cut to 6,000: the LM head at full width is
     covered by A).

Weights are random and seeded, drawn on the GPU and written to a folder that exists for the length of this file's
tests; the plain implementation reads the folder.  Each model is checked whole (a prompt of more than 300 tokens
in one step, so the tensor-core prompt attention, the CTA-pair expert product and the tensor-core router run),
with the last 32 tokens one by one (through the CUDA graphs that generation replays), and in two batches of
unequal lengths one after another, in float32 and in bfloat16.  The third test runs the float32 path on a batch
of 16 prompts of 1 to 2,048 tokens followed by 64 decoded tokens each and checks sampled positions.

Every check prints its worst logit error and the smallest router margin it met (pytest -s shows them)."""
import json
import tempfile

import numpy as np
import pytest

from replay_util import batched, check_against_plain, run_schedule, whole, with_tail

pytestmark = pytest.mark.gpu

COMMON = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe", "norm_topk_prob": False,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "use_sliding_window": False, "sliding_window": 0,
    "tie_word_embeddings": False, "decoder_sparse_step": 1, "mlp_only_layers": [], "hidden_act": "silu",
    "torch_dtype": "bfloat16",
}
WIDTHS = {
    "A": dict(COMMON, num_hidden_layers=2, max_window_layers=2, hidden_size=2048, num_attention_heads=16,
              num_key_value_heads=16, num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408,
              shared_expert_intermediate_size=5632, intermediate_size=5632, vocab_size=151936,
              max_position_embeddings=8192),
    "B": dict(COMMON, num_hidden_layers=1, max_window_layers=1, hidden_size=3584, num_attention_heads=28,
              num_key_value_heads=4, num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560,
              shared_expert_intermediate_size=20480, intermediate_size=20480, vocab_size=6000,
              max_position_embeddings=32768),
}


@pytest.fixture(scope="module")
def folders():
    """name -> (folder, plain model); the folders are deleted when the module's tests are done."""
    import turboquant_cpp_b200 as tq
    from plain.qwen2_moe_plain import PlainModel
    made, out = [], {}

    def get(name):
        if name not in out:
            for other in list(out):            # one model's float64 copy at a time on the host
                del out[other]
            d = tempfile.TemporaryDirectory(prefix=f"tq_widths_{name}_")
            made.append(d)
            tq.write_random_folder(d.name, WIDTHS[name], seed=21, device="cuda:0")
            out[name] = (d.name, PlainModel(d.name))
        return out[name]
    yield get
    out.clear()
    for d in made:
        d.cleanup()


def sampled(n, every=9, tail=6):
    """Positions whose logits are compared: every few, and the last ones (the LM head is wide)."""
    return set(range(0, n, every)) | set(range(max(0, n - tail), n))


def three_schedules(folders, name, dtype):
    import torch
    import turboquant_cpp_b200 as tq
    folder, plain = folders(name)
    V = WIDTHS[name]["vocab_size"]
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=4096, record_routing=True)
    rng = np.random.default_rng(31)
    report = {}
    toks = rng.integers(0, V, size=330).tolist()
    keep = sampled(len(toks)) | set(range(298, 330))
    logits, routing = run_schedule(eng, *whole("r", toks, keep))                      # one step of 330 tokens
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} whole", report)
    logits, routing = run_schedule(eng, *with_tail("r", toks, 32, keep))              # 298 tokens, then 32 single ones
    assert eng.graphs.graphs and eng.graphs.replays > 0, "the decoded tail did not run as CUDA graphs"
    assert set(logits["r"]) == {p for p in keep if p < 298} | set(range(298, 330))
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} tail", report)
    # two batches of unequal lengths, one after the other on the same engine (slots and pages come back)
    free_before = [p.n_free for p in eng.cache.book.pools]
    for lens, seed in (({"a": (140, 6), "b": (9, 3), "c": (66, 6)}, 41), ({"d": (1, 5), "e": (51, 2)}, 43)):
        r2 = np.random.default_rng(seed)
        reqs = {r: r2.integers(0, V, size=p + d).tolist() for r, (p, d) in lens.items()}
        logits, routing = run_schedule(eng, *batched(reqs, {r: lens[r][0] for r in lens}, sampled(140, 13, 3)))
        for r, t in reqs.items():
            check_against_plain(plain, t, logits[r], routing[r], dtype, f"{name} batch {r}", report)
        eng.cache.book.check_invariants()
        assert [p.n_free for p in eng.cache.book.pools] == free_before
    eng.check_kernels()
    print(f"\n[{name} {dtype}] worst logit error {report['worst']:.2e} of scale; smallest router margin "
          f"{report['margin']:.2e}; expert choices that fell the other way {report['flips']}")
    eng.release()
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_schedules_at_the_widths_of_a2_7b(folders, dtype):
    three_schedules(folders, "A", dtype)


def test_float32_batch_of_16_unequal_prompts_then_64_tokens(folders):
    """Batch 16, prompt lengths uniform in [1, 2048] (seed 3), then 64 more tokens each, in float32, at A's
    widths with 2 of its 24 layers: the prompts in one step, then one token each through the CUDA graphs.
    Three of the requests (the shortest, the longest and one between) are compared with the plain implementation
    at sampled positions of their prompts and at every decoded position; one of them is then replayed alone,
    whole and with its tail one by one, against the same plain result."""
    import torch
    import turboquant_cpp_b200 as tq
    folder, plain = folders("A")
    V = WIDTHS["A"]["vocab_size"]
    rng = np.random.default_rng(3)
    prompt_lens = rng.integers(1, 2049, size=16).tolist()
    reqs = {f"r{i}": rng.integers(0, V, size=n + 64).tolist() for i, n in enumerate(prompt_lens)}
    lens = {f"r{i}": n for i, n in enumerate(prompt_lens)}
    order = sorted(lens, key=lambda r: lens[r])
    checked = [order[0], order[len(order) // 2], order[-1]]
    need = sum(-(-len(t) // 64) * 64 for t in reqs.values())
    eng = tq.Engine(tq.load_model(folder, "float32", "cuda:0"), max_tokens=need, max_slots=16, record_routing=True)
    keep = sampled(2048, 97, 2)
    logits, routing = run_schedule(eng, *batched(reqs, lens, keep))
    assert eng.graphs.replays >= 60
    report = {}
    for r in checked:
        assert set(range(lens[r], lens[r] + 64)) <= set(logits[r])
        check_against_plain(plain, reqs[r], logits[r], routing[r], "float32", f"batch of 16, {r} ({lens[r]} + 64)", report)
    eng.cache.book.check_invariants()
    mid = checked[1]
    alone, routing = run_schedule(eng, *whole(mid, reqs[mid], set(logits[mid])))
    check_against_plain(plain, reqs[mid], alone[mid], routing[mid], "float32", f"{mid} alone", report)
    tail, routing = run_schedule(eng, *with_tail(mid, reqs[mid], 32, set(logits[mid])))
    check_against_plain(plain, reqs[mid], tail[mid], routing[mid], "float32", f"{mid} tail", report)
    print(f"\n[float32 batch of 16, prompts {sorted(prompt_lens)}] worst logit error {report['worst']:.2e} of scale; "
          f"smallest router margin {report['margin']:.2e}; flips {report['flips']}")
    eng.release()
    del eng
    torch.cuda.empty_cache()


def test_a_prompt_of_900_tokens_in_bfloat16_with_both_experts_products_in_one_launch(folders):
    """At 900 tokens the routed experts' tiles are wide enough for pairs of CTAs and the shared expert's product has
    few rounds of tiles: its tiles ride in the routed experts' launches (one launch for both gate/up products,
    one for both down projections).  Whole, and in two pieces of 600 and 300 tokens (the second piece runs the
    launches of their own), against the plain implementation."""
    import torch
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.kernels import gemm_tc as KT
    folder, plain = folders("A")
    V = WIDTHS["A"]["vocab_size"]
    eng = tq.Engine(tq.load_model(folder, "bfloat16", "cuda:0"), max_tokens=1024, record_routing=True)
    toks = np.random.default_rng(77).integers(0, V, size=900).tolist()
    keep = sampled(len(toks), 31, 4)
    before = KT.DUAL_CALLS
    logits, routing = run_schedule(eng, *whole("r", toks, keep))
    assert KT.DUAL_CALLS == before + 2 * WIDTHS["A"]["num_hidden_layers"], "the step did not take the two-product launches"
    report = {}
    check_against_plain(plain, toks, logits["r"], routing["r"], "bfloat16", "A 900 whole", report)
    steps = [[("r", toks[:600], sorted(p for p in keep if p < 600))],
             [("r", toks[600:], sorted(p - 600 for p in keep if p >= 600))]]
    pieces, routing = run_schedule(eng, steps, {1: ["r"]})
    check_against_plain(plain, toks, pieces["r"], routing["r"], "bfloat16", "A 900 in pieces", report)
    eng.check_kernels()
    print(f"\n[A bfloat16, 900 tokens] worst logit error {report['worst']:.2e} of scale; smallest router margin "
          f"{report['margin']:.2e}; flips {report['flips']}")
    eng.release()
    del eng
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_three_schedules_at_the_widths_of_57b_a14b(folders, dtype):
    three_schedules(folders, "B", dtype)
