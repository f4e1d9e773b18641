"""The engine at head size 128 and widths of the benchmark model's order (one layer, small vocabulary),
where the tensor-core kernels take over: prompt attention on tcgen05 (head 128), router logits of a long
step as a tensor-core product, expert tiles of 128 tokens, packed expert weights — against the plain
implementation, in bfloat16 and in float32, whole and with the last tokens one by one."""
import numpy as np
import pytest

from replay_util import batched, check_against_plain, run_schedule, whole, with_tail

pytestmark = pytest.mark.gpu

WIDE = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 1, "hidden_size": 1024, "num_attention_heads": 8, "num_key_value_heads": 2,
    "num_experts": 12, "num_experts_per_tok": 4, "moe_intermediate_size": 704, "norm_topk_prob": False,
    "shared_expert_intermediate_size": 1408, "intermediate_size": 1408, "vocab_size": 512, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 1024, "use_sliding_window": False, "sliding_window": 0,
    "max_window_layers": 1, "tie_word_embeddings": False, "decoder_sparse_step": 1, "mlp_only_layers": [],
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
WINDOWED = dict(WIDE, num_attention_heads=4, num_key_value_heads=4, head_dim=64, use_sliding_window=True,
                sliding_window=200, max_window_layers=0, num_experts=5, num_experts_per_tok=2, norm_topk_prob=True)


@pytest.fixture(scope="module")
def wide(tmp_path_factory):
    import turboquant_cpp_b200 as tq
    from plain.qwen2_moe_plain import PlainModel
    out = {}
    for name, cfg in (("wide", WIDE), ("windowed", WINDOWED)):
        d = str(tmp_path_factory.mktemp(name))
        tq.write_random_folder(d, cfg, seed=3)
        out[name] = (d, PlainModel(d))
    return out


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["wide", "windowed"])
def test_long_prompt_and_tail(wide, name, dtype):
    import turboquant_cpp_b200 as tq
    folder, plain = wide[name]
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=2048, record_routing=True)
    rng = np.random.default_rng(5)
    toks = rng.integers(0, 512, size=420).tolist()
    logits, routing = run_schedule(eng, *whole("r", toks))                   # one step of 420 tokens
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} whole")
    logits, routing = run_schedule(eng, *with_tail("r", toks, 32))           # 388 tokens, then 32 single ones
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} tail")
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["bfloat16"])
def test_unequal_prompts_in_one_step(wide, dtype):
    import turboquant_cpp_b200 as tq
    folder, plain = wide["wide"]
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=2048, record_routing=True)
    rng = np.random.default_rng(6)
    reqs = {"a": rng.integers(0, 512, size=300).tolist(), "b": rng.integers(0, 512, size=70).tolist(),
            "c": rng.integers(0, 512, size=131).tolist()}
    logits, routing = run_schedule(eng, *batched(reqs, {"a": 290, "b": 64, "c": 129}))
    for r, t in reqs.items():
        check_against_plain(plain, t, logits[r], routing[r], dtype, f"wide batch {r}")
    eng.check_kernels()


def in_pieces(rid, tokens, cuts):
    """The request alone, its tokens cut into steps of the given sizes (the rest one by one), logits everywhere."""
    steps, at = [], 0
    for n in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        steps.append([(rid, list(tokens[at:at + n]), list(range(n)))])
        at += n
    assert at == len(tokens)
    return steps, {len(steps) - 1: [rid]}


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["wide", "windowed"])
def test_a_prompt_in_pieces(wide, name, dtype):
    """A prompt that arrives in pieces long enough for the prompt kernel (48 tokens and more), so that its later
    pieces start in the middle of the sequence, of a page and of a key tile; then two tokens in one step, another
    long piece, and single tokens.  On the windowed model the first pages have been given back by then: their
    entries in the page table are -1 and nothing may read them."""
    import turboquant_cpp_b200 as tq
    folder, plain = wide[name]
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=2048, record_routing=True)
    rng = np.random.default_rng(7)
    toks = rng.integers(0, 512, size=470).tolist()
    steps, ends = in_pieces("r", toks, [260, 130, 2, 70])
    seen_holes = []
    book_close = eng.close

    def close_and_look(seq):                     # what the page lists looked like when the request ended
        seen_holes.append([sum(p is None for p in pages) for pages in seq.pages])
        book_close(seq)
    eng.close = close_and_look
    logits, routing = run_schedule(eng, steps, ends)
    eng.close = book_close
    if name == "windowed":
        assert max(seen_holes[0]) >= 3, f"the window gave no page back: {seen_holes}"
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} pieces")
    logits, routing = run_schedule(eng, *in_pieces("r", toks, [140, 140, 140]))
    check_against_plain(plain, toks, logits["r"], routing["r"], dtype, f"{name} three pieces of 140")
    eng.check_kernels()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["wide", "windowed"])
def test_a_long_piece_beside_single_tokens(wide, name, dtype):
    """One step that mixes a 300-token piece of one sequence with single tokens of two sequences that already
    hold about 500 (the whole step takes the prompt kernel's route)."""
    import turboquant_cpp_b200 as tq
    folder, plain = wide[name]
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=4096, record_routing=True)
    rng = np.random.default_rng(8)
    reqs = {"a": rng.integers(0, 512, size=503).tolist(), "b": rng.integers(0, 512, size=499).tolist(),
            "c": rng.integers(0, 512, size=420).tolist()}
    every = lambda n: list(range(n))
    steps = [[("a", reqs["a"][:500], every(500)), ("b", reqs["b"][:497], every(497)), ("c", reqs["c"][:118], every(118))],
             [("a", reqs["a"][500:501], [0]), ("c", reqs["c"][118:418], every(300)), ("b", reqs["b"][497:498], [0])],
             [("a", reqs["a"][501:502], [0]), ("b", reqs["b"][498:499], [0]), ("c", reqs["c"][418:419], [0])],
             [("a", reqs["a"][502:503], [0]), ("c", reqs["c"][419:420], [0])]]
    logits, routing = run_schedule(eng, steps, {2: ["b"], 3: ["a", "c"]})
    for r, t in reqs.items():
        assert sorted(logits[r]) == list(range(len(t)))
        check_against_plain(plain, t, logits[r], routing[r], dtype, f"{name} mixed step {r}")
    eng.check_kernels()
    eng.cache.book.check_invariants()
