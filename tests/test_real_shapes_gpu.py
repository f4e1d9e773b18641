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
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=2048)
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
    eng = tq.Engine(tq.load_model(folder, dtype, "cuda:0"), max_tokens=2048)
    rng = np.random.default_rng(6)
    reqs = {"a": rng.integers(0, 512, size=300).tolist(), "b": rng.integers(0, 512, size=70).tolist(),
            "c": rng.integers(0, 512, size=131).tolist()}
    logits, routing = run_schedule(eng, *batched(reqs, {"a": 290, "b": 64, "c": 129}))
    for r, t in reqs.items():
        check_against_plain(plain, t, logits[r], routing[r], dtype, f"wide batch {r}")
    eng.check_kernels()
