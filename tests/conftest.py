"""Shared fixtures: tiny configurations of the architecture, random model folders, the plain model.

Model folders are written into pytest's temporary folders and never kept.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


# Two tiny configurations that differ in every size and option, and a third with odd sizes
# (a head size that is not hidden/heads, one KV head, no shared expert, a dense layer by sparse step).
TINY_A = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 4,
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 32, "norm_topk_prob": False,
    "shared_expert_intermediate_size": 64, "intermediate_size": 96, "vocab_size": 256, "rope_theta": 10000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 128, "use_sliding_window": False, "sliding_window": 0,
    "max_window_layers": 2, "tie_word_embeddings": False, "decoder_sparse_step": 1, "mlp_only_layers": [],
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 2,
    "num_experts": 6, "num_experts_per_tok": 3, "moe_intermediate_size": 48, "norm_topk_prob": True,
    "shared_expert_intermediate_size": 128, "intermediate_size": 160, "vocab_size": 320, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 256, "use_sliding_window": True, "sliding_window": 32,
    "max_window_layers": 1, "tie_word_embeddings": True, "decoder_sparse_step": 1, "mlp_only_layers": [1],
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY_C = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48,
    "num_experts": 5, "num_experts_per_tok": 1, "moe_intermediate_size": 40, "norm_topk_prob": False,
    "shared_expert_intermediate_size": 0, "intermediate_size": 72, "vocab_size": 257, "rope_theta": 50000.0,
    "rms_norm_eps": 3e-6, "max_position_embeddings": 200, "use_sliding_window": True, "sliding_window": 8,
    "max_window_layers": 0, "tie_word_embeddings": False, "decoder_sparse_step": 2, "mlp_only_layers": [],
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """name -> folder with config.json and model.safetensors (random weights, seeded)."""
    import turboquant_cpp_b200 as tq
    out = {}
    for name, (cfg, seed) in TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        tq.write_random_folder(d, cfg, seed)
        out[name] = d
    return out


@pytest.fixture(scope="session")
def plain_models(tiny_folders):
    from plain.qwen2_moe_plain import PlainModel
    return {n: PlainModel(d) for n, d in tiny_folders.items()}
