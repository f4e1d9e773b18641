"""Configuration and registry (CPU)."""
import copy
import json

import pytest

import turboquant_cpp_b200 as tq
from turboquant_cpp_b200.config import ConfigError, Qwen2MoeConfig, load_config, parse_config
from conftest import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_tiny_b():
    arch, cfg = parse_config(TINY_B)
    assert arch.name == "Qwen2MoeForCausalLM" and isinstance(cfg, Qwen2MoeConfig)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 192, 6, 2)
    assert cfg.head_dim == 32 and cfg.vocab_size == 320 and cfg.max_position_embeddings == 256
    assert cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5
    assert (cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size) == (6, 3, 48)
    assert cfg.shared_expert_intermediate_size == 128 and cfg.intermediate_size == 160
    assert cfg.norm_topk_prob is True and cfg.tie_word_embeddings is True
    assert [cfg.layer_is_sparse(l) for l in range(3)] == [True, False, True]
    assert [cfg.layer_window(l) for l in range(3)] == [0, 32, 32]


def test_layer_plans_of_a_and_c():
    _, a = parse_config(TINY_A)
    assert all(a.layer_is_sparse(l) for l in range(2)) and all(a.layer_window(l) == 0 for l in range(2))
    _, c = parse_config(TINY_C)
    assert c.head_dim == 48                                   # given, not hidden/heads
    assert [c.layer_is_sparse(l) for l in range(2)] == [False, True]   # decoder_sparse_step = 2
    assert [c.layer_window(l) for l in range(2)] == [8, 8]


def test_round_trip_through_to_dict():
    _, b = parse_config(TINY_B)
    _, again = parse_config(b.to_dict())
    assert again == b


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size", "rope_theta",
                                 "rms_norm_eps", "max_position_embeddings", "num_experts", "num_experts_per_tok",
                                 "moe_intermediate_size", "hidden_act"])
def test_missing_required_key_is_named(key):
    raw = copy.deepcopy(TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        parse_config(raw)


@pytest.mark.parametrize("key,value", [("hidden_size", "64"), ("num_experts_per_tok", 9), ("num_key_value_heads", 3),
                                       ("hidden_act", "gelu"), ("rms_norm_eps", 0), ("norm_topk_prob", 1),
                                       ("mlp_only_layers", [5]), ("vocab_size", 2.5)])
def test_bad_value_is_named(key, value):
    raw = copy.deepcopy(TINY_A)
    raw[key] = value
    with pytest.raises(ConfigError, match=key):
        parse_config(raw)


def test_dense_layers_need_intermediate_size():
    raw = copy.deepcopy(TINY_B)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        parse_config(raw)
    raw = copy.deepcopy(TINY_A)       # every layer sparse: not needed
    del raw["intermediate_size"]
    parse_config(raw)


def test_window_needs_a_size():
    raw = copy.deepcopy(TINY_A)
    raw["use_sliding_window"] = True
    with pytest.raises(ConfigError, match="sliding_window"):
        parse_config(raw)


def test_unknown_architecture_lists_registered():
    raw = copy.deepcopy(TINY_A)
    raw["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError, match="Qwen2MoeForCausalLM"):
        parse_config(raw)
    del raw["architectures"]
    with pytest.raises(ConfigError, match="architectures"):
        parse_config(raw)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_config(str(tmp_path))
    assert cfg.hidden_size == 64
    with pytest.raises(FileNotFoundError):
        load_config(str(tmp_path / "nope"))
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))


def test_registry_accepts_a_new_architecture():
    class C:
        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls()

    class M:
        def __init__(self, cfg, dtype):
            pass

    tq.register_architecture("ToyTestArch", C, M)
    try:
        with pytest.raises(ValueError):
            tq.register_architecture("ToyTestArch", C, M)
        arch, cfg = parse_config({"architectures": ["ToyTestArch"]})
        assert arch.model_class is M and isinstance(cfg, C)
    finally:
        from turboquant_cpp_b200.config import unregister_architecture
        unregister_architecture("ToyTestArch")


def test_sizes_no_kernel_takes_are_refused_when_the_configuration_is_read():
    from turboquant_cpp_b200.config import ConfigError
    from turboquant_cpp_b200.config.qwen2_moe import Qwen2MoeConfig
    from conftest import TINY_A
    for key, value, needle in (("head_dim", 24, "multiple of 16"), ("head_dim", 272, "multiple of 16"),
                               ("num_experts", 5000, "num_experts")):
        raw = dict(TINY_A)
        raw[key] = value
        with pytest.raises(ConfigError, match=needle):
            Qwen2MoeConfig.from_dict(raw, "config.json")
