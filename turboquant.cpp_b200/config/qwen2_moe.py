"""Typed configuration of the Qwen2 MoE sparse decoder ("Qwen2MoeForCausalLM").

Every size and constant of the model comes from the architecture's own
config.json keys; nothing that config.json gives is repeated in code.

The reference carries the same knobs in one flat struct for all its model
families (include/turboquant/tq_engine.h:15-77) plus a MoE side struct
(include/turboquant/tq_gguf.h:220-228), filled from GGUF metadata
(src/engine/tq_model.c:2867-2905, 3000-3029).  Its ``norm_topk_prob`` field
is never read (always renormalised, src/engine/tq_moe.c:600-682) and it has
no per-layer window for this family (src/engine/tq_transformer.c:1646-1654
is Gemma only); both are honoured here.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Any, Dict, List, Tuple

from .reader import ConfigError, KeyReader

ARCHITECTURE = "Qwen2MoeForCausalLM"
# limits of the kernels this architecture's parts launch, checked when the configuration is read so that a model
# that cannot run is refused before its weights are loaded (csrc/attention.cu TQ_MAX_HEAD_DIM, csrc/moe.cu
# ROUTER_MAX_EXPERTS)
MAX_HEAD_DIM = 256
MAX_EXPERTS = 4096


@dataclass(frozen=True)
class Qwen2MoeConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    hidden_act: str
    intermediate_size: int                  # dense feed-forward width (non-sparse layers)
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int    # 0: no shared expert
    norm_topk_prob: bool
    decoder_sparse_step: int
    mlp_only_layers: Tuple[int, ...]
    use_sliding_window: bool
    sliding_window: int
    max_window_layers: int
    tie_word_embeddings: bool
    qkv_bias: bool
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    architecture: str = ARCHITECTURE

    # ---- derived, layer by layer ------------------------------------------------
    def layer_is_sparse(self, layer: int) -> bool:
        """A layer has routed experts unless it is listed in mlp_only_layers or
        falls between sparse steps."""
        return (layer not in self.mlp_only_layers and self.num_experts > 0
                and (layer + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, layer: int) -> int:
        """Number of positions a query of this layer sees (itself included); 0 = all."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    # ---- reading ----------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "Qwen2MoeConfig":
        r = KeyReader(raw, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        if r.has("head_dim"):
            head_dim = r.integer("head_dim", minimum=1)
        else:
            if hidden % heads:
                raise ConfigError(f"{where}: 'hidden_size' ({hidden}) is not a multiple of "
                                  f"'num_attention_heads' ({heads}) and no 'head_dim' is given")
            head_dim = hidden // heads
        if heads % kv_heads:
            raise ConfigError(f"{where}: 'num_attention_heads' ({heads}) is not a multiple of "
                              f"'num_key_value_heads' ({kv_heads})")
        if head_dim % 16 or not 16 <= head_dim <= MAX_HEAD_DIM:
            raise ConfigError(f"{where}: 'head_dim' ({head_dim}) must be a multiple of 16 between 16 and "
                              f"{MAX_HEAD_DIM}: the attention kernels take no other head size")
        layers = r.integer("num_hidden_layers", minimum=1)
        act = r.string("hidden_act")
        if act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' must be 'silu' for this architecture, got '{act}'")
        n_experts = r.integer("num_experts", minimum=0)
        if n_experts > 0:
            top_k = r.integer("num_experts_per_tok", minimum=1)
        else:
            top_k = r.integer("num_experts_per_tok", default=0, minimum=0)
        if n_experts > MAX_EXPERTS:
            raise ConfigError(f"{where}: 'num_experts' ({n_experts}) exceeds the {MAX_EXPERTS} experts the router "
                              f"kernels take")
        if n_experts > 0 and not (1 <= top_k <= n_experts):
            raise ConfigError(f"{where}: 'num_experts_per_tok' ({top_k}) must be in 1..num_experts ({n_experts})")
        moe_inter = r.integer("moe_intermediate_size", minimum=1) if n_experts > 0 else \
            r.integer("moe_intermediate_size", default=0, minimum=0)
        shared = r.integer("shared_expert_intermediate_size", default=0, minimum=0)
        sparse_step = r.integer("decoder_sparse_step", default=1, minimum=1)
        mlp_only = tuple(r.int_list("mlp_only_layers", default=[]))
        for l in mlp_only:
            if not 0 <= l < layers:
                raise ConfigError(f"{where}: 'mlp_only_layers' names layer {l}, but there are {layers} layers")
        use_win = r.boolean("use_sliding_window", default=False)
        window = r.integer("sliding_window", default=0, minimum=0)
        max_win_layers = r.integer("max_window_layers", default=layers, minimum=0)
        if use_win and window < 1:
            raise ConfigError(f"{where}: 'use_sliding_window' is true but 'sliding_window' is {window}")
        cfg = cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            rope_theta=r.real("rope_theta", positive=True),
            rms_norm_eps=r.real("rms_norm_eps", positive=True),
            hidden_act=act,
            intermediate_size=0,
            num_experts=n_experts,
            num_experts_per_tok=top_k,
            moe_intermediate_size=moe_inter,
            shared_expert_intermediate_size=shared,
            norm_topk_prob=r.boolean("norm_topk_prob", default=False),
            decoder_sparse_step=sparse_step,
            mlp_only_layers=mlp_only,
            use_sliding_window=use_win,
            sliding_window=window,
            max_window_layers=max_win_layers,
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            qkv_bias=r.boolean("qkv_bias", default=True),
            eos_token_ids=tuple(r.token_ids("eos_token_id")),
            torch_dtype=r.string("torch_dtype", default="bfloat16"),
            architecture=ARCHITECTURE,
        )
        has_dense = any(not cfg.layer_is_sparse(l) for l in range(layers))
        dense = r.integer("intermediate_size", minimum=1) if has_dense else \
            r.integer("intermediate_size", default=0, minimum=0)
        object.__setattr__(cfg, "intermediate_size", dense)
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.pop("architecture")
        eos = d.pop("eos_token_ids")
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2_moe"
        if eos:
            d["eos_token_id"] = list(eos) if len(eos) > 1 else eos[0]
        return d
