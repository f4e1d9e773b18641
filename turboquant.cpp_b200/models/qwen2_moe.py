"""The Qwen2 MoE sparse decoder ("Qwen2MoeForCausalLM") as a list of parts.

Every layer: RMSNorm, attention with QKV bias and rotary encoding (windowed on the layers the
configuration says), RMSNorm, then routed experts with a shared expert on sparse layers or a dense
SwiGLU on the others.  Tensor names are those of safetensors checkpoints of this family; the
reference loads the same tensors under GGUF names (src/engine/tq_model.c:3271-3322 attention and
biases, :3440-3569 router/experts/shared expert, :3570-3581 dense layers, :3705-3769 embedding,
output norm and head)."""
from __future__ import annotations

import torch

from ..config.qwen2_moe import ARCHITECTURE, Qwen2MoeConfig
from ..config.registry import register_architecture
from ..parts import PreNormBlock, make_feed_forward, make_mixer, make_norm, make_position_encoding
from .decoder import DecoderModel, Embedding, LMHead, ScheduleEntry


class Qwen2MoeModel(DecoderModel):
    def __init__(self, cfg: Qwen2MoeConfig, dtype: torch.dtype):
        H = cfg.hidden_size
        rotary = make_position_encoding("rotary", head_dim=cfg.head_dim, theta=cfg.rope_theta,
                                        max_position=cfg.max_position_embeddings, pairing="half")
        blocks = []
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}."
            mixer = make_mixer("attention", prefix=p + "self_attn.", hidden=H, n_heads=cfg.num_attention_heads,
                               n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, qkv_bias=cfg.qkv_bias,
                               window=cfg.layer_window(l), position=rotary)
            if cfg.layer_is_sparse(l):
                ffn = make_feed_forward("moe", prefix=p + "mlp.", hidden=H, n_experts=cfg.num_experts,
                                        top_k=cfg.num_experts_per_tok, intermediate=cfg.moe_intermediate_size,
                                        norm_topk=cfg.norm_topk_prob,
                                        shared_intermediate=cfg.shared_expert_intermediate_size, shared_gate=True)
            else:
                ffn = make_feed_forward("swiglu", prefix=p + "mlp.", hidden=H, intermediate=cfg.intermediate_size)
            blocks.append(PreNormBlock(
                make_norm("rmsnorm", name=p + "input_layernorm.weight", size=H, eps=cfg.rms_norm_eps), mixer,
                make_norm("rmsnorm", name=p + "post_attention_layernorm.weight", size=H, eps=cfg.rms_norm_eps), ffn))
        head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
        super().__init__(
            cfg, dtype,
            embedding=Embedding("model.embed_tokens.weight", cfg.vocab_size, H),
            blocks=blocks,
            schedule=[ScheduleEntry(l) for l in range(cfg.num_hidden_layers)],
            final_norm=make_norm("rmsnorm", name="model.norm.weight", size=H, eps=cfg.rms_norm_eps),
            head=LMHead(head_name, cfg.vocab_size, H))


register_architecture(ARCHITECTURE, Qwen2MoeConfig, Qwen2MoeModel)
