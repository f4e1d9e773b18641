"""Attention mixer: fused QKV projection with bias, position encoding, cache write, attention over
the paged cache (grouped-query, causal, optional window), output projection.

Order of the reference (src/engine/tq_transformer.c): projections :1027-1083, biases :1044-1047
and :1086-1093, rotary :1343, cache write :1371 and :1452-1455, scores/softmax/PV :1909-2191 with
head h reading KV head h/(nh/nkv) :1679 and scale 1/sqrt(hd) :1633, output projection :2231-2240.
The window (a query sees the last `window` positions, itself included) follows the mask of the
reference's Gemma branch :1646-1654."""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..kernels import attention as KA
from ..kernels import elementwise as KE
from ..kernels import gemv as KG
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import KVNeed, LayerCache, Mixer, PositionEncoding, StepContext, register_mixer


class AttentionMixer(Mixer):
    PREFILL_MIN_RUN = 48      # steps whose longest run of new tokens is at least this use the prompt kernel

    def __init__(self, prefix: str, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 qkv_bias: bool, window: int = 0, position: Optional[PositionEncoding] = None,
                 scale: Optional[float] = None):
        if n_heads < 1 or n_kv_heads < 1 or n_heads % n_kv_heads:
            raise ValueError(f"attention '{prefix}': {n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        KA.check_head_dim(head_dim)
        if window < 0:
            raise ValueError(f"attention '{prefix}': negative window {window}")
        self.prefix, self.hidden = prefix, int(hidden)
        self.n_heads, self.n_kv_heads, self.head_dim = int(n_heads), int(n_kv_heads), int(head_dim)
        self.qkv_bias, self.window, self.position = bool(qkv_bias), int(window), position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size, self.kv_size = n_heads * head_dim, n_kv_heads * head_dim
        self.w_qkv = self.b_qkv = self.w_o = None

    def weight_specs(self) -> List[WeightSpec]:
        p, H = self.prefix, self.hidden
        specs = [WeightSpec(p + "q_proj.weight", (self.q_size, H)), WeightSpec(p + "k_proj.weight", (self.kv_size, H)),
                 WeightSpec(p + "v_proj.weight", (self.kv_size, H)), WeightSpec(p + "o_proj.weight", (H, self.q_size))]
        if self.qkv_bias:
            specs += [WeightSpec(p + "q_proj.bias", (self.q_size,)), WeightSpec(p + "k_proj.bias", (self.kv_size,)),
                      WeightSpec(p + "v_proj.bias", (self.kv_size,))]
        return specs

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        ws = [store.take(p + n + "_proj.weight") for n in "qkv"]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_qkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()      # one product for q, k and v
        if self.qkv_bias:
            bs = [store.take(p + n + "_proj.bias") for n in "qkv"]
            bdt = torch.float32 if any(b.dtype == torch.float32 for b in bs) else bs[0].dtype
            self.b_qkv = torch.cat([b.to(bdt) for b in bs], dim=0).contiguous()
        self.w_o = store.get(p + "o_proj.weight")
        if self.position is not None:
            self.position.prepare(store.device)

    def kernels(self) -> List[str]:
        names = ["attention", "elementwise"]
        if getattr(self, "run_dtype", None) == torch.bfloat16:
            names.append("gemv")
        if getattr(self, "run_dtype", None) == torch.bfloat16 and self.head_dim in (64, 128):
            names.append("attention_prefill")
        return names

    def cache_need(self) -> KVNeed:
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        proj = self.hidden * (self.q_size + 2 * self.kv_size) + self.q_size * self.hidden
        kv_el = 2 if getattr(self, "run_dtype", None) == torch.bfloat16 else 4
        seen = min(kv_tokens, n_tokens * self.window) if self.window else kv_tokens
        return {"matmul": (wb(self.w_qkv) + wb(self.w_o), 2.0 * n_tokens * proj),
                "attn": (2.0 * self.kv_size * kv_el * seen, 4.0 * self.q_size * seen)}

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = xn.shape[0]
        act = ctx.act_dtype
        q = torch.empty((T, self.n_heads, self.head_dim), dtype=act, device=xn.device)
        tables = self.position.tables() if self.position is not None else None
        fused = (KG.fused_pays(xn, self.w_qkv) and (self.position is None or (tables is not None and tables[2] == "half"))
                 and (cache.kv is None or cache.kv.dtype == torch.bfloat16))
        if fused:
            # one or two tokens: the projection is a stream of its weights; bias, rotation and the cache write
            # ride on the same launch instead of a library product and a kernel behind it
            cos, sin = (tables[0], tables[1]) if tables is not None else (None, None)
            KG.qkv_gemv_rope(xn, self.w_qkv, self.b_qkv, cos, sin, ctx.positions, ctx.seq_of_token, cache.page_table,
                             cache.page_size, q, cache.kv if cache.writes else None, self.n_heads, self.n_kv_heads,
                             self.head_dim)
            return self._attend(q, T, act, ctx, cache)
        qkv = linear(xn, self.w_qkv, out_dtype=act)
        bias = self.b_qkv
        if self.position is not None and tables is None:
            # an encoding that is not a table-driven rotation: the bias first, then the encoding's own pass over
            # the projection's queries and keys in place, then the fused kernel only splits and writes the cache
            if bias is not None:
                KE.add_bias(qkv, bias)
                bias = None
            rows = qkv.view(T, self.n_heads + 2 * self.n_kv_heads, self.head_dim)
            self.position.apply(rows[:, :self.n_heads], rows[:, self.n_heads:self.n_heads + self.n_kv_heads], ctx.positions)
        cos, sin, pairing = tables if tables is not None else (None, None, "half")
        KA.qkv_rope_cache(qkv, bias, cos, sin, pairing, ctx.positions, ctx.seq_of_token, cache.page_table,
                          cache.page_size, q, cache.kv if cache.writes else None,
                          self.n_heads, self.n_kv_heads, self.head_dim)
        return self._attend(q, T, act, ctx, cache)

    def _attend(self, q: torch.Tensor, T: int, act: torch.dtype, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """Attention of the step's queries over the cache (the step's keys and values are in it), then the output
        projection."""
        xn = q
        o = torch.empty((T, self.q_size), dtype=act, device=xn.device)
        if ctx.max_q_len >= self.PREFILL_MIN_RUN and KA.prefill_usable(act, self.head_dim, cache.page_size):
            # long runs of new tokens (prompts): tensor cores
            KA.attention_prefill(q, cache.kv, ctx.cu_seqlens, ctx.seq_start, cache.page_table, cache.page_size,
                                 self.window, self.scale, o, ctx.n_seqs, ctx.max_q_len, self.n_heads, self.n_kv_heads,
                                 self.head_dim, status=ctx.status)
        elif ctx.max_q_len >= self.PREFILL_MIN_RUN and self.head_dim % 4 == 0:
            # long runs where the tensor-core kernel does not apply (float32, other head sizes): exact fp32 on CUDA
            # cores, 32 queries sharing each tile of keys
            KA.attention_tiled(q, cache.kv, ctx.cu_seqlens, ctx.seq_start, cache.page_table, cache.page_size,
                               self.window, self.scale, o, ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim)
        elif KA.split_usable(self.n_heads, self.n_kv_heads, self.head_dim, cache.page_size):
            n_splits = KA.splits_for(T, self.n_kv_heads * KA.head_chunks(self.n_heads, self.n_kv_heads),
                                     KA.split_resident(act, self.n_heads, self.n_kv_heads, self.head_dim, xn.device))
            if KA.gqa_mma_usable(act, self.n_heads, self.n_kv_heads, self.head_dim):
                n_splits = min(n_splits, KA.GQA_MAX_SPLITS)
            partial = torch.empty(T * self.n_heads * n_splits * (self.head_dim + 2), dtype=torch.float32,
                                  device=xn.device) if n_splits > 1 else None
            KA.attention_split(q, cache.kv, ctx.positions, ctx.seq_of_token, cache.page_table, cache.page_size,
                               self.window, self.scale, o, self.n_heads, self.n_kv_heads, self.head_dim, n_splits, partial,
                               early_keys=KA.EARLY_KEYS and ctx.max_q_len == 1)
        else:
            KA.attention(q, cache.kv, ctx.positions, ctx.seq_of_token, cache.page_table, cache.page_size,
                         self.window, self.scale, o, self.n_heads, self.n_kv_heads, self.head_dim)
        if KG.pays(o, self.w_o):
            return KG.gemv(o, self.w_o, torch.empty((T, self.hidden), dtype=torch.float32, device=o.device))
        return linear(o, self.w_o, out_dtype=torch.float32)


register_mixer("attention", AttentionMixer)
