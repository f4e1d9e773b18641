"""A decoder put together from parts: embedding, a list of blocks, the order in which they run,
a final norm and an LM head.  Architectures subclass it and only say which parts they have.

The order of the layers is data: ``schedule`` is a list of entries, each naming a block; a block
may be named twice (it then runs twice, each run with a cache of its own), and an entry may read
the cache another entry wrote (``cache_of``) instead of keeping one.

Forward of the reference for one token (src/engine/tq_transformer.c:2281-3029): embedding row
:2298-2329, layers :2410-2830, final norm :2922, logits :2931-2942 — here for all tokens of a
step, with the LM head on the wanted rows only (the reference's multi-token path computes the
last row only, :3571-3587)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import elementwise as K
from ..kernels.linear import linear
from ..parts.base import Block, KVNeed, LayerCache, Norm, Part, StateNeed, StepContext
from ..weights.loader import WeightSpec, WeightStore


@dataclass(frozen=True)
class ScheduleEntry:
    block: int                       # index into the model's blocks
    cache_of: Optional[int] = None   # index of the schedule entry whose cache this entry reads


class Embedding(Part):
    """x = table[token], no scaling (src/engine/tq_transformer.c:2298-2329)."""

    def __init__(self, name: str, vocab: int, hidden: int):
        self.name, self.vocab, self.hidden = name, int(vocab), int(hidden)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store: WeightStore) -> None:
        self.table = store.get(self.name)

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        x = torch.empty((tokens.shape[0], self.hidden), dtype=torch.float32, device=tokens.device)
        return K.embed_rows(tokens, self.table, x)


class LMHead(Part):
    """logits = W x in float32; ``name`` may be the embedding's tensor (tied weights:
    src/engine/tq_model.c:1499-1516)."""

    def __init__(self, name: str, vocab: int, hidden: int):
        self.name, self.vocab, self.hidden = name, int(vocab), int(hidden)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store: WeightStore) -> None:
        self.weight = store.get(self.name)

    def forward(self, xn: torch.Tensor) -> torch.Tensor:
        return linear(xn, self.weight, out_dtype=torch.float32)

    def step_work(self, n_tokens, kv_tokens):
        w = self.weight
        return {"matmul": (0 if w is None else w.numel() * w.element_size(), 2.0 * n_tokens * self.vocab * self.hidden)}


class DecoderModel:
    def __init__(self, config, dtype: torch.dtype, embedding: Embedding, blocks: Sequence[Block],
                 schedule: Sequence[ScheduleEntry], final_norm: Norm, head: LMHead):
        self.config, self.dtype = config, dtype
        self.embedding, self.blocks, self.schedule = embedding, list(blocks), list(schedule)
        self.final_norm, self.head = final_norm, head
        for part in self.parts():            # parts may ask which dtype the run keeps activations in
            for sub in (part.parts() if hasattr(part, "parts") else [part]):
                sub.run_dtype = dtype
        for i, e in enumerate(self.schedule):
            if not 0 <= e.block < len(self.blocks):
                raise ValueError(f"schedule entry {i} names block {e.block}, but there are {len(self.blocks)} blocks")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_of}, which keeps none of its own")
                a, b = self.blocks[e.block].cache_need(), self.blocks[self.schedule[e.cache_of].block].cache_need()
                if a is None or b is None or (a.n_kv_heads, a.head_dim) != (b.n_kv_heads, b.head_dim):
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {e.cache_of}: different shapes")

    # ---- sizes the engine asks for -----------------------------------------------------------
    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    @property
    def max_position(self) -> int:
        return int(self.config.max_position_embeddings)

    def parts(self) -> List[Part]:
        return [self.embedding] + self.blocks + [self.final_norm, self.head]

    def weight_specs(self) -> List[WeightSpec]:
        seen: Dict[str, WeightSpec] = {}
        for p in self.parts():
            for s in p.weight_specs():
                if s.name in seen and tuple(seen[s.name].shape) != tuple(s.shape):
                    raise ValueError(f"tensor '{s.name}' is wanted with shapes {seen[s.name].shape} and {s.shape}")
                seen.setdefault(s.name, s)
        return list(seen.values())

    def bind(self, store: WeightStore) -> None:
        for p in self.parts():
            p.bind(store)
        store.release()

    def kernels(self) -> List[str]:
        return sorted({k for p in self.parts() for k in p.kernels()})

    def cache_needs(self) -> List[Optional[KVNeed]]:
        """Per schedule entry: the key/value need of an entry that keeps a cache, else None."""
        return [self.blocks[e.block].cache_need() if e.cache_of is None else None for e in self.schedule]

    def state_needs(self) -> List[Optional[StateNeed]]:
        return [self.blocks[e.block].state_need() for e in self.schedule]

    def capturable(self) -> bool:
        """Whether decode steps can be recorded into CUDA graphs: every block says so of its own parts."""
        return all(b.capturable() for b in self.blocks)

    def step_work(self, n_tokens: int, kv_tokens: int, n_want: int = None):
        """{bucket: (bytes, flops)} of one step, summed over the schedule's entries and the head."""
        total = {}
        runs = [self.blocks[e.block] for e in self.schedule]
        for part in runs:
            for sub in (part.parts() if hasattr(part, "parts") else [part]):
                for bucket, (b, f) in sub.step_work(n_tokens, kv_tokens).items():
                    tb, tf = total.get(bucket, (0.0, 0.0))
                    total[bucket] = (tb + b, tf + f)
        for bucket, (b, f) in self.head.step_work(n_tokens if n_want is None else n_want, kv_tokens).items():
            tb, tf = total.get(bucket, (0.0, 0.0))
            total[bucket] = (tb + b, tf + f)
        return total

    # ---- one step ------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, layer_caches: Sequence[LayerCache]) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the schedule; float32 logits [n_want, vocab] (None if
        nothing is wanted)."""
        x = self.embedding.forward(ctx.tokens)
        pending = None
        dump = ctx.debug.get("layer_sums") if ctx.debug is not None else None
        for i, (e, cache) in enumerate(zip(self.schedule, layer_caches)):
            x, pending = self.blocks[e.block].forward(x, pending, ctx, cache)
            if dump is not None:             # sum and sum of magnitudes of the residual stream after this layer
                full = x if pending is None else x + pending.float()
                dump.append((i, full.sum(dim=1, dtype=torch.float64), full.abs().sum(dim=1, dtype=torch.float64)))
        if ctx.n_want == 0:
            return None
        xn = self.final_norm.forward(x, ctx.act_dtype, rows=ctx.want_rows, add=pending)
        return self.head.forward(xn)
