"""Pre-norm block: x += mixer(norm(x)); x += feed_forward(norm(x))
(src/engine/tq_transformer.c:2494, 2268, 2685, 2701).

The residual sums are fused into the norm that follows them: a block receives the previous
sub-layer's output as `pending` and hands its own feed-forward output on the same way, so each
sum is one fp32 pass together with the next norm's statistics."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..weights.loader import WeightSpec, WeightStore
from .base import Block, FeedForward, KVNeed, LayerCache, Mixer, Norm, StateNeed, StepContext


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def parts(self):
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def cache_need(self) -> Optional[KVNeed]:
        return self.mixer.cache_need()

    def state_need(self) -> Optional[StateNeed]:
        return self.mixer.state_need()

    def capturable(self) -> bool:
        return self.mixer.capturable() and self.ffn.capturable()

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def bind(self, store: WeightStore) -> None:
        for p in self.parts():
            p.bind(store)

    def kernels(self) -> List[str]:
        return [k for p in self.parts() for k in p.kernels()]

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, torch.Tensor]:
        if pending is None:
            xn = self.mixer_norm.forward(x, ctx.act_dtype)
        else:
            xn = self.mixer_norm.add_forward(x, pending, ctx.act_dtype)
        y = self.mixer.forward(xn, ctx, cache)
        xn = self.ffn_norm.add_forward(x, y, ctx.act_dtype)
        return x, self.ffn.forward(xn, ctx)
