"""Dense SwiGLU feed-forward: down(silu(gate x) * (up x)) (src/engine/tq_transformer.c:2771-2806;
silu with exact exp, src/engine/tq_ops.c:1454-1478).  Gate and up are one fused product."""
from __future__ import annotations

from typing import List

import torch

from ..kernels import elementwise as K
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import FeedForward, StepContext, register_feed_forward


class SwiGLUFeedForward(FeedForward):
    def __init__(self, prefix: str, hidden: int, intermediate: int):
        if hidden < 1 or intermediate < 1:
            raise ValueError(f"feed-forward '{prefix}': sizes must be positive, got {hidden}, {intermediate}")
        self.prefix, self.hidden, self.intermediate = prefix, int(hidden), int(intermediate)
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        p, H, I = self.prefix, self.hidden, self.intermediate
        return [WeightSpec(p + "gate_proj.weight", (I, H)), WeightSpec(p + "up_proj.weight", (I, H)),
                WeightSpec(p + "down_proj.weight", (H, I))]

    def bind(self, store: WeightStore) -> None:
        p = self.prefix
        g, u = store.take(p + "gate_proj.weight"), store.take(p + "up_proj.weight")
        dt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous()
        self.w_down = store.get(p + "down_proj.weight")

    def kernels(self) -> List[str]:
        return ["elementwise"]

    def step_work(self, n_tokens, kv_tokens):
        wb = lambda w: 0 if w is None else w.numel() * w.element_size()
        return {"matmul": (wb(self.w_gate_up) + wb(self.w_down), 6.0 * n_tokens * self.hidden * self.intermediate)}

    def forward(self, xn: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(xn, self.w_gate_up, out_dtype=torch.float32)     # gate and up stay fp32 until the product
        h = torch.empty((xn.shape[0], self.intermediate), dtype=ctx.act_dtype, device=xn.device)
        K.silu_mul(gu, h)
        return linear(h, self.w_down, out_dtype=torch.float32)


register_feed_forward("swiglu", SwiGLUFeedForward)
