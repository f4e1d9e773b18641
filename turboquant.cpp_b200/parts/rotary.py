"""Rotary position encoding: for pair index i < hd/2, freq_i = theta^(-2i/hd), angle = pos*freq_i,
(a, b) <- (a cos - b sin, a sin + b cos) (src/engine/tq_ops.c:1418-1448).

pairing "half" rotates (x[i], x[i+hd/2]), the layout of safetensors checkpoints of this family;
"interleaved" rotates (x[2i], x[2i+1]) as the reference does.  The reference recomputes
powf/cosf/sinf for every head of every token; here cos and sin are float32 tables over positions,
built once (angles in float64, rounded once to float32)."""
from __future__ import annotations

from typing import Optional

import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_position: int, pairing: str = "half"):
        if head_dim % 2:
            raise ValueError(f"rotary: head size {head_dim} must be even")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary: pairing must be 'half' or 'interleaved', got '{pairing}'")
        if not theta > 0 or max_position < 1:
            raise ValueError(f"rotary: theta {theta} and max_position {max_position} must be positive")
        self.head_dim, self.theta, self.max_position, self.pairing = int(head_dim), float(theta), int(max_position), pairing
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        if self.cos is not None and self.cos.device == torch.device(device):
            return
        i = torch.arange(self.head_dim // 2, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.head_dim)
        ang = torch.arange(self.max_position, dtype=torch.float64)[:, None] * freq[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(device).contiguous()

    def tables(self):
        return self.cos, self.sin, self.pairing


register_position_encoding("rotary", RotaryEncoding)
