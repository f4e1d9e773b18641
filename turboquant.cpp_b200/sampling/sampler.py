"""Greedy and temperature / top-p sampling from the step's logits.

The reference samples with argmax when temperature <= 0 or top_p <= 0 and with a temperature-scaled
nucleus otherwise (src/engine/tq_generate.c:30-40, 81-156); it keeps one xorshift64* state per
generation call (:53-58), so a draw depends on everything sampled before it.  Here each draw's
uniform number is a pure function of (seed, index of the request, index of the generated token):
a request's tokens do not depend on what else is in its batch.

Before it samples, the reference lowers the logits of the last tokens of the request (rep_penalty 1.1
over rep_window 32 by default, include/turboquant/tq_engine.h:408-409, src/engine/tq_generate.c:586-600).
Here the penalty is off unless asked for (rep_penalty > 1), so that greedy output is the model's argmax.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import sampling as KS

_M = (1 << 64) - 1


def _mix(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniforms_for(seed: int, requests: Sequence[int], steps: Sequence[int]) -> np.ndarray:
    """float32 uniforms in [0, 1): splitmix64 over (seed, request, step), top 24 bits."""
    with np.errstate(over="ignore"):
        r = np.asarray(requests, dtype=np.uint64)
        s = np.asarray(steps, dtype=np.uint64)
        z = (np.uint64(int(seed) & _M) * np.uint64(0x9E3779B97F4A7C15) + r * np.uint64(0xBF58476D1CE4E5B9)
             + s * np.uint64(0x94D049BB133111EB) + np.uint64(0x2545F4914F6CDD1D))
        z = _mix(_mix(z))
    return ((z >> np.uint64(40)).astype(np.float64) / float(1 << 24)).astype(np.float32)


REP_WINDOW_MAX = 128      # the reference keeps at most this many recent tokens (src/engine/tq_generate.c:367)


class Sampler:
    def __init__(self, temperature: float = 0.0, top_p: float = 1.0, seed: int = 42, rep_penalty: float = 1.0,
                 rep_window: int = 32):
        self.temperature, self.top_p = float(temperature), float(top_p)
        self.seed = int(seed) if int(seed) != 0 else 42      # 0 means "the default", as in the reference's CLI
        self.rep_penalty = float(rep_penalty)
        self.rep_window = max(0, min(int(rep_window), REP_WINDOW_MAX))
        self._work: Optional[torch.Tensor] = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_p <= 0.0

    @property
    def penalizes(self) -> bool:
        """Whether sample() wants each request's recent tokens."""
        return self.rep_penalty > 1.0 and self.rep_window > 0

    def sample(self, logits: torch.Tensor, requests: Sequence[int], steps: Sequence[int],
               recent: Optional[Sequence[Sequence[int]]] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row of float32 logits [R, V] (int32, on the device).  recent: for each row the tokens
        of its request so far (prompt, then generated); with a repetition penalty the last rep_window of them
        lower their logits first, in place.  out: where to put the tokens (int32 [R] on the logits' device)."""
        R, V = logits.shape
        if out is None:
            out = torch.empty(R, dtype=torch.int32, device=logits.device)
        elif out.shape != (R,) or out.dtype != torch.int32 or out.device != logits.device or not out.is_contiguous():
            raise ValueError(f"sample: out must be a contiguous int32 tensor of {R} elements on {logits.device}")
        if self.penalizes and recent is not None:
            W = self.rep_window
            table = np.full((R, W), -1, dtype=np.int32)
            for r, toks in enumerate(recent):
                tail = list(toks)[-W:]
                table[r, :len(tail)] = tail
            KS.rep_penalty(logits, torch.from_numpy(table).to(logits.device, non_blocking=True), self.rep_penalty)
        if self.greedy:
            return KS.argmax_rows(logits, out)
        u = torch.from_numpy(uniforms_for(self.seed, requests, steps)).to(logits.device, non_blocking=True)
        if self._work is None or self._work.numel() < R * V or self._work.device != logits.device:
            self._work = torch.empty(R * V, dtype=torch.float32, device=logits.device)
        return KS.sample_rows(logits, self.temperature, self.top_p, u, self._work, out)
