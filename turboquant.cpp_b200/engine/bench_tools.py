"""The command line's built-in measurements, after the reference's --bench-prefill and
--bench-memory modes (tools/quant.c:804-859 and :726-797): prompt speed, and decode speed at
growing context lengths.  Synthetic token ids; times from CUDA events."""
from __future__ import annotations

import sys

import torch

from .step import StepEntry


def _time_ms(fn) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


def bench_prefill(m, n_tokens: int = 0, file=sys.stderr) -> float:
    eng = m.engine
    n = n_tokens or min(2048, m.context_length)
    toks = [i % eng.model.vocab_size for i in range(n)]
    best = float("inf")
    for _ in range(3):
        seq = eng.open()
        ms = _time_ms(lambda: eng.step([StepEntry(seq, toks, [n - 1])]))
        eng.close(seq)
        best = min(best, ms)
    print(f"PREFILL_CSV:{n},{best:.3f},{n / best * 1e3:.1f}", file=file)
    print(f"prefill: {n} tokens in {best:.2f} ms ({n / best * 1e3:.0f} tok/s)", file=file)
    return n / best * 1e3


def bench_memory(m, file=sys.stderr) -> None:
    eng = m.engine
    V = eng.model.vocab_size
    for ctx in (16, 64, 256, 1024, 4096, 16384):
        if ctx + 20 > m.context_length:
            break
        seq = eng.open()
        eng.step([StepEntry(seq, [i % V for i in range(ctx)], [])])
        ms = _time_ms(lambda: [eng.step([StepEntry(seq, [1], [0])]) for _ in range(20)])
        eng.close(seq)
        print(f"BENCH_CSV:{ctx},{20 / ms * 1e3:.2f}", file=file)
        print(f"decode at context {ctx}: {20 / ms * 1e3:.1f} tok/s", file=file)
